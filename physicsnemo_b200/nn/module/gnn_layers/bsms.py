"""Bi-stride multi-scale message passing (a graph U-Net over a hierarchy of coarsened meshes).

Parity: ``physicsnemo/nn/module/gnn_layers/bsms.py`` (``BistrideGraphMessagePassing``,
``GraphMessagePassing``, ``WeightedEdgeConv``, ``Unpool``, ``degree``, ``scatter_sum``): on the way
down every level runs one message-passing block, then features and positions are transferred to
the kept nodes by a normalised weighted edge convolution; on the way up features are un-pooled,
convolved back with the stored weights, processed and added to the skip.  Tensors may carry a
leading batch dimension.  Scatter sums go through ``index_add_`` on the node axis.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .mesh_graph_mlp import MeshGraphMLP


def degree(index: torch.Tensor, num_nodes: Optional[int] = None, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    n = int(index.max()) + 1 if index.numel() else 0
    return torch.zeros(n, dtype=dtype, device=index.device).index_add_(0, index, torch.ones(index.shape[0], dtype=dtype, device=index.device))


def scatter_sum(src: torch.Tensor, index: torch.Tensor, dim: int = -1, out: Optional[torch.Tensor] = None,
                dim_size: Optional[int] = None) -> torch.Tensor:
    """Sum ``src`` slices along ``dim`` into rows given by the 1-D ``index``."""
    dim = dim % src.dim()
    if out is None:
        size = list(src.shape)
        size[dim] = dim_size if dim_size is not None else (int(index.max()) + 1 if index.numel() else 0)
        out = torch.zeros(size, dtype=src.dtype, device=src.device)
    return out.index_add_(dim, index, src)


def _take(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    if x.dim() == 3:
        return x[:, idx]
    if x.dim() == 2:
        return x[idx]
    raise ValueError(f"Only implemented for dim 2 and 3, got {tuple(x.shape)}")


class GraphMessagePassing(nn.Module):
    """One residual message-passing block; edge inputs are (direction, length, x_i, x_j)."""

    def __init__(self, latent_dim, hidden_layer, pos_dim):
        super().__init__()
        self.mlp_node = MeshGraphMLP(2 * latent_dim, latent_dim, latent_dim, hidden_layer)
        self.mlp_edge = MeshGraphMLP(2 * latent_dim + pos_dim + 1, latent_dim, latent_dim, hidden_layer)
        self.pos_dim = pos_dim

    def forward(self, x, g, pos):
        i, j = g[0], g[1]
        x_i, x_j = _take(x, i), _take(x, j)
        d = _take(pos, i) - _take(pos, j)
        fiber = torch.cat([d, torch.norm(d, dim=-1, keepdim=True)], dim=-1)
        if x.dim() == 3 and pos.dim() == 2:
            fiber = fiber.unsqueeze(0).expand(x.shape[0], -1, -1)
        edge = self.mlp_edge(torch.cat([fiber, x_i, x_j], dim=-1))
        agg = scatter_sum(edge, j, dim=-2, dim_size=x.shape[-2])
        return self.mlp_node(torch.cat([x, agg], dim=-1)) + x


class WeightedEdgeConv(nn.Module):
    def __init__(self, *args):
        super().__init__()

    def forward(self, x, g, ew, aggragating=True):
        i, j = g[0], g[1]
        info = _take(x, i if aggragating else j) * ew.unsqueeze(-1)
        return scatter_sum(info, j if aggragating else i, dim=-2, dim_size=x.shape[-2])

    @torch.no_grad()
    def cal_ew(self, w, g):
        """Edge weights that split every sender's weight evenly over its edges and normalise per receiver."""
        i, j = g[0], g[1]
        normed = w.squeeze(-1) / degree(i, dtype=torch.float, num_nodes=w.shape[0])
        sent = normed[i]
        received = scatter_sum(sent, j, dim=-1, dim_size=normed.size(0)) + 1e-12
        return sent / received[j], received


class Unpool(nn.Module):
    def __init__(self, *args):
        super().__init__()

    def forward(self, h, pre_node_num, idx):
        out = h.new_zeros((*h.shape[:-2], pre_node_num, h.shape[-1]))
        if h.dim() == 2:
            out[idx] = h
        else:
            out[:, idx] = h
        return out


class BistrideGraphMessagePassing(nn.Module):
    def __init__(self, unet_depth, latent_dim, hidden_layer, pos_dim):
        super().__init__()
        self.bottom_gmp = GraphMessagePassing(latent_dim, hidden_layer, pos_dim)
        self.down_gmps, self.up_gmps, self.unpools = nn.ModuleList(), nn.ModuleList(), nn.ModuleList()
        self.unet_depth = unet_depth
        self.edge_conv = WeightedEdgeConv()
        for _ in range(unet_depth):
            self.down_gmps.append(GraphMessagePassing(latent_dim, hidden_layer, pos_dim))
            self.up_gmps.append(GraphMessagePassing(latent_dim, hidden_layer, pos_dim))
            self.unpools.append(Unpool())

    def forward(self, h, m_ids, m_gs, pos):
        skips, positions, weights = [], [], []
        w = pos.new_ones((pos.shape[-2], 1))
        for lvl in range(self.unet_depth):
            h = self.down_gmps[lvl](h, m_gs[lvl], pos)
            skips.append(h)
            positions.append(pos)
            ew, w = self.edge_conv.cal_ew(w, m_gs[lvl])
            h = _take(self.edge_conv(h, m_gs[lvl], ew), m_ids[lvl])
            pos = _take(self.edge_conv(pos, m_gs[lvl], ew), m_ids[lvl])
            weights.append(ew)
            w = w[m_ids[lvl]]
        h = self.bottom_gmp(h, m_gs[self.unet_depth], pos)
        for k in range(self.unet_depth):
            lvl = self.unet_depth - k - 1
            g = m_gs[lvl]
            h = self.unpools[k](h, skips[lvl].shape[-2], m_ids[lvl])
            h = self.edge_conv(h, g, weights[lvl], aggragating=False)
            h = self.up_gmps[k](h, g, positions[lvl]) + skips[lvl]
        return h

"""Mesh-reduced encoder / decoder: MeshGraphNet on the full mesh, k-NN interpolation to pivotal nodes.

Parity: ``physicsnemo/models/mesh_reduced/mesh_reduced.py`` (``Mesh_Reduced``: ``encoder_processor``,
``decoder_processor``, ``PivotalNorm``; ``knn_interpolate`` with inverse-squared-distance weights;
``encode`` mesh → pivotal and ``decode`` pivotal → mesh over a batch of identical meshes).  The
reference depends on ``torch_cluster`` / ``torch_scatter``; here neighbours come from this package's
``knn`` functional, one call per batch item (all items share the same positions, so the neighbour
table is computed once and reused), and the weighted sums are dense ``[N, k]`` reductions.
"""
from __future__ import annotations

from typing import Literal, Tuple

import torch
from torch import Tensor

from ..meshgraphnet.meshgraphnet import MeshGraphNet


class Mesh_Reduced(torch.nn.Module):
    def __init__(self, input_dim_nodes: int, input_dim_edges: int, output_decode_dim: int, output_encode_dim: int = 3,
                 processor_size: int = 15, num_layers_node_processor: int = 2, num_layers_edge_processor: int = 2,
                 hidden_dim_processor: int = 128, hidden_dim_node_encoder: int = 128, num_layers_node_encoder: int = 2,
                 hidden_dim_edge_encoder: int = 128, num_layers_edge_encoder: int = 2, hidden_dim_node_decoder: int = 128,
                 num_layers_node_decoder: int = 2, k: int = 3, aggregation: Literal["sum", "mean"] = "mean"):
        super().__init__()
        self.knn_encoder_already = False
        self.knn_decoder_already = False
        common = (processor_size, "relu", num_layers_node_processor, num_layers_edge_processor, hidden_dim_processor,
                  hidden_dim_node_encoder, num_layers_node_encoder, hidden_dim_edge_encoder, num_layers_edge_encoder,
                  hidden_dim_node_decoder, num_layers_node_decoder, aggregation)
        self.encoder_processor = MeshGraphNet(input_dim_nodes, input_dim_edges, output_encode_dim, *common)
        self.decoder_processor = MeshGraphNet(output_encode_dim, input_dim_edges, output_decode_dim, *common)
        self.k = k
        self.PivotalNorm = torch.nn.LayerNorm(output_encode_dim)
        self.input_dim_nodes, self.input_dim_edges = input_dim_nodes, input_dim_edges
        self.output_encode_dim, self.output_decode_dim = output_encode_dim, output_decode_dim

    def knn_interpolate(self, x: Tensor, pos_x: Tensor, pos_y: Tensor, batch_x: Tensor | None = None,
                        batch_y: Tensor | None = None, k: int = 3, num_workers: int = 1) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
        """Values at ``pos_y`` from the ``k`` nearest ``pos_x`` of the same batch item, weights ``1 / d²``.

        Returns ``(y, col, row, weights)`` with ``col`` / ``row`` the flattened source / target indices.
        """
        from ...nn.functional.neighbors import knn

        with torch.no_grad():
            if batch_x is None:
                idx, _ = knn(pos_x.float(), pos_y.float(), k)
            else:
                idx = torch.empty(pos_y.shape[0], k, dtype=torch.long, device=pos_y.device)
                for b in torch.unique(batch_y).tolist():
                    sx, sy = (batch_x == b).nonzero().squeeze(1), (batch_y == b).nonzero().squeeze(1)
                    local, _ = knn(pos_x[sx].float(), pos_y[sy].float(), k)
                    idx[sy] = sx[local.long()]
            idx = idx.long()
            d2 = (pos_x[idx] - pos_y[:, None]).pow(2).sum(-1, keepdim=True)
            w = 1.0 / d2.clamp_min(1e-16)                                        # [Ny, k, 1]
        y = (x[idx] * w).sum(1) / w.sum(1)
        row = torch.arange(pos_y.shape[0], device=pos_y.device).repeat_interleave(k)
        return y.float(), idx.reshape(-1), row, w.reshape(-1, 1)

    @staticmethod
    def _batch_of(graph, n_nodes: int, device) -> Tuple[Tensor, int]:
        batch = getattr(graph, "batch", None)
        if batch is None:
            return torch.zeros(n_nodes, dtype=torch.long, device=device), 1
        return batch, int(batch.max().item()) + 1 if batch.numel() > 0 else 1

    def _batched_positions(self, graph, x, position_mesh, position_pivotal):
        batch_mesh, bs = self._batch_of(graph, position_mesh.shape[0], x.device)
        batch_piv = torch.arange(bs, device=x.device).repeat_interleave(len(position_pivotal))
        return position_mesh.repeat(bs, 1), position_pivotal.repeat(bs, 1), batch_mesh, batch_piv

    def encode(self, x: Tensor, edge_features: Tensor, graph, position_mesh: Tensor, position_pivotal: Tensor) -> Tensor:
        if not torch.compiler.is_compiling():
            if x.ndim != 2:
                raise ValueError(f"Expected 2D node features (N_nodes, D_in) but got shape {tuple(x.shape)}")
            if edge_features.ndim != 2:
                raise ValueError(f"Expected 2D edge features (N_edges, D_in) but got shape {tuple(edge_features.shape)}")
            if position_mesh.ndim != 2 or position_pivotal.ndim != 2:
                raise ValueError(f"Expected position tensors to be 2D, got {tuple(position_mesh.shape)} and {tuple(position_pivotal.shape)}")
        x = self.PivotalNorm(self.encoder_processor(x, edge_features, graph))
        pm, pp, bm, bp = self._batched_positions(graph, x, position_mesh, position_pivotal)
        return self.knn_interpolate(x=x, pos_x=pm, pos_y=pp, batch_x=bm, batch_y=bp, k=self.k)[0]

    def decode(self, x: Tensor, edge_features: Tensor, graph, position_mesh: Tensor, position_pivotal: Tensor) -> Tensor:
        if not torch.compiler.is_compiling():
            if edge_features.ndim != 2 or edge_features.shape[1] != self.input_dim_edges:
                raise ValueError(f"Expected tensor of shape (N_edges, {self.input_dim_edges}) but got tensor of shape {tuple(edge_features.shape)}")
            if position_mesh.ndim != 2 or position_pivotal.ndim != 2:
                raise ValueError(f"Expected position tensors to be 2D, got shapes {tuple(position_mesh.shape)} and {tuple(position_pivotal.shape)}")
        pm, pp, bm, bp = self._batched_positions(graph, x, position_mesh, position_pivotal)
        x = self.knn_interpolate(x=x, pos_x=pp, pos_y=pm, batch_x=bp, batch_y=bm, k=self.k)[0]
        return self.decoder_processor(x, edge_features, graph)

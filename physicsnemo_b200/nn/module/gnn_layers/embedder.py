"""Feature embedders of the GraphCast encoder and decoder.

Parity: ``physicsnemo/nn/module/gnn_layers/embedder.py`` (``GraphCastEncoderEmbedder`` with the four
MLPs ``grid_node_mlp``, ``mesh_node_mlp``, ``mesh_edge_mlp``, ``grid2mesh_edge_mlp``;
``GraphCastDecoderEmbedder`` with ``mesh2grid_edge_mlp``).
"""
from typing import Tuple

import torch.nn as nn
from torch import Tensor

from .mesh_graph_mlp import MeshGraphMLP


def _mlp(input_dim, output_dim, hidden_dim, hidden_layers, activation_fn, norm_type, recompute_activation):
    return MeshGraphMLP(input_dim=input_dim, output_dim=output_dim, hidden_dim=hidden_dim, hidden_layers=hidden_layers,
                        activation_fn=activation_fn, norm_type=norm_type, recompute_activation=recompute_activation)


class GraphCastEncoderEmbedder(nn.Module):
    def __init__(self, input_dim_grid_nodes: int = 474, input_dim_mesh_nodes: int = 3, input_dim_edges: int = 4,
                 output_dim: int = 512, hidden_dim: int = 512, hidden_layers: int = 1,
                 activation_fn: nn.Module = nn.SiLU(), norm_type: str = "LayerNorm", recompute_activation: bool = False):
        super().__init__()
        common = (output_dim, hidden_dim, hidden_layers, activation_fn, norm_type, recompute_activation)
        self.grid_node_mlp = _mlp(input_dim_grid_nodes, *common)
        self.mesh_node_mlp = _mlp(input_dim_mesh_nodes, *common)
        self.mesh_edge_mlp = _mlp(input_dim_edges, *common)
        self.grid2mesh_edge_mlp = _mlp(input_dim_edges, *common)

    def forward(self, grid_nfeat: Tensor, mesh_nfeat: Tensor, g2m_efeat: Tensor,
                mesh_efeat: Tensor) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
        return (self.grid_node_mlp(grid_nfeat), self.mesh_node_mlp(mesh_nfeat), self.grid2mesh_edge_mlp(g2m_efeat),
                self.mesh_edge_mlp(mesh_efeat))


class GraphCastDecoderEmbedder(nn.Module):
    def __init__(self, input_dim_edges: int = 4, output_dim: int = 512, hidden_dim: int = 512, hidden_layers: int = 1,
                 activation_fn: nn.Module = nn.SiLU(), norm_type: str = "LayerNorm", recompute_activation: bool = False):
        super().__init__()
        self.mesh2grid_edge_mlp = _mlp(input_dim_edges, output_dim, hidden_dim, hidden_layers, activation_fn, norm_type,
                                       recompute_activation)

    def forward(self, m2g_efeat: Tensor) -> Tensor:
        return self.mesh2grid_edge_mlp(m2g_efeat)

"""Bipartite grid → mesh encoder block.

Parity: ``physicsnemo/nn/module/gnn_layers/mesh_graph_encoder.py`` (``edge_mlp`` on (edge, grid
source, mesh destination) features, sum / mean aggregation onto the mesh nodes, residual
``dst_node_mlp`` on ``cat(aggregated, mesh)`` and residual ``src_node_mlp`` on the grid nodes).
"""
from typing import Tuple

import torch.nn as nn
from torch import Tensor

from ._bipartite import BipartiteMessagePassing


class MeshGraphEncoder(BipartiteMessagePassing):
    """Returns ``(grid, mesh)``: the mesh nodes receive the aggregated grid → mesh messages, the grid nodes get their own
    residual MLP."""

    def __init__(self, aggregation: str = "sum", input_dim_src_nodes: int = 512, input_dim_dst_nodes: int = 512,
                 input_dim_edges: int = 512, output_dim_src_nodes: int = 512, output_dim_dst_nodes: int = 512,
                 output_dim_edges: int = 512, hidden_dim: int = 512, hidden_layers: int = 1,
                 activation_fn: nn.Module = nn.SiLU(), norm_type: str = "LayerNorm", do_concat_trick: bool = False,
                 recompute_activation: bool = False):
        super().__init__()
        self.aggregation = aggregation
        shared = {"norm_type": norm_type, "activation_fn": activation_fn, "hidden_layers": hidden_layers, "hidden_dim": hidden_dim,
                  "recompute_activation": recompute_activation}
        self._make_mlps(src_width=input_dim_src_nodes, dst_width=input_dim_dst_nodes, edge_width=input_dim_edges,
                        edge_out=output_dim_edges, concat_trick=do_concat_trick, shared=shared)
        self.src_node_mlp = self.node_mlp_for(input_dim_src_nodes, output_dim_src_nodes, shared)
        self.dst_node_mlp = self.node_mlp_for(output_dim_edges + input_dim_dst_nodes, output_dim_dst_nodes, shared)

    def forward(self, g2m_efeat: Tensor, grid_nfeat: Tensor, mesh_nfeat: Tensor, graph) -> Tuple[Tensor, Tensor]:
        incoming = self.messages_to_dst(g2m_efeat, grid_nfeat, mesh_nfeat, graph)
        mesh_new = self.dst_node_mlp((incoming, mesh_nfeat), post=mesh_nfeat)
        grid_new = self.src_node_mlp(grid_nfeat, post=grid_nfeat)
        return grid_new, mesh_new

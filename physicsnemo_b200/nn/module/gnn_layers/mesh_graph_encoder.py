"""Bipartite grid → mesh encoder block.

Parity: ``physicsnemo/nn/module/gnn_layers/mesh_graph_encoder.py`` (``edge_mlp`` on (edge, grid
source, mesh destination) features, sum / mean aggregation onto the mesh nodes, residual
``dst_node_mlp`` on ``cat(aggregated, mesh)`` and residual ``src_node_mlp`` on the grid nodes).
"""
from typing import Tuple

import torch.nn as nn
from torch import Tensor

from .mesh_graph_mlp import MeshGraphEdgeMLPConcat, MeshGraphEdgeMLPSum, MeshGraphMLP
from .utils import aggregate


class MeshGraphEncoder(nn.Module):
    def __init__(self, aggregation: str = "sum", input_dim_src_nodes: int = 512, input_dim_dst_nodes: int = 512,
                 input_dim_edges: int = 512, output_dim_src_nodes: int = 512, output_dim_dst_nodes: int = 512,
                 output_dim_edges: int = 512, hidden_dim: int = 512, hidden_layers: int = 1,
                 activation_fn: nn.Module = nn.SiLU(), norm_type: str = "LayerNorm", do_concat_trick: bool = False,
                 recompute_activation: bool = False):
        super().__init__()
        self.aggregation = aggregation
        edge_cls = MeshGraphEdgeMLPSum if do_concat_trick else MeshGraphEdgeMLPConcat
        kw = dict(hidden_dim=hidden_dim, hidden_layers=hidden_layers, activation_fn=activation_fn, norm_type=norm_type,
                  recompute_activation=recompute_activation)
        self.edge_mlp = edge_cls(efeat_dim=input_dim_edges, src_dim=input_dim_src_nodes, dst_dim=input_dim_dst_nodes,
                                 output_dim=output_dim_edges, **kw)
        self.src_node_mlp = MeshGraphMLP(input_dim=input_dim_src_nodes, output_dim=output_dim_src_nodes, **kw)
        self.dst_node_mlp = MeshGraphMLP(input_dim=input_dim_dst_nodes + output_dim_edges, output_dim=output_dim_dst_nodes, **kw)

    def forward(self, g2m_efeat: Tensor, grid_nfeat: Tensor, mesh_nfeat: Tensor, graph) -> Tuple[Tensor, Tensor]:
        efeat = self.edge_mlp(g2m_efeat, (grid_nfeat, mesh_nfeat), graph)
        agg = aggregate(efeat, mesh_nfeat.shape[0], graph, self.aggregation)
        # the MLP takes the two column blocks without materialising their concatenation; residual added in its epilogue
        mesh_out = self.dst_node_mlp((agg, mesh_nfeat), post=mesh_nfeat)
        grid_out = self.src_node_mlp(grid_nfeat, post=grid_nfeat)
        return grid_out, mesh_out

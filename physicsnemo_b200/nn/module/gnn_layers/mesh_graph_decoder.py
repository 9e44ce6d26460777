"""Bipartite mesh → grid decoder block.

Parity: ``physicsnemo/nn/module/gnn_layers/mesh_graph_decoder.py`` (``edge_mlp`` on (edge, mesh
source, grid destination), aggregation onto the grid nodes, residual ``node_mlp``).
"""
import torch.nn as nn
from torch import Tensor

from .mesh_graph_mlp import MeshGraphEdgeMLPConcat, MeshGraphEdgeMLPSum, MeshGraphMLP
from .utils import aggregate


class MeshGraphDecoder(nn.Module):
    def __init__(self, aggregation: str = "sum", input_dim_src_nodes: int = 512, input_dim_dst_nodes: int = 512,
                 input_dim_edges: int = 512, output_dim_dst_nodes: int = 512, output_dim_edges: int = 512,
                 hidden_dim: int = 512, hidden_layers: int = 1, activation_fn: nn.Module = nn.SiLU(),
                 norm_type: str = "LayerNorm", do_concat_trick: bool = False, recompute_activation: bool = False):
        super().__init__()
        self.aggregation = aggregation
        edge_cls = MeshGraphEdgeMLPSum if do_concat_trick else MeshGraphEdgeMLPConcat
        kw = dict(hidden_dim=hidden_dim, hidden_layers=hidden_layers, activation_fn=activation_fn, norm_type=norm_type,
                  recompute_activation=recompute_activation)
        self.edge_mlp = edge_cls(efeat_dim=input_dim_edges, src_dim=input_dim_src_nodes, dst_dim=input_dim_dst_nodes,
                                 output_dim=output_dim_edges, **kw)
        self.node_mlp = MeshGraphMLP(input_dim=input_dim_dst_nodes + output_dim_edges, output_dim=output_dim_dst_nodes, **kw)

    def forward(self, m2g_efeat: Tensor, grid_nfeat: Tensor, mesh_nfeat: Tensor, graph) -> Tensor:
        efeat = self.edge_mlp(m2g_efeat, (mesh_nfeat, grid_nfeat), graph)
        agg = aggregate(efeat, grid_nfeat.shape[0], graph, self.aggregation)
        return self.node_mlp((agg, grid_nfeat), post=grid_nfeat)

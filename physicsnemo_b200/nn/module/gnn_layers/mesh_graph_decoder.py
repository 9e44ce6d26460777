"""Bipartite mesh → grid decoder block.

Parity: ``physicsnemo/nn/module/gnn_layers/mesh_graph_decoder.py`` (``edge_mlp`` on (edge, mesh
source, grid destination), aggregation onto the grid nodes, residual ``node_mlp``).
"""
import torch.nn as nn
from torch import Tensor

from ._bipartite import BipartiteMessagePassing


class MeshGraphDecoder(BipartiteMessagePassing):
    """``grid ← grid + node_mlp(cat(Σ_edges edge_mlp(e, mesh_src, grid_dst), grid))``."""

    def __init__(self, aggregation: str = "sum", input_dim_src_nodes: int = 512, input_dim_dst_nodes: int = 512,
                 input_dim_edges: int = 512, output_dim_dst_nodes: int = 512, output_dim_edges: int = 512,
                 hidden_dim: int = 512, hidden_layers: int = 1, activation_fn: nn.Module = nn.SiLU(),
                 norm_type: str = "LayerNorm", do_concat_trick: bool = False, recompute_activation: bool = False):
        super().__init__()
        self.aggregation = aggregation
        shared = {"norm_type": norm_type, "activation_fn": activation_fn, "hidden_layers": hidden_layers, "hidden_dim": hidden_dim,
                  "recompute_activation": recompute_activation}
        self._make_mlps(src_width=input_dim_src_nodes, dst_width=input_dim_dst_nodes, edge_width=input_dim_edges,
                        edge_out=output_dim_edges, concat_trick=do_concat_trick, shared=shared)
        self.node_mlp = self.node_mlp_for(output_dim_edges + input_dim_dst_nodes, output_dim_dst_nodes, shared)

    def forward(self, m2g_efeat: Tensor, grid_nfeat: Tensor, mesh_nfeat: Tensor, graph) -> Tensor:
        incoming = self.messages_to_dst(m2g_efeat, mesh_nfeat, grid_nfeat, graph)
        # two column blocks, no materialised concatenation; the residual is added by the MLP's last kernel
        return self.node_mlp((incoming, grid_nfeat), post=grid_nfeat)

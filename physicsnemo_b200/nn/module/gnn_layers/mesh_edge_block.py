"""Edge update block (parity: ``physicsnemo/nn/module/gnn_layers/mesh_edge_block.py:31-97``)."""
import torch.nn as nn
from torch import Tensor

from .mesh_graph_mlp import MeshGraphEdgeMLPConcat, MeshGraphEdgeMLPSum


class MeshEdgeBlock(nn.Module):
    """``efeat ← efeat + MLP(efeat, nfeat[src], nfeat[dst])``; returns ``(efeat, nfeat)``."""

    def __init__(self, input_dim_nodes: int = 512, input_dim_edges: int = 512, output_dim: int = 512,
                 hidden_dim: int = 512, hidden_layers: int = 1, activation_fn: nn.Module = nn.SiLU(),
                 norm_type: str = "LayerNorm", do_concat_trick: bool = False, recompute_activation: bool = False):
        super().__init__()
        MLP = MeshGraphEdgeMLPSum if do_concat_trick else MeshGraphEdgeMLPConcat
        self.edge_mlp = MLP(efeat_dim=input_dim_edges, src_dim=input_dim_nodes, dst_dim=input_dim_nodes,
                            output_dim=output_dim, hidden_dim=hidden_dim, hidden_layers=hidden_layers,
                            activation_fn=activation_fn, norm_type=norm_type,
                            recompute_activation=recompute_activation)

    def forward(self, efeat: Tensor, nfeat: Tensor, graph):
        return self.edge_mlp(efeat, nfeat, graph, post=efeat), nfeat


class HybridMeshEdgeBlock(nn.Module):
    """Edge update with separate MLPs for mesh edges and world (contact) edges of one graph.

    Parity: ``physicsnemo/nn/module/gnn_layers/mesh_edge_block.py`` (``HybridMeshEdgeBlock``); the graph
    lists the mesh edges first and the world edges after them.
    """

    def __init__(self, input_dim_nodes: int = 512, input_dim_edges: int = 512, output_dim: int = 512,
                 hidden_dim: int = 512, hidden_layers: int = 1, activation_fn: nn.Module = nn.SiLU(),
                 norm_type: str = "LayerNorm", do_concat_trick: bool = False, recompute_activation: bool = False):
        super().__init__()
        from .mesh_graph_mlp import MeshGraphHeteroEdgeMLPConcat

        self.edge_mlp = MeshGraphHeteroEdgeMLPConcat(efeat_dim=input_dim_edges, src_dim=input_dim_nodes,
                                                     dst_dim=input_dim_nodes, output_dim=output_dim, hidden_dim=hidden_dim,
                                                     hidden_layers=hidden_layers, activation_fn=activation_fn,
                                                     norm_type=norm_type, recompute_activation=recompute_activation)

    def forward(self, mesh_efeat: Tensor, world_efeat: Tensor, nfeat: Tensor, graph):
        mesh_new, world_new = self.edge_mlp(mesh_efeat, world_efeat, nfeat, graph)
        return mesh_new + mesh_efeat, world_new + world_efeat, nfeat

"""Node update block (parity: ``physicsnemo/nn/module/gnn_layers/mesh_node_block.py:27-91``)."""
import torch
import torch.nn as nn
from torch import Tensor

from .... import ops
from .mesh_graph_mlp import MeshGraphMLP
from .utils import aggregate, aggregate_and_concat


class MeshNodeBlock(nn.Module):
    """``nfeat ← nfeat + MLP(cat(aggregate(efeat → dst), nfeat))``; returns ``(efeat, nfeat)``."""

    def __init__(self, aggregation: str = "sum", input_dim_nodes: int = 512, input_dim_edges: int = 512,
                 output_dim: int = 512, hidden_dim: int = 512, hidden_layers: int = 1,
                 activation_fn: nn.Module = nn.SiLU(), norm_type: str = "LayerNorm",
                 recompute_activation: bool = False):
        super().__init__()
        self.aggregation = aggregation
        self.node_mlp = MeshGraphMLP(input_dim=input_dim_nodes + input_dim_edges, output_dim=output_dim,
                                     hidden_dim=hidden_dim, hidden_layers=hidden_layers, activation_fn=activation_fn,
                                     norm_type=norm_type, recompute_activation=recompute_activation)

    def forward(self, efeat: Tensor, nfeat: Tensor, graph):
        if ops.fused_path_enabled(efeat) and efeat.dtype == torch.bfloat16 and nfeat.dtype == torch.bfloat16:
            agg = aggregate(efeat, nfeat.shape[0], graph, self.aggregation)
            return efeat, self.node_mlp((agg, nfeat), post=nfeat)
        cat_feat = aggregate_and_concat(efeat, nfeat, graph, self.aggregation)
        return efeat, self.node_mlp(cat_feat, post=nfeat)


class HybridMeshNodeBlock(nn.Module):
    """Node update aggregating mesh and world edge features together.

    Parity: ``physicsnemo/nn/module/gnn_layers/mesh_node_block.py`` (``HybridMeshNodeBlock``).
    """

    def __init__(self, aggregation: str = "sum", input_dim_nodes: int = 512, input_dim_edges: int = 512,
                 output_dim: int = 512, hidden_dim: int = 512, hidden_layers: int = 1,
                 activation_fn: nn.Module = nn.SiLU(), norm_type: str = "LayerNorm", recompute_activation: bool = False):
        super().__init__()
        self.aggregation = aggregation
        self.node_mlp = MeshGraphMLP(input_dim=input_dim_nodes + input_dim_edges, output_dim=output_dim,
                                     hidden_dim=hidden_dim, hidden_layers=hidden_layers, activation_fn=activation_fn,
                                     norm_type=norm_type, recompute_activation=recompute_activation)

    def forward(self, mesh_efeat: Tensor, world_efeat: Tensor, nfeat: Tensor, graph):
        agg = aggregate(torch.cat((mesh_efeat, world_efeat), dim=0), nfeat.shape[0], graph, self.aggregation)
        return mesh_efeat, world_efeat, self.node_mlp((agg, nfeat), post=nfeat)

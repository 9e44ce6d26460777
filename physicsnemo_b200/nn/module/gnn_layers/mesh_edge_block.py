"""Edge update blocks of the MeshGraphNet processor (parity: ``physicsnemo/nn/module/gnn_layers/mesh_edge_block.py:31-97``).

Both blocks own one ``edge_mlp`` (the state-dict key) and differ in the MLP behind it: one edge set, or separate
weights for the mesh edges and the world (contact) edges of a hybrid graph.
"""
import torch.nn as nn
from torch import Tensor

from . import mesh_graph_mlp as _mlps


class _EdgeBlock(nn.Module):
    """Builds ``self.edge_mlp`` from the block's sizes; ``_pick`` names the MLP class for a given concat-trick flag."""

    @staticmethod
    def _pick(do_concat_trick: bool):
        raise NotImplementedError

    def __init__(self, input_dim_nodes: int = 512, input_dim_edges: int = 512, output_dim: int = 512,
                 hidden_dim: int = 512, hidden_layers: int = 1, activation_fn: nn.Module = nn.SiLU(),
                 norm_type: str = "LayerNorm", do_concat_trick: bool = False, recompute_activation: bool = False):
        super().__init__()
        widths = {"src_dim": input_dim_nodes, "dst_dim": input_dim_nodes, "efeat_dim": input_dim_edges}
        trunk = {"hidden_layers": hidden_layers, "hidden_dim": hidden_dim, "output_dim": output_dim}
        extras = {"norm_type": norm_type, "activation_fn": activation_fn, "recompute_activation": recompute_activation}
        self.edge_mlp = self._pick(do_concat_trick)(**widths, **trunk, **extras)


class MeshEdgeBlock(_EdgeBlock):
    """``efeat ← efeat + MLP(efeat, nfeat[src], nfeat[dst])``; returns ``(efeat, nfeat)``.

    The residual is handed to the MLP (``post``), whose last kernel adds it while writing the result."""

    @staticmethod
    def _pick(do_concat_trick: bool):
        return _mlps.MeshGraphEdgeMLPSum if do_concat_trick else _mlps.MeshGraphEdgeMLPConcat

    def forward(self, efeat: Tensor, nfeat: Tensor, graph):
        updated = self.edge_mlp(efeat, nfeat, graph, post=efeat)
        return updated, nfeat


class HybridMeshEdgeBlock(_EdgeBlock):
    """Edge update with separate MLPs for mesh edges and world (contact) edges of one graph, whose edge list holds the
    mesh edges first and the world edges after them.  Returns ``(mesh_efeat, world_efeat, nfeat)``."""

    @staticmethod
    def _pick(do_concat_trick: bool):
        return _mlps.MeshGraphHeteroEdgeMLPConcat

    def forward(self, mesh_efeat: Tensor, world_efeat: Tensor, nfeat: Tensor, graph):
        deltas = self.edge_mlp(mesh_efeat, world_efeat, nfeat, graph)
        return deltas[0] + mesh_efeat, deltas[1] + world_efeat, nfeat

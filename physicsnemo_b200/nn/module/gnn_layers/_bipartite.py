"""Shared pieces of the bipartite encoder / decoder blocks of GraphCast-style models: an edge MLP over
(edge, source node, destination node) features followed by an aggregation onto the destination nodes."""
import torch.nn as nn

from . import mesh_graph_mlp as _mlps
from .utils import aggregate


class BipartiteMessagePassing(nn.Module):
    """Owns ``edge_mlp`` (checkpoint key) and ``aggregation``; ``messages_to_dst`` returns the aggregated edge
    features per destination node."""

    def _make_mlps(self, *, src_width: int, dst_width: int, edge_width: int, edge_out: int, concat_trick: bool, shared: dict):
        edge_type = _mlps.MeshGraphEdgeMLPSum if concat_trick else _mlps.MeshGraphEdgeMLPConcat
        self.edge_mlp = edge_type(efeat_dim=edge_width, src_dim=src_width, dst_dim=dst_width, output_dim=edge_out, **shared)

    def node_mlp_for(self, width_in: int, width_out: int, shared: dict) -> nn.Module:
        return _mlps.MeshGraphMLP(input_dim=width_in, output_dim=width_out, **shared)

    def messages_to_dst(self, efeat, src_nfeat, dst_nfeat, graph):
        per_edge = self.edge_mlp(efeat, (src_nfeat, dst_nfeat), graph)
        return aggregate(per_edge, dst_nfeat.shape[0], graph, self.aggregation)

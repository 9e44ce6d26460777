"""Graph container used by the GNN layers.

The reference accepts PyTorch-Geometric ``Data`` / ``HeteroData`` objects
(``physicsnemo/nn/module/gnn_layers/graph_types.py``).  Here any object exposing
``edge_index`` (a ``(2, E)`` integer tensor, row 0 = source, row 1 = destination) is
accepted — PyG ``Data`` included — and ``Graph`` is the package's own light container.
Sorted (CSC / CSR) edge orders are computed once per graph and cached on the object, which
is what lets the aggregation kernels run without atomics.
"""
from __future__ import annotations

from typing import Optional, Union

import torch

from ....ops.graph import SegmentIndex


class Graph:
    """Directed graph given by ``edge_index`` (2, E) and ``num_nodes`` (optionally bipartite)."""

    def __init__(self, edge_index: torch.Tensor, num_nodes: Optional[int] = None,
                 num_src_nodes: Optional[int] = None, num_dst_nodes: Optional[int] = None, **attrs):
        if edge_index.dim() != 2 or edge_index.shape[0] != 2:
            raise ValueError(f"edge_index must have shape (2, E), got {tuple(edge_index.shape)}")
        self.edge_index = edge_index
        n = int(edge_index.max().item()) + 1 if (num_nodes is None and edge_index.numel()) else (num_nodes or 0)
        self.num_nodes = n
        self.num_src_nodes = num_src_nodes if num_src_nodes is not None else n
        self.num_dst_nodes = num_dst_nodes if num_dst_nodes is not None else n
        for k, v in attrs.items():
            setattr(self, k, v)

    @property
    def num_edges(self) -> int:
        return self.edge_index.shape[1]

    def to(self, device):
        g = Graph(self.edge_index.to(device), self.num_nodes, self.num_src_nodes, self.num_dst_nodes)
        for k, v in self.__dict__.items():
            if k not in ("edge_index", "num_nodes", "num_src_nodes", "num_dst_nodes", "_pnm_cache"):
                setattr(g, k, v.to(device) if isinstance(v, torch.Tensor) else v)
        return g


GraphType = Union[Graph, object]


def edge_index_of(graph) -> torch.Tensor:
    """``(2, E)`` edge index of a ``Graph`` / PyG ``Data`` / PyG ``HeteroData`` (first edge type)."""
    if hasattr(graph, "edge_types") and not hasattr(graph, "edge_index"):
        return graph[graph.edge_types[0]].edge_index
    if not hasattr(graph, "edge_index"):
        raise ValueError(f"Unsupported graph type: {type(graph)}")
    return graph.edge_index


def segments(graph, which: str, num_nodes: int) -> SegmentIndex:
    """Cached ``SegmentIndex`` of the edges by ``"src"`` or ``"dst"`` node."""
    cache = getattr(graph, "_pnm_cache", None)
    if cache is None:
        cache = {}
        try:
            object.__setattr__(graph, "_pnm_cache", cache)
        except Exception:  # objects that refuse new attributes: no caching
            pass
    ei = edge_index_of(graph)
    key = (which, num_nodes, ei.data_ptr(), ei.shape[1], str(ei.device))
    if key not in cache:
        cache[key] = SegmentIndex(ei[0 if which == "src" else 1], num_nodes)
    return cache[key]

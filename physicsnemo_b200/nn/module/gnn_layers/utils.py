"""Edge / node feature plumbing of the message-passing layers.

Parity: ``physicsnemo/nn/module/gnn_layers/utils.py`` — ``set_checkpoint_fn`` (``:55-79``),
``concat_efeat`` (``:105-133``), ``sum_efeat`` / ``sum_edge_node_feat`` (``:193-222``),
``aggregate_and_concat`` / ``agg_concat_pyg`` (``:266-280``).  Gathers and the aggregation go
through ``physicsnemo_b200.ops.graph`` (sorted segment reduction instead of
``torch_scatter`` atomics); no dependency on PyTorch Geometric.
"""
from __future__ import annotations

from typing import Callable, Tuple, Union

import torch
from torch import Tensor
from torch.utils.checkpoint import checkpoint

from .... import ops
from .graph_types import edge_index_of, segments


def checkpoint_identity(layer: Callable, *args, **kwargs):
    """Stand-in for ``torch.utils.checkpoint.checkpoint`` that just calls ``layer``."""
    kwargs.pop("use_reentrant", None)
    kwargs.pop("preserve_rng_state", None)
    return layer(*args)


def set_checkpoint_fn(do_checkpointing: bool) -> Callable:
    return checkpoint if do_checkpointing else checkpoint_identity


def _src_dst(nfeat):
    return nfeat if isinstance(nfeat, (tuple, list)) else (nfeat, nfeat)


def gather_src_dst(nfeat: Union[Tensor, Tuple[Tensor, Tensor]], graph) -> Tuple[Tensor, Tensor]:
    """``(src_feat[src], dst_feat[dst])`` for every edge."""
    src_feat, dst_feat = _src_dst(nfeat)
    if hasattr(graph, "gather_src"):
        # partitioned graph: sources may live on another rank; the gather reads them from their owners
        return graph.gather_src(src_feat), ops.gather_rows(dst_feat, segments(graph, "dst", dst_feat.shape[0]))
    return (ops.gather_rows(src_feat, segments(graph, "src", src_feat.shape[0])),
            ops.gather_rows(dst_feat, segments(graph, "dst", dst_feat.shape[0])))


def concat_efeat(efeat: Tensor, nfeat: Union[Tensor, Tuple[Tensor, Tensor]], graph) -> Tensor:
    """``cat(efeat, src_feat[src], dst_feat[dst])`` along the feature dimension."""
    gs, gd = gather_src_dst(nfeat, graph)
    return torch.cat((efeat, gs, gd), dim=1)


def concat_efeat_hetero(mesh_efeat: Tensor, world_efeat: Tensor, nfeat, graph) -> Tensor:
    return concat_efeat(torch.cat((mesh_efeat, world_efeat), dim=0), nfeat, graph)


def sum_edge_node_feat(efeat: Tensor, src_feat: Tensor, dst_feat: Tensor, src_idx: Tensor, dst_idx: Tensor) -> Tensor:
    return efeat + src_feat[src_idx] + dst_feat[dst_idx]


def sum_efeat(efeat: Tensor, nfeat: Union[Tensor, Tuple[Tensor, Tensor]], graph) -> Tensor:
    """``efeat + src_feat[src] + dst_feat[dst]`` (the "concat trick" after splitting the first linear layer)."""
    gs, gd = gather_src_dst(nfeat, graph)
    return efeat + gs + gd


def aggregate(efeat: Tensor, num_dst: int, graph, aggregation: str = "sum") -> Tensor:
    """Reduce edge features onto their destination nodes."""
    return ops.segment_reduce(efeat, segments(graph, "dst", num_dst), aggregation)


def aggregate_and_concat(efeat: Tensor, nfeat: Tensor, graph, aggregation: str) -> Tensor:
    """``cat(aggregate(efeat → dst nodes), nfeat)``."""
    return torch.cat((aggregate(efeat, nfeat.shape[0], graph, aggregation), nfeat), -1)


def aggregate_and_concat_hetero(mesh_efeat: Tensor, world_efeat: Tensor, nfeat: Tensor, graph, aggregation: str) -> Tensor:
    """``cat(aggregate(cat(mesh, world) edge features → dst nodes), nfeat)``; ``graph`` lists mesh edges first."""
    return aggregate_and_concat(torch.cat((mesh_efeat, world_efeat), dim=0), nfeat, graph, aggregation)

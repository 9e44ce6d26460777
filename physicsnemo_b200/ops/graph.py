"""Graph message-passing primitives: row gather and sorted segment reduction.

``gather_rows(x, idx)``            edge ← node features (``x[idx]``)
``segment_reduce(x, graph_csc)``   node ← incident edges (sum / mean over edges sorted by node)

They replace ``x[idx]`` indexing + ``torch_scatter.scatter`` of the reference
(``physicsnemo/nn/module/gnn_layers/utils.py:105-133, 266-280``).  The reduction walks
edges pre-sorted by destination (CSC order, computed once per graph), so it needs no
atomics and sums in a fixed order.  Each op is the other's backward.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from . import gemm as _g


class SegmentIndex:
    """Edges grouped by a node index: ``perm`` (edge ids sorted by node) and CSR ``offsets``."""

    def __init__(self, index: torch.Tensor, num_segments: int):
        index = index.to(torch.long)
        order = torch.argsort(index, stable=True)
        counts = torch.bincount(index, minlength=num_segments)
        offsets = torch.zeros(num_segments + 1, dtype=torch.long, device=index.device)
        offsets[1:] = torch.cumsum(counts, 0)
        self.index = index
        self.index32 = index.to(torch.int32).contiguous()
        self.perm = order.to(torch.int32).contiguous()
        self.offsets = offsets.to(torch.int32).contiguous()
        self.counts = counts
        self.inv_count = (1.0 / counts.clamp_min(1).float()).contiguous()
        self.num_segments = num_segments
        self.num_items = index.numel()


def _gather_raw(x: torch.Tensor, idx32: torch.Tensor, scale: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    lib = _lib.load(required=True)
    E, C = idx32.numel(), x.shape[1]
    if out is None:
        out = torch.empty((E, C), dtype=torch.bfloat16, device=x.device)
    code = lib.pnm_gather_rows(x.data_ptr(), x.stride(0), idx32.data_ptr(), None if scale is None else scale.data_ptr(),
                               out.data_ptr(), out.stride(0), E, C, _g._stream())
    _g._check(code, "pnm_gather_rows")
    _g.launch_count += 1
    return out


def _segment_raw(x: torch.Tensor, seg: SegmentIndex, mean: bool = False, out: Optional[torch.Tensor] = None,
                 accumulate: bool = False) -> torch.Tensor:
    lib = _lib.load(required=True)
    C = x.shape[1]
    if out is None:
        out = torch.empty((seg.num_segments, C), dtype=torch.bfloat16, device=x.device)
    code = lib.pnm_segment_sum(x.data_ptr(), x.stride(0), seg.perm.data_ptr(), seg.offsets.data_ptr(), out.data_ptr(),
                               out.stride(0), seg.num_segments, C, int(accumulate), int(mean), _g._stream())
    _g._check(code, "pnm_segment_sum")
    _g.launch_count += 1
    return out


def _ok(x: torch.Tensor) -> torch.Tensor:
    if x.stride(1) != 1 or x.stride(0) % 8 or x.data_ptr() % 16:
        x = x.contiguous()
    return x


class _GatherFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, seg):
        ctx.seg = seg
        return _gather_raw(_ok(x), seg.index32)

    @staticmethod
    def backward(ctx, g):
        return _segment_raw(_ok(g), ctx.seg), None


class _SegmentFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, seg, mean):
        ctx.seg, ctx.mean = seg, mean
        return _segment_raw(_ok(x), seg, mean)

    @staticmethod
    def backward(ctx, g):
        seg = ctx.seg
        return _gather_raw(_ok(g), seg.index32, seg.inv_count if ctx.mean else None), None, None


def _fused(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] % 8 == 0 and _lib.available()


def gather_rows(x: torch.Tensor, seg: SegmentIndex) -> torch.Tensor:
    """``x[seg.index]`` (differentiable; backward is the sorted segment sum)."""
    if _fused(x):
        return _GatherFn.apply(x, seg)
    return x[seg.index]


def segment_reduce(x: torch.Tensor, seg: SegmentIndex, reduce: str = "sum") -> torch.Tensor:
    """Sum (or mean) of the rows of ``x`` that share a segment id; result has ``seg.num_segments`` rows."""
    if reduce not in ("sum", "mean"):
        raise ValueError(f"unsupported reduction {reduce}")
    if _fused(x):
        return _SegmentFn.apply(x, seg, reduce == "mean")
    out = torch.zeros((seg.num_segments, x.shape[1]), dtype=x.dtype, device=x.device)
    out.index_add_(0, seg.index, x)
    if reduce == "mean":
        out = out * seg.inv_count.to(out.dtype).unsqueeze(1)
    return out

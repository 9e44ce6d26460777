"""Bucketed gradient reduction overlapped with backward.

Reference behaviour: ``torch.nn.parallel.DistributedDataParallel`` (25 MB fp32 buckets reduced by
NCCL while backward continues) and, for domain parallelism, one all-reduce per parameter
(``physicsnemo/domain_parallel/shard_utils/grad_ops.py:107-139``); ``fused_all_reduce``
(``physicsnemo/distributed/fused_all_reduce.py:148-271``) packs, reduces and unpacks in three steps.

Here every parameter's ``.grad`` is a view into one flat fp32 buffer, so a bucket is a contiguous range
of that buffer and nothing is packed or unpacked.  When the last gradient of a bucket has been
accumulated (post-accumulate-grad hooks) the bucket is handed to ONE kernel on a side stream
(``pnm_peer_allreduce_bf16``): it casts to bf16 with the ``1/world`` (or any) scale into symmetric
memory, reduce-scatters with fp32 accumulation over direct peer loads, and all-gathers the result
straight back into the fp32 gradient range.  Backward keeps running on the main stream meanwhile.
Without CUDA / NCCL (CPU tests with gloo) the same bucket logic calls ``dist.all_reduce``.
"""
from __future__ import annotations

from typing import Iterable, List, Optional

import torch
import torch.distributed as dist


class GradBucketReducer:
    """Owns the flat gradient buffer of ``params`` and reduces it over ``group`` bucket by bucket.

    ``scale``: factor applied before the sum (``1/world`` for data-parallel averaging, ``1.0`` when the
    ranks hold partial sums of one global gradient, as under domain parallelism).
    ``wire``: ``"bf16"`` (default on the peer path) or ``"fp32"``.
    """

    def __init__(self, params: Iterable[torch.nn.Parameter], group: Optional[dist.ProcessGroup] = None,
                 bucket_mb: float = 25.0, scale: float = 1.0, wire: str = "bf16", overlap: bool = True,
                 max_ctas: int = 48):
        self.params: List[torch.nn.Parameter] = [p for p in params if p.requires_grad]
        if not self.params:
            raise ValueError("no parameters require gradients")
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.scale, self.wire, self.overlap, self.max_ctas = float(scale), wire, overlap, int(max_ctas)
        dev = self.params[0].device
        self.device = dev
        # layout: reverse parameter order (gradients arrive roughly last-to-first), every tensor on a 32-byte boundary
        order = list(reversed(self.params))
        offs, total = [], 0
        for p in order:
            offs.append(total)
            total += (p.numel() + 7) // 8 * 8
        self.flat = torch.zeros(total, dtype=torch.float32, device=dev)
        self._views = []
        for p, o in zip(order, offs):
            v = self.flat[o:o + p.numel()].view_as(p)
            self._views.append(v)
        elems = max(8, int(bucket_mb * (1 << 20) / (2 if wire == "bf16" else 4)) // 8 * 8)
        self.buckets = []          # (start, end, number of parameters)
        self._bucket_of = {}
        start, count = 0, 0
        for i, (p, o) in enumerate(zip(order, offs)):
            end = o + (p.numel() + 7) // 8 * 8
            self._bucket_of[id(p)] = len(self.buckets)
            count += 1
            if end - start >= elems or i == len(order) - 1:
                self.buckets.append((start, end, count))
                start, count = end, 0
        self._order = order
        self._idx = {id(p): i for i, p in enumerate(order)}
        self._pending = [0] * len(self.buckets)
        self._launched = [False] * len(self.buckets)
        self._rt = None
        self.loopback = False      # measurement aid: run the step with every reduction skipped
        self.sync = True           # False while accumulating micro-batches: hooks do nothing until the last one
        self._comm_stream = None
        self._ev_bwd_end = self._ev_comm_end = None
        if self.world > 1 and dev.type == "cuda":
            from .peer import PeerRuntime, peer_available

            if peer_available():
                biggest = max(e - s for s, e, _ in self.buckets)
                cap = biggest // 2 + 8 if wire == "bf16" else biggest
                self._rt = PeerRuntime(group, capacity_floats=cap)
            self._comm_stream = torch.cuda.Stream(device=dev) if overlap else None
        if self.world > 1:
            from .peer import register_loopback

            register_loopback(self)
        self.attach()
        self._hooks = [p.register_post_accumulate_grad_hook(self._on_grad) for p in self.params]

    # ------------------------------------------------------------------------------------------------
    def attach(self) -> None:
        """(Re)install the flat views as ``.grad`` (needed after ``zero_grad(set_to_none=True)`` elsewhere)."""
        for p, v in zip(self._order, self._views):
            p.grad = v

    def zero_grad(self) -> None:
        """One memset for all gradients; keeps ``.grad`` pointing into the flat buffer."""
        self.flat.zero_()
        for p, v in zip(self._order, self._views):
            if p.grad is None or p.grad.data_ptr() != v.data_ptr():
                p.grad = v

    def _on_grad(self, p: torch.nn.Parameter) -> None:
        b = self._bucket_of.get(id(p))
        if b is None or self.world == 1 or not self.sync:
            return
        view = self._views[self._idx[id(p)]]
        if p.grad is not None and p.grad.data_ptr() != view.data_ptr():
            # a fresh tensor replaced the view (set_to_none elsewhere): copy into the flat buffer
            view.copy_(p.grad)
            p.grad = view
        self._pending[b] += 1
        if self._pending[b] == self.buckets[b][2] and not self._launched[b]:
            self._launch(b)

    def _reduce_range(self, lo: int, hi: int) -> None:
        seg = self.flat[lo:hi]
        if self.loopback:
            if self.scale != 1.0:
                seg.mul_(self.scale)
            return
        if self._rt is not None:
            if self.wire == "bf16":
                self._rt.all_reduce_bf16_(seg, scale=self.scale, max_ctas=self.max_ctas)
            else:
                self._rt.all_reduce(seg, scale=self.scale, out=seg, two_shot=self.world > 2, max_ctas=self.max_ctas)
        else:
            if self.scale != 1.0:
                seg.mul_(self.scale)
            dist.all_reduce(seg, group=self.group)

    def _launch(self, b: int) -> None:
        lo, hi, _ = self.buckets[b]
        self._launched[b] = True
        if self._comm_stream is None:
            self._reduce_range(lo, hi)
            return
        cur = torch.cuda.current_stream()
        self._comm_stream.wait_stream(cur)
        with torch.cuda.stream(self._comm_stream):
            self._reduce_range(lo, hi)

    def finish(self) -> None:
        """Call after ``backward``: reduces buckets that did not fill (unused parameters) and joins the side stream."""
        if self.world == 1:
            return
        for b in range(len(self.buckets)):
            if not self._launched[b]:
                self._launch(b)
        if self._comm_stream is not None:
            cur = torch.cuda.current_stream()
            timing = not torch.cuda.is_current_stream_capturing()
            if timing:
                self._ev_bwd_end = torch.cuda.Event(enable_timing=True)
                self._ev_comm_end = torch.cuda.Event(enable_timing=True)
                self._ev_bwd_end.record(cur)
                self._ev_comm_end.record(self._comm_stream)
            cur.wait_stream(self._comm_stream)
        if self._rt is not None:
            self._rt.step_done()
        self._pending = [0] * len(self.buckets)
        self._launched = [False] * len(self.buckets)

    def exposed_ms(self) -> float:
        """Time the main stream had to wait for the last bucket after backward ended (last finished step); syncs."""
        if self._ev_bwd_end is None:
            return 0.0
        self._ev_comm_end.synchronize()
        return max(0.0, self._ev_bwd_end.elapsed_time(self._ev_comm_end))

    def remove(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []

"""Point (token) sharding for slice-attention models on replicated parameters.

Each rank holds ``N / P`` points of every sample; parameters are replicated.  Only two
kinds of data cross ranks (reference: ``physicsnemo/nn/module/physics_attention.py:120-206``
comments on partial sums, resolved there by ShardTensor all-reduces, one per tensor):

* per attention block, the ``H*S*(D+1)`` partial slice-token / slice-norm sums forward and
  the matching small gradient sums backward — ``reduce_fn`` below (one peer-memory kernel);
* the parameter gradients (every rank saw a different shard of the points): bucketed, cast to
  bf16 and reduced on a side stream while backward is still running (``GradBucketReducer``).

``PointParallel`` installs ``reduce_fn`` on every physics-attention module and owns the
gradient reducer.  A training step is ``pp.zero_grad(); loss.backward(); pp.reduce_gradients()``.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .grad_reducer import GradBucketReducer


class _CollectiveExchange:
    """``PeerRegions`` look-alike on ``torch.distributed`` all-reduce (the selectable baseline, ``backend="nccl"``):
    the producers fill a local buffer, ``publish`` reduces it in place, the consumer reads the reduced copy."""

    def __init__(self, group):
        self.group = group
        self.world = dist.get_world_size(group)
        self._last = None

    def region(self, floats: int, device=None):
        self._last = torch.empty(floats, dtype=torch.float32, device=device)
        return self._last, [self._last.data_ptr()]

    def publish(self):
        dist.all_reduce(self._last, group=self.group)
        return None

    def step_done(self) -> None:
        self._last = None


class PointParallel:
    """Wraps a model whose inputs are sharded over points on ``group``.

    ``backend="nccl"`` uses ``torch.distributed`` all-reduce for the small reductions; ``backend="peer"`` (and
    ``"auto"`` on a CUDA + NCCL job) uses the package's peer-memory kernels (``physicsnemo_b200.parallel.peer``).
    """

    def __init__(self, model: torch.nn.Module, group: Optional[dist.ProcessGroup] = None, backend: str = "auto",
                 bucket_mb: float = 25.0, wire: str = "bf16"):
        self.model = model
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.backend = backend
        self._peer = None
        self._regions = None
        if backend in ("auto", "peer") and self.world > 1 and torch.cuda.is_available():
            try:
                from .peer import PeerAllReduce, PeerRegions

                self._peer = PeerAllReduce(group=group, max_numel=1 << 20)
                self._regions = PeerRegions(group=group, region_floats=1 << 18, n_regions=32)
            except Exception:
                if backend == "peer":
                    raise
                self._peer = self._regions = None
        self.params = [p for p in model.parameters() if p.requires_grad]
        self.reducer = GradBucketReducer(self.params, group=group, bucket_mb=bucket_mb, scale=1.0, wire=wire) \
            if self.world > 1 else None
        for m in model.modules():
            if hasattr(m, "in_project_slice") and hasattr(m, "qkv_project"):
                m._reduce_fn = self.reduce_small
                # partial sums are added inside the consuming kernels (peer) or by an all-reduce before them (nccl)
                m._exchange = self._regions if self._regions is not None else (
                    _CollectiveExchange(group) if self.world > 1 else None)

    # small latency-bound reductions (slice tokens, small gradient sums)
    def reduce_small(self, flat: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return flat
        if self._peer is not None and flat.numel() <= self._peer.max_numel and flat.dtype == torch.float32:
            return self._peer.all_reduce(flat)
        flat = flat.contiguous()
        dist.all_reduce(flat, group=self.group)
        return flat

    def zero_grad(self) -> None:
        """Clear the gradients (one memset of the reducer's flat buffer when sharded)."""
        if self.reducer is not None:
            self.reducer.zero_grad()
        else:
            for p in self.params:
                p.grad = None

    def reduce_gradients(self) -> None:
        """Finish the gradient reduction started by the backward hooks; last peer operation of the step."""
        if self.world == 1:
            return
        self.reducer.finish()
        if self._peer is not None:
            self._peer.step_done()      # lets a captured step advance its call numbers
        if self._regions is not None:
            self._regions.step_done()

    def exposed_ms(self) -> float:
        return self.reducer.exposed_ms() if self.reducer is not None else 0.0

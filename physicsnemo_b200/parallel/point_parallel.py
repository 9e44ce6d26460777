"""Point (token) sharding for slice-attention models on replicated parameters.

Each rank holds ``N / P`` points of every sample; parameters are replicated.  Only two
kinds of data cross ranks (reference: ``physicsnemo/nn/module/physics_attention.py:120-206``
comments on partial sums, resolved there by ShardTensor all-reduces, one per tensor):

* per attention block, the ``H*S*(D+1)`` partial slice-token / slice-norm sums forward and
  the matching small gradient sums backward — ``reduce_fn`` below;
* once per step, the parameter gradients (every rank saw a different shard of the points).

``PointParallel`` installs ``reduce_fn`` on every physics-attention module and owns one flat
fp32 gradient bucket so that the whole model needs a single reduction per step.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


class PointParallel:
    """Wraps a model whose inputs are sharded over points on ``group``.

    ``backend="nccl"`` uses ``torch.distributed`` all-reduce; ``backend="peer"`` uses the
    package's peer-memory all-reduce kernel (``physicsnemo_b200.parallel.peer``).
    """

    def __init__(self, model: torch.nn.Module, group: Optional[dist.ProcessGroup] = None, backend: str = "auto"):
        self.model = model
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.backend = backend
        self._peer = None
        if backend in ("auto", "peer") and self.world > 1 and torch.cuda.is_available():
            try:
                from .peer import PeerAllReduce

                self._peer = PeerAllReduce(group=group, max_numel=1 << 23)
            except Exception:
                if backend == "peer":
                    raise
                self._peer = None
        self.params = [p for p in model.parameters() if p.requires_grad]
        self._flat: Optional[torch.Tensor] = None
        for m in model.modules():
            if hasattr(m, "in_project_slice") and hasattr(m, "qkv_project"):
                m._reduce_fn = self.reduce_small

    # small latency-bound reductions (slice tokens, small gradient sums)
    def reduce_small(self, flat: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return flat
        if self._peer is not None and flat.numel() <= self._peer.max_numel and flat.dtype == torch.float32:
            return self._peer.all_reduce(flat)
        flat = flat.contiguous()
        dist.all_reduce(flat, group=self.group)
        return flat

    def reduce_gradients(self) -> None:
        """Sum parameter gradients over the point shards (one flat fp32 reduction)."""
        if self.world == 1:
            return
        grads = [p.grad for p in self.params if p.grad is not None]
        if not grads:
            return
        total = sum(g.numel() for g in grads)
        if self._flat is None or self._flat.numel() != total:
            self._flat = torch.empty(total, dtype=torch.float32, device=grads[0].device)
        flat = self._flat
        torch._foreach_copy_(list(flat.split([g.numel() for g in grads])), [g.reshape(-1) for g in grads])
        if self._peer is not None and total <= self._peer.max_numel:
            flat = self._peer.all_reduce(flat)
        else:
            dist.all_reduce(flat, group=self.group)
        torch._foreach_copy_([g.reshape(-1) for g in grads], list(flat.split([g.numel() for g in grads])))
        if self._peer is not None:
            self._peer.step_done()      # last peer call of the step: lets a captured step advance its call numbers

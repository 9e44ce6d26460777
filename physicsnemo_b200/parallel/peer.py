"""Peer-memory runtime: symmetric buffers mapped on every rank + the in-kernel collectives.

The reference communicates only through ``torch.distributed`` / NCCL calls
(``physicsnemo/distributed/utils.py``, ``domain_parallel/shard_utils/*``).  Here the
latency-bound collectives of the hot paths run inside this package's own kernels
(``csrc/peer.cuh``): every rank allocates one buffer, the ranks exchange handles once
(``torch.distributed._symmetric_memory`` rendezvous), and afterwards a kernel reads its
peers' buffers directly over NVLink with plain loads, ordered by per-CTA epoch flags.
All device-side waits are bounded; a time-out surfaces as ``PeerTimeoutError`` on the host.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import gemm as _g


class PeerTimeoutError(RuntimeError):
    """A bounded device-side wait on a peer flag ran out."""


class PeerRuntime:
    """One symmetric buffer per rank of ``group`` with the peer pointers of all ranks."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None, capacity_floats: int = 1 << 23):
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("PeerRuntime needs an initialised process group")
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.lib = _lib.load(required=True)
        self.lib.pnm_peer_allreduce.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_float,
                                                ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                                ctypes.c_uint, ctypes.c_longlong, ctypes.c_double, ctypes.c_void_p,
                                                ctypes.c_void_p]
        self.lib.pnm_peer_allreduce.restype = ctypes.c_int
        self.flag_bytes = self.lib.pnm_peer_flag_bytes()
        self.capacity = int(capacity_floats)
        nbytes = self.flag_bytes + 4 * self.capacity * 4  # 2 slots x 2 stages
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.buffer = symm.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.buffer.zero_()
        torch.cuda.synchronize()
        self.handle = symm.rendezvous(self.buffer, group=self.group.group_name)
        ptrs = list(self.handle.buffer_ptrs)
        self._bases = (ctypes.c_void_p * self.world)(*ptrs)
        self.epoch = 0
        self.budget_s = 2.0
        # Call numbers are ``epoch_base (device) + epoch (host offset)``.  The host offset restarts at every
        # ``step_done()``, which moves it into the device counter with a one-element add on the stream; a CUDA graph
        # that contains a whole step (its all-reduces and that add) therefore advances the call numbers at each replay.
        self.epoch_base = torch.zeros(1, dtype=torch.int32, device=self.device)
        dist.barrier(group=self.group)  # zeroed flags are visible before the first kernel

    def all_reduce(self, x: torch.Tensor, scale: float = 1.0, out: Optional[torch.Tensor] = None,
                   two_shot: Optional[bool] = None) -> torch.Tensor:
        """Sum of the fp32 vector ``x`` over the ranks (times ``scale``), computed by one kernel."""
        assert x.dtype == torch.float32 and x.is_cuda and x.is_contiguous()
        n = x.numel()
        if n > self.capacity:
            raise ValueError(f"{n} floats exceed the symmetric buffer capacity {self.capacity}")
        if out is None:
            out = torch.empty_like(x)
        if two_shot is None:
            two_shot = n >= (1 << 16) and self.world > 2
        self.epoch += 1
        code = self.lib.pnm_peer_allreduce(x.data_ptr(), out.data_ptr(), n, float(scale), int(two_shot), self._bases,
                                           self.rank, self.world, self.epoch, self.capacity, self.budget_s,
                                           _g._stream(), self.epoch_base.data_ptr())
        _g._check(code, "pnm_peer_allreduce")
        _g.launch_count += 1
        return out

    def step_done(self) -> None:
        """Fold the calls made since the last ``step_done`` into the device-side call counter.

        Must be the last peer operation of a step that is captured into a CUDA graph; harmless otherwise.
        """
        if self.epoch:
            self.epoch_base.add_(self.epoch)
            self.epoch = 0

    def check(self) -> None:
        """Raise ``PeerTimeoutError`` if any bounded wait has run out (synchronises the device)."""
        err = self.lib.pnm_get_error()
        if err != 0:
            raise PeerTimeoutError(f"device error word = {err} (6 = wait on a peer flag ran out)")


class PeerAllReduce:
    """Callable all-reduce used by ``PointParallel`` (fp32 vectors up to ``max_numel``)."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None, max_numel: int = 1 << 23):
        self.rt = PeerRuntime(group, capacity_floats=max_numel)
        self.max_numel = max_numel

    def all_reduce(self, flat: torch.Tensor) -> torch.Tensor:
        return self.rt.all_reduce(flat.contiguous())

    def step_done(self) -> None:
        self.rt.step_done()

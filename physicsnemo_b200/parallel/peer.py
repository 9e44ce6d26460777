"""Peer-memory runtime: symmetric buffers mapped on every rank + the in-kernel collectives.

The reference communicates only through ``torch.distributed`` / NCCL calls
(``physicsnemo/distributed/utils.py``, ``domain_parallel/shard_utils/*``).  Here the
collectives of the hot paths run inside this package's own kernels (``csrc/peer.cuh``):
every rank allocates one buffer, the ranks exchange handles once
(``torch.distributed._symmetric_memory`` rendezvous), and afterwards a kernel reads its
peers' buffers directly over NVLink with plain loads, ordered by epoch flags.

Failure handling.  Every device-side wait is bounded by ``budget_s``.  A wait that runs out
sets the library's error word and fills the outputs it could not produce with NaN.  The
host notices it without stalling the pipeline: ``step_done()`` enqueues a copy of the error
word into pinned memory and looks at the copy made by the *previous* call; ``check()`` is the
synchronising form.  After a ``PeerTimeoutError`` every rank calls ``recover()``
(host barrier, flags and call numbers back to zero) before the runtime is used again.
"""
from __future__ import annotations

import ctypes
import weakref
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import gemm as _g


class PeerTimeoutError(RuntimeError):
    """A bounded device-side wait on a peer flag ran out."""


_LOOPBACK_AWARE = weakref.WeakSet()


def register_loopback(obj) -> None:
    """Objects with a ``loopback`` attribute (runtimes, reducers) that ``set_loopback`` should switch."""
    _LOOPBACK_AWARE.add(obj)


def set_loopback(flag: bool) -> None:
    """Measurement aid: run the same kernels with all peer traffic off (every rank talks to itself, halos read as
    zero padding, gradient buckets are not reduced).  The time of a step in this mode is its communication-free
    time; ``step time - loopback time`` is the communication that the step does not hide."""
    for obj in list(_LOOPBACK_AWARE):
        obj.loopback = bool(flag)


def _declare(lib) -> None:
    if getattr(lib, "_peer_declared", False):
        return
    c = ctypes
    vp, i, u, ll, f, d = c.c_void_p, c.c_int, c.c_uint, c.c_longlong, c.c_float, c.c_double
    lib.pnm_peer_allreduce.argtypes = [vp, vp, ll, f, i, vp, i, i, u, ll, d, vp, vp, i]
    lib.pnm_peer_allreduce_bf16.argtypes = [vp, ll, f, vp, i, i, u, ll, d, vp, vp, i]
    lib.pnm_peer_signal.argtypes = [vp, i, i, u, ll, vp, vp]
    lib.pnm_peer_pull.argtypes = [vp, vp, ll, i, vp, i, i, u, ll, d, vp, vp, i]
    lib.pnm_peer_pull_reduce.argtypes = [vp, ll, vp, i, i, u, ll, d, vp, vp, i]
    lib.pnm_error_copy_async.argtypes = [vp, vp]
    lib.pnm_peer_wait_probe.argtypes = [vp, u, d, vp, vp]
    for name in ("pnm_peer_allreduce", "pnm_peer_allreduce_bf16", "pnm_peer_signal", "pnm_peer_pull",
                 "pnm_peer_pull_reduce", "pnm_error_copy_async", "pnm_peer_wait_probe", "pnm_peer_flag_bytes"):
        getattr(lib, name).restype = i
    lib._peer_declared = True


class PeerRuntime:
    """One symmetric buffer per rank of ``group`` with the peer pointers of all ranks."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None, capacity_floats: int = 1 << 23,
                 budget_s: float = 30.0, poll_every: int = 1):
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("PeerRuntime needs an initialised process group")
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.lib = _lib.load(required=True)
        _declare(self.lib)
        self.flag_bytes = self.lib.pnm_peer_flag_bytes()
        self.capacity = (int(capacity_floats) + 7) // 8 * 8
        nbytes = self.flag_bytes + 4 * self.capacity * 4  # 2 slots x 2 stages
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.buffer = symm.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.buffer.zero_()
        torch.cuda.synchronize()
        self.handle = symm.rendezvous(self.buffer, group=self.group.group_name)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self._bases = (ctypes.c_void_p * self.world)(*self.ptrs)
        self._own = (ctypes.c_void_p * 1)(self.ptrs[self.rank])
        self.loopback = False   # measurement aid: same kernels, no peer traffic (every sum is over this rank only)
        self.epoch = 0
        # training-sized default: a rank may legitimately be seconds late (checkpoint write, data stall, lazy init)
        self.budget_s = float(budget_s)
        self.poll_every = max(1, int(poll_every))
        # Call numbers are ``epoch_base (device) + epoch (host offset)``.  The host offset restarts at every
        # ``step_done()``, which moves it into the device counter with a one-element add on the stream; a CUDA graph
        # that contains a whole step (its collectives and that add) therefore advances the call numbers at each replay.
        self.epoch_base = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._err_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._err_event: Optional[torch.cuda.Event] = None
        self._steps = 0
        self._folded = 0   # host mirror of epoch_base (valid as long as no captured graph replays the add)
        register_loopback(self)
        dist.barrier(group=self.group)  # zeroed flags are visible before the first kernel

    def _brw(self):
        """(bases, rank, world) as the kernels see them; in loopback mode the rank talks only to itself."""
        if self.loopback:
            return self._own, 0, 1
        return self._bases, self.rank, self.world

    # ------------------------------------------------------------------ call numbers
    def next_epoch(self) -> int:
        """Reserve the next call number (every rank must make the same sequence of calls)."""
        self.epoch += 1
        return self.epoch

    def peer_args(self, epoch: int) -> Tuple:
        """``(bases, rank, world, epoch, capacity, budget_s, epoch_base)`` as the C entry points take them."""
        return (*self._brw(), epoch, self.capacity, self.budget_s, self.epoch_base.data_ptr())

    def stage_ptr(self, rank: int, epoch: int, stage: int = 0) -> int:
        """Address (peer-mapped) of stage ``stage`` of the data slot that call ``epoch`` uses on ``rank``.

        Only meaningful outside CUDA-graph replay, where ``epoch_base`` is folded in by the kernels themselves.
        """
        return self.ptrs[rank] + self.flag_bytes + (((epoch + self._folded) & 1) * 2 + stage) * self.capacity * 4

    # ------------------------------------------------------------------ collectives
    def all_reduce(self, x: torch.Tensor, scale: float = 1.0, out: Optional[torch.Tensor] = None,
                   two_shot: Optional[bool] = None, max_ctas: int = 0) -> torch.Tensor:
        """Sum of the fp32 vector ``x`` over the ranks (times ``scale``), computed by one kernel."""
        assert x.dtype == torch.float32 and x.is_cuda and x.is_contiguous()
        n = x.numel()
        if n > self.capacity:
            raise ValueError(f"{n} floats exceed the symmetric buffer capacity {self.capacity}")
        if out is None:
            out = torch.empty_like(x)
        if two_shot is None:
            two_shot = n >= (1 << 16) and self.world > 2
        code = self.lib.pnm_peer_allreduce(x.data_ptr(), out.data_ptr(), n, float(scale), int(two_shot), *self._brw(),
                                           self.next_epoch(), self.capacity, self.budget_s,
                                           _g._stream(), self.epoch_base.data_ptr(), int(max_ctas))
        _g._check(code, "pnm_peer_allreduce")
        _g.launch_count += 1
        return out

    def all_reduce_bf16_(self, x: torch.Tensor, scale: float = 1.0, max_ctas: int = 0) -> torch.Tensor:
        """In-place gradient all-reduce with bf16 on the wire: ``x <- sum_r bf16(scale * x_r)`` (fp32 accumulate)."""
        assert x.dtype == torch.float32 and x.is_cuda and x.is_contiguous()
        n = x.numel()
        if n % 8 or x.data_ptr() % 32:
            raise ValueError("all_reduce_bf16_ needs a 32-byte aligned vector whose length is a multiple of 8")
        if n > 2 * self.capacity:
            raise ValueError(f"{n} bf16 values exceed the symmetric buffer capacity {2 * self.capacity}")
        code = self.lib.pnm_peer_allreduce_bf16(x.data_ptr(), n, float(scale), *self._brw(),
                                                self.next_epoch(), self.capacity, self.budget_s, _g._stream(),
                                                self.epoch_base.data_ptr(), int(max_ctas))
        _g._check(code, "pnm_peer_allreduce_bf16")
        _g.launch_count += 1
        return x

    def signal(self, epoch: int) -> None:
        """Raise this rank's flag of call ``epoch`` on every peer (after everything already enqueued on the stream)."""
        code = self.lib.pnm_peer_signal(*self._brw(), epoch, self.capacity, _g._stream(),
                                        self.epoch_base.data_ptr())
        _g._check(code, "pnm_peer_signal")
        _g.launch_count += 1

    def pull(self, src_ptr: int, dst: torch.Tensor, nbytes: int, epoch: int, flag_from: int = -1, max_ctas: int = 0) -> None:
        """Copy ``nbytes`` from the peer-mapped address ``src_ptr`` into ``dst`` once ``flag_from`` signalled ``epoch``."""
        code = self.lib.pnm_peer_pull(src_ptr, dst.data_ptr(), int(nbytes), int(flag_from), *self._brw(), epoch, self.capacity, self.budget_s, _g._stream(),
                                      self.epoch_base.data_ptr(), int(max_ctas))
        _g._check(code, "pnm_peer_pull")
        _g.launch_count += 1

    def pull_reduce(self, dst: torch.Tensor, block: int, epoch: int, max_ctas: int = 0) -> None:
        """``dst[i] = sum_r stageA_r[rank * block + i]`` after every rank signalled ``epoch`` (pull-model reduce-scatter)."""
        code = self.lib.pnm_peer_pull_reduce(dst.data_ptr(), int(block), *self._brw(), epoch,
                                             self.capacity, self.budget_s, _g._stream(), self.epoch_base.data_ptr(),
                                             int(max_ctas))
        _g._check(code, "pnm_peer_pull_reduce")
        _g.launch_count += 1

    # ------------------------------------------------------------------ step bookkeeping / failure handling
    def step_done(self) -> None:
        """Fold the calls made since the last ``step_done`` into the device-side call counter and poll for time-outs.

        Must be the last peer operation of a step that is captured into a CUDA graph; harmless otherwise.  The poll
        is non-blocking: it inspects the copy of the error word enqueued ``poll_every`` steps ago.
        """
        if self.epoch:
            self.epoch_base.add_(self.epoch)
            self._folded += self.epoch
            self.epoch = 0
        if torch.cuda.is_current_stream_capturing():
            return
        self.poll()

    def poll(self) -> None:
        """Raise ``PeerTimeoutError`` if an earlier enqueued copy of the error word shows a time-out; enqueue a new copy."""
        if self._err_event is not None and self._err_event.query():
            code = int(self._err_host.item())
            self._err_event = None
            if code:
                raise PeerTimeoutError(f"device error word = {code} (6 = wait on a peer flag ran out); call recover() on every rank")
        self._steps += 1
        if self._err_event is None and self._steps % self.poll_every == 0:
            self.lib.pnm_error_copy_async(self._err_host.data_ptr(), _g._stream())
            self._err_event = torch.cuda.Event()
            self._err_event.record()

    def check(self) -> None:
        """Raise ``PeerTimeoutError`` if any bounded wait has run out (synchronises the device)."""
        err = self.lib.pnm_get_error()
        if err != 0:
            raise PeerTimeoutError(f"device error word = {err} (6 = wait on a peer flag ran out); call recover() on every rank")

    def audit_flags(self) -> dict:
        """Collective consistency check of this rank's flag block at a quiescent point (debug aid against stray or
        reordered signals).  Flags hold the call number of the last signal that peer ``r`` raised for CTA ``c`` in
        ``[slot][phase]``; after a device synchronisation and a barrier every signal of every finished call has landed,
        so: no flag may exceed the current call number, the columns of ranks that do not exist must still be zero,
        and the flags of one (slot, phase, CTA) row that were written may differ between peers by at most the calls
        still allowed in flight (one per slot).  Returns the per-peer maxima; raises ``RuntimeError`` on a violation."""
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        words = self.buffer[: self.flag_bytes].view(torch.int32).cpu().view(2, 2, -1, 8)      # [slot][phase][cta][rank]
        now = int(self.epoch_base.item()) + self.epoch
        if int(words.max()) > now:
            raise RuntimeError(f"a flag carries call number {int(words.max())} but only {now} calls were made")
        if self.world < 8 and int(words[..., self.world:].abs().max()) != 0:
            raise RuntimeError("a flag column of a rank outside the group was written")
        live = words[..., : self.world]
        written = live.max(dim=-1).values > 0
        spread = (live.max(dim=-1).values - live.min(dim=-1).values)[written]
        if spread.numel() and int(spread.max()) > 2:
            raise RuntimeError(f"peers disagree by {int(spread.max())} calls on one flag row (at most 2 may be in flight)")
        dist.barrier(group=self.group)
        return {"calls": now, "max_per_peer": [int(live[..., r].max()) for r in range(self.world)]}

    def recover(self) -> None:
        """Collective: bring flags, call numbers and the error word back to their initial state after a time-out."""
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self.buffer[: self.flag_bytes].zero_()
        self.epoch_base.zero_()
        self.epoch = 0
        self._folded = 0
        self._err_event = None
        self.lib.pnm_reset_error()
        torch.cuda.synchronize()
        dist.barrier(group=self.group)


_runtimes: Dict[Tuple[str, str], PeerRuntime] = {}


def get_runtime(group: Optional[dist.ProcessGroup] = None, purpose: str = "compute", capacity_floats: int = 1 << 20) -> PeerRuntime:
    """Process-wide runtime of ``group`` for one ``purpose`` (one stream of calls: every purpose has its own call numbers)."""
    g = group if group is not None else dist.group.WORLD
    key = (g.group_name, purpose)
    rt = _runtimes.get(key)
    if rt is None or rt.capacity < capacity_floats:
        rt = PeerRuntime(g, capacity_floats=capacity_floats)
        _runtimes[key] = rt
    return rt


def peer_available(t: Optional[torch.Tensor] = None) -> bool:
    """Whether the peer-memory kernels can serve this process (CUDA, NCCL group initialised, library present)."""
    if not (torch.cuda.is_available() and dist.is_available() and dist.is_initialized()):
        return False
    if t is not None and not t.is_cuda:
        return False
    return dist.get_backend() == "nccl" and _lib.available()


class PeerAllReduce:
    """Callable all-reduce used by ``PointParallel`` (fp32 vectors up to ``max_numel``)."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None, max_numel: int = 1 << 23):
        self.rt = PeerRuntime(group, capacity_floats=max_numel)
        self.max_numel = max_numel
        self.world = self.rt.world

    def all_reduce(self, flat: torch.Tensor) -> torch.Tensor:
        return self.rt.all_reduce(flat.contiguous())

    def step_done(self) -> None:
        self.rt.step_done()


class PeerRegions:
    """Fixed regions of one symmetric buffer for producer → consumer exchanges that are summed by the consumer.

    A producer kernel of every rank writes its partial result into ``region()`` (this rank's copy, ordinary local
    memory that the peers have mapped), ``publish()`` raises the rank's flag of a fresh call number on every peer,
    and the consuming kernel — given the addresses of all ranks' copies and the peer arguments — waits for the flags
    and adds the copies with direct loads.  Regions are handed out round-robin within a step (``step_done()`` rewinds),
    so their addresses are the same in every step and a captured CUDA graph stays valid; a region is reused only after
    at least one other exchange, whose flags order the reuse behind every peer's reads.
    """

    def __init__(self, group: Optional[dist.ProcessGroup] = None, region_floats: int = 1 << 18, n_regions: int = 32,
                 budget_s: float = 30.0):
        self.region_floats = (int(region_floats) + 63) // 64 * 64
        self.n_regions = max(2, int(n_regions))
        total = self.region_floats * self.n_regions
        self.rt = PeerRuntime(group, capacity_floats=(total + 3) // 4, budget_s=budget_s)
        self.world = self.rt.world
        self._i = 0

    def region(self, floats: int, device=None):
        """``(fp32 view of this rank's copy, [address of every rank's copy])`` of the next region of the step."""
        if floats > self.region_floats:
            raise ValueError(f"{floats} floats exceed the region size {self.region_floats}")
        rt = self.rt
        off = rt.flag_bytes + (self._i % self.n_regions) * self.region_floats * 4
        self._i += 1
        view = rt.buffer[off: off + floats * 4].view(torch.float32)
        ptrs = [rt.ptrs[rt.rank] + off] if rt.loopback else [p + off for p in rt.ptrs]
        return view, ptrs

    def publish(self):
        """Raise the flags of a new call number (after the producers already enqueued); returns the peer arguments."""
        rt = self.rt
        epoch = rt.next_epoch()
        rt.signal(epoch)
        return rt.peer_args(epoch)

    def step_done(self) -> None:
        self._i = 0
        self.rt.step_done()

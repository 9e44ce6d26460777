"""Adam / AdamW whose whole step is one kernel launch.

The reference trains with ``torch.optim.Adam(fused=True)`` (recipes under ``examples/``); here
the multi-tensor kernel of ``csrc/optim.cu`` walks a device table of (param, grad, m, v)
pointers, so a step costs one small host→device table copy and one launch regardless of the
number of parameters.  CPU tensors (and anything that is not fp32 parameters with fp32 / bf16
gradients) take the plain PyTorch formula, which is also the test oracle.
"""
from __future__ import annotations

import ctypes
import math
from typing import Callable, Iterable, Optional

import torch
from torch.optim import Optimizer

from ..ops import _lib
from ..ops import gemm as _g

_ENTRY_WORDS = 6  # 48 bytes: p, g, m, v, n, (g_bf16 | pad)


def _declare(lib):
    if getattr(lib, "_opt_declared", False):
        return
    c = ctypes
    lib.pnm_opt_chunk.restype = c.c_int
    lib.pnm_adam_multi.argtypes = [c.c_void_p, c.c_void_p, c.c_int] + [c.c_float] * 7 + [c.c_int, c.c_float, c.c_void_p, c.c_void_p]
    lib.pnm_adam_multi.restype = c.c_int
    lib.pnm_grad_sqnorm_multi.argtypes = [c.c_void_p, c.c_void_p, c.c_int, c.c_void_p, c.c_void_p]
    lib.pnm_grad_sqnorm_multi.restype = c.c_int
    lib._opt_declared = True


class _Tables:
    """Device copy of the entry / block tables of one parameter group, fed from a ring of pinned host buffers.

    The upload is an asynchronous copy, and a GPU-bound training loop runs the host several steps ahead of the device:
    a host buffer is therefore rewritten only after the copy that last read it has executed (one event per ring slot),
    and not at all while the pointers are the ones already on the device.  Under stream capture the copy becomes a node
    that re-reads its host buffer at every replay, so captured uploads get a buffer of their own that is never reused.
    """

    RING = 3

    def __init__(self, n_entries: int, n_blocks: int, device, blocks: torch.Tensor):
        words = n_entries * _ENTRY_WORDS + n_blocks
        self.n_entries, self.n_blocks = n_entries, n_blocks
        self.blocks = blocks
        self.hosts = [self._new_host(words) for _ in range(self.RING)]
        self.events = [None] * self.RING
        self.slot = 0
        self.dev = torch.empty(words, dtype=torch.int64, device=device)
        self.rows_on_device = None
        self.captured_hosts = []
        self.spare = self._new_host(words)       # pinned memory cannot be allocated while a stream is capturing

    def _new_host(self, words: int) -> torch.Tensor:
        h = torch.empty(words, dtype=torch.int64).pin_memory()
        h[self.n_entries * _ENTRY_WORDS:] = self.blocks
        return h

    def upload(self, rows):
        """Make the device table hold ``rows`` (a flat list of ints); returns the entry and block table addresses."""
        capturing = torch.cuda.is_current_stream_capturing()
        if capturing or rows != self.rows_on_device:
            if capturing:
                host, self.spare = self.spare, None
                if host is None:
                    raise RuntimeError("FusedAdam: run one eager step between two captures of step() (staging buffers "
                                       "for a captured step are set aside outside of capture)")
                self.captured_hosts.append(host)
            else:
                if self.spare is None:
                    self.spare = self._new_host(self.dev.numel())
                self.slot = (self.slot + 1) % self.RING
                ev = self.events[self.slot]
                if ev is not None:
                    ev.synchronize()                      # the copy that last read this buffer has run
                host = self.hosts[self.slot]
            host[: len(rows)] = torch.tensor(rows, dtype=torch.int64)
            self.dev.copy_(host, non_blocking=True)
            if not capturing:
                ev = self.events[self.slot] or torch.cuda.Event()
                ev.record()
                self.events[self.slot] = ev
            # a captured upload is replayed later with these rows; an eager step in between must upload again
            self.rows_on_device = None if capturing else list(rows)
        base = self.dev.data_ptr()
        return base, base + self.n_entries * _ENTRY_WORDS * 8


def build_tables(params, grads, ms, vs, chunk: int, cache: dict):
    """The (cached by shape signature) tables for the given tensors and the rows that describe them."""
    key = tuple(p.numel() for p in params)
    t = cache.get(key)
    if t is None:
        blocks = []
        for i, n in enumerate(key):
            blocks += [i | (j << 32) for j in range((n + chunk - 1) // chunk)]  # int2 {entry, chunk} little-endian
        t = cache[key] = _Tables(len(params), len(blocks), params[0].device, torch.tensor(blocks, dtype=torch.int64))
    rows = []
    for p, g, m, v in zip(params, grads, ms, vs):
        rows += [p.data_ptr(), g.data_ptr(), m.data_ptr() if m is not None else 0, v.data_ptr() if v is not None else 0,
                 p.numel(), 1 if g.dtype == torch.bfloat16 else 0]
    return t, rows


class FusedAdam(Optimizer):
    """``Adam`` (``adam_w_mode=False``) or ``AdamW`` with the semantics of ``torch.optim``."""

    def __init__(self, params: Iterable, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, adam_w_mode: bool = False, grad_scale: float = 1.0, capturable: bool = False):
        if lr < 0 or eps < 0 or not 0 <= betas[0] < 1 or not 0 <= betas[1] < 1:
            raise ValueError("invalid Adam hyper-parameters")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, adam_w_mode=adam_w_mode,
                                      grad_scale=grad_scale))
        self._tables: dict = {}
        self.kernel_launches = 0
        # capturable: learning rate and step count live in a device tensor per group ({lr, step}); ``step()`` then
        # contains no host-computed scalar, so it can be captured into a CUDA graph and replayed.  Change the learning
        # rate of a captured optimizer with ``set_lr`` (writes the device value), not through ``param_groups``.
        self.capturable = capturable
        self._hyper: dict = {}

    def _state_of(self, p):
        st = self.state[p]
        if not st:
            st["step"] = 0
            st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.preserve_format)
            st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.preserve_format)
        return st

    def _hyper_of(self, gi: int, group, device) -> torch.Tensor:
        h = self._hyper.get(gi)
        if h is None:
            done = max((int(self.state[p]["step"]) for p in group["params"] if p in self.state and self.state[p]), default=1) - 1
            h = self._hyper[gi] = torch.tensor([float(group["lr"]), float(max(done, 0))], dtype=torch.float32, device=device)
        return h

    def set_lr(self, lr: float, group: Optional[int] = None) -> None:
        """Set the learning rate of one group (or all): host value and, if capturable, the device value."""
        for gi, g in enumerate(self.param_groups):
            if group is None or gi == group:
                g["lr"] = lr
                if gi in self._hyper:
                    self._hyper[gi][0] = float(lr)

    def _sync_host_from_device(self) -> None:
        """Capturable mode keeps {lr, step} on the device and graph replays advance them without running ``step()``:
        bring the host copies (``param_groups[i]["lr"]``, ``state[p]["step"]``) up to date."""
        for gi, group in enumerate(self.param_groups):
            h = self._hyper.get(gi)
            if h is None:
                continue
            lr, t = (float(v) for v in h.tolist())
            group["lr"] = lr
            for p in group["params"]:
                if p in self.state and self.state[p]:
                    self.state[p]["step"] = int(round(t))

    def state_dict(self):
        if self.capturable:
            self._sync_host_from_device()
        return super().state_dict()

    def load_state_dict(self, state_dict) -> None:
        super().load_state_dict(state_dict)
        for gi, group in enumerate(self.param_groups):
            steps = [int(self.state[p]["step"]) for p in group["params"] if p in self.state and "step" in self.state[p]]
            for p in group["params"]:
                if p in self.state and "step" in self.state[p]:
                    self.state[p]["step"] = int(self.state[p]["step"])
            if self.capturable and steps:
                dev = next((p.device for p in group["params"] if p.is_cuda), None)
                if dev is None:
                    continue
                vals = torch.tensor([float(group["lr"]), float(steps[0])], dtype=torch.float32, device=dev)
                if gi in self._hyper:
                    self._hyper[gi].copy_(vals)          # in place: a captured graph keeps reading this tensor
                else:
                    self._hyper[gi] = vals

    @torch.no_grad()
    def step(self, closure: Optional[Callable] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for gi, group in enumerate(self.param_groups):
            ps = [p for p in group["params"] if p.grad is not None]
            if not ps:
                continue
            lr = float(group["lr"])
            b1, b2 = group["betas"]
            fused, plain = [], []
            for p in ps:
                ok = (p.is_cuda and p.dtype == torch.float32 and p.is_contiguous() and p.grad.is_contiguous()
                      and p.grad.dtype in (torch.float32, torch.bfloat16) and not p.grad.is_sparse)
                (fused if ok else plain).append(p)
            for p in plain:
                st = self._state_of(p)
                st["step"] += 1
                g = p.grad.float() * group["grad_scale"]
                pf = p.float() if p.dtype != torch.float32 else p
                if group["adam_w_mode"]:
                    pf.mul_(1 - lr * group["weight_decay"])
                elif group["weight_decay"]:
                    g = g + group["weight_decay"] * pf
                st["exp_avg"].lerp_(g, 1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
                bc1, bc2 = 1 - b1 ** st["step"], 1 - b2 ** st["step"]
                pf.addcdiv_(st["exp_avg"], (st["exp_avg_sq"].sqrt() / math.sqrt(bc2)).add_(group["eps"]), value=-lr / bc1)
                if pf is not p:
                    p.copy_(pf)
            if fused:
                lib = _lib.load(required=True)
                _declare(lib)
                sts = [self._state_of(p) for p in fused]
                for st in sts:
                    st["step"] += 1
                t = sts[0]["step"]
                if any(st["step"] != t for st in sts):
                    raise RuntimeError("parameters of one group must share the step count")
                tab, rows = build_tables(fused, [p.grad for p in fused], [s["exp_avg"] for s in sts],
                                         [s["exp_avg_sq"] for s in sts], lib.pnm_opt_chunk(), self._tables.setdefault(gi, {}))
                e_ptr, b_ptr = tab.upload(rows)
                hyper = None
                if self.capturable:
                    hyper = self._hyper_of(gi, group, fused[0].device)
                    hyper[1:2].add_(1.0)                  # device-side step count (captured with the step)
                err = lib.pnm_adam_multi(e_ptr, b_ptr, tab.n_blocks, lr, b1, b2, group["eps"], group["weight_decay"],
                                         lr / (1 - b1 ** t), 1.0 / math.sqrt(1 - b2 ** t), int(group["adam_w_mode"]),
                                         group["grad_scale"], torch.cuda.current_stream().cuda_stream,
                                         hyper.data_ptr() if hyper is not None else None)
                if err:
                    raise RuntimeError(f"pnm_adam_multi failed with CUDA error {err}")
                self.kernel_launches += 1
                _g.launch_count += 1
        return loss


def FusedAdamW(params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, **kw) -> FusedAdam:
    return FusedAdam(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, adam_w_mode=True, **kw)


def grad_global_norm(params: Iterable[torch.Tensor]) -> torch.Tensor:
    """L2 norm of all gradients: one kernel on CUDA (fp32 / bf16 gradients), ``torch`` otherwise."""
    ps = [p for p in params if p.grad is not None]
    if not ps:
        return torch.zeros(())
    if all(p.is_cuda and p.grad.is_contiguous() and p.grad.dtype in (torch.float32, torch.bfloat16) for p in ps):
        lib = _lib.load(required=True)
        _declare(lib)
        cache = grad_global_norm.__dict__.setdefault("_cache", {})
        tab, rows = build_tables(ps, [p.grad for p in ps], [None] * len(ps), [None] * len(ps), lib.pnm_opt_chunk(), cache)
        e_ptr, b_ptr = tab.upload(rows)
        out = torch.zeros(1, device=ps[0].device, dtype=torch.float32)
        err = lib.pnm_grad_sqnorm_multi(e_ptr, b_ptr, tab.n_blocks, out.data_ptr(), torch.cuda.current_stream().cuda_stream)
        if err:
            raise RuntimeError(f"pnm_grad_sqnorm_multi failed with CUDA error {err}")
        return out.sqrt()[0]
    return torch.linalg.vector_norm(torch.stack([torch.linalg.vector_norm(p.grad.float()) for p in ps]))

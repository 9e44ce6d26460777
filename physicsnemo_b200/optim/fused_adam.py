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
    """Pinned host + device copies of the entry / block tables of one parameter group."""

    def __init__(self, n_entries: int, n_blocks: int, device):
        self.host = torch.empty(n_entries * _ENTRY_WORDS + n_blocks, dtype=torch.int64).pin_memory()
        self.dev = torch.empty_like(self.host, device=device)
        self.n_entries, self.n_blocks = n_entries, n_blocks

    def upload(self):
        self.dev.copy_(self.host, non_blocking=True)
        base = self.dev.data_ptr()
        return base, base + self.n_entries * _ENTRY_WORDS * 8


def build_tables(params, grads, ms, vs, chunk: int, cache: dict):
    """Fill (and cache by shape signature) the tables for the given tensors."""
    key = tuple(p.numel() for p in params)
    n_blocks = sum((n + chunk - 1) // chunk for n in key)
    t = cache.get(key)
    if t is None:
        t = cache[key] = _Tables(len(params), n_blocks, params[0].device)
        blocks = []
        for i, n in enumerate(key):
            blocks += [i | (j << 32) for j in range((n + chunk - 1) // chunk)]  # int2 {entry, chunk} little-endian
        t.host[len(params) * _ENTRY_WORDS:] = torch.tensor(blocks, dtype=torch.int64)
    rows = []
    for p, g, m, v in zip(params, grads, ms, vs):
        rows += [p.data_ptr(), g.data_ptr(), m.data_ptr() if m is not None else 0, v.data_ptr() if v is not None else 0,
                 p.numel(), 1 if g.dtype == torch.bfloat16 else 0]
    t.host[: len(rows)] = torch.tensor(rows, dtype=torch.int64)
    return t


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
            h = self._hyper[gi] = torch.tensor([float(group["lr"]), 0.0], dtype=torch.float32, device=device)
        return h

    def set_lr(self, lr: float, group: Optional[int] = None) -> None:
        """Set the learning rate of one group (or all): host value and, if capturable, the device value."""
        for gi, g in enumerate(self.param_groups):
            if group is None or gi == group:
                g["lr"] = lr
                if gi in self._hyper:
                    self._hyper[gi][0] = float(lr)

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
                tab = build_tables(fused, [p.grad for p in fused], [s["exp_avg"] for s in sts],
                                   [s["exp_avg_sq"] for s in sts], lib.pnm_opt_chunk(), self._tables.setdefault(gi, {}))
                e_ptr, b_ptr = tab.upload()
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
        tab = build_tables(ps, [p.grad for p in ps], [None] * len(ps), [None] * len(ps), lib.pnm_opt_chunk(), cache)
        e_ptr, b_ptr = tab.upload()
        out = torch.zeros(1, device=ps[0].device, dtype=torch.float32)
        err = lib.pnm_grad_sqnorm_multi(e_ptr, b_ptr, tab.n_blocks, out.data_ptr(), torch.cuda.current_stream().cuda_stream)
        if err:
            raise RuntimeError(f"pnm_grad_sqnorm_multi failed with CUDA error {err}")
        return out.sqrt()[0]
    return torch.linalg.vector_norm(torch.stack([torch.linalg.vector_norm(p.grad.float()) for p in ps]))

"""Muon: momentum + Newton–Schulz orthogonalised updates for 2-D parameters.

Parity: ``physicsnemo/optim/muon.py:54-118`` (batched quintic Newton–Schulz iteration in bf16 on
a ``(G, M, N)`` stack) and ``:121-293`` (parameters of equal shape are stacked so each shape
costs three batched GEMMs per iteration).  Hyper-parameters and learning-rate adjustment
follow ``torch.optim.Muon``.
"""
from __future__ import annotations

import math
from collections import defaultdict
from typing import Callable, Iterable

import torch
from torch import Tensor
from torch.optim import Optimizer

__all__ = ["Muon"]


def _batched_newton_schulz(updates: Tensor, ns_coefficients: tuple[float, float, float], ns_steps: int,
                           eps: float) -> Tensor:
    """Approximate ``U Vᵀ`` of every matrix of the stack ``updates`` (G, M, N)."""
    if ns_steps >= 100:
        raise ValueError("Number of steps must be less than 100 for computational efficiency")
    if updates.ndim != 3:
        raise ValueError("Batched Newton-Schulz expects a 3D (G, M, N) tensor")
    if len(ns_coefficients) != 3:
        raise ValueError("Coefficients must be a tuple of exactly 3 values")
    a, b, c = ns_coefficients
    x = updates.bfloat16()
    wide = x.size(1) <= x.size(2)
    if not wide:
        x = x.transpose(1, 2)
    x = x / x.norm(dim=(1, 2), keepdim=True).clamp(min=eps)
    for _ in range(ns_steps):
        gram = torch.bmm(x, x.transpose(1, 2))
        poly = torch.baddbmm(gram, gram, gram, beta=b, alpha=c)      # b·A + c·A²
        x = torch.baddbmm(x, poly, x, beta=a, alpha=1.0)             # a·X + (b·A + c·A²)·X
    return x if wide else x.transpose(1, 2)


def _adjust_lr(lr: float, adjust_lr_fn: str | None, shape) -> float:
    rows, cols = shape[:2]
    if adjust_lr_fn is None or adjust_lr_fn == "original":
        return lr * math.sqrt(max(1, rows / cols))
    if adjust_lr_fn == "match_rms_adamw":
        return lr * 0.2 * math.sqrt(max(rows, cols))
    return lr


class Muon(Optimizer):
    def __init__(self, params: Iterable, lr: float = 1e-3, weight_decay: float = 0.1, momentum: float = 0.95,
                 nesterov: bool = True, ns_coefficients: tuple[float, float, float] = (3.4445, -4.775, 2.0315),
                 eps: float = 1e-7, ns_steps: int = 5, adjust_lr_fn: str | None = None):
        if lr < 0 or momentum < 0 or weight_decay < 0:
            raise ValueError("lr, momentum and weight_decay must be non-negative")
        if adjust_lr_fn not in (None, "original", "match_rms_adamw"):
            raise ValueError(f"Adjust learning rate function {adjust_lr_fn} is not supported")
        super().__init__(params, dict(lr=lr, weight_decay=weight_decay, momentum=momentum, nesterov=nesterov,
                                      ns_coefficients=ns_coefficients, eps=eps, ns_steps=ns_steps,
                                      adjust_lr_fn=adjust_lr_fn))
        for group in self.param_groups:
            for p in group["params"]:
                if p.ndim != 2:
                    raise ValueError(f"Muon only supports 2D parameters whereas we found a parameter with size: {p.size()}")

    @staticmethod
    def _group_params_by_shape(params: list[Tensor]) -> dict[tuple, list[int]]:
        by_shape: dict[tuple, list[int]] = defaultdict(list)
        for i, p in enumerate(params):
            by_shape[(tuple(p.shape), p.dtype, p.device)].append(i)
        return by_shape

    @torch.no_grad()
    def step(self, closure: Callable[[], float] | None = None) -> float | None:
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            lr = group["lr"].item() if isinstance(group["lr"], Tensor) else group["lr"]
            mu = group["momentum"]
            ps, gs, bufs = [], [], []
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.ndim != 2:
                    raise ValueError("Param gradient must be a 2D matrix")
                st = self.state[p]
                if "momentum_buffer" not in st:
                    st["momentum_buffer"] = torch.zeros_like(p.grad, memory_format=torch.preserve_format)
                ps.append(p), gs.append(p.grad), bufs.append(st["momentum_buffer"])
            if not ps:
                continue
            torch._foreach_lerp_(bufs, gs, 1 - mu)
            updates = torch._foreach_lerp(gs, bufs, mu) if group["nesterov"] else list(bufs)
            torch._foreach_mul_(ps, 1 - lr * group["weight_decay"])
            for (shape, _, _), idxs in self._group_params_by_shape(ps).items():
                ortho = _batched_newton_schulz(torch.stack([updates[i] for i in idxs]), group["ns_coefficients"],
                                               group["ns_steps"], group["eps"])
                members = [ps[i] for i in idxs]
                torch._foreach_add_(members, [ortho[j].to(members[j].dtype) for j in range(len(idxs))],
                                    alpha=-_adjust_lr(lr, group["adjust_lr_fn"], shape))
        return loss

    def __repr__(self) -> str:
        return f"{self.__class__.__name__} (fused Newton-Schulz)"

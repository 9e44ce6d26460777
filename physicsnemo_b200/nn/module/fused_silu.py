"""SiLU whose 1st–3rd derivatives are themselves single-kernel autograd functions.

Parity: ``physicsnemo/nn/module/fused_silu.py`` (``FusedSiLU``, ``FusedSiLU_deriv_1/2/3`` built on
nvFuser fusion definitions with activation recomputation).  Here every order is one launch of
``pnm_silu_derivative`` (``csrc/elementwise.cu``), which evaluates ``silu^(k)(x) · g`` in closed
form from ``sigmoid(x)``; the chain goes one order further than the reference (the backward of
the third derivative is again one kernel), so fourth-order input derivatives stay fused.  Only
``x`` is saved for backward.  On CPU the same closed forms run as tensor expressions.
"""
from __future__ import annotations

import ctypes

import torch
from torch.autograd import Function

from ...ops import _lib
from ...ops import gemm as _g

_DT = {torch.bfloat16: 0, torch.float32: 1}


def silu_derivative_reference(x: torch.Tensor, order: int) -> torch.Tensor:
    """Closed-form ``silu^(order)(x)``, ``order`` in 0..4 (tensor expression; CPU path and oracle)."""
    s = torch.sigmoid(x)
    if order == 0:
        return x * s
    d1 = s * (1 - s)
    if order == 1:
        return s + x * d1
    t = 1 - 2 * s
    d2 = d1 * t
    if order == 2:
        return 2 * d1 + x * d2
    d3 = d2 * t - 2 * d1 * d1
    if order == 3:
        return 3 * d2 + x * d3
    if order == 4:
        return 4 * d3 + x * (d3 * t - 6 * d1 * d2)
    raise ValueError(f"order must be in 0..4, got {order}")


def _kernel(x: torch.Tensor, g, order: int) -> torch.Tensor:
    if not (x.is_cuda and x.dtype in _DT):
        out = silu_derivative_reference(x, order)
        return out if g is None else out * g
    lib = _lib.load(required=True)
    if not getattr(lib, "_silu_declared", False):
        vp = ctypes.c_void_p
        lib.pnm_silu_derivative.argtypes = [vp, vp, vp, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, vp]
        lib.pnm_silu_derivative.restype = ctypes.c_int
        lib._silu_declared = True
    xc = x.contiguous()
    gc = None if g is None else g.to(x.dtype).expand_as(x).contiguous()
    out = torch.empty_like(xc)
    err = lib.pnm_silu_derivative(xc.data_ptr(), None if gc is None else gc.data_ptr(), out.data_ptr(), xc.numel(), order,
                                  _DT[x.dtype], torch.cuda.current_stream().cuda_stream)
    if err == -2:                                     # a view at an odd offset: 16-byte alignment not met
        out = silu_derivative_reference(x, order)
        return out if g is None else out * g
    if err:
        raise RuntimeError(f"pnm_silu_derivative failed ({err})")
    _g.launch_count += 1
    return out


def _make(order: int, name: str):
    class _Fn(Function):
        @staticmethod
        def forward(ctx, x):
            ctx.save_for_backward(x)
            return _kernel(x, None, order)

        @staticmethod
        def backward(ctx, grad_output):
            (x,) = ctx.saved_tensors
            if order >= 4:
                raise RuntimeError("SiLU derivatives are fused up to the fourth order")
            nxt = _ORDERS[order + 1]
            if torch.is_grad_enabled() and (x.requires_grad or grad_output.requires_grad):
                return nxt.apply(x) * grad_output          # keep the chain differentiable
            return _kernel(x, grad_output, order + 1)     # leaf of the chain: derivative and product in one launch

    _Fn.__name__ = _Fn.__qualname__ = name
    return _Fn


_ORDERS: list = []
for _k, _n in enumerate(["FusedSiLU", "FusedSiLU_deriv_1", "FusedSiLU_deriv_2", "FusedSiLU_deriv_3", "FusedSiLU_deriv_4"]):
    _ORDERS.append(_make(_k, _n))
FusedSiLU, FusedSiLU_deriv_1, FusedSiLU_deriv_2, FusedSiLU_deriv_3, FusedSiLU_deriv_4 = _ORDERS


def fused_silu(x: torch.Tensor) -> torch.Tensor:
    return FusedSiLU.apply(x)


class FusedSiLUModule(torch.nn.Module):
    """``nn.Module`` face of ``FusedSiLU`` (drop-in for ``nn.SiLU`` in networks differentiated to high order)."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return FusedSiLU.apply(x)

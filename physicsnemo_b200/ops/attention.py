"""Scaled-dot-product attention on the library's tcgen05 flash kernel (``csrc/flash_attn.cuh``).

``sdpa(q, k, v, is_causal=False, scale=None)`` takes ``[..., S, D]`` tensors like
``torch.nn.functional.scaled_dot_product_attention``.  The kernel covers CUDA bf16 tensors with head dimension 64 or
128, no additive mask and no dropout (``supported``); everything else goes to the PyTorch operator.  The forward keeps
the row-wise log-sum-exp; the backward recomputes the attention with the PyTorch operator under autograd, so the
gradients are those of the reference operator on the same inputs.

``flash_forward`` is the raw kernel call and returns ``(out, lse)``; ``v_layout`` selects how V reaches the tensor
core: ``"natural"`` reads ``[keys, D]`` tiles as an MN-major operand, ``"transposed"`` makes one ``[D, keys]`` copy
and reads it K-major.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _lib
from . import gemm as _g

V_LAYOUT = "natural"
P_IN_TMEM = False


def _lib_fa():
    lib = _lib.load(required=True)
    if not getattr(lib, "_fa_declared", False):
        c = ctypes
        vp, i, f = c.c_void_p, c.c_int, c.c_float
        lib.pnm_flash_attn_fwd.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, f, i, i, i, vp]
        lib.pnm_flash_attn_fwd.restype = i
        lib._fa_declared = True
    return lib


def supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    if not (q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == v.dtype == q.dtype):
        return False
    if q.dim() < 3 or q.shape[-1] not in (64, 128) or k.shape[-1] != q.shape[-1] or v.shape != k.shape:
        return False
    if q.shape[:-2] != k.shape[:-2] or q.shape[-2] == 0 or k.shape[-2] == 0:
        return False
    return math.prod(q.shape[:-2]) * ((q.shape[-2] + 127) // 128) < 2 ** 31


def flash_forward(q, k, v, is_causal: bool = False, scale: float | None = None, v_layout: str | None = None, p_in_tmem: bool | None = None):
    if not supported(q, k, v):
        raise ValueError("flash_forward needs CUDA bf16 tensors [..., S, D] with D in (64, 128) and matching batch dimensions")
    lead, Sq, D = q.shape[:-2], q.shape[-2], q.shape[-1]
    Skv = k.shape[-2]
    BH = math.prod(lead)
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(D)
    if not scale > 0:
        raise ValueError("scale must be positive")
    q3, k3 = q.reshape(BH, Sq, D).contiguous(), k.reshape(BH, Skv, D).contiguous()
    layout = v_layout or V_LAYOUT
    if layout == "transposed":
        ldv = (Skv + 7) // 8 * 8
        v3 = torch.zeros(BH, D, ldv, dtype=v.dtype, device=v.device) if ldv != Skv else torch.empty(BH, D, ldv, dtype=v.dtype, device=v.device)
        v3[:, :, :Skv].copy_(v.reshape(BH, Skv, D).transpose(1, 2))
        vt = 1
    elif layout == "natural":
        v3, ldv, vt = v.reshape(BH, Skv, D).contiguous(), 0, 0
    else:
        raise ValueError(f"v_layout must be 'natural' or 'transposed', got {layout!r}")
    out = torch.empty(BH, Sq, D, dtype=q.dtype, device=q.device)
    lse = torch.empty(BH, Sq, dtype=torch.float32, device=q.device)
    err = _lib_fa().pnm_flash_attn_fwd(q3.data_ptr(), k3.data_ptr(), v3.data_ptr(), out.data_ptr(), lse.data_ptr(), BH, Sq, Skv, D,
                                       ldv, scale, int(bool(is_causal)), vt, int(P_IN_TMEM if p_in_tmem is None else p_in_tmem),
                                       torch.cuda.current_stream().cuda_stream)
    if err:
        raise RuntimeError(f"pnm_flash_attn_fwd failed ({err})")
    _g.launch_count += 1
    return out.reshape(*lead, Sq, D), lse.reshape(*lead, Sq)


class _Flash(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, is_causal, scale):
        out, lse = flash_forward(q, k, v, is_causal, scale)
        ctx.save_for_backward(q, k, v)
        ctx.cfg = (is_causal, scale)
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, grad_out, _grad_lse):
        q, k, v = ctx.saved_tensors
        is_causal, scale = ctx.cfg
        with torch.enable_grad():
            qq, kk, vv = (t.detach().requires_grad_(True) for t in (q, k, v))
            o = torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, is_causal=is_causal, scale=scale)
            gq, gk, gv = torch.autograd.grad(o, (qq, kk, vv), grad_out)
        return gq, gk, gv, None, None


def sdpa(q, k, v, attn_mask=None, dropout_p: float = 0.0, is_causal: bool = False, scale: float | None = None):
    """Drop-in for ``F.scaled_dot_product_attention``; uses the flash kernel when it covers the call."""
    if attn_mask is None and dropout_p == 0.0 and supported(q, k, v) and (scale is None or scale > 0):
        return _Flash.apply(q, k, v, bool(is_causal), scale)[0]
    return torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask, dropout_p=dropout_p,
                                                            is_causal=is_causal, scale=scale)

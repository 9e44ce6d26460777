"""Stride-1 "same" 2-D convolution on the tensor cores, channels-last, bf16.

The kernel is the library's persistent tcgen05 GEMM run as an implicit GEMM: an M tile is an 8 × 16
patch of output pixels, the K loop runs over (filter tap, 64 input channels), and the A operand of each
K block is fetched by ONE 4-D TMA copy of the input window shifted by the tap — coordinates outside the
image read as zeros, which is the padding; no im2col buffer and no padded copy of the input exist.  Bias
and an activation are applied in the epilogue and the result leaves through 4-D TMA stores that the copy
engine clips at the image edge.

Backward: the input gradient is the same kernel on the flipped, transposed filter; the weight gradient
(a reduction over all pixels) uses the framework's convolution-weight-gradient on channels-last views.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib
from . import gemm as _g

_ACT = {None: 0, "none": 0, "gelu": 1, "silu": 2, "relu": 3}


def _lib_conv():
    lib = _lib.load(required=True)
    if not getattr(lib, "_conv_declared", False):
        vp, i = ctypes.c_void_p, ctypes.c_int
        lib.pnm_conv2d_nhwc.argtypes = [vp, vp, vp, i, i, i, i, i, i, vp, i, i, i, vp]
        lib.pnm_conv2d_nhwc.restype = i
        lib._conv_declared = True
    return lib


def supported(x: torch.Tensor, weight: torch.Tensor, stride=1, padding=None, dilation=1, groups=1) -> bool:
    """Whether ``conv2d_same`` covers this call (CUDA, 4-D, square odd filter, stride 1, Cin % 64 == 0, Cout % 8 == 0)."""
    if not (x.is_cuda and x.dim() == 4 and weight.dim() == 4):
        return False
    cout, cin, kh, kw = weight.shape
    one = lambda v: v == 1 or tuple(v) == (1, 1)  # noqa: E731
    if not (one(stride) and one(dilation) and groups == 1 and kh == kw and kh % 2 == 1 and kh <= 7):
        return False
    if padding is not None and padding != "same":
        p = (padding, padding) if isinstance(padding, int) else tuple(padding)
        if p != (kh // 2, kh // 2):
            return False
    return cin % 64 == 0 and cout % 8 == 0 and x.shape[1] == cin


def _pack_weight(weight: torch.Tensor) -> torch.Tensor:
    """``[Cout, Cin, k, k]`` → ``[Cout, k*k*Cin]`` bf16, tap-major."""
    return weight.detach().permute(0, 2, 3, 1).reshape(weight.shape[0], -1).to(torch.bfloat16).contiguous()


def _launch(x_nhwc: torch.Tensor, w_packed: torch.Tensor, bias, ksize: int, act: int) -> torch.Tensor:
    n, h, w, cin = x_nhwc.shape
    cout = w_packed.shape[0]
    y = torch.empty(n, h, w, cout, dtype=torch.bfloat16, device=x_nhwc.device)
    b = None if bias is None else bias.detach().float().contiguous()
    err = _lib_conv().pnm_conv2d_nhwc(x_nhwc.data_ptr(), w_packed.data_ptr(), y.data_ptr(), n, h, w, cin, cout, ksize,
                                      None if b is None else b.data_ptr(), act, 0, 0, torch.cuda.current_stream().cuda_stream)
    if err:
        raise RuntimeError(f"pnm_conv2d_nhwc failed ({err})")
    _g.launch_count += 1
    return y


def _as_nhwc_bf16(t: torch.Tensor) -> torch.Tensor:
    """``[N, C, H, W]`` (any memory format) → contiguous ``[N, H, W, C]`` bf16; free for channels-last bf16 input."""
    return t.permute(0, 2, 3, 1).to(torch.bfloat16).contiguous()


class _ConvSame(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, act: int):
        xh = _as_nhwc_bf16(x)
        y = _launch(xh, _pack_weight(weight), bias, weight.shape[-1], act)
        if act != 0:
            raise RuntimeError("fused activations are inference-only in conv2d_same; apply the activation separately when training")
        ctx.save_for_backward(xh, weight)
        ctx.has_bias = bias is not None
        ctx.x_dtype = x.dtype
        return y.permute(0, 3, 1, 2)                   # NCHW view of channels-last storage

    @staticmethod
    def backward(ctx, dy):
        xh, weight = ctx.saved_tensors
        cout, cin, k, _ = weight.shape
        dyh = _as_nhwc_bf16(dy)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            if cout % 64 == 0 and cin % 8 == 0:
                wt = weight.detach().flip(2, 3).transpose(0, 1)                       # [Cin, Cout, k, k]
                dx = _launch(dyh, _pack_weight(wt), None, k, 0).permute(0, 3, 1, 2).to(ctx.x_dtype)
            else:
                dx = torch.nn.grad.conv2d_input((xh.shape[0], cin, xh.shape[1], xh.shape[2]), weight.to(torch.bfloat16),
                                                dyh.permute(0, 3, 1, 2), padding=k // 2).to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            dw = torch.nn.grad.conv2d_weight(xh.permute(0, 3, 1, 2), weight.shape, dyh.permute(0, 3, 1, 2),
                                             padding=k // 2).to(weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dyh.float().sum(dim=(0, 1, 2))
        return dx, dw, db, None


def conv2d_same(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, act: str | None = None) -> torch.Tensor:
    """``act(conv2d(x, weight, bias, padding=k//2))`` in bf16; returns an NCHW tensor in channels-last memory format.

    ``supported(x, weight)`` must hold.  With ``act`` the call is forward-only (inference).
    """
    code = _ACT[act]
    if code and not (torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad)):
        return _launch(_as_nhwc_bf16(x), _pack_weight(weight), bias, weight.shape[-1], code).permute(0, 3, 1, 2)
    y = _ConvSame.apply(x, weight, bias, 0)
    if code:
        y = {1: F.gelu, 2: F.silu, 3: F.relu}[code](y)
    return y

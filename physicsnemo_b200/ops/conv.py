"""Stride-1 "same" 2-D convolution on the tensor cores, channels-last, bf16 — forward, input gradient, weight gradient.

The forward kernel is the library's persistent tcgen05 GEMM run as an implicit GEMM: an M tile is an 8 × 16
patch of output pixels, the K loop runs over (filter tap, 64 input channels), and the A operand of each
K block is fetched by ONE 4-D TMA copy of the input window shifted by the tap — coordinates outside the
image read as zeros, which is the padding; no im2col buffer and no padded copy of the input exist.  Bias
and an activation are applied in the epilogue and the result leaves through 4-D TMA stores that the copy
engine clips at the image edge.

Backward: the input gradient is the same kernel on the flipped, transposed filter.  The weight gradient of a
3 × 3 filter is the library's reduction GEMM in convolution mode (``pnm_conv2d_wgrad_nhwc``): the reduction runs
over 4 × 16 patches of pixels, both operands arrive as tap-shifted 4-D TMA boxes, the M range is split over the
SMs and the fp32 tiles are added with vector reductions; the bias gradient comes out of the same pass (a
ones-column MMA).  Other filter sizes use the framework's convolution-weight-gradient on channels-last views.

Channel counts that the kernels do not cover directly (``C_in % 64 != 0``, ``C_out < 64``) are zero-padded to 64:
the first (16 → 128) and last (128 → 4) convolutions of a U-Net then run on the same kernels.
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
        vp, i, u, d = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_double
        lib.pnm_conv2d_nhwc.argtypes = [vp, vp, vp, i, i, i, i, i, i, vp, i, i, i, vp]
        lib.pnm_conv2d_nhwc.restype = i
        lib.pnm_conv2d_wgrad_nhwc.argtypes = [vp, vp, vp, vp, i, i, i, i, i, vp, vp, vp, vp, u, d, i, vp]
        lib.pnm_conv2d_wgrad_nhwc.restype = i
        lib._conv_declared = True
    return lib


def _pad64(c: int) -> int:
    return max(64, (c + 63) // 64 * 64)


def supported(x: torch.Tensor, weight: torch.Tensor, stride=1, padding=None, dilation=1, groups=1) -> bool:
    """Whether ``conv2d_same`` covers this call (CUDA, 4-D, square odd filter ≤ 7, stride 1, "same" padding)."""
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
    if x.shape[1] != cin:
        return False
    # padded channel counts must not blow the work up by more than 4x (C_in 16 -> 64 is the intended case)
    return _pad64(cin) <= 4 * cin and (cout % 8 == 0 or cout <= 64)


def _pack_weight(weight: torch.Tensor, cin_pad: int | None = None, cout_pad: int | None = None) -> torch.Tensor:
    """``[Cout, Cin, k, k]`` → ``[Cout', k*k*Cin']`` bf16, tap-major, zero-padded to ``Cout' × Cin'`` channels."""
    w = weight.detach().permute(0, 2, 3, 1)                       # [Cout, k, k, Cin]
    cout, k, _, cin = w.shape
    cin_pad, cout_pad = cin_pad or cin, cout_pad or cout
    if cin_pad != cin or cout_pad != cout:
        w = F.pad(w, (0, cin_pad - cin, 0, 0, 0, 0, 0, cout_pad - cout))
    return w.reshape(cout_pad, -1).to(torch.bfloat16).contiguous()


def _conv_dims(weight: torch.Tensor):
    """Padded channel counts of the kernels for this filter: (cin', cout').

    ``cin'`` is a multiple of 64 (the K blocks of the forward); ``cout'`` is the forward's output width (a multiple of
    8, at least 64).  The backward pads the output gradient to ``_cout_bwd`` channels instead, a multiple of 64,
    because there the output channels are the K dimension."""
    cout, cin = weight.shape[:2]
    cin_p = cin if cin % 64 == 0 else _pad64(cin)
    cout_p = cout if (cout % 8 == 0 and cout >= 64) else _pad64(cout)
    return cin_p, cout_p


def _cout_bwd(weight: torch.Tensor) -> int:
    cout = weight.shape[0]
    return cout if cout % 64 == 0 else _pad64(cout)


def _launch(x_nhwc: torch.Tensor, w_packed: torch.Tensor, bias, ksize: int, act: int) -> torch.Tensor:
    n, h, w, cin = x_nhwc.shape
    cout = w_packed.shape[0]
    y = torch.empty(n, h, w, cout, dtype=torch.bfloat16, device=x_nhwc.device)
    b = None if bias is None else bias.detach().float().contiguous()
    if b is not None and b.numel() != cout:
        b = F.pad(b, (0, cout - b.numel()))
    err = _lib_conv().pnm_conv2d_nhwc(x_nhwc.data_ptr(), w_packed.data_ptr(), y.data_ptr(), n, h, w, cin, cout, ksize,
                                      None if b is None else b.data_ptr(), act, 0, 0, torch.cuda.current_stream().cuda_stream)
    if err:
        raise RuntimeError(f"pnm_conv2d_nhwc failed ({err})")
    _g.launch_count += 1
    return y


def _as_nhwc_bf16(t: torch.Tensor, c_pad: int | None = None) -> torch.Tensor:
    """``[N, C, H, W]`` (any memory format) → contiguous ``[N, H, W, C']`` bf16; free for channels-last bf16 input."""
    t = t.permute(0, 2, 3, 1)
    if c_pad is not None and c_pad != t.shape[-1]:
        return F.pad(t.to(torch.bfloat16), (0, c_pad - t.shape[-1])).contiguous()
    return t.to(torch.bfloat16).contiguous()


def wgrad3x3(dy_nhwc: torch.Tensor, x_nhwc: torch.Tensor, want_bias: bool, up_rows=None, down_rows=None):
    """``(dW [Cout', 9*Cin'] fp32 tap-major, db [Cout'] fp32 or None)`` of a 3 × 3 "same" convolution on the tensor cores.

    ``up_rows`` / ``down_rows``: optional ``[N, 1, W, Cin']`` input rows just above / below a height slab.
    """
    n, h, w, cin = x_nhwc.shape
    cout = dy_nhwc.shape[-1]
    dw = torch.zeros(cout, 9 * cin, dtype=torch.float32, device=x_nhwc.device)
    db = torch.zeros(cout, dtype=torch.float32, device=x_nhwc.device) if want_bias else None
    err = _lib_conv().pnm_conv2d_wgrad_nhwc(
        dy_nhwc.data_ptr(), x_nhwc.data_ptr(), dw.data_ptr(), None if db is None else db.data_ptr(), n, h, w, cin, cout,
        None if up_rows is None else up_rows.data_ptr(), None if down_rows is None else down_rows.data_ptr(), None, None,
        0, 0.0, 0, torch.cuda.current_stream().cuda_stream)
    if err:
        raise RuntimeError(f"pnm_conv2d_wgrad_nhwc failed ({err})")
    _g.launch_count += 1
    return dw, db


def unpack_wgrad(dw: torch.Tensor, weight: torch.Tensor, cin_pad: int) -> torch.Tensor:
    """``[Cout', 9*Cin']`` tap-major → the gradient of ``weight [Cout, Cin, 3, 3]``."""
    cout, cin = weight.shape[:2]
    return dw.reshape(dw.shape[0], 3, 3, cin_pad)[:cout, :, :, :cin].permute(0, 3, 1, 2).to(weight.dtype)


class _ConvSame(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, act: int):
        cin_p, cout_p = _conv_dims(weight)
        xh = _as_nhwc_bf16(x, cin_p)
        y = _launch(xh, _pack_weight(weight, cin_p, cout_p), bias, weight.shape[-1], act)
        if act != 0:
            raise RuntimeError("fused activations are inference-only in conv2d_same; apply the activation separately when training")
        ctx.save_for_backward(xh, weight)
        ctx.has_bias = bias is not None
        ctx.x_dtype = x.dtype
        if cout_p != weight.shape[0]:
            y = y[..., :weight.shape[0]]
        return y.permute(0, 3, 1, 2)                   # NCHW view of channels-last storage

    @staticmethod
    def backward(ctx, dy):
        xh, weight = ctx.saved_tensors
        cout, cin, k, _ = weight.shape
        cin_p, _ = _conv_dims(weight)
        cout_p = _cout_bwd(weight)
        dyh = _as_nhwc_bf16(dy, cout_p)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            wt = weight.detach().flip(2, 3).transpose(0, 1)                           # [Cin, Cout, k, k]
            dxh = _launch(dyh, _pack_weight(wt, cout_p, cin_p), None, k, 0)
            dx = dxh[..., :cin].permute(0, 3, 1, 2).to(ctx.x_dtype)
        need_w, need_b = ctx.needs_input_grad[1], ctx.has_bias and ctx.needs_input_grad[2]
        if k == 3 and (need_w or need_b):
            dwp, dbp = wgrad3x3(dyh, xh, need_b)
            if need_w:
                dw = unpack_wgrad(dwp, weight, cin_p)
            if need_b:
                db = dbp[:cout]
        elif k == 1 and (need_w or need_b):
            # 1 x 1: the plain reduction GEMM dY^T X over all pixels (+ column sums of dY for the bias)
            res = _g.gemm_nt(dyh.reshape(-1, cout_p), xh.reshape(-1, cin_p), colsum=need_b)
            dwp, dbp = res if need_b else (res, None)
            if need_w:
                dw = dwp[:cout, :cin].reshape(cout, cin, 1, 1).to(weight.dtype)
            if need_b:
                db = dbp[:cout]
        else:
            if need_w:
                dw = torch.nn.grad.conv2d_weight(xh[..., :cin].permute(0, 3, 1, 2), weight.shape,
                                                 dyh[..., :cout].permute(0, 3, 1, 2), padding=k // 2).to(weight.dtype)
            if need_b:
                db = dyh[..., :cout].float().sum(dim=(0, 1, 2))
        return dx, dw, db, None


def conv2d_same(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, act: str | None = None) -> torch.Tensor:
    """``act(conv2d(x, weight, bias, padding=k//2))`` in bf16; returns an NCHW tensor in channels-last memory format.

    ``supported(x, weight)`` must hold.  With ``act`` the call is forward-only (inference).
    """
    code = _ACT[act]
    if code and not (torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad)):
        cin_p, cout_p = _conv_dims(weight)
        y = _launch(_as_nhwc_bf16(x, cin_p), _pack_weight(weight, cin_p, cout_p), bias, weight.shape[-1], code)
        return y[..., :weight.shape[0]].permute(0, 3, 1, 2)
    y = _ConvSame.apply(x, weight, bias, 0)
    if code:
        y = {1: F.gelu, 2: F.silu, 3: F.relu}[code](y)
    return y

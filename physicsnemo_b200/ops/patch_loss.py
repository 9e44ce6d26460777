"""Un-patchify and the fused squared-error loss: the two memory-bound tails of a patch-token model.

``unpatchify`` is the rearrangement ``b h w (p0 p1 c) -> b c (h p0) (w p1)`` that follows the linear head of AFNO /
ModAFNO (``physicsnemo/models/afno/afno.py`` ``forward``: the ``rearrange`` after ``self.head``); ``squared_error`` is
``sum((pred - target)^2) * scale`` as one reduction kernel with a one-kernel gradient, which replaces the cast /
subtract / square / sum chain of an fp32 loss on bf16 predictions.  Both fall back to plain tensor expressions on the
host and for layouts the kernels do not cover.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from . import gemm as _g


def _lib_pl():
    lib = _lib.load(required=True)
    if not getattr(lib, "_patch_loss_declared", False):
        c = ctypes
        vp, i, ll = c.c_void_p, c.c_int, c.c_longlong
        lib.pnm_unpatchify_bf16.argtypes = [vp, vp, i, i, i, i, i, i, i, vp]
        lib.pnm_unpatchify_bf16.restype = i
        lib.pnm_sq_err_partials.argtypes = []
        lib.pnm_sq_err_partials.restype = i
        lib.pnm_sq_err_sum.argtypes = [vp, vp, ll, i, i, c.c_double, vp, vp, vp]
        lib.pnm_sq_err_sum.restype = i
        lib.pnm_sq_err_grad.argtypes = [vp, vp, vp, ll, i, i, c.c_float, vp, vp]
        lib.pnm_sq_err_grad.restype = i
        lib._patch_loss_declared = True
    return lib


def _unpatchify_reference(tokens: torch.Tensor, h: int, w: int, p0: int, p1: int, C: int) -> torch.Tensor:
    B = tokens.shape[0]
    image = tokens.reshape(B, h, w, p0, p1, C).permute(0, 5, 1, 3, 2, 4)
    return image.reshape(B, C, h * p0, w * p1)


def _patchify_reference(image: torch.Tensor, h: int, w: int, p0: int, p1: int, C: int) -> torch.Tensor:
    B = image.shape[0]
    return image.reshape(B, C, h, p0, w, p1).permute(0, 2, 4, 3, 5, 1).reshape(B, h, w, p0 * p1 * C)


def _launch_unpatchify(tokens: torch.Tensor, image: torch.Tensor, dims, to_image: bool) -> bool:
    """Run the kernel; False when it declines the shape (nothing was written then)."""
    B, h, w, p0, p1, C = dims
    rc = _lib_pl().pnm_unpatchify_bf16(tokens.data_ptr(), image.data_ptr(), B, h, w, p0, p1, C, int(to_image),
                                       torch.cuda.current_stream().cuda_stream)
    if rc == -2:
        return False
    _g._check(rc, "pnm_unpatchify_bf16")
    _g.launch_count += 1
    return True


class _UnpatchifyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, h, w, p0, p1, C):
        B = tokens.shape[0]
        ctx.dims = (B, h, w, p0, p1, C)
        src = tokens.contiguous()
        image = torch.empty(B, C, h * p0, w * p1, dtype=tokens.dtype, device=tokens.device)
        if not _launch_unpatchify(src, image, ctx.dims, True):
            image = _unpatchify_reference(src, h, w, p0, p1, C).contiguous()
        return image

    @staticmethod
    def backward(ctx, dimage):
        B, h, w, p0, p1, C = ctx.dims
        d = dimage.to(torch.bfloat16).contiguous()
        dtokens = torch.empty(B, h, w, p0 * p1 * C, dtype=d.dtype, device=d.device)
        if not _launch_unpatchify(dtokens, d, ctx.dims, False):
            dtokens = _patchify_reference(d, h, w, p0, p1, C).contiguous()
        return dtokens, None, None, None, None, None


def unpatchify(tokens: torch.Tensor, h: int, w: int, p0: int, p1: int, channels: int) -> torch.Tensor:
    """``tokens[B, h, w, p0 * p1 * channels]`` (features ordered patch row, patch column, channel) as the image
    ``[B, channels, h * p0, w * p1]``."""
    if tokens.shape[1:] != (h, w, p0 * p1 * channels):
        tokens = tokens.reshape(tokens.shape[0], h, w, p0 * p1 * channels)
    if tokens.is_cuda and tokens.dtype == torch.bfloat16 and type(tokens) is torch.Tensor:
        return _UnpatchifyFn.apply(tokens, h, w, p0, p1, channels)
    return _unpatchify_reference(tokens, h, w, p0, p1, channels)


_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class _SquaredErrorFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pred, target, scale):
        lib = _lib_pl()
        p, t = pred.contiguous(), target.contiguous()
        if p.data_ptr() % 16:
            p = p.clone()
        if t.data_ptr() % 16:
            t = t.clone()
        partial = torch.empty(lib.pnm_sq_err_partials(), dtype=torch.float32, device=p.device)
        out = torch.empty(1, dtype=torch.float32, device=p.device)
        rc = lib.pnm_sq_err_sum(p.data_ptr(), t.data_ptr(), p.numel(), _DTYPE_CODE[p.dtype], _DTYPE_CODE[t.dtype], float(scale),
                                partial.data_ptr(), out.data_ptr(), torch.cuda.current_stream().cuda_stream)
        _g._check(rc, "pnm_sq_err_sum")
        _g.launch_count += 2
        ctx.save_for_backward(p, t)
        ctx.scale = float(scale)
        return out.reshape(())

    @staticmethod
    def backward(ctx, gout):
        p, t = ctx.saved_tensors
        g = gout.detach().to(torch.float32).reshape(1).contiguous()
        grad = torch.empty_like(p)
        rc = _lib_pl().pnm_sq_err_grad(p.data_ptr(), t.data_ptr(), g.data_ptr(), p.numel(), _DTYPE_CODE[p.dtype],
                                       _DTYPE_CODE[t.dtype], 2.0 * ctx.scale, grad.data_ptr(),
                                       torch.cuda.current_stream().cuda_stream)
        _g._check(rc, "pnm_sq_err_grad")
        _g.launch_count += 1
        return grad, None, None


def squared_error(pred: torch.Tensor, target: torch.Tensor, scale: float | None = None) -> torch.Tensor:
    """``scale * sum((pred - target)^2)`` in fp32 (``scale`` defaults to ``1 / numel``: the mean squared error).

    ``target`` is a constant of the loss (no gradient flows to it).  On the device, for bf16 / fp32 operands of equal
    shape, forward is one reduction pass and backward one elementwise pass."""
    if pred.shape != target.shape:
        raise ValueError(f"pred {tuple(pred.shape)} and target {tuple(target.shape)} must have the same shape")
    if scale is None:
        scale = 1.0 / max(pred.numel(), 1)
    fused = (pred.is_cuda and target.is_cuda and pred.numel() > 0 and type(pred) is torch.Tensor and type(target) is torch.Tensor
             and pred.dtype in _DTYPE_CODE and target.dtype in _DTYPE_CODE and not target.requires_grad)
    if fused:
        return _SquaredErrorFn.apply(pred, target, scale)
    return ((pred.float() - target.float()) ** 2).sum() * scale

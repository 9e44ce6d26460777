"""2 × 2 box down- / up-sampling of channels-last bf16 images on the library's kernels (``csrc/resample2x.cu``).

The ``[1, 1]`` resample filter of the diffusion U-Nets (reference: ``physicsnemo/nn/module/conv_layers.py:Conv2d`` applies
it as a depth-wise strided (transposed) convolution) is a 2 × 2 mean on the way down and a 2 × 2 replication on the way
up; each is the other's adjoint up to a factor, so two kernels cover both directions and both backward passes.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib
from . import gemm as _g


def _fn():
    lib = _lib.load(required=True)
    if not getattr(lib, "_resample_declared", False):
        c = ctypes
        lib.pnm_resample2x_nhwc.argtypes = [c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_float, c.c_void_p]
        lib.pnm_resample2x_nhwc.restype = c.c_int
        lib._resample_declared = True
    return lib.pnm_resample2x_nhwc


def supported(x: torch.Tensor) -> bool:
    return (type(x) is torch.Tensor and x.is_cuda and x.dim() == 4 and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.is_contiguous(memory_format=torch.channels_last) and _lib.available())


def _run(x: torch.Tensor, mode: int, scale: float) -> torch.Tensor:
    n, c, h, w = x.shape
    ho, wo = (h // 2, w // 2) if mode == 0 else (2 * h, 2 * w)
    y = torch.empty((n, c, ho, wo), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
    rc = _fn()(x.data_ptr(), y.data_ptr(), n, h, w, c, mode, float(scale), torch.cuda.current_stream().cuda_stream)
    _g._check(rc, "pnm_resample2x_nhwc")
    _g.launch_count += 1
    return y


class _Down2x(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _run(x, 0, 0.25)

    @staticmethod
    def backward(ctx, dy):
        return _run(dy.contiguous(memory_format=torch.channels_last), 1, 0.25)


class _Up2x(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _run(x, 1, 1.0)

    @staticmethod
    def backward(ctx, dy):
        return _run(dy.contiguous(memory_format=torch.channels_last), 0, 1.0)


def down2x(x: torch.Tensor) -> torch.Tensor:
    """2 × 2 mean (``F.avg_pool2d(x, 2)``)."""
    if supported(x) and x.shape[2] % 2 == 0 and x.shape[3] % 2 == 0:
        return _Down2x.apply(x)
    return F.avg_pool2d(x, 2)


def up2x(x: torch.Tensor) -> torch.Tensor:
    """2 × 2 replication (``F.interpolate(x, scale_factor=2, mode="nearest")``)."""
    if supported(x):
        return _Up2x.apply(x)
    return F.interpolate(x, scale_factor=2, mode="nearest")


# ------------------------------------------------------------------------------------------------ residual join
def _add_scale_fn():
    lib = _lib.load(required=True)
    if not getattr(lib, "_add_scale_declared", False):
        c = ctypes
        lib.pnm_add_scale_bf16.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_longlong, c.c_float, c.c_void_p]
        lib.pnm_add_scale_bf16.restype = c.c_int
        lib._add_scale_declared = True
    return lib.pnm_add_scale_bf16


def _same_dense_layout(a: torch.Tensor, b: torch.Tensor) -> bool:
    return a.shape == b.shape and a.stride() == b.stride() and (a.is_contiguous() or a.is_contiguous(memory_format=torch.channels_last))


class _AddScale(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, scale: float):
        out = torch.empty_like(a)
        rc = _add_scale_fn()(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), float(scale), torch.cuda.current_stream().cuda_stream)
        _g._check(rc, "pnm_add_scale_bf16")
        _g.launch_count += 1
        ctx.scale = float(scale)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous(memory_format=torch.channels_last) if g.dim() == 4 and not g.is_contiguous() else g.contiguous() if not (
            g.is_contiguous() or (g.dim() == 4 and g.is_contiguous(memory_format=torch.channels_last))) else g
        d = torch.empty_like(g)
        rc = _add_scale_fn()(g.data_ptr(), None, d.data_ptr(), g.numel(), ctx.scale, torch.cuda.current_stream().cuda_stream)
        _g._check(rc, "pnm_add_scale_bf16")
        _g.launch_count += 1
        return d, d, None                      # both branches receive the same scaled gradient


def add_scale(a: torch.Tensor, b: torch.Tensor, scale: float) -> torch.Tensor:
    """``(a + b) * scale``: one kernel (forward) and one (backward, shared by both inputs) for bf16 CUDA tensors of the
    same dense layout; the PyTorch expression otherwise."""
    if (type(a) is torch.Tensor and type(b) is torch.Tensor and a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
            and a.numel() % 8 == 0 and _same_dense_layout(a, b) and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0 and _lib.available()):
        return _AddScale.apply(a, b, scale)
    return (a + b) * scale

"""Grouped normalisation of spherical-harmonic grids ``[B, L, M, 2, C]`` (``csrc/sh_norm.cu``).

One operator expresses the three equivariant norms of ``experimental.nn.symmetry`` (RMS over all degrees, per-degree
layer norm, tied norm with a plain layer norm on ``l = 0``).  With ``xc`` the masked input, centred over the channels
of the ``(l, m, r) = (0, 0, 0)`` row when ``subtract_mean``::

    S_g   = (1 / C) * sum_{l in g} sum_m wstat[l, m] * sum_{r, c} xc[l, m, r, c]^2
    y     = mask * (xc * rsqrt(S_{group[l]} + eps) * affine[l, c] + [l = m = r = 0] * bias[c])

``sh_norm`` runs one CTA per sample (read once, write once; masked rows are never read) and has a hand-written
backward kernel; ``reference`` is the same formula in tensor operations (used on the CPU and as the test oracle).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib
from . import gemm as _g

_DTYPES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def _lib_sh():
    lib = _lib.load(required=True)
    if not getattr(lib, "_sh_declared", False):
        vp, i, i64, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        lib.pnm_sh_norm_fits.argtypes = [i, i, i, i]
        lib.pnm_sh_norm_fits.restype = i
        lib.pnm_sh_norm_bwd_grid.argtypes = [i64, i, i, i]
        lib.pnm_sh_norm_bwd_grid.restype = i
        lib.pnm_sh_norm_fwd.argtypes = [vp] * 7 + [i64, i, i, i, f, i, i, vp]
        lib.pnm_sh_norm_fwd.restype = i
        lib.pnm_sh_norm_bwd.argtypes = [vp] * 9 + [i64, i, i, i, f, i, i, i, vp]
        lib.pnm_sh_norm_bwd.restype = i
        lib._sh_declared = True
    return lib


def reference(x, affine, bias, wstat, mask, group, eps: float, subtract_mean: bool):
    """Tensor-operation form of the operator (any device); statistics in fp32 (fp64 for fp64 input)."""
    cd = torch.float64 if x.dtype == torch.float64 else torch.float32
    B, L, M, _, C = x.shape
    mk = mask.to(cd)[None, :, :, :, None]
    xc = x.to(cd) * mk
    first = torch.zeros(L, M, 2, 1, dtype=cd, device=x.device)       # indicator of the (0, 0, 0) row
    first[0, 0, 0, 0] = 1.0
    if subtract_mean:
        xc = xc - xc[:, :1, :1, :1, :].mean(dim=-1, keepdim=True) * first
    per_l = torch.einsum("blmrc,lm->bl", xc * xc, wstat.to(cd)) / C                      # [B, L]
    onehot = torch.nn.functional.one_hot(group.long(), L).to(cd)                           # [L, G]
    inv = ((per_l @ onehot) + eps).rsqrt() @ onehot.t()                                    # back to [B, L]
    y = xc * inv[:, :, None, None, None] * affine.to(cd)[None, :, None, None, :]
    if bias is not None:
        y = y + first * bias.to(cd)
    return (y * mk).to(x.dtype)


def supported(x: torch.Tensor) -> bool:
    if not (x.is_cuda and x.dim() == 5 and x.shape[3] == 2 and x.dtype in _DTYPES and x.shape[0] > 0):
        return False
    L, M, C = x.shape[1], x.shape[2], x.shape[4]
    return bool(_lib_sh().pnm_sh_norm_fits(L, M, C, 1))


class _ShNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, affine, bias, wstat, mask, group, eps, subtract_mean):
        B, L, M, _, C = x.shape
        xc = x.detach().contiguous()
        if xc.data_ptr() % 16:
            xc = xc.clone()
        a32 = affine.detach().float().contiguous()
        b32 = None if bias is None else bias.detach().float().contiguous()
        w32, m32, g32 = wstat.float().contiguous(), mask.float().contiguous(), group.to(torch.int32).contiguous()
        y = torch.empty_like(xc)
        err = _lib_sh().pnm_sh_norm_fwd(xc.data_ptr(), y.data_ptr(), a32.data_ptr(), None if b32 is None else b32.data_ptr(),
                                        w32.data_ptr(), m32.data_ptr(), g32.data_ptr(), B, L, M, C, float(eps), int(subtract_mean),
                                        _DTYPES[x.dtype], torch.cuda.current_stream().cuda_stream)
        if err:
            raise RuntimeError(f"pnm_sh_norm_fwd failed ({err})")
        _g.launch_count += 1
        ctx.save_for_backward(xc, a32, w32, m32, g32)
        ctx.meta = (float(eps), int(subtract_mean), affine.dtype, None if bias is None else bias.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, a32, w32, m32, g32 = ctx.saved_tensors
        eps, sub, a_dtype, b_dtype = ctx.meta
        B, L, M, _, C = xc.shape
        dy = dy.contiguous()
        if dy.data_ptr() % 16:
            dy = dy.clone()
        lib = _lib_sh()
        grid = lib.pnm_sh_norm_bwd_grid(B, L, M, C)
        dx = torch.empty_like(xc)
        daw = torch.empty(grid, L, C, dtype=torch.float32, device=xc.device)
        dbias = torch.empty(grid, C, dtype=torch.float32, device=xc.device)
        err = lib.pnm_sh_norm_bwd(xc.data_ptr(), dy.data_ptr(), dx.data_ptr(), a32.data_ptr(), w32.data_ptr(), m32.data_ptr(),
                                  g32.data_ptr(), daw.data_ptr(), dbias.data_ptr(), B, L, M, C, eps, sub, _DTYPES[xc.dtype], grid,
                                  torch.cuda.current_stream().cuda_stream)
        if err:
            raise RuntimeError(f"pnm_sh_norm_bwd failed ({err})")
        _g.launch_count += 1
        d_aff = daw.sum(0).to(a_dtype) if ctx.needs_input_grad[1] else None
        d_bias = dbias.sum(0).to(b_dtype) if b_dtype is not None and ctx.needs_input_grad[2] else None
        return dx, d_aff, d_bias, None, None, None, None, None


def sh_norm(x: torch.Tensor, affine: torch.Tensor, bias: Optional[torch.Tensor], wstat: torch.Tensor, mask: torch.Tensor,
            group: torch.Tensor, eps: float = 1e-5, subtract_mean: bool = True) -> torch.Tensor:
    """Grouped spherical-harmonic normalisation; CUDA kernel when ``supported(x)``, tensor operations otherwise."""
    if supported(x):
        return _ShNorm.apply(x, affine, bias, wstat, mask, group, eps, subtract_mean)
    return reference(x, affine, bias, wstat, mask, group, eps, subtract_mean)

"""Spectral-convolution mode contraction on the library kernel (``csrc/spectral.cu``).

``corner_contract(x_ft, weights, starts, out_ft)`` adds ``einsum("bi…,io…->bo…", x_ft[corner], weights)`` into the same
corner of ``out_ft`` in one launch: the corner of the input spectrum is read in place through its strides and the result is
written in place into the output spectrum, so neither the sliced copy of ``x_ft`` nor a separate scatter exists.  The
backward uses the same kernel twice (input gradient into a zero spectrum, weight gradient with the batch contracted).
``weights`` is the real view ``[I, O, *modes, 2]`` that the spectral layers store; spectra are complex64.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from . import gemm as _g


def _lib_sp():
    lib = _lib.load(required=True)
    if not getattr(lib, "_sp_declared", False):
        vp, i = ctypes.c_void_p, ctypes.c_int
        lib.pnm_spectral_contract.argtypes = [vp, vp, vp, i, vp, vp, vp, vp, vp, i, i, i, i, i, i, vp]
        lib.pnm_spectral_contract.restype = i
        lib._sp_declared = True
    return lib


def supported(x_ft: torch.Tensor, weights: torch.Tensor) -> bool:
    nd = x_ft.dim() - 2
    return (x_ft.is_cuda and x_ft.dtype == torch.complex64 and weights.dtype == torch.float32 and 1 <= nd <= 4
            and weights.dim() == nd + 3 and weights.shape[-1] == 2 and weights.is_contiguous() and x_ft.shape[0] <= 65535)


def _launch(a, a_p, a_r, a_modes, b, b_r, b_q, b_modes, out, o_p, o_q, o_modes, shape, P, Q, R, conj_a, conj_b, accumulate):
    nd = len(shape)
    arr = lambda vals, ty: (ty * len(vals))(*vals)  # noqa: E731
    shp, sa, sb, so = arr(shape, ctypes.c_int), arr(a_modes, ctypes.c_longlong), arr(b_modes, ctypes.c_longlong), arr(o_modes, ctypes.c_longlong)
    ch = arr([a_p, a_r, b_r, b_q, o_p, o_q], ctypes.c_longlong)
    err = _lib_sp().pnm_spectral_contract(a.data_ptr(), b.data_ptr(), out.data_ptr(), nd, shp, sa, sb, so, ch, P, Q, R, int(conj_a), int(conj_b),
                                          int(accumulate), torch.cuda.current_stream().cuda_stream)
    if err:
        raise RuntimeError(f"pnm_spectral_contract failed ({err})")
    _g.launch_count += 1


def _corner(t: torch.Tensor, starts, modes):
    """View of ``t[:, :, s0:s0+m0, …]`` (strides only)."""
    idx = (slice(None), slice(None)) + tuple(slice(s, s + m) for s, m in zip(starts, modes))
    return t[idx]


class _CornerContract(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_ft, weights, out_ft, starts):
        modes = tuple(weights.shape[2:-1])
        B, I = x_ft.shape[:2]
        O = weights.shape[1]
        wc = torch.view_as_complex(weights)
        xc, oc = _corner(x_ft, starts, modes), _corner(out_ft, starts, modes)
        _launch(xc, xc.stride(0), xc.stride(1), xc.stride()[2:], wc, wc.stride(0), wc.stride(1), wc.stride()[2:], oc, oc.stride(0), oc.stride(1),
                oc.stride()[2:], modes, B, O, I, False, False, True)
        ctx.save_for_backward(x_ft, weights)
        ctx.starts = starts
        ctx.mark_dirty(out_ft)
        return out_ft

    @staticmethod
    def backward(ctx, g):
        x_ft, weights = ctx.saved_tensors
        starts, modes = ctx.starts, tuple(weights.shape[2:-1])
        B, I = x_ft.shape[:2]
        O = weights.shape[1]
        g = g.contiguous()
        gc, wc = _corner(g, starts, modes), torch.view_as_complex(weights)
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx = torch.zeros_like(x_ft)
            gxc = _corner(gx, starts, modes)                       # dx[b,i,m] = sum_o dy[b,o,m] conj(w[i,o,m])
            _launch(gc, gc.stride(0), gc.stride(1), gc.stride()[2:], wc, wc.stride(1), wc.stride(0), wc.stride()[2:], gxc, gxc.stride(0),
                    gxc.stride(1), gxc.stride()[2:], modes, B, I, O, False, True, False)
        if ctx.needs_input_grad[1]:
            gwc = torch.empty_like(wc)                             # dw[i,o,m] = sum_b conj(x[b,i,m]) dy[b,o,m]
            xc = _corner(x_ft, starts, modes)
            _launch(xc, xc.stride(1), xc.stride(0), xc.stride()[2:], gc, gc.stride(0), gc.stride(1), gc.stride()[2:], gwc, gwc.stride(0),
                    gwc.stride(1), gwc.stride()[2:], modes, I, O, B, True, False, False)
            gw = torch.view_as_real(gwc)
        return gx, gw, g, None


def corner_contract(x_ft: torch.Tensor, weights: torch.Tensor, starts, out_ft: torch.Tensor) -> torch.Tensor:
    """``out_ft[:, :, corner] += einsum(x_ft[:, :, corner], weights)``; returns ``out_ft`` (modified in place)."""
    return _CornerContract.apply(x_ft, weights, out_ft, tuple(int(s) for s in starts))

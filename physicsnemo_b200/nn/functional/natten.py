"""Neighbourhood attention (1-, 2-, 3-D).

Parity: ``physicsnemo/nn/functional/natten.py`` wraps the NATTEN extension; here the operation is
implemented directly.  Semantics follow NATTEN: tensors are ``[B, *spatial, heads, head_dim]``; every query
attends to a ``kernel_size`` (per axis) window of keys centred on it, the window being *shifted* (not
truncated) at the borders so that each query sees exactly ``prod(kernel_size)`` keys; ``dilation`` strides
the window.  Formulation: the neighbour index table ``[L, K]`` is built once per (shape, kernel, dilation)
and cached; keys / values are gathered and reduced with a batched softmax (CPU path and oracle).
On CUDA tensors (bf16 / fp32) the warp-per-query kernels of ``csrc/natten.cu`` run instead: no index table and no
gathered ``[L, K, D]`` copies of the keys and values exist, forward or backward.
"""
from __future__ import annotations

from functools import lru_cache
from typing import Any, Sequence

import torch
from torch.overrides import handle_torch_function, has_torch_function


def _tuple(v, n):
    return tuple(int(v) for _ in range(n)) if isinstance(v, int) else tuple(int(x) for x in v)


@lru_cache(maxsize=64)
def _neighbour_table(shape: tuple, kernel: tuple, dilation: tuple, device_str: str) -> torch.Tensor:
    device = torch.device(device_str)
    per_axis = []
    for n, k, d in zip(shape, kernel, dilation):
        if k * d > n + (d - 1) and k > n:
            raise ValueError(f"kernel_size {k} (dilation {d}) exceeds the extent {n}")
        i = torch.arange(n, device=device)
        if d == 1:
            start = (i - k // 2).clamp(0, n - k)
            idx = start[:, None] + torch.arange(k, device=device)[None]
        else:
            # positions congruent to i modulo d form a sub-lattice; shift the window inside it
            phase, pos = i % d, i // d
            count = (n - phase + d - 1) // d
            start = torch.minimum((pos - k // 2).clamp_min(0), count - k)
            idx = (start[:, None] + torch.arange(k, device=device)[None]) * d + phase[:, None]
        per_axis.append(idx)                                  # [n, k]
    flat = per_axis[0]
    for a in range(1, len(shape)):
        flat = (flat[:, None, :, None] * shape[a] + per_axis[a][None, :, None, :]).reshape(
            flat.shape[0] * shape[a], -1)
    return flat                                               # [L, K]


_DT = {torch.bfloat16: 0, torch.float32: 1}


def _lib_na():
    import ctypes

    from ...ops import _lib

    lib = _lib.load(required=True)
    if not getattr(lib, "_na_declared", False):
        c = ctypes
        vp, i, f = c.c_void_p, c.c_int, c.c_float
        ip = c.POINTER(c.c_int)
        lib.pnm_natten_fwd.argtypes = [vp, vp, vp, vp, i, i, i, i, ip, ip, ip, f, i, vp]
        lib.pnm_natten_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, i, i, i, i, ip, ip, ip, f, i, vp]
        lib.pnm_natten_fwd.restype = lib.pnm_natten_bwd.restype = i
        lib._na_declared = True
    return lib


def _cuda_ok(q, kern, dil, shape) -> bool:
    import math

    if not (q.is_cuda and q.dtype in _DT and q.shape[-1] <= 256 and math.prod(kern) <= 512):
        return False
    return all(k <= n and (d == 1 or k <= n // d) for n, k, d in zip(shape, kern, dil))


class _NattenFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, shape, kern, dil, scale):
        import ctypes

        from ...ops import gemm as _g

        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        B, H, D = q.shape[0], q.shape[-2], q.shape[-1]
        nd = len(shape)
        arr = lambda t: (ctypes.c_int * nd)(*t)  # noqa: E731
        out = torch.empty_like(q)
        err = _lib_na().pnm_natten_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, H, D, nd, arr(shape),
                                       arr(kern), arr(dil), float(scale), _DT[q.dtype],
                                       torch.cuda.current_stream().cuda_stream)
        if err:
            raise RuntimeError(f"pnm_natten_fwd failed ({err})")
        _g.launch_count += 1
        ctx.save_for_backward(q, k, v)
        ctx.cfg = (shape, kern, dil, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        import ctypes

        from ...ops import gemm as _g

        q, k, v = ctx.saved_tensors
        shape, kern, dil, scale = ctx.cfg
        B, H, D = q.shape[0], q.shape[-2], q.shape[-1]
        nd = len(shape)
        arr = lambda t: (ctypes.c_int * nd)(*t)  # noqa: E731
        dout = dout.contiguous().to(q.dtype)
        dq = torch.empty_like(q)
        dkv = torch.zeros(2, *q.shape, dtype=torch.float32, device=q.device)
        err = _lib_na().pnm_natten_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), dout.data_ptr(), dq.data_ptr(),
                                       dkv[0].data_ptr(), dkv[1].data_ptr(), B, H, D, nd, arr(shape), arr(kern), arr(dil),
                                       float(scale), _DT[q.dtype], torch.cuda.current_stream().cuda_stream)
        if err:
            raise RuntimeError(f"pnm_natten_bwd failed ({err})")
        _g.launch_count += 1
        return dq, dkv[0].to(q.dtype), dkv[1].to(q.dtype), None, None, None, None


def _neighborhood_attention(q, k, v, kernel_size, dilation, scale=None, is_causal=False, implementation=None, **kwargs):
    nd = q.ndim - 3
    if is_causal:
        raise NotImplementedError("causal neighbourhood attention is not supported")
    shape = tuple(q.shape[1:1 + nd])
    kern, dil = _tuple(kernel_size, nd), _tuple(dilation, nd)
    if implementation != "torch" and _cuda_ok(q, kern, dil, shape):
        return _NattenFn.apply(q, k, v, shape, kern, dil, q.shape[-1] ** -0.5 if scale is None else float(scale))
    if implementation == "cuda":
        raise RuntimeError("neighbourhood attention kernels need CUDA bf16 / fp32 tensors, head_dim <= 256 and <= 512 neighbours")
    table = _neighbour_table(shape, kern, dil, str(q.device))
    B, H, D = q.shape[0], q.shape[-2], q.shape[-1]
    L = table.shape[0]
    qf = q.reshape(B, L, H, D).permute(0, 2, 1, 3)            # [B, H, L, D]
    kf = k.reshape(B, L, H, D).permute(0, 2, 1, 3)
    vf = v.reshape(B, L, H, D).permute(0, 2, 1, 3)
    kn, vn = kf[:, :, table], vf[:, :, table]                 # [B, H, L, K, D]
    s = D ** -0.5 if scale is None else scale
    att = torch.einsum("bhld,bhlkd->bhlk", qf, kn) * s
    att = torch.softmax(att.float(), dim=-1).to(q.dtype)
    out = torch.einsum("bhlk,bhlkd->bhld", att, vn)
    return out.permute(0, 2, 1, 3).reshape(q.shape)


def _make(nd: int, name: str):
    def fn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kernel_size, dilation=1, **kwargs: Any) -> torch.Tensor:
        if has_torch_function((q, k, v)):
            return handle_torch_function(fn, (q, k, v), q, k, v, kernel_size, dilation=dilation, **kwargs)
        if q.ndim != nd + 3:
            raise ValueError(f"{name} expects [B, {'*' * nd}spatial, heads, head_dim] tensors, got {tuple(q.shape)}")
        return _neighborhood_attention(q, k, v, kernel_size, dilation, **kwargs)

    fn.__name__ = fn.__qualname__ = name
    return fn


na1d = _make(1, "na1d")
na2d = _make(2, "na2d")
na3d = _make(3, "na3d")

__all__ = ["na1d", "na2d", "na3d"]

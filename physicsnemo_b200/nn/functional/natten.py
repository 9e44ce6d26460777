"""Neighbourhood attention (1-, 2-, 3-D).

Parity: ``physicsnemo/nn/functional/natten.py`` wraps the NATTEN extension; here the operation is
implemented directly.  Semantics follow NATTEN: tensors are ``[B, *spatial, heads, head_dim]``; every query
attends to a ``kernel_size`` (per axis) window of keys centred on it, the window being *shifted* (not
truncated) at the borders so that each query sees exactly ``prod(kernel_size)`` keys; ``dilation`` strides
the window.  Formulation: the neighbour index table ``[L, K]`` is built once per (shape, kernel, dilation)
and cached; keys / values are gathered and reduced with a batched softmax.
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


def _neighborhood_attention(q, k, v, kernel_size, dilation, scale=None, is_causal=False, **kwargs):
    nd = q.ndim - 3
    if is_causal:
        raise NotImplementedError("causal neighbourhood attention is not supported")
    shape = tuple(q.shape[1:1 + nd])
    kern, dil = _tuple(kernel_size, nd), _tuple(dilation, nd)
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

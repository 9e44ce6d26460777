"""Right-sided padding of channels-last fields (``[B, *spatial, ...]``) to a multiple of a block size.

Counterpart of ``physicsnemo/experimental/models/xdeeponet/_padding.py`` (``compute_right_pad_to_multiple`` :37,
``pad_right_nd`` :93, ``pad_spatial_right`` :164).  Every axis is padded by one gather (replicate) or one slice
copy (constant) directly on the channels-last tensor: no permutation to channels-first and back, and any number of
spatial axes is handled by the same code.
"""

from __future__ import annotations

from typing import Literal, Sequence

import torch
from torch import Tensor

__all__ = ["compute_right_pad_to_multiple", "pad_right_nd", "pad_spatial_right"]


def compute_right_pad_to_multiple(spatial_shape: Sequence[int], *, multiple: int = 8, min_right_pad: int = 0) -> tuple:
    """Smallest right pads ``>= min_right_pad`` that make every extent a multiple of ``multiple``."""
    if multiple <= 0:
        raise ValueError(f"multiple must be > 0, got {multiple}")
    if min_right_pad < 0:
        raise ValueError(f"min_right_pad must be >= 0, got {min_right_pad}")
    if any(d <= 0 for d in spatial_shape):
        raise ValueError(f"spatial dimensions must be positive, got {spatial_shape}")
    # the padded extent is the first multiple of `multiple` at or above d + min_right_pad
    return tuple(int(-(-(d + min_right_pad) // multiple) * multiple - d) for d in spatial_shape)


def pad_right_nd(x: Tensor, *, dims: Sequence[int], right_pad: Sequence[int],
                 mode: Literal["replicate", "constant"] = "replicate", constant_value: float = 0.0) -> Tensor:
    """Pad the axes ``dims`` of ``x`` on their right side by ``right_pad`` entries."""
    if len(dims) != len(right_pad):
        raise ValueError("dims and right_pad must have the same length")
    if mode not in ("replicate", "constant"):
        raise ValueError(f"pad_right_nd supports mode='replicate' or 'constant', got {mode}")
    todo = []
    for dim, pad in zip(dims, right_pad):
        d = dim + x.dim() if dim < 0 else dim
        if not 0 <= d < x.dim():
            raise ValueError(f"invalid dim {dim} for x.dim()={x.dim()}")
        if int(pad) > 0:
            todo.append((d, int(pad)))
    if not todo:
        return x
    if mode == "constant":
        shape = list(x.shape)
        for d, pad in todo:
            shape[d] += pad
        out = x.new_full(shape, float(constant_value))
        out[tuple(slice(0, s) for s in x.shape)] = x
        return out
    for d, pad in todo:
        n = x.shape[d]
        x = x.index_select(d, torch.arange(n + pad, device=x.device).clamp_(max=n - 1))
    return x


def pad_spatial_right(x: Tensor, *, spatial_ndim: int, right_pad: Sequence[int],
                      mode: Literal["replicate", "constant"] = "replicate", constant_value: float = 0.0) -> Tensor:
    """Pad the ``spatial_ndim`` axes that follow the batch axis of a channels-last tensor."""
    if spatial_ndim not in (2, 3, 4):
        raise ValueError(f"spatial_ndim must be 2, 3, or 4, got {spatial_ndim}")
    if len(right_pad) != spatial_ndim:
        raise ValueError(f"right_pad must have length {spatial_ndim}, got {len(right_pad)}")
    if x.dim() < 1 + spatial_ndim:
        raise ValueError(f"expected x.dim() >= {1 + spatial_ndim}, got x.dim()={x.dim()}")
    return pad_right_nd(x, dims=range(1, 1 + spatial_ndim), right_pad=right_pad, mode=mode, constant_value=constant_value)

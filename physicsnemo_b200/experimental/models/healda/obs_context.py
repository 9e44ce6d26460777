"""Packed observation context for pixel / observation cross attention.

Counterpart of ``physicsnemo/experimental/models/healda/obs_context.py`` (``PixelGroupMap`` :44, ``ObsContext`` :85,
``sort_and_pack`` :176, ``counts_to_cu_seqlens`` :211, ``build_pixel_group_map`` :233, ``prepare_obs_context`` :306).
Observations are sorted by their target pixel (a counting sort on the GPU) so that every pixel owns the contiguous
slice ``[cu_seqlens_k[p], cu_seqlens_k[p+1])`` of the packed arrays.
"""

from __future__ import annotations

import dataclasses
from typing import Optional, Tuple

import torch

from ....ops.pixel_attention import counting_sort_and_pack

__all__ = ["PixelGroupMap", "ObsContext", "sort_and_pack", "counts_to_cu_seqlens", "build_pixel_group_map", "prepare_obs_context"]


def _move(t: torch.Tensor, device, dtype, non_blocking: bool) -> torch.Tensor:
    return t.to(device=device, dtype=dtype if dtype is not None and t.is_floating_point() else None, non_blocking=non_blocking)


@dataclasses.dataclass
class PixelGroupMap:
    """Work list that pairs pixels with few observations (``program_ptr`` CSR offsets into ``program_pixels``).

    The attention kernel of this package balances work by itself (one warp per pixel and block of heads), so the map
    is optional metadata kept for interface compatibility.
    """

    program_ptr: torch.Tensor
    program_pixels: torch.Tensor

    def to(self, device=None, dtype=None, non_blocking: bool = True) -> "PixelGroupMap":
        if isinstance(device, torch.dtype):
            device, dtype = None, device
        return PixelGroupMap(_move(self.program_ptr, device, dtype, non_blocking), _move(self.program_pixels, device, dtype, non_blocking))


@dataclasses.dataclass
class ObsContext:
    """Observations packed by pixel: values, float metadata, integer type / channel / platform codes, CSR offsets."""

    obs: torch.Tensor
    float_metadata: torch.Tensor
    obs_type: torch.Tensor
    channel: torch.Tensor
    platform: torch.Tensor
    cu_seqlens_k: torch.Tensor
    max_seqlen_k: int
    group_map: Optional[PixelGroupMap] = None

    def __post_init__(self) -> None:
        if self.cu_seqlens_k.ndim != 1:
            raise ValueError(f"cu_seqlens_k must be 1D of shape (total_pixels + 1,); got shape {tuple(self.cu_seqlens_k.shape)}")

    def to(self, device=None, dtype=None, non_blocking: bool = True) -> "ObsContext":
        if isinstance(device, torch.dtype):
            device, dtype = None, device
        mv = lambda t: _move(t, device, dtype, non_blocking)  # noqa: E731
        return ObsContext(obs=mv(self.obs), float_metadata=mv(self.float_metadata), obs_type=mv(self.obs_type), channel=mv(self.channel),
                          platform=mv(self.platform), cu_seqlens_k=mv(self.cu_seqlens_k), max_seqlen_k=self.max_seqlen_k,
                          group_map=None if self.group_map is None else self.group_map.to(device, dtype, non_blocking))


def sort_and_pack(flat_idx: torch.Tensor, total_pixels: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(order, counts)`` such that ``flat_idx[order]`` is grouped by pixel and ``counts[p]`` observations hit pixel ``p``."""
    return counting_sort_and_pack(flat_idx, total_pixels)


def counts_to_cu_seqlens(counts: torch.Tensor) -> torch.Tensor:
    cu = torch.zeros(counts.shape[0] + 1, dtype=torch.int32, device=counts.device)
    cu[1:] = counts.cumsum(0).to(torch.int32)
    return cu


def build_pixel_group_map(cu_seqlens_k: torch.Tensor, thresh_mult: float = 2.0) -> PixelGroupMap:
    """Non-empty pixels with fewer than ``thresh_mult x median`` observations are paired, the others stand alone."""
    dev = cu_seqlens_k.device
    counts = (cu_seqlens_k[1:] - cu_seqlens_k[:-1]).to(torch.int64)
    busy = torch.nonzero(counts > 0).flatten()
    if busy.numel() == 0:
        return PixelGroupMap(torch.zeros(1, dtype=torch.int32, device=dev), torch.empty(0, dtype=torch.int32, device=dev))
    c = counts[busy].float()
    small = c < c.median() * thresh_mult
    small_px, large_px = busy[small], busy[~small]
    pairs, odd = small_px.numel() // 2, small_px.numel() % 2
    sizes = torch.cat([torch.ones(large_px.numel(), dtype=torch.int64, device=dev), torch.full((pairs,), 2, dtype=torch.int64, device=dev),
                       torch.ones(odd, dtype=torch.int64, device=dev)])
    ptr = torch.zeros(sizes.numel() + 1, dtype=torch.int32, device=dev)
    ptr[1:] = torch.cumsum(sizes, 0).to(torch.int32)
    return PixelGroupMap(ptr.contiguous(), torch.cat([large_px, small_px]).to(torch.int32).contiguous())


def prepare_obs_context(obs: torch.Tensor, float_metadata: torch.Tensor, obs_type: torch.Tensor, channel: torch.Tensor,
                        platform: torch.Tensor, flat_idx: torch.Tensor, total_pixels: int, *, build_group_map: bool = True,
                        group_thresh_mult: float = 2.0) -> ObsContext:
    """Sort all per-observation arrays by target pixel and build the CSR offsets."""
    if obs.ndim != 1:
        raise ValueError(f"Expected obs of shape (nobs,), got {obs.ndim}D tensor with shape {tuple(obs.shape)}")
    nobs = obs.shape[0]
    if float_metadata.ndim != 2 or float_metadata.shape[0] != nobs:
        raise ValueError(f"Expected float_metadata of shape ({nobs}, meta_dim), got tensor with shape {tuple(float_metadata.shape)}")
    for name, t in (("obs_type", obs_type), ("channel", channel), ("platform", platform), ("flat_idx", flat_idx)):
        if t.ndim != 1 or t.shape[0] != nobs:
            raise ValueError(f"Expected {name} of shape ({nobs},), got tensor with shape {tuple(t.shape)}")
    if nobs == 0:
        counts = torch.zeros(total_pixels, dtype=torch.int64, device=obs.device)
        order = torch.empty(0, dtype=torch.long, device=obs.device)
    else:
        order, counts = sort_and_pack(flat_idx, total_pixels)
        order = order.long()
    cu = counts_to_cu_seqlens(counts)
    return ObsContext(obs=obs[order], float_metadata=float_metadata[order], obs_type=obs_type[order], channel=channel[order],
                      platform=platform[order], cu_seqlens_k=cu, max_seqlen_k=int(counts.max()) if nobs > 0 else 0,
                      group_map=build_pixel_group_map(cu, group_thresh_mult) if build_group_map else None)

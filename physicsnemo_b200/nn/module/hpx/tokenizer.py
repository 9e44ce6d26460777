"""HEALPix patch tokenizer / detokenizer for transformer backbones, with calendar (local time, day of year) embedding.

Counterpart of ``physicsnemo/nn/module/hpx/tokenizer.py`` (``HEALPixPatchTokenizer`` :58, ``HEALPixPatchDetokenizer``
:176, ``FrequencyEmbedding`` :288, ``CalendarEmbedding`` :318); parameter names are the same.  The reference takes the
pixel longitudes from the ``earth2grid`` package; here ``healpix_xy_lonlat`` computes the pixel centres directly
(standard HEALPix ring geometry of the nested scheme).

Pixel order: ``index = face * nside^2 + row * nside + column`` with the face-local origin at the northern corner,
``column`` running towards the eastern corner and ``row`` towards the western corner (the order used by the HEALPix
padding layers of this package).  A patch is the ``p x p`` block of fine pixels inside one coarse pixel, so the patch
convolution (stride = kernel) is a GEMM on unfolded patches and writes the token matrix directly; the detokenizer is
the transposed GEMM followed by the inverse unfolding.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

__all__ = ["HEALPixPatchTokenizer", "HEALPixPatchDetokenizer", "FrequencyEmbedding", "CalendarEmbedding", "healpix_xy_lonlat", "healpix_lonlat_to_xy"]

_JRLL = (2, 2, 2, 2, 3, 3, 3, 3, 4, 4, 4, 4)
_JPLL = (1, 3, 5, 7, 0, 2, 4, 6, 1, 3, 5, 7)


def healpix_xy_lonlat(level: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Longitude and latitude (degrees, float64) of the ``12 * 4**level`` pixel centres in the order described above."""
    n = 2 ** level
    face = torch.arange(12).view(12, 1, 1)
    row = torch.arange(n).view(1, n, 1)              # towards the western corner, from the northern corner
    col = torch.arange(n).view(1, 1, n)              # towards the eastern corner
    # nested face coordinates: ix runs south -> east corner direction (north-east), iy runs north-west, origin south
    ix, iy = (n - 1 - row).expand(12, n, n), (n - 1 - col).expand(12, n, n)
    jrll, jpll = torch.tensor(_JRLL).view(12, 1, 1), torch.tensor(_JPLL).view(12, 1, 1)
    jr = jrll * n - ix - iy - 1                                           # ring number, 1 .. 4n - 1
    north, south = jr < n, jr > 3 * n
    nr = torch.where(north, jr, torch.where(south, 4 * n - jr, torch.full_like(jr, n)))
    z = torch.where(north, 1 - nr.double() ** 2 / (3 * n * n),
                    torch.where(south, nr.double() ** 2 / (3 * n * n) - 1, (2 * n - jr).double() * 2 / (3 * n)))
    kshift = torch.where(north | south, torch.zeros_like(jr), (jr - n) & 1)
    jp = (jpll * nr + ix - iy + 1 + kshift) // 2
    jp = torch.where(jp > 4 * nr, jp - 4 * nr, jp)
    jp = torch.where(jp < 1, jp + 4 * nr, jp)
    phi = (jp.double() - (kshift.double() + 1) * 0.5) * (math.pi / 2) / nr.double()
    return torch.rad2deg(phi).reshape(-1), torch.rad2deg(torch.asin(z.expand(12, n, n))).reshape(-1)


def healpix_lonlat_to_xy(lon: torch.Tensor, lat: torch.Tensor, level: int) -> torch.Tensor:
    """Index (in the order of :func:`healpix_xy_lonlat`) of the pixel that contains each point; degrees in, int64 out.

    Standard HEALPix point location: the equatorial belt ``|z| <= 2/3`` uses the two diagonal line
    counters ``jp``, ``jm`` of the cylindrical projection, the polar caps the Collignon coordinates;
    both give the face and the in-face ``(ix, iy)``, which map to ``row = n - 1 - ix``, ``col = n - 1 - iy``.
    """
    n = 2 ** level
    z = torch.sin(torch.deg2rad(lat.double()))
    za = z.abs()
    tt = torch.remainder(lon.double(), 360.0) / 90.0                       # [0, 4)
    # equatorial belt
    t1, t2 = n * (0.5 + tt), n * z * 0.75
    jp, jm = torch.floor(t1 - t2).long(), torch.floor(t1 + t2).long()
    ifp, ifm = jp // n, jm // n
    face_eq = torch.where(ifp == ifm, (ifp % 4) + 4, torch.where(ifp < ifm, ifp % 4, (ifm % 4) + 8))
    ix_eq, iy_eq = jm % n, n - 1 - (jp % n)
    # polar caps
    ntt = tt.floor().clamp(max=3)
    tp = tt - ntt
    tmp = n * torch.sqrt(3 * (1 - za))
    jp_c = torch.floor(tp * tmp).long().clamp(max=n - 1)
    jm_c = torch.floor((1 - tp) * tmp).long().clamp(max=n - 1)
    up = z >= 0
    face_cap = torch.where(up, ntt.long(), ntt.long() + 8)
    ix_cap, iy_cap = torch.where(up, n - 1 - jm_c, jp_c), torch.where(up, n - 1 - jp_c, jm_c)
    belt = za <= 2.0 / 3.0
    face = torch.where(belt, face_eq, face_cap)
    ix, iy = torch.where(belt, ix_eq, ix_cap), torch.where(belt, iy_eq, iy_cap)
    return face * (n * n) + (n - 1 - ix) * n + (n - 1 - iy)


class FrequencyEmbedding(nn.Module):
    """``[cos(2 pi k x), sin(2 pi k x)]`` for ``k = 1 .. num_channels`` of a ``[B, T, X]`` phase, channels on axis 1."""

    def __init__(self, num_channels: int):
        super().__init__()
        self.register_buffer("freqs", torch.arange(1, num_channels + 1), persistent=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ang = x[:, None] * (2 * math.pi * self.freqs[None, :, None, None]).to(x.dtype)
        return torch.cat([ang.cos(), ang.sin()], dim=1)


class CalendarEmbedding(nn.Module):
    """Harmonics of the local solar time of every pixel and of the day of year: ``[B, 4 * embed_channels, T, X]``."""

    def __init__(self, lon: torch.Tensor, embed_channels: int, include_legacy_bug: bool = False):
        super().__init__()
        self.register_buffer("lon", lon, persistent=False)
        self.embed_channels, self.out_channels, self.include_legacy_bug = embed_channels, embed_channels * 4, include_legacy_bug
        self.embed_second = FrequencyEmbedding(embed_channels)
        self.embed_day = FrequencyEmbedding(embed_channels)

    def forward(self, day_of_year: torch.Tensor, second_of_day: torch.Tensor) -> torch.Tensor:
        if second_of_day.shape != day_of_year.shape:
            raise ValueError(f"second_of_day and day_of_year must share a shape; got {tuple(second_of_day.shape)} and "
                             f"{tuple(day_of_year.shape)}")
        offset = self.lon * 86400 // 360
        local = (second_of_day.unsqueeze(2) - offset if self.include_legacy_bug else second_of_day.unsqueeze(2) + offset) % 86400
        a = self.embed_second(local / 86400)
        b = self.embed_day(day_of_year.unsqueeze(2) / 365.25 % 1)
        a, b = torch.broadcast_tensors(a, b)
        return torch.cat([a, b], dim=1)


def _unfold_faces(x: torch.Tensor, nside: int, p: int) -> torch.Tensor:
    """``[B, C, T, 12 n^2] -> [B, T, 12 (n/p)^2, C p p]``: the ``p x p`` fine pixels of every coarse pixel as one row."""
    B, C, T, _ = x.shape
    m = nside // p
    x = x.view(B, C, T, 12, m, p, m, p).permute(0, 2, 3, 4, 6, 1, 5, 7)
    return x.reshape(B, T, 12 * m * m, C * p * p)


class HEALPixPatchTokenizer(nn.Module):
    """``[B, C, T, npix_fine] -> [B, T * npix_coarse, hidden]`` (or ``[B, T, npix_coarse, hidden]``): patch projection
    plus a learned per-pixel position embedding and the calendar embedding."""

    def __init__(self, *, in_channels: int, hidden_size: int, level_fine: int, level_coarse: int, separate_time_axis: bool = False,
                 **kwargs):
        super().__init__()
        if hidden_size % 4 != 0:
            raise ValueError(f"hidden_size must be divisible by 4, got {hidden_size}")
        self.in_channels, self.hidden_size, self.level_fine, self.level_coarse = in_channels, hidden_size, level_fine, level_coarse
        self.separate_time_axis = separate_time_axis
        self.nside, self.nside_coarse, self.patch_size = 2 ** level_fine, 2 ** level_coarse, 2 ** (level_fine - level_coarse)
        self.conv = nn.Conv2d(in_channels, hidden_size, kernel_size=self.patch_size, stride=self.patch_size)
        self.pos_embed = nn.Parameter(torch.randn(12 * 4 ** level_coarse, hidden_size))
        self.calendar_embed = CalendarEmbedding(healpix_xy_lonlat(level_coarse)[0], hidden_size // 4).float()

    def initialize_weights(self) -> None:
        pass

    def forward(self, x: torch.Tensor, second_of_day: torch.Tensor, day_of_year: torch.Tensor) -> torch.Tensor:
        B, _, T, _ = x.shape
        rows = _unfold_faces(x, self.nside, self.patch_size)
        tok = F.linear(rows, self.conv.weight.reshape(self.hidden_size, -1).to(rows.dtype), self.conv.bias.to(rows.dtype))
        cal = self.calendar_embed(second_of_day=second_of_day, day_of_year=day_of_year).permute(0, 2, 3, 1)       # [B, T, X, C]
        tok = tok + cal + self.pos_embed
        return tok if self.separate_time_axis else tok.reshape(B, -1, self.hidden_size)


class HEALPixPatchDetokenizer(nn.Module):
    """Adaptive layer norm on the conditioning vector, then the transposed patch projection back to the fine grid:
    ``[B, T * npix_coarse, hidden]`` (or with a separate time axis) ``-> [B, C_out, T, npix_fine]``."""

    def __init__(self, *, hidden_size: int, out_channels: int, level_coarse: int, level_fine: int, time_length: int = 1,
                 condition_dim: Optional[int] = None, **kwargs):
        super().__init__()
        self.hidden_size, self.out_channels, self.level_coarse, self.level_fine, self.time_length = hidden_size, out_channels, level_coarse, level_fine, time_length
        self.nside_coarse, self.patch_size = 2 ** level_coarse, 2 ** (level_fine - level_coarse)
        self.adaptive_modulation = nn.Sequential(nn.SiLU(), nn.Linear(hidden_size if condition_dim is None else condition_dim, 2 * hidden_size))
        self.norm_out = nn.LayerNorm(hidden_size, elementwise_affine=False, eps=1e-6)
        self.conv_t = nn.ConvTranspose2d(hidden_size, out_channels, kernel_size=self.patch_size, stride=self.patch_size)

    def initialize_weights(self) -> None:
        nn.init.zeros_(self.adaptive_modulation[-1].weight)
        nn.init.zeros_(self.adaptive_modulation[-1].bias)

    def forward(self, x: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
        B, m, p = x.shape[0], self.nside_coarse, self.patch_size
        if x.ndim != 4:
            x = x.reshape(B, self.time_length, 12 * m * m, self.hidden_size)
        T = x.shape[1]
        shift, scale = self.adaptive_modulation(c).chunk(2, dim=-1)
        x = torch.addcmul(shift[:, None, None, :], self.norm_out(x), 1 + scale[:, None, None, :])
        # conv_t weight [hidden, C_out, p, p]: one GEMM to (C_out, p, p) per coarse pixel, then fold the patches back
        w = self.conv_t.weight.reshape(self.hidden_size, -1).to(x.dtype)
        y = (x @ w).view(B, T, 12, m, m, self.out_channels, p, p) + self.conv_t.bias.to(x.dtype).view(1, 1, 1, 1, 1, -1, 1, 1)
        return y.permute(0, 5, 1, 2, 3, 6, 4, 7).reshape(B, self.out_channels, T, 12 * m * p * m * p)

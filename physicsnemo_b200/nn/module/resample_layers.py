"""Patch-merging / patch-splitting resamplers of the Pangu / FengWu transformers.

Parity: ``physicsnemo/nn/module/resample_layers.py`` — tokens ``[B, N, C]`` on a (pressure,) lat, lon lattice;
down: zero-pad to even extents, merge 2×2 horizontal patches (4C) → LayerNorm → Linear(4C→2C); up:
Linear(C→4·out) → split into 2×2 → crop to the target extents → LayerNorm → Linear.
"""
import torch
from torch import nn


def _crop(pad):
    lo = pad // 2
    return lo, pad - lo


class _Up(nn.Module):
    def __init__(self, in_dim, out_dim, input_resolution, output_resolution):
        super().__init__()
        self.linear1 = nn.Linear(in_dim, out_dim * 4, bias=False)
        self.linear2 = nn.Linear(out_dim, out_dim, bias=False)
        self.norm = nn.LayerNorm(out_dim)
        self.input_resolution, self.output_resolution = input_resolution, output_resolution

    def forward(self, x: torch.Tensor):
        B, _, C = x.shape
        *lead_in, ilat, ilon = self.input_resolution
        *lead_out, olat, olon = self.output_resolution
        lead = tuple(lead_in)
        x = self.linear1(x).reshape(B, *lead, ilat, ilon, 2, 2, C // 2)
        n = len(lead)
        x = x.permute(*range(0, n + 2), n + 3, n + 2, n + 4, n + 5).reshape(B, *lead, ilat * 2, ilon * 2, -1)
        top, bottom = _crop(ilat * 2 - olat)
        left, right = _crop(ilon * 2 - olon)
        if lead:
            x = x[:, :lead_out[0]]
        x = x[..., top:2 * ilat - bottom, left:2 * ilon - right, :]
        x = x.reshape(B, -1, x.shape[-1])
        return self.linear2(self.norm(x))


class UpSample3D(_Up):
    pass


class UpSample2D(_Up):
    pass


class _Down(nn.Module):
    def __init__(self, in_dim, input_resolution, output_resolution):
        super().__init__()
        self.linear = nn.Linear(in_dim * 4, in_dim * 2, bias=False)
        self.norm = nn.LayerNorm(4 * in_dim)
        self.input_resolution, self.output_resolution = input_resolution, output_resolution
        *_, ilat, ilon = input_resolution
        *_, olat, olon = output_resolution
        top, bottom = _crop(olat * 2 - ilat)
        left, right = _crop(olon * 2 - ilon)
        if len(input_resolution) == 3:
            self.pad = nn.ZeroPad3d((left, right, top, bottom, 0, 0))
        else:
            self.pad = nn.ZeroPad2d((left, right, top, bottom))

    def forward(self, x: torch.Tensor):
        B, _, C = x.shape
        *lead, ilat, ilon = self.input_resolution
        *lead_out, olat, olon = self.output_resolution
        lead = tuple(lead)
        n = len(lead)
        x = x.reshape(B, *lead, ilat, ilon, C)
        x = self.pad(x.movedim(-1, 1)).movedim(1, -1)
        x = x.reshape(B, *lead, olat, 2, olon, 2, C).permute(*range(0, n + 2), n + 3, n + 2, n + 4, n + 5)
        x = x.reshape(B, -1, 4 * C)
        return self.linear(self.norm(x))


class DownSample3D(_Down):
    pass


class DownSample2D(_Down):
    pass

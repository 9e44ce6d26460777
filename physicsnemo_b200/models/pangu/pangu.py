"""Pangu-Weather 3-D earth-specific transformer.

Parity: ``physicsnemo/models/pangu/pangu.py`` — surface (4 + 3 mask channels) and upper-air (5 variables × 13
levels) inputs are patch-embedded (2-D / 3-D), stacked to 8 pressure slabs, and processed by four ``FuserLayer``
stages (2-6-6-2 blocks, one down / up sampling with a skip) before 2-D / 3-D patch recovery.
"""
import math
from dataclasses import dataclass

import numpy as np
import torch

from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.resample_layers import DownSample3D, UpSample3D
from ...nn.module.transformer_layers import FuserLayer
from ...nn.module.utils import PatchEmbed2D, PatchEmbed3D, PatchRecovery2D, PatchRecovery3D


@dataclass
class MetaData(ModelMetaData):
    jit: bool = False
    cuda_graphs: bool = True
    amp: bool = True
    onnx_cpu: bool = False
    onnx_gpu: bool = True
    onnx_runtime: bool = True
    var_dim: int = 1
    func_torch: bool = False
    auto_grad: bool = False


def _expect(cond, msg):
    if not cond:
        raise ValueError(msg)


def _check_field(name: str, tensor, wanted: tuple) -> None:
    """``tensor`` must have exactly the shape ``wanted`` (batch first where there is one); the message names the first
    axis that differs: sample, channel, pressure level or grid."""
    got = tuple(tensor.shape)
    if got == tuple(wanted):
        return
    if len(got) != len(wanted):
        raise ValueError(f"'{name}' should have {len(wanted)} dimensions {tuple(wanted)}, but its shape is {got}")
    axis = next(i for i, (g, w) in enumerate(zip(got, wanted)) if g != w)
    from_end = len(wanted) - axis
    if from_end <= 2:
        what = "grid size"
    elif axis == 0 and len(wanted) >= 4:
        what = "batch size"
    elif len(wanted) == 5 and axis == 2:
        what = "number of pressure levels"
    else:
        what = "channel count"
    raise ValueError(f"'{name}' has the wrong {what}: expected shape {tuple(wanted)}, got {got}")


class Pangu(Module):
    def __init__(self, img_size: tuple[int, int] = (721, 1440), patch_size: tuple[int, int, int] = (2, 4, 4),
                 embed_dim: int = 192, num_heads: tuple[int, int, int, int] = (6, 12, 12, 6),
                 window_size: tuple[int, int, int] = (2, 6, 12)) -> None:
        super().__init__(meta=MetaData())
        self.img_size, self.patch_size, self.embed_dim = tuple(img_size), tuple(patch_size), embed_dim
        self.surface_channels, self.surface_mask_channels = 4, 3
        self.upper_air_channels, self.upper_air_levels = 5, 13
        self.surface_input_channels = self.surface_channels + self.surface_mask_channels
        self.in_channels = self.surface_input_channels + self.upper_air_channels * self.upper_air_levels
        drop_path = np.linspace(0, 0.2, 8).tolist()
        self.patchembed2d = PatchEmbed2D(img_size=img_size, patch_size=patch_size[1:], in_chans=7, embed_dim=embed_dim)
        self.patchembed3d = PatchEmbed3D(img_size=(13, img_size[0], img_size[1]), patch_size=patch_size, in_chans=5,
                                         embed_dim=embed_dim)
        fine = (8, math.ceil(img_size[0] / patch_size[1]), math.ceil(img_size[1] / patch_size[2]))
        coarse = (8, math.ceil(fine[1] / 2), math.ceil(fine[2] / 2))
        self.layer1 = FuserLayer(dim=embed_dim, input_resolution=fine, depth=2, num_heads=num_heads[0],
                                 window_size=window_size, drop_path=drop_path[:2])
        self.downsample = DownSample3D(in_dim=embed_dim, input_resolution=fine, output_resolution=coarse)
        self.layer2 = FuserLayer(dim=embed_dim * 2, input_resolution=coarse, depth=6, num_heads=num_heads[1],
                                 window_size=window_size, drop_path=drop_path[2:])
        self.layer3 = FuserLayer(dim=embed_dim * 2, input_resolution=coarse, depth=6, num_heads=num_heads[2],
                                 window_size=window_size, drop_path=drop_path[2:])
        self.upsample = UpSample3D(embed_dim * 2, embed_dim, coarse, fine)
        self.layer4 = FuserLayer(dim=embed_dim, input_resolution=fine, depth=2, num_heads=num_heads[3],
                                 window_size=window_size, drop_path=drop_path[:2])
        self.patchrecovery2d = PatchRecovery2D(img_size, patch_size[1:], 2 * embed_dim, 4)
        self.patchrecovery3d = PatchRecovery3D((13, img_size[0], img_size[1]), patch_size, 2 * embed_dim, 5)

    def prepare_input(self, surface, surface_mask, upper_air):
        """Concatenate ``surface [B,4,H,W]``, ``surface_mask [3,H,W]`` (or batched) and ``upper_air [B,5,13,H,W]``."""
        if not torch.compiler.is_compiling():
            batch = surface.shape[0]
            _check_field("surface", surface, (batch, self.surface_channels, *self.img_size))
            _expect(surface_mask.ndim in (3, 4), f"'surface_mask' is either one [C, H, W] mask for all samples or a batch "
                                                  f"[B, C, H, W] of masks; its shape is {tuple(surface_mask.shape)}")
            lead = (batch,) if surface_mask.ndim == 4 else ()
            _check_field("surface_mask", surface_mask, (*lead, self.surface_mask_channels, *self.img_size))
            _check_field("upper_air", upper_air, (batch, self.upper_air_channels, self.upper_air_levels, *self.img_size))
        if surface_mask.ndim == 3:
            surface_mask = surface_mask.unsqueeze(0).repeat(surface.shape[0], 1, 1, 1)
        return torch.cat([surface, surface_mask, upper_air.flatten(1, 2)], dim=1)

    def forward(self, x):
        if not torch.compiler.is_compiling():
            _check_field("x", x, (x.shape[0], self.in_channels, *self.img_size))
        n_s = self.surface_input_channels
        surface = self.patchembed2d(x[:, :n_s])
        upper = self.patchembed3d(x[:, n_s:].reshape(x.shape[0], self.upper_air_channels, self.upper_air_levels, *x.shape[2:]))
        x = torch.cat([surface.unsqueeze(2), upper], dim=2)
        B, C, Pl, Lat, Lon = x.shape
        x = self.layer1(x.reshape(B, C, -1).transpose(1, 2))
        skip = x
        x = self.layer3(self.layer2(self.downsample(x)))
        x = self.layer4(self.upsample(x))
        out = torch.cat([x, skip], dim=-1).transpose(1, 2).reshape(B, -1, Pl, Lat, Lon)
        return self.patchrecovery2d(out[:, :, 0]), self.patchrecovery3d(out[:, :, 1:])

"""FengWu: per-variable 2-D encoders / decoders around a 3-D fuser.

Parity: ``physicsnemo/models/fengwu/fengwu.py`` — six modalities (surface, z, r, u, v, t), each with its own
``EncoderLayer`` / ``DecoderLayer``; the six latent maps are stacked as pressure slabs and mixed by a 6-block
``FuserLayer``.  Sub-module names (``encoder_surface``, ``encoder_z``, …, ``fuser``, ``decoder_t``) follow the
reference so checkpoints are interchangeable.
"""
import math
from dataclasses import dataclass

import numpy as np
import torch

from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.transformer_layers import DecoderLayer, EncoderLayer, FuserLayer

_NAMES = ("surface", "z", "r", "u", "v", "t")


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


class Fengwu(Module):
    def __init__(self, img_size: tuple[int, int] = (721, 1440), pressure_level: int = 37, embed_dim: int = 192,
                 patch_size: tuple[int, int] = (4, 4), num_heads: tuple[int, int, int, int] = (6, 12, 12, 6),
                 window_size: tuple[int, int, int] = (2, 6, 12)) -> None:
        super().__init__(meta=MetaData())
        self.img_size, self.pressure_level = tuple(img_size), pressure_level
        self.patch_size, self.embed_dim = tuple(patch_size), embed_dim
        self.surface_channels = 4
        self.in_channels = self.surface_channels + 5 * pressure_level
        drop_path = np.linspace(0, 0.2, 8).tolist()
        fine = (math.ceil(img_size[0] / patch_size[0]), math.ceil(img_size[1] / patch_size[1]))
        coarse = (math.ceil(fine[0] / 2), math.ceil(fine[1] / 2))
        common = dict(img_size=img_size, patch_size=patch_size, dim=embed_dim, middle_resolution=coarse, depth=2,
                      depth_middle=6, num_heads=num_heads[:2], window_size=window_size[1:], drop_path=drop_path)
        for name in _NAMES:
            ch = self.surface_channels if name == "surface" else pressure_level
            setattr(self, f"encoder_{name}", EncoderLayer(in_chans=ch, input_resolution=fine, **common))
        self.fuser = FuserLayer(dim=embed_dim * 2, input_resolution=(6, coarse[0], coarse[1]), depth=6,
                                num_heads=num_heads[1], window_size=window_size, drop_path=[0.2] * 6)
        for name in _NAMES:
            ch = self.surface_channels if name == "surface" else pressure_level
            setattr(self, f"decoder_{name}", DecoderLayer(out_chans=ch, output_resolution=fine, **common))

    def prepare_input(self, surface, z, r, u, v, t):
        if not torch.compiler.is_compiling():
            for name, ten in zip(_NAMES, (surface, z, r, u, v, t)):
                ch = self.surface_channels if name == "surface" else self.pressure_level
                if ten.ndim != 4:
                    raise ValueError(f"Expected '{name}' to be a 4D tensor, got {ten.ndim}D tensor with shape {tuple(ten.shape)}")
                if ten.shape[1] != ch:
                    raise ValueError(f"Expected '{name}' to have {ch} channels, got tensor with shape {tuple(ten.shape)}")
                if tuple(ten.shape[2:]) != self.img_size:
                    raise ValueError(f"Expected '{name}' spatial shape {self.img_size}, got tensor with shape {tuple(ten.shape)}")
                if ten.shape[0] != surface.shape[0]:
                    raise ValueError(f"Expected '{name}' batch size {surface.shape[0]}, got tensor with shape {tuple(ten.shape)}")
        return torch.cat([surface, z, r, u, v, t], dim=1)

    def forward(self, x):
        if not torch.compiler.is_compiling():
            if x.ndim != 4:
                raise ValueError(f"Expected 'x' to be a 4D tensor, got {x.ndim}D tensor with shape {tuple(x.shape)}")
            if x.shape[1] != self.in_channels:
                raise ValueError(f"Expected 'x' to have {self.in_channels} channels, got tensor with shape {tuple(x.shape)}")
            if tuple(x.shape[2:]) != self.img_size:
                raise ValueError(f"Expected 'x' spatial shape {self.img_size}, got tensor with shape {tuple(x.shape)}")
        sizes = [self.surface_channels] + [self.pressure_level] * 5
        latents, skips = [], []
        for name, part in zip(_NAMES, torch.split(x, sizes, dim=1)):
            lat, skip = getattr(self, f"encoder_{name}")(part)
            latents.append(lat)
            skips.append(skip)
        z = torch.stack(latents, dim=1)                           # [B, 6, L, C]
        B, P, L, C = z.shape
        z = self.fuser(z.reshape(B, -1, C)).reshape(B, P, L, C)
        return tuple(getattr(self, f"decoder_{name}")(z[:, i], skips[i]) for i, name in enumerate(_NAMES))

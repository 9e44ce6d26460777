"""SwinRNN: Swin-transformer encoder / decoder pyramid with recurrent skip fusion.

Parity: ``physicsnemo/models/swinvrnn/swinvrnn.py`` — cube embedding of a ``(T, lat, lon)`` history, four
resolution levels of ``SwinTransformer`` blocks joined by strided ``ConvBlock``s; at every level the latest
input frame (down-sampled alongside) is concatenated with the features, projected and refined by a
12-block decoder; an up-sampling pyramid predicts the increment of the last frame.
"""
from dataclasses import dataclass

import torch
from torch import nn

from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.conv_layers import ConvBlock, CubeEmbedding
from ...nn.module.transformer_layers import SwinTransformer


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


class SwinRNN(Module):
    def __init__(self, img_size: tuple[int, int, int] = (2, 721, 1440), patch_size: tuple[int, int, int] = (2, 4, 4),
                 in_chans: int = 70, out_chans: int = 70, embed_dim: int = 1536, num_groups: int = 32, num_heads: int = 8,
                 window_size: int = 7) -> None:
        super().__init__(meta=MetaData())
        self.img_size, self.patch_size = tuple(img_size), tuple(patch_size)
        self.in_chans, self.out_chans, self.embed_dim = in_chans, out_chans, embed_dim
        res = tuple(img_size[1:])
        self.cube_embedding = CubeEmbedding(img_size, patch_size, in_chans, embed_dim)
        for level in range(1, 5):
            setattr(self, f"swin_block{level}", SwinTransformer(embed_dim, res, num_heads, window_size, depth=2))
            if level < 4:
                setattr(self, f"down{level}", ConvBlock(embed_dim, embed_dim, num_groups, upsample=-1))
                setattr(self, f"down{level}x", ConvBlock(in_chans, in_chans, in_chans, upsample=-1))
            setattr(self, f"lin_proj{level}", nn.Linear(embed_dim + in_chans, embed_dim))
            setattr(self, f"swin_decoder{level}", SwinTransformer(embed_dim, res, num_heads, window_size, depth=12))
            if level < 4:
                res = (res[0] // 2, res[1] // 2)
        self.up3x = ConvBlock(embed_dim, embed_dim, num_groups, upsample=1)
        self.up2x = ConvBlock(embed_dim * 2, embed_dim, num_groups, upsample=1)
        self.up1x = ConvBlock(embed_dim * 2, embed_dim, num_groups, upsample=1)
        self.pred = ConvBlock(embed_dim * 2, out_chans, out_chans, upsample=0)
        self.input_resolution = res

    def _fuse(self, level, frame, feat):
        B, C, H, W = frame.shape
        z = torch.cat([frame.reshape(B, C, -1), feat.reshape(B, self.embed_dim, -1)], dim=1).transpose(1, 2)
        z = getattr(self, f"lin_proj{level}")(z).transpose(1, 2).reshape(B, self.embed_dim, H, W)
        return feat + getattr(self, f"swin_decoder{level}")(z)

    def forward(self, x):
        if not torch.compiler.is_compiling():
            if x.ndim != 5:
                raise ValueError(f"Expected 'x' to be a 5D tensor, got {x.ndim}D tensor with shape {tuple(x.shape)}")
            if x.shape[1] != self.in_chans:
                raise ValueError(f"Expected 'x' to have {self.in_chans} channels, got tensor with shape {tuple(x.shape)}")
            if x.shape[2] != self.img_size[0]:
                raise ValueError(f"Expected 'x' time dimension {self.img_size[0]}, got tensor with shape {tuple(x.shape)}")
            if tuple(x.shape[3:]) != self.img_size[1:]:
                raise ValueError(f"Expected 'x' spatial shape {self.img_size[1:]}, got tensor with shape {tuple(x.shape)}")
        last = x[:, :, -1]
        z = self.cube_embedding(x).squeeze(2)
        feats, frames, frame = [], [], last
        for level in range(1, 5):
            h = getattr(self, f"swin_block{level}")(z)
            feats.append(h)
            frames.append(frame)
            if level < 4:
                z = getattr(self, f"down{level}")(h)
                frame = getattr(self, f"down{level}x")(frame)
        h1, h2, h3, h4 = (self._fuse(i + 1, frames[i], feats[i]) for i in range(4))
        up = self.up3x(h4)
        up = self.up2x(torch.cat([h3, up], dim=1))
        up = self.up1x(torch.cat([h2, up], dim=1))
        return last + self.pred(torch.cat([h1, up], dim=1))

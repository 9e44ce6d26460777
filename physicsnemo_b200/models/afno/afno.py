"""Adaptive Fourier Neural Operator (FourCastNet backbone).

Parity: ``physicsnemo/models/afno/afno.py`` — ``Block`` (``:38-125``) and ``AFNO`` (``:144-359``):
patch embedding + learned position embedding → ``depth`` × {LN → AFNO2DLayer → (+res) → LN → MLP
→ +res} → linear head → un-patchify.  Keys: ``pos_embed``, ``patch_embed.proj.*``,
``blocks.#.{norm1,norm2,filter.{w1,b1,w2,b2},mlp.{fc1,fc2}}``, ``head.weight``.
"""
from __future__ import annotations

from dataclasses import dataclass
from functools import partial
from typing import List

import torch
import torch.nn as nn
from torch import Tensor

from ... import ops
from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.afno_layers import AFNO2DLayer, AFNOMlp, AFNOPatchEmbed
from ...nn.module.layer_norm import LayerNorm


class Block(nn.Module):
    """AFNO transformer block on (B, H, W, C) tokens."""

    def __init__(self, embed_dim: int, num_blocks: int = 8, mlp_ratio: float = 4.0, drop: float = 0.0,
                 activation_fn: nn.Module = nn.GELU(), norm_layer=LayerNorm, double_skip: bool = True,
                 sparsity_threshold: float = 0.01, hard_thresholding_fraction: float = 1.0):
        super().__init__()
        self.norm1 = norm_layer(embed_dim)
        self.filter = AFNO2DLayer(embed_dim, num_blocks, sparsity_threshold, hard_thresholding_fraction)
        self.norm2 = norm_layer(embed_dim)
        self.mlp = AFNOMlp(in_features=embed_dim, latent_features=int(embed_dim * mlp_ratio), out_features=embed_dim,
                           activation_fn=activation_fn, drop=drop)
        self.double_skip = double_skip

    def forward(self, x: Tensor) -> Tensor:
        residual = x
        x = self.filter(self.norm1(x))
        if self.double_skip:
            x = x + residual
            residual = x
        return self.mlp(self.norm2(x), residual=residual)


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


class AFNO(Module):
    """AFNO model: (B, in_channels, H, W) → (B, out_channels, H, W)."""

    def __init__(self, inp_shape: List[int], in_channels: int, out_channels: int, patch_size: List[int] = [16, 16],
                 embed_dim: int = 256, depth: int = 4, mlp_ratio: float = 4.0, drop_rate: float = 0.0,
                 num_blocks: int = 16, sparsity_threshold: float = 0.01,
                 hard_thresholding_fraction: float = 1.0) -> None:
        super().__init__(meta=MetaData())
        if len(inp_shape) != 2:
            raise ValueError("inp_shape should be a list of length 2")
        if len(patch_size) != 2:
            raise ValueError("patch_size should be a list of length 2")
        if not (inp_shape[0] % patch_size[0] == 0 and inp_shape[1] % patch_size[1] == 0):
            raise ValueError(f"input shape {inp_shape} should be divisible by patch_size {patch_size}")
        self.in_chans, self.out_chans = in_channels, out_channels
        self.inp_shape, self.patch_size = inp_shape, patch_size
        self.num_features = self.embed_dim = embed_dim
        self.num_blocks = num_blocks
        norm_layer = partial(LayerNorm, eps=1e-6)
        self.patch_embed = AFNOPatchEmbed(inp_shape=inp_shape, in_channels=in_channels, patch_size=patch_size,
                                          embed_dim=embed_dim)
        self.pos_embed = nn.Parameter(torch.zeros(1, self.patch_embed.num_patches, embed_dim))
        self.pos_drop = nn.Dropout(p=drop_rate)
        self.h = inp_shape[0] // patch_size[0]
        self.w = inp_shape[1] // patch_size[1]
        self.blocks = nn.ModuleList([
            Block(embed_dim=embed_dim, num_blocks=num_blocks, mlp_ratio=mlp_ratio, drop=drop_rate,
                  norm_layer=norm_layer, sparsity_threshold=sparsity_threshold,
                  hard_thresholding_fraction=hard_thresholding_fraction)
            for _ in range(depth)
        ])
        self.head = nn.Linear(embed_dim, out_channels * patch_size[0] * patch_size[1], bias=False)
        torch.nn.init.trunc_normal_(self.pos_embed, std=0.02)
        self.apply(self._init_weights)

    def _init_weights(self, m: nn.Module) -> None:
        if isinstance(m, nn.Linear):
            torch.nn.init.trunc_normal_(m.weight, std=0.02)
            if m.bias is not None:
                nn.init.constant_(m.bias, 0)
        elif isinstance(m, nn.LayerNorm):
            nn.init.constant_(m.bias, 0)
            nn.init.constant_(m.weight, 1.0)

    def _forward_features(self, x: Tensor) -> Tensor:
        B = x.shape[0]
        x = self.patch_embed(x)
        x = self.pos_drop(x + self.pos_embed)
        x = x.reshape(B, self.h, self.w, self.embed_dim)
        for blk in self.blocks:
            x = blk(x)
        return x

    def forward(self, x: Tensor) -> Tensor:
        if not torch.compiler.is_compiling():
            expected = (self.in_chans, self.inp_shape[0], self.inp_shape[1])
            if x.ndim != 4 or tuple(x.shape[1:]) != expected:
                raise ValueError(f"Expected input shape (B, {expected[0]}, {expected[1]}, {expected[2]}), got {tuple(x.shape)}")
        x = self._forward_features(x)
        x = ops.linear(x, self.head.weight, None)
        out = x.view(list(x.shape[:-1]) + [self.patch_size[0], self.patch_size[1], -1])
        out = torch.permute(out, (0, 5, 1, 3, 2, 4))
        return out.reshape(list(out.shape[:2]) + [self.inp_shape[0], self.inp_shape[1]])

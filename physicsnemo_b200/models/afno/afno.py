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
    """AFNO transformer block on (B, H, W, C) tokens: spectral token mixing, then a channel MLP, both pre-normed.

    With ``double_skip`` the block has two residual connections (around the filter and around the MLP); without it a
    single one spans both.  The MLP adds its residual inside its last GEMM."""

    def __init__(self, embed_dim: int, num_blocks: int = 8, mlp_ratio: float = 4.0, drop: float = 0.0,
                 activation_fn: nn.Module = nn.GELU(), norm_layer=LayerNorm, double_skip: bool = True,
                 sparsity_threshold: float = 0.01, hard_thresholding_fraction: float = 1.0):
        super().__init__()
        hidden = int(mlp_ratio * embed_dim)
        self.double_skip = double_skip
        self.norm1, self.norm2 = norm_layer(embed_dim), norm_layer(embed_dim)
        self.filter = AFNO2DLayer(embed_dim, num_blocks=num_blocks, sparsity_threshold=sparsity_threshold,
                                  hard_thresholding_fraction=hard_thresholding_fraction)
        self.mlp = AFNOMlp(embed_dim, hidden, embed_dim, activation_fn=activation_fn, drop=drop)

    def forward(self, x: Tensor) -> Tensor:
        if self._fused_residuals(x):
            return self._forward_fused(x)
        mixed = self.filter(self.norm1(x))
        skip = x
        if self.double_skip:
            mixed = skip = mixed + x
        return self.mlp(self.norm2(mixed), residual=skip)

    def _fused_residuals(self, x: Tensor) -> bool:
        return (type(x) is torch.Tensor and x.is_cuda and x.dtype == torch.bfloat16 and type(self.norm1) is LayerNorm
                and type(self.norm2) is LayerNorm and type(self.filter) is AFNO2DLayer and ops.fused_path_enabled(x))

    def _forward_fused(self, x: Tensor) -> Tensor:
        """Same block with no separate elementwise kernels: each LayerNorm hands its input on as the skip tensor (the
        LayerNorm backward then sums the two gradient paths), the filter adds its own residual and the skip while it
        stores its result, the MLP adds its residual in its last GEMM."""
        n1, x_skip = ops.layer_norm(x, self.norm1.weight, self.norm1.bias, self.norm1.eps, return_residual=True)
        if self.double_skip:
            mixed = self.filter(n1, residual=x_skip)
            n2, skip = ops.layer_norm(mixed, self.norm2.weight, self.norm2.bias, self.norm2.eps, return_residual=True)
        else:
            mixed = self.filter(n1)
            n2, skip = ops.layer_norm(mixed, self.norm2.weight, self.norm2.bias, self.norm2.eps), x_skip
        return self.mlp(n2, residual=skip)


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
        for name, pair in (("inp_shape", inp_shape), ("patch_size", patch_size)):
            if len(pair) != 2:
                raise ValueError(f"{name} must give (height, width); got {list(pair)}")
        if any(n % p for n, p in zip(inp_shape, patch_size)):
            raise ValueError(f"a {list(inp_shape)} grid cannot be cut into {list(patch_size)} patches without remainder")
        self.inp_shape, self.patch_size = inp_shape, patch_size
        self.in_chans, self.out_chans = in_channels, out_channels
        self.embed_dim = self.num_features = embed_dim
        self.num_blocks = num_blocks
        self.h, self.w = (n // p for n, p in zip(inp_shape, patch_size))        # token grid
        self.patch_embed = AFNOPatchEmbed(inp_shape=inp_shape, in_channels=in_channels, patch_size=patch_size,
                                          embed_dim=embed_dim)
        self.pos_embed = nn.Parameter(torch.zeros(1, self.patch_embed.num_patches, embed_dim))
        self.pos_drop = nn.Dropout(p=drop_rate)
        block_args = dict(num_blocks=num_blocks, mlp_ratio=mlp_ratio, drop=drop_rate, norm_layer=partial(LayerNorm, eps=1e-6),
                          sparsity_threshold=sparsity_threshold, hard_thresholding_fraction=hard_thresholding_fraction)
        self.blocks = nn.ModuleList(Block(embed_dim, **block_args) for _ in range(depth))
        self.head = nn.Linear(embed_dim, patch_size[0] * patch_size[1] * out_channels, bias=False)
        nn.init.trunc_normal_(self.pos_embed, std=0.02)
        self.apply(self._init_weights)

    @staticmethod
    def _init_weights(m: nn.Module) -> None:
        """Linear layers: truncated normal weights (std 0.02), zero bias; LayerNorm: unit scale, zero shift."""
        if isinstance(m, nn.LayerNorm):
            nn.init.ones_(m.weight)
            nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Linear):
            nn.init.trunc_normal_(m.weight, std=0.02)
            if m.bias is not None:
                nn.init.zeros_(m.bias)

    def _forward_features(self, x: Tensor) -> Tensor:
        tokens = self.pos_drop(self.patch_embed(x) + self.pos_embed)
        tokens = tokens.reshape(x.shape[0], self.h, self.w, self.embed_dim)
        for blk in self.blocks:
            tokens = blk(tokens)
        return tokens

    def forward(self, x: Tensor) -> Tensor:
        if not torch.compiler.is_compiling():
            wanted = (self.in_chans, *self.inp_shape)
            if x.ndim != 4 or tuple(x.shape[1:]) != wanted:
                raise ValueError(f"AFNO was built for inputs [B, {wanted[0]}, {wanted[1]}, {wanted[2]}]; got {tuple(x.shape)}")
        tokens = ops.linear(self._forward_features(x), self.head.weight, None)           # [B, h, w, p0 * p1 * C_out]
        p0, p1 = self.patch_size
        # un-patchify: the head's features are ordered (p0, p1, channel)
        return ops.unpatchify(tokens, self.h, self.w, p0, p1, self.out_chans)

"""Modulated AFNO: an AFNO whose spectral filters and MLPs are scaled / shifted by an embedding of a side input
(for instance the forecast lead time).

Parity: ``physicsnemo/models/afno/modafno.py`` — ``Block`` (``:46-181``) and ``ModAFNO`` (``:198-``): constructor
arguments, attribute names (``patch_embed``, ``pos_embed``, ``blocks.#.{norm1,filter,norm2,mlp}``, ``head``,
``mod_additive_proj``, ``mod_embed_net``) and therefore the state-dict keys are the reference's.  The modulation
embedding is also projected and added to every token before the first block.
"""
from __future__ import annotations

from dataclasses import dataclass
from functools import partial
from typing import List, Literal, Union

import torch
import torch.nn as nn
from torch import Tensor

from ... import ops
from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.afno_layers import AFNO2DLayer, AFNOMlp, AFNOPatchEmbed, ModAFNO2DLayer, ModAFNOMlp
from .modembed import ModEmbedNet


class Block(Module):
    """AFNO block on (B, H, W, C) tokens with optional modulation of the filter and of the MLP."""

    def __init__(self, embed_dim: int, mod_dim: int, num_blocks: int = 8, mlp_ratio: float = 4.0, drop: float = 0.0,
                 activation_fn: nn.Module = nn.GELU(), norm_layer=nn.LayerNorm, double_skip: bool = True,
                 sparsity_threshold: float = 0.01, hard_thresholding_fraction: float = 1.0, modulate_filter: bool = True,
                 modulate_mlp: bool = True, scale_shift_mode: Literal["complex", "real"] = "real"):
        super().__init__()
        self.norm1 = norm_layer(embed_dim)
        if modulate_filter:
            self.filter = ModAFNO2DLayer(embed_dim, mod_dim, num_blocks, sparsity_threshold, hard_thresholding_fraction,
                                         scale_shift_mode=scale_shift_mode)
        else:
            self.filter = AFNO2DLayer(embed_dim, num_blocks, sparsity_threshold, hard_thresholding_fraction)
        self.norm2 = norm_layer(embed_dim)
        latent = int(embed_dim * mlp_ratio)
        if modulate_mlp:
            self.mlp = ModAFNOMlp(in_features=embed_dim, latent_features=latent, out_features=embed_dim, mod_features=mod_dim,
                                  activation_fn=activation_fn, drop=drop)
        else:
            self.mlp = AFNOMlp(in_features=embed_dim, latent_features=latent, out_features=embed_dim,
                               activation_fn=activation_fn, drop=drop)
        self.double_skip, self.modulate_filter, self.modulate_mlp = double_skip, modulate_filter, modulate_mlp

    def forward(self, x: Tensor, mod_embed: Tensor) -> Tensor:
        skip = x
        y = self.norm1(x)
        y = self.filter(y, mod_embed) if self.modulate_filter else self.filter(y)
        if self.double_skip:
            y = y + skip
            skip = y
        y = self.norm2(y)
        y = self.mlp(y, mod_embed) if self.modulate_mlp else self.mlp(y)
        return y + skip


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


class ModAFNO(Module):
    """``forward(x (B, C_in, H, W), mod (B,) or (B, 1)) -> (B, C_out, H, W)``."""

    def __init__(self, inp_shape: List[int], in_channels: int = 155, out_channels: int = 73,
                 embed_model: Union[dict, None] = None, patch_size: List[int] = [2, 2], embed_dim: int = 512,
                 mod_dim: int = 64, modulate_filter: bool = True, modulate_mlp: bool = True,
                 scale_shift_mode: Literal["complex", "real"] = "complex", depth: int = 12, mlp_ratio: float = 2.0,
                 drop_rate: float = 0.0, num_blocks: int = 1, sparsity_threshold: float = 0.01,
                 hard_thresholding_fraction: float = 1.0) -> None:
        super().__init__(meta=MetaData())
        if len(inp_shape) != 2 or len(patch_size) != 2:
            raise ValueError("inp_shape and patch_size must both have two entries (height, width)")
        if inp_shape[0] % patch_size[0] or inp_shape[1] % patch_size[1]:
            raise ValueError(f"the grid {inp_shape} is not a whole number of {patch_size} patches")
        self.in_chans, self.out_chans = in_channels, out_channels
        self.inp_shape, self.patch_size = inp_shape, patch_size
        self.num_features = self.embed_dim = embed_dim
        self.num_blocks = num_blocks
        self.modulate_filter, self.modulate_mlp, self.scale_shift_mode = modulate_filter, modulate_mlp, scale_shift_mode
        self.patch_embed = AFNOPatchEmbed(inp_shape=inp_shape, in_channels=in_channels, patch_size=patch_size, embed_dim=embed_dim)
        self.pos_embed = nn.Parameter(torch.zeros(1, self.patch_embed.num_patches, embed_dim))
        self.pos_drop = nn.Dropout(p=drop_rate)
        self.h, self.w = inp_shape[0] // patch_size[0], inp_shape[1] // patch_size[1]
        norm_layer = partial(nn.LayerNorm, eps=1e-6)
        self.blocks = nn.ModuleList([
            Block(embed_dim=embed_dim, mod_dim=mod_dim, num_blocks=num_blocks, mlp_ratio=mlp_ratio, drop=drop_rate,
                  norm_layer=norm_layer, sparsity_threshold=sparsity_threshold,
                  hard_thresholding_fraction=hard_thresholding_fraction, modulate_filter=modulate_filter,
                  modulate_mlp=modulate_mlp, scale_shift_mode=scale_shift_mode)
            for _ in range(depth)])
        self.head = nn.Linear(embed_dim, out_channels * patch_size[0] * patch_size[1], bias=False)
        torch.nn.init.trunc_normal_(self.pos_embed, std=0.02)
        self.apply(self._init_weights)
        self.mod_additive_proj = nn.Linear(mod_dim, embed_dim)
        if modulate_mlp or modulate_filter:
            self.mod_embed_net = ModEmbedNet(**(embed_model or {}))
        else:
            self.mod_embed_net = nn.Identity()

    @staticmethod
    def _init_weights(m: nn.Module) -> None:
        if isinstance(m, nn.Linear):
            torch.nn.init.trunc_normal_(m.weight, std=0.02)
            if m.bias is not None:
                nn.init.constant_(m.bias, 0)
        elif isinstance(m, nn.LayerNorm):
            nn.init.constant_(m.bias, 0)
            nn.init.constant_(m.weight, 1.0)

    def _forward_features(self, x: Tensor, mod: Tensor) -> Tensor:
        B = x.shape[0]
        tokens = self.pos_drop(self.patch_embed(x) + self.pos_embed)
        mod_embed = self.mod_embed_net(mod)
        tokens = tokens + self.mod_additive_proj(mod_embed).unsqueeze(1)
        tokens = tokens.reshape(B, self.h, self.w, self.embed_dim)
        for blk in self.blocks:
            tokens = blk(tokens, mod_embed=mod_embed)
        return tokens

    def forward(self, x: Tensor, mod: Tensor) -> Tensor:
        if not torch.compiler.is_compiling():
            want = (self.in_chans, self.inp_shape[0], self.inp_shape[1])
            if x.ndim != 4 or tuple(x.shape[1:]) != want:
                raise ValueError(f"ModAFNO takes (B, {want[0]}, {want[1]}, {want[2]}) inputs, received {tuple(x.shape)}")
        y = self.head(self._forward_features(x, mod))
        p0, p1 = self.patch_size
        return ops.unpatchify(y, self.h, self.w, p0, p1, y.shape[-1] // (p0 * p1))

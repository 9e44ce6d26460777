"""3-D transformer backbone for fields on (level, latitude, longitude) tiles.

Counterpart of ``physicsnemo/experimental/models/strata/transformer.py`` (``StrataTransformer3D`` :71): patch
embedding, a stack of pre-norm transformer blocks with global / neighbourhood / vertical-column attention and optional
rotary embedding (axial, or stereographic about the tile centroid from per-pixel latitude / longitude), and a linear
head that un-patchifies.  A deterministic field-to-field regressor: no noise or timestep conditioning.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Literal, Optional, Tuple, Union

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from ....core.meta import ModelMetaData
from ....core.module import Module
from ...nn.rope import build_axial_rope_cos_sin_2d_continuous
from .coords import build_axial_token_coords, build_stereographic_token_coords
from .layers import FinalLayer3D, PatchEmbed3D, RopeTables, StrataTransformer3DBlock

__all__ = ["StrataTransformer3D"]


@dataclass
class StrataTransformer3DMetaData(ModelMetaData):
    amp_gpu: bool = True
    bf16: bool = True


def checkpoint_ratio(value: Union[bool, float]) -> float:
    """``True`` / ``False`` or a fraction of the blocks (from the first) whose activations are recomputed."""
    if isinstance(value, bool):
        return 1.0 if value else 0.0
    if not isinstance(value, (int, float)):
        raise TypeError(f"activation_checkpointing must be bool or numeric, got {type(value).__name__}")
    if not 0.0 <= float(value) <= 1.0:
        raise ValueError(f"activation_checkpointing must be bool or a float in [0, 1], got {float(value)}")
    return float(value)


def init_linear_xavier(module: nn.Module) -> None:
    if isinstance(module, nn.Linear):
        nn.init.xavier_uniform_(module.weight)
        if module.bias is not None:
            nn.init.zeros_(module.bias)


def init_patch_embed(embed: PatchEmbed3D) -> None:
    w = embed.proj.weight.data
    nn.init.xavier_uniform_(w.view(w.shape[0], -1))
    nn.init.zeros_(embed.proj.bias)


class StrataTransformer3D(Module):
    __model_checkpoint_version__ = "1.0.0"

    def __init__(self, in_channels: int, out_channels: Optional[int] = None, input_shape: Tuple[int, int, int] = (16, 64, 64),
                 patch_size: Union[int, Tuple[int, int, int]] = 1, embed_dim: int = 768, num_heads: int = 8, num_layers: int = 12,
                 mlp_ratio: float = 4.0, qkv_bias: bool = True, qk_norm: bool = False, qk_norm_affine: bool = False,
                 attn_kernel: Union[int, Tuple[int, int, int]] = 3, na_dilation: int = 1, do_interleaved_dilation: bool = False,
                 do_alt_depthwise_attn: bool = False, gated_attention: bool = False, na3d_backend: Optional[str] = None,
                 rope_mode: Literal["none", "axial", "stereographic"] = "none", rope_base: float = 100.0,
                 rope_length_scale: float = 1.0, activation_checkpointing: Union[bool, float] = False, bf16_mixed: bool = False,
                 include_head: bool = True):
        super().__init__(meta=StrataTransformer3DMetaData())
        if embed_dim % num_heads != 0:
            raise ValueError(f"embed_dim ({embed_dim}) must be divisible by num_heads ({num_heads})")
        if rope_mode not in ("none", "axial", "stereographic"):
            raise ValueError(f"rope_mode must be 'none', 'axial', or 'stereographic'; got {rope_mode!r}")
        head_dim = embed_dim // num_heads
        if rope_mode != "none" and head_dim % 4 != 0:
            raise ValueError(f"RoPE requires head_dim (embed_dim // num_heads = {head_dim}) divisible by 4")
        patch_size = (patch_size,) * 3 if isinstance(patch_size, int) else tuple(patch_size)
        self.in_channels, self.out_channels = in_channels, (out_channels if out_channels is not None else in_channels)
        self.depth, self.height, self.width = self.input_shape = tuple(input_shape)
        self.patch_size, self.patch_size_vert, self.patch_size_horiz = patch_size, patch_size[0], patch_size[1]
        self.embed_dim, self.num_heads, self.num_layers, self.head_dim, self.mlp_ratio = embed_dim, num_heads, num_layers, head_dim, mlp_ratio
        self.attn_kernel, self.rope_mode, self.rope_base, self.rope_length_scale = attn_kernel, rope_mode, rope_base, rope_length_scale
        self.bf16_mixed = bf16_mixed
        self._activation_checkpointing_ratio = checkpoint_ratio(activation_checkpointing)
        self.patch_embed = PatchEmbed3D(self.depth, self.height, self.width, patch_size=patch_size, in_chans=in_channels, embed_dim=embed_dim)
        self.blocks = nn.ModuleList(
            StrataTransformer3DBlock(dim=embed_dim, num_heads=num_heads, mlp_ratio=mlp_ratio, qkv_bias=qkv_bias, qk_norm=qk_norm,
                                     qk_norm_affine=qk_norm_affine, attn_kernel=attn_kernel,
                                     do_depthwise_attention=(i % 2 == 1 and do_alt_depthwise_attn),
                                     na_dilation=(na_dilation if do_interleaved_dilation and i % 4 == 2 else 1),
                                     gated_attention=gated_attention, na3d_backend=na3d_backend) for i in range(num_layers))
        if rope_mode == "axial":
            self._set_axial_rope()
        self.final_layer = FinalLayer3D(embed_dim, patch_size[0] * patch_size[1] * patch_size[2] * self.out_channels) if include_head else None
        self.initialize_weights()

    _parse_checkpointing_param = staticmethod(checkpoint_ratio)

    def _set_axial_rope(self) -> None:
        pd, ph, pw = self.patch_size
        coords = build_axial_token_coords(self.depth // pd, self.height // ph, self.width // pw)
        cos, sin = build_axial_rope_cos_sin_2d_continuous(coords[:, 0], coords[:, 1], self.head_dim, theta=self.rope_base)
        device = self._rope_cos.device if hasattr(self, "_rope_cos") else None
        self.register_buffer("_rope_cos", cos.to(device), persistent=False)
        self.register_buffer("_rope_sin", sin.to(device), persistent=False)

    def _should_checkpoint_block(self, i: int) -> bool:
        r = self._activation_checkpointing_ratio
        return self.training and r > 0.0 and (r >= 1.0 or i < round(r * len(self.blocks)))

    def initialize_weights(self) -> None:
        self.apply(init_linear_xavier)
        init_patch_embed(self.patch_embed)
        if self.final_layer is not None:
            nn.init.zeros_(self.final_layer.linear.weight)
            nn.init.zeros_(self.final_layer.linear.bias)

    def set_tile_size(self, height: int, width: int) -> None:
        """Change the horizontal tile extent (the weights do not depend on it; axial rotary tables are rebuilt)."""
        for extent, p, what in ((height, self.patch_size[1], "Height"), (width, self.patch_size[2], "Width")):
            if extent % p != 0:
                raise ValueError(f"{what} ({extent}) must be divisible by horizontal patch size ({p})")
        self.height, self.width = height, width
        self.input_shape = (self.depth, height, width)
        if self.rope_mode == "axial":
            self._set_axial_rope()

    def _build_rope_tables(self, pos: Optional[torch.Tensor], latent_dhw) -> Optional[RopeTables]:
        if self.rope_mode == "none":
            return None
        if self.rope_mode == "axial":
            return self._rope_cos, self._rope_sin
        coords = build_stereographic_token_coords(pos, self.patch_size[1:], d_patch=latent_dhw[0], length_scale=self.rope_length_scale)
        cos, sin = build_axial_rope_cos_sin_2d_continuous(coords[..., 0], coords[..., 1], self.head_dim, theta=self.rope_base)
        return cos.unsqueeze(1), sin.unsqueeze(1)

    def forward_tokens(self, x: torch.Tensor, pos: Optional[torch.Tensor] = None):
        """Backbone features ``[B, tokens, embed_dim]`` and the token grid ``(d, h, w)``."""
        if not torch.compiler.is_compiling():
            if x.ndim != 5:
                raise ValueError(f"Expected 5D input (B, C, D, H, W), got tensor of shape {tuple(x.shape)}")
            if x.shape[1] != self.in_channels:
                raise ValueError(f"Expected {self.in_channels} input channels, got {x.shape[1]}")
            if tuple(x.shape[2:]) != self.input_shape:
                raise ValueError(f"Expected spatial shape {self.input_shape}, got {tuple(x.shape[2:])}")
            if self.rope_mode == "stereographic":
                if pos is None:
                    raise ValueError("pos (lat/lon of shape (B, 2, H, W)) is required when rope_mode='stereographic'")
                if tuple(pos.shape) != (x.shape[0], 2, x.shape[3], x.shape[4]):
                    raise ValueError(f"Expected pos of shape {(x.shape[0], 2, x.shape[3], x.shape[4])}, got {tuple(pos.shape)}")
        tok, dhw = self.patch_embed.tokens(x)
        rope = self._build_rope_tables(pos, dhw)
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=self.bf16_mixed and x.is_cuda):
            for i, blk in enumerate(self.blocks):
                r = None if blk.do_depthwise_attention else rope
                if self._should_checkpoint_block(i):
                    tok = checkpoint(lambda t, b=blk, r=r: b(t, latent_dhw=dhw, rope_tables=r), tok, use_reentrant=False)
                else:
                    tok = blk(tok, latent_dhw=dhw, rope_tables=r)
        return tok, dhw

    def _unpatchify(self, x: torch.Tensor, depth=None, height=None, width=None) -> torch.Tensor:
        pd, ph, pw = self.patch_size
        d, h, w = (depth or self.depth) // pd, (height or self.height) // ph, (width or self.width) // pw
        x = x.reshape(x.shape[0], d, h, w, pd, ph, pw, self.out_channels).permute(0, 7, 1, 4, 2, 5, 3, 6)
        return x.reshape(x.shape[0], self.out_channels, d * pd, h * ph, w * pw)

    def forward(self, x: torch.Tensor, pos: Optional[torch.Tensor] = None) -> torch.Tensor:
        tok, _ = self.forward_tokens(x, pos)
        return tok if self.final_layer is None else self._unpatchify(self.final_layer(tok))

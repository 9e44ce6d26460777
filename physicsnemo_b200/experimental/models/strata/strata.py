"""Two-stage Strata regressor: a patch-level transformer backbone conditions a pixel-resolution transformer.

Counterpart of ``physicsnemo/experimental/models/strata/strata.py`` (``Strata`` :77).  The backbone (a head-less
``StrataTransformer3D``) produces one feature vector per patch; the pixel stage embeds every grid point, runs
neighbourhood-attention blocks whose layer norms are modulated per pixel by those features, and projects to the
output channels.  Both stages are deterministic (no diffusion conditioning).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Literal, Optional, Tuple, Union

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from ....core.meta import ModelMetaData
from ....core.module import Module
from ...nn.rope import build_axial_rope_cos_sin_2d_continuous
from .coords import build_axial_token_coords, build_stereographic_token_coords
from .layers import FinalLayer3D, PatchEmbed3D, RopeTables, StrataPixel3DBlock, StrataTransformer3DBlock
from .transformer import StrataTransformer3D, checkpoint_ratio, init_linear_xavier, init_patch_embed

__all__ = ["Strata"]


@dataclass
class StrataMetaData(ModelMetaData):
    amp_gpu: bool = True
    bf16: bool = True


class Strata(Module):
    __model_checkpoint_version__ = "1.0.0"

    def __init__(self, backbone_config: Optional[Dict[str, Any]] = None, embed_dim_pixel: int = 128, num_layers_pixel: int = 4,
                 num_heads_pixel: Optional[int] = None, mlp_ratio_pixel: float = 4.0,
                 attn_kernel_pixel: Union[int, Tuple[int, int, int]] = 3, gated_attention_pixel: bool = False, qk_norm_pixel: bool = False,
                 qk_norm_affine_pixel: bool = False, na3d_backend_pixel: Optional[str] = None,
                 adaln_mode: Literal["pixel_proj", "bilinear_dw"] = "pixel_proj", first_block_only_adaln: bool = False,
                 use_chunked_depthwise_conv: bool = True, chunk_size_grouped_conv: int = 2,
                 rope_mode_pixel: Literal["none", "axial", "stereographic"] = "none", rope_base_pixel: float = 100.0,
                 rope_length_scale_pixel: float = 1.0, bf16_mixed_pixel: bool = False,
                 activation_checkpointing_pixel: Union[bool, float] = False):
        super().__init__(meta=StrataMetaData())
        self.backbone = StrataTransformer3D(**{**(backbone_config or {}), "include_head": False})
        bb = self.backbone
        num_heads_pixel = num_heads_pixel if num_heads_pixel is not None else max(1, embed_dim_pixel // 64)
        if embed_dim_pixel % num_heads_pixel != 0:
            raise ValueError(f"embed_dim_pixel ({embed_dim_pixel}) must be divisible by num_heads_pixel ({num_heads_pixel})")
        head_dim = embed_dim_pixel // num_heads_pixel
        if rope_mode_pixel not in ("none", "axial", "stereographic"):
            raise ValueError(f"rope_mode_pixel must be 'none', 'axial', or 'stereographic'; got {rope_mode_pixel!r}")
        if rope_mode_pixel != "none" and head_dim % 4 != 0:
            raise ValueError(f"Pixel RoPE requires head_dim_pixel (embed_dim_pixel // num_heads_pixel = {head_dim}) divisible by 4")
        if first_block_only_adaln and num_layers_pixel < 1:
            raise ValueError(f"first_block_only_adaln requires num_layers_pixel >= 1; got num_layers_pixel={num_layers_pixel}")
        self.in_channels, self.out_channels = bb.in_channels, bb.out_channels
        self.depth, self.height, self.width = bb.depth, bb.height, bb.width
        self.embed_dim_pixel, self.num_layers_pixel, self.num_heads_pixel, self.head_dim_pixel = embed_dim_pixel, num_layers_pixel, num_heads_pixel, head_dim
        self.adaln_mode, self.first_block_only_adaln = adaln_mode, first_block_only_adaln
        self.rope_mode_pixel, self.rope_base_pixel, self.rope_length_scale_pixel = rope_mode_pixel, rope_base_pixel, rope_length_scale_pixel
        self.bf16_mixed_pixel = bf16_mixed_pixel
        self._activation_checkpointing_ratio_pixel = checkpoint_ratio(activation_checkpointing_pixel)
        self.pixel_patch_embed = PatchEmbed3D(self.depth, self.height, self.width, patch_size=(1, 1, 1), in_chans=self.in_channels,
                                              embed_dim=embed_dim_pixel)
        shared = dict(dim=embed_dim_pixel, num_heads=num_heads_pixel, mlp_ratio=mlp_ratio_pixel, qk_norm=qk_norm_pixel,
                      qk_norm_affine=qk_norm_affine_pixel, attn_kernel=attn_kernel_pixel, gated_attention=gated_attention_pixel,
                      na3d_backend=na3d_backend_pixel)
        pd, ph, pw = bb.patch_size
        modulated = lambda: StrataPixel3DBlock(cond_dim=bb.embed_dim, pixels_per_patch=pd * ph * pw, adaln_mode=adaln_mode,  # noqa: E731
                                               use_chunked_depthwise_conv=use_chunked_depthwise_conv,
                                               chunk_size_grouped_conv=chunk_size_grouped_conv, **shared)
        n_mod = min(1, num_layers_pixel) if first_block_only_adaln else num_layers_pixel
        self.pixel_blocks = nn.ModuleList([modulated() for _ in range(n_mod)]
                                          + [StrataTransformer3DBlock(**shared) for _ in range(num_layers_pixel - n_mod)])
        self.pixel_final_layer = FinalLayer3D(embed_dim_pixel, self.out_channels)
        if rope_mode_pixel == "axial":
            coords = build_axial_token_coords(self.depth, self.height, self.width)
            cos, sin = build_axial_rope_cos_sin_2d_continuous(coords[:, 0], coords[:, 1], head_dim, theta=rope_base_pixel)
            self.register_buffer("_rope_cos_pixel", cos, persistent=False)
            self.register_buffer("_rope_sin_pixel", sin, persistent=False)
        self.initialize_weights()

    def initialize_weights(self) -> None:
        self.pixel_blocks.apply(init_linear_xavier)
        for blk in self.pixel_blocks:
            if isinstance(blk, StrataPixel3DBlock):
                blk.reset_adaln_zero()
        init_patch_embed(self.pixel_patch_embed)
        nn.init.zeros_(self.pixel_final_layer.linear.weight)
        nn.init.zeros_(self.pixel_final_layer.linear.bias)

    def _should_checkpoint_pixel_block(self, i: int) -> bool:
        r = self._activation_checkpointing_ratio_pixel
        return self.training and r > 0.0 and (r >= 1.0 or i < round(r * len(self.pixel_blocks)))

    def _build_pixel_rope_tables(self, pos: Optional[torch.Tensor]) -> Optional[RopeTables]:
        if self.rope_mode_pixel == "none":
            return None
        if self.rope_mode_pixel == "axial":
            return self._rope_cos_pixel, self._rope_sin_pixel
        coords = build_stereographic_token_coords(pos, (1, 1), d_patch=self.depth, length_scale=self.rope_length_scale_pixel)
        cos, sin = build_axial_rope_cos_sin_2d_continuous(coords[..., 0], coords[..., 1], self.head_dim_pixel, theta=self.rope_base_pixel)
        return cos.unsqueeze(1), sin.unsqueeze(1)

    def forward(self, x: torch.Tensor, pos: Optional[torch.Tensor] = None) -> torch.Tensor:
        if not torch.compiler.is_compiling():
            if x.ndim != 5:
                raise ValueError(f"Expected 5D input (B, C, D, H, W), got tensor of shape {tuple(x.shape)}")
            if self.rope_mode_pixel == "stereographic" and pos is None:
                raise ValueError("pos (lat/lon of shape (B, 2, H, W)) is required when rope_mode_pixel='stereographic'")
            if pos is not None and tuple(pos.shape) != (x.shape[0], 2, x.shape[3], x.shape[4]):
                raise ValueError(f"Expected pos of shape {(x.shape[0], 2, x.shape[3], x.shape[4])}, got {tuple(pos.shape)}")
        B, _, dd, hh, ww = x.shape
        cond, backbone_dhw = self.backbone.forward_tokens(x, pos)
        pixel_dhw = (dd, hh, ww)
        pix, _ = self.pixel_patch_embed.tokens(x)
        bilinear = None
        if any(isinstance(b, StrataPixel3DBlock) and b.adaln_mode == "bilinear_dw" for b in self.pixel_blocks):
            bilinear = StrataPixel3DBlock.precompute_bilinear_cond(cond, pixel_dhw, backbone_dhw)
        rope = self._build_pixel_rope_tables(pos)
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=self.bf16_mixed_pixel and x.is_cuda):
            for i, blk in enumerate(self.pixel_blocks):
                if isinstance(blk, StrataPixel3DBlock):
                    run = lambda t, c, s, b=blk: b(t, backbone_cond=c, pixel_dhw=pixel_dhw, backbone_dhw=backbone_dhw,  # noqa: E731
                                                   s_cond_bilinear=s, rope_tables=rope)
                    args = (pix, cond, bilinear)
                else:
                    run = lambda t, b=blk: b(t, latent_dhw=pixel_dhw, rope_tables=rope)  # noqa: E731
                    args = (pix,)
                pix = checkpoint(run, *args, use_reentrant=False) if self._should_checkpoint_pixel_block(i) else run(*args)
            pix = self.pixel_final_layer(pix)
        return pix.reshape(B, dd, hh, ww, -1).permute(0, 4, 1, 2, 3)

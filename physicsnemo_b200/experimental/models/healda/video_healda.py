"""VideoHealDA: space-time diffusion transformer on the HEALPix grid that reads point observations by cross attention.

Counterpart of ``physicsnemo/experimental/models/healda/video_healda.py`` (``VideoHealDA`` :52).  Observations are
tokenised by the FiLM tokenizer; every block of the ``VideoDiT`` lets each coarse ``(batch, time, pixel)`` site attend
to its own packed tokens (``ObsContext`` built on the coarse grid), followed by causal linear attention along time.
"""

from __future__ import annotations

from dataclasses import dataclass
from functools import partial
from typing import Literal, Optional

import torch

from ....core.meta import ModelMetaData
from ....core.module import Module
from ....nn.module.hpx.tokenizer import HEALPixPatchDetokenizer, HEALPixPatchTokenizer
from .attention_layers import PixelCrossAttention
from .obs_context import ObsContext
from .obs_tokenizer import ObsTokenizerFiLM
from .video_dit import VideoDiT

__all__ = ["VideoHealDA"]


@dataclass
class VideoHealDAMetaData(ModelMetaData):
    amp_gpu: bool = True
    bf16: bool = True


class VideoHealDA(Module):
    def __init__(self, in_channels: int = 2, out_channels: int = 74, hidden_size: int = 1536, num_layers: int = 32, num_heads: int = 16,
                 mlp_ratio: float = 4.0, level_in: int = 6, level_model: int = 5, time_length: int = 8, condition_embed_dim: int = 128,
                 noise_channels: int = 128, condition_dim: int = 0, temporal_attention: bool = True, is_causal: bool = True,
                 linear_attention: bool = True, use_rope: bool = True, rope_base: int = 100, max_seq_len: int = 100,
                 temporal_causal_window: Optional[int] = None, drop_path: float = 0.1, drop_path_zero_first_n_blocks: int = 4,
                 qk_norm_type: Optional[Literal["RMSNorm", "LayerNorm"]] = "RMSNorm", qk_norm_affine: bool = False,
                 attention_backend: str = "timm", layernorm_backend: str = "torch", obs_token_dim: int = 32, obs_meta_dim: int = 50,
                 obs_type_embed_dim: int = 4, channel_embed_dim: int = 16, platform_embed_dim: int = 8, obs_film_hidden_dim: int = 64,
                 use_fused_obs_mlp: bool = True, pixel_attn_n_q_heads: int = 64, pixel_attn_n_kv_heads: int = 2, pixel_attn_head_dim: int = 32,
                 pixel_attn_use_proj_bias: bool = True):
        super().__init__(meta=VideoHealDAMetaData())
        self.in_channels, self.out_channels, self.hidden_size = in_channels, out_channels, hidden_size
        self.level_in, self.level_model, self.time_length, self.condition_dim = level_in, level_model, time_length, condition_dim
        self.npix = 12 * 4 ** level_in
        self.obs_tokenizer = ObsTokenizerFiLM(meta_dim=obs_meta_dim, out_dim=obs_token_dim, obs_type_embed_dim=obs_type_embed_dim,
                                              channel_embed_dim=channel_embed_dim, platform_embed_dim=platform_embed_dim,
                                              hidden_dim=obs_film_hidden_dim, use_fused_mlp=use_fused_obs_mlp)
        cross = partial(PixelCrossAttention, hidden_size=hidden_size, token_dim=obs_token_dim, n_q_heads=pixel_attn_n_q_heads,
                        n_kv_heads=pixel_attn_n_kv_heads, d_head=pixel_attn_head_dim, use_proj_bias=pixel_attn_use_proj_bias)
        attn_kwargs = {"qk_norm_type": qk_norm_type, "qk_norm_affine": qk_norm_affine} if qk_norm_type else {}
        n_zero = min(drop_path_zero_first_n_blocks, num_layers)
        tokenizer = HEALPixPatchTokenizer(in_channels=in_channels, hidden_size=hidden_size, level_fine=level_in, level_coarse=level_model,
                                          separate_time_axis=True)
        detokenizer = HEALPixPatchDetokenizer(hidden_size=hidden_size, out_channels=out_channels, level_coarse=level_model, level_fine=level_in,
                                              time_length=time_length, condition_dim=condition_embed_dim)
        self.dit = VideoDiT(tokenizer, detokenizer, hidden_size=hidden_size, num_heads=num_heads, num_layers=num_layers,
                            emb_channels=condition_embed_dim, noise_channels=noise_channels, condition_dim=condition_dim,
                            temporal_attention=temporal_attention, use_rope=use_rope, rope_base=rope_base, max_seq_len=max_seq_len,
                            temporal_kwargs={"linear_attention": linear_attention, "causal_window": temporal_causal_window},
                            cross_attention=cross, is_causal=is_causal, attention_backend=attention_backend, layernorm_backend=layernorm_backend,
                            mlp_ratio=mlp_ratio, drop_path_rates=[0.0] * n_zero + [drop_path] * (num_layers - n_zero),
                            conditioning_embedder="edm", attn_kwargs=attn_kwargs)

    def set_context_parallel(self, mode: Optional[str], target=None) -> None:
        self.dit.set_context_parallel(mode, target)

    def forward(self, x: torch.Tensor, t: torch.Tensor, second_of_day: torch.Tensor, day_of_year: torch.Tensor, obs_ctx: ObsContext,
                class_labels: Optional[torch.Tensor] = None) -> torch.Tensor:
        if not torch.compiler.is_compiling():
            if x.ndim != 4:
                raise ValueError(f"Expected 4D input (B, C, T, X), got {x.ndim}D tensor with shape {tuple(x.shape)}")
            b, c, tl, xd = x.shape
            if c != self.in_channels:
                raise ValueError(f"Expected {self.in_channels} input channels, got {c} channels")
            if tl != self.time_length:
                raise ValueError(f"Expected time_length {self.time_length}, got {tl} frames")
            if xd != self.npix:
                raise ValueError(f"Expected npix {self.npix}, got {xd} pixels")
            if t.ndim != 1 or t.shape[0] != b:
                raise ValueError(f"Expected t of shape ({b},), got tensor with shape {tuple(t.shape)}")
            if tuple(second_of_day.shape) != (b, tl) or tuple(day_of_year.shape) != (b, tl):
                raise ValueError(f"Expected calendar tensors of shape ({b}, {tl}), got second_of_day {tuple(second_of_day.shape)} and "
                                 f"day_of_year {tuple(day_of_year.shape)}")
            want = b * tl * 12 * 4 ** self.level_model + 1
            if obs_ctx.cu_seqlens_k.numel() != want:
                raise ValueError(f"Expected cu_seqlens_k length {want} (B*T*npix_model+1), got {obs_ctx.cu_seqlens_k.numel()}")
            if self.condition_dim > 0:
                if class_labels is None:
                    raise ValueError(f"condition_dim={self.condition_dim} but class_labels was not provided")
                if tuple(class_labels.shape) != (b, self.condition_dim):
                    raise ValueError(f"Expected class_labels of shape ({b}, {self.condition_dim}), got tensor with shape "
                                     f"{tuple(class_labels.shape)}")
            elif class_labels is not None:
                raise ValueError("class_labels was provided but condition_dim=0 (noise-only conditioning)")
        tokens = self.obs_tokenizer(obs_ctx.obs, obs_ctx.float_metadata, obs_ctx.obs_type, obs_ctx.channel, obs_ctx.platform)
        cross = {"tokens": tokens, "cu_seqlens_k": obs_ctx.cu_seqlens_k, "max_seqlen_k": obs_ctx.max_seqlen_k, "group_map": obs_ctx.group_map}
        return self.dit(x, t, condition=class_labels, cross_attn_kwargs=cross,
                        tokenizer_kwargs={"second_of_day": second_of_day, "day_of_year": day_of_year})

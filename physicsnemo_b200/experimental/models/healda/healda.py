"""HealDA (first generation): diffusion transformer on the HEALPix grid conditioned on embedded point observations.

Counterpart of ``physicsnemo/experimental/models/healda/healda.py`` (``HealDA`` :57).  The multi-sensor embedder turns
the flat observation arrays into ``fusion_dim`` extra input channels on the fine HEALPix grid; a DiT with HEALPix patch
tokenizer / detokenizer (patches are the ``4**(level_in - level_model)`` children of a coarse pixel) maps the
concatenated state to the output channels, with EDM noise conditioning unless ``diffusion_conditioning=False``.
"""

from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import List, Literal, Optional

import torch

from ....core.meta import ModelMetaData
from ....core.module import Module
from ....models.dit import DiT
from .point_embed import MultiSensorObsEmbedder

__all__ = ["HealDA"]


@dataclass
class HealDAMetaData(ModelMetaData):
    amp_gpu: bool = True
    bf16: bool = True


class HealDA(Module):
    def __init__(self, in_channels: int, out_channels: int, nchannel_per_sensor: List[int], nplatform_per_sensor: List[int],
                 sensor_names: Optional[List[str]] = None, hidden_size: int = 1024, num_layers: int = 24, num_heads: int = 16,
                 mlp_ratio: float = 4.0, level_in: int = 6, level_model: int = 5, time_length: int = 1, embed_dim: int = 32,
                 meta_dim: int = 28, fusion_dim: int = 512, obs_gradient_checkpointing: bool = False, compile_obs_embedder: bool = False,
                 qk_norm_type: Optional[Literal["RMSNorm", "LayerNorm"]] = "RMSNorm", qk_norm_affine: bool = False, drop_path: float = 0.0,
                 dropout: float = 0.0, diffusion_conditioning: bool = True, condition_dim: int = 0,
                 condition_embed_dim: Optional[int] = None, noise_channels: Optional[int] = None, legacy_condition_bias: bool = True,
                 condition_dropout: float = 0.0, norm_eps: float = 1e-5, attention_backend: str = "timm", layernorm_backend: str = "torch"):
        warnings.warn("HealDA (v1) is deprecated and will be removed in a future release. Use VideoHealDA instead.", DeprecationWarning,
                      stacklevel=2)
        super().__init__(meta=HealDAMetaData())
        self.in_channels, self.out_channels, self.hidden_size = in_channels, out_channels, hidden_size
        self.level_in, self.level_model, self.time_length = level_in, level_model, time_length
        self.diffusion_conditioning, self.condition_dim, self.fusion_dim = diffusion_conditioning, condition_dim, fusion_dim
        self.qk_norm_type, self.qk_norm_affine, self.attention_backend = qk_norm_type, qk_norm_affine, attention_backend
        self.npix = 12 * 4 ** level_in
        self.obs_embedder = MultiSensorObsEmbedder(nchannel_per_sensor=nchannel_per_sensor, nplatform_per_sensor=nplatform_per_sensor,
                                                   sensor_names=sensor_names, embed_dim=embed_dim, meta_dim=meta_dim, fusion_dim=fusion_dim,
                                                   gradient_checkpointing=obs_gradient_checkpointing, torch_compile=compile_obs_embedder)
        attn_kwargs = {"qk_norm_type": qk_norm_type, "qk_norm_affine": qk_norm_affine} if qk_norm_type else {}
        if attention_backend == "transformer_engine":
            attn_kwargs["qkv_format"] = "bshd"
        if diffusion_conditioning:
            condition_embed_dim = 4 * hidden_size if condition_embed_dim is None else condition_embed_dim
            embedder, embedder_kwargs = "edm", {"emb_channels": condition_embed_dim,
                                                "noise_channels": hidden_size if noise_channels is None else noise_channels,
                                                "condition_dropout": condition_dropout, "legacy_condition_bias": legacy_condition_bias}
        else:
            condition_embed_dim, embedder, embedder_kwargs = 0, "zero", {}
        patch = 2 ** (level_in - level_model)
        self.dit = DiT(input_size=(12 * 4 ** level_model * time_length,), in_channels=in_channels + fusion_dim, patch_size=(patch, patch),
                       tokenizer="hpx_patch_embed", detokenizer="hpx_patch_detokenizer", out_channels=out_channels, hidden_size=hidden_size,
                       depth=num_layers, num_heads=num_heads, mlp_ratio=mlp_ratio, attention_backend=attention_backend,
                       layernorm_backend=layernorm_backend, condition_dim=condition_dim, conditioning_embedder=embedder,
                       conditioning_embedder_kwargs=embedder_kwargs,
                       drop_path_rates=[drop_path * i / max(1, num_layers - 1) for i in range(num_layers)], attn_kwargs=attn_kwargs,
                       block_kwargs={"proj_drop_rate": dropout, "mlp_drop_rate": dropout, "norm_eps": norm_eps, "final_mlp_dropout": False},
                       tokenizer_kwargs={"level_fine": level_in, "level_coarse": level_model},
                       detokenizer_kwargs={"level_coarse": level_model, "level_fine": level_in, "time_length": time_length,
                                           "condition_dim": condition_embed_dim})

    def forward(self, x: torch.Tensor, t: torch.Tensor, obs: torch.Tensor, float_metadata: torch.Tensor, pix: torch.Tensor,
                local_channel: torch.Tensor, local_platform: torch.Tensor, obs_type: torch.Tensor, offsets: torch.Tensor,
                second_of_day: torch.Tensor, day_of_year: torch.Tensor, class_labels: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x`` ``[B, C_in, T, npix]`` -> ``[B, C_out, T, npix]``; the observation arguments are those of ``MultiSensorObsEmbedder``."""
        obs_channels = self.obs_embedder(obs=obs, float_metadata=float_metadata, pix=pix, local_channel=local_channel,
                                         local_platform=local_platform, obs_type=obs_type, offsets=offsets, npix=self.npix)
        return self.dit(torch.cat([x, obs_channels], dim=1), t, condition=class_labels,
                        tokenizer_kwargs={"second_of_day": second_of_day, "day_of_year": day_of_year})

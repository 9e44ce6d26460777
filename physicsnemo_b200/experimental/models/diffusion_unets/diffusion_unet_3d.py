"""Volumetric diffusion U-Net (DDPM++ / NCSN++ style encoder-decoder on ``[B, C, D, H, W]``).

Counterpart of ``physicsnemo/experimental/models/diffusion_unets/diffusion_unet_3d.py:54`` (``DiffusionUNet3D``);
module names inside ``enc`` / ``dec`` are the same, so reference state dicts load strictly.  The network is described
once as an ordered plan of named steps (built in ``__init__``), and ``forward`` interprets that plan; activation
checkpointing is decided per step from the largest spatial extent of its input.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Literal, Mapping, Optional

import numpy as np
import torch
from torch.nn.functional import silu
from torch.utils.checkpoint import checkpoint

from ....core.meta import ModelMetaData
from ....core.module import Module
from ....nn.module.embedding_layers import FourierEmbedding, PositionalEmbedding
from ....nn.module.fully_connected_layers import Linear
from ...nn.diffusion_unet_3d_blocks import Conv3D, GroupNorm3D, UNetBlock3D

__all__ = ["DiffusionUNet3D"]


@dataclass
class MetaData(ModelMetaData):
    amp_gpu: bool = True
    bf16: bool = True


class DiffusionUNet3D(Module):
    """Noise-conditioned 3-D U-Net ``(x, t, condition) -> x``.

    ``condition`` is an optional mapping with the keys ``"vector"`` ``[B, vec_cond_dim]`` (added to the noise
    embedding) and ``"volume"`` ``[B, vol_cond_channels, D, H, W]`` (concatenated to the input channels).
    Spatial sizes must be multiples of ``2**(num_levels-1)`` or smaller powers of two.
    """

    def __init__(self, x_channels: int, vol_cond_channels: int = 0, vec_cond_dim: int = 0, num_levels: int = 4,
                 model_channels: int = 128, channel_mult: List[int] = [1, 2, 2, 2], channel_mult_emb: int = 4,
                 num_blocks: int = 4, attention_levels: List[int] = [], dropout: float = 0.1,
                 embedding_type: Literal["fourier", "positional", "zero"] = "positional", channel_mult_noise: int = 1,
                 encoder_type: Literal["standard", "skip", "residual"] = "standard",
                 decoder_type: Literal["standard", "skip"] = "standard", resample_filter: List[int] = [1, 1],
                 checkpoint_level: int = 0, bottleneck_attention: bool = True,
                 activation: Literal["silu", "gelu"] = "silu"):
        if len(channel_mult) != num_levels:
            raise ValueError(f"len(channel_mult) must equal num_levels, got len(channel_mult)={len(channel_mult)} and "
                             f"num_levels={num_levels}")
        if any(not 0 <= lvl < num_levels for lvl in attention_levels):
            raise ValueError(f"All values in attention_levels must be in [0, num_levels={num_levels}), got {attention_levels}")
        if embedding_type == "zero" and vec_cond_dim > 0:
            raise ValueError("embedding_type='zero' disables the conditioning embedding; vec_cond_dim must be 0 in that "
                             f"case (got vec_cond_dim={vec_cond_dim}).")
        super().__init__(meta=MetaData())
        self.x_channels, self.vol_cond_channels, self.vec_cond_dim = x_channels, vol_cond_channels, vec_cond_dim
        self.embedding_type, self.num_levels, self.checkpoint_level = embedding_type, num_levels, checkpoint_level
        self._input_shape_mult = 2 ** (num_levels - 1)
        emb_channels = self.emb_channels = model_channels * channel_mult_emb
        noise_channels = model_channels * channel_mult_noise
        init = dict(init_mode="xavier_uniform")
        init_zero = dict(init_mode="xavier_uniform", init_weight=1e-5)
        init_attn = dict(init_mode="xavier_uniform", init_weight=np.sqrt(0.2))
        block = dict(emb_channels=emb_channels, num_heads=1, dropout=dropout, skip_scale=np.sqrt(0.5), eps=1e-6,
                     resample_filter=resample_filter, resample_proj=True, adaptive_scale=False, activation=activation,
                     init=init, init_zero=init_zero, init_attn=init_attn)

        if embedding_type != "zero":
            self.map_noise = (PositionalEmbedding(num_channels=noise_channels, endpoint=True) if embedding_type == "positional"
                              else FourierEmbedding(num_channels=noise_channels))
            self.map_condition = Linear(vec_cond_dim, noise_channels, **init) if vec_cond_dim > 0 else None
            self.map_layer0 = Linear(noise_channels, emb_channels, **init)
            self.map_layer1 = Linear(emb_channels, emb_channels, **init)
        else:
            self.register_buffer("zero_emb", torch.zeros(1, emb_channels), persistent=False)
            self.map_condition = None

        # ---- encoder ---------------------------------------------------------------------------------------
        self.enc = torch.nn.ModuleDict()
        cin0 = x_channels + vol_cond_channels
        cout, caux = cin0, cin0
        for level, mult in enumerate(channel_mult):
            if level == 0:
                self.enc["l0_conv"] = Conv3D(cout, model_channels, kernel=3, **init)
                cout = model_channels
            else:
                self.enc[f"l{level}_down"] = UNetBlock3D(cout, cout, down=True, **block)
                if encoder_type == "skip":
                    self.enc[f"l{level}_aux_down"] = Conv3D(caux, caux, kernel=0, down=True, resample_filter=resample_filter)
                    self.enc[f"l{level}_aux_skip"] = Conv3D(caux, cout, kernel=1, **init)
                elif encoder_type == "residual":
                    self.enc[f"l{level}_aux_residual"] = Conv3D(caux, cout, kernel=3, down=True,
                                                                resample_filter=resample_filter, **init)
                    caux = cout
            for idx in range(num_blocks):
                cin, cout = cout, model_channels * mult
                self.enc[f"l{level}_block{idx}"] = UNetBlock3D(cin, cout, attention=level in attention_levels, **block)
        skips = [m.out_channels for name, m in self.enc.items() if "aux" not in name]

        # ---- decoder ---------------------------------------------------------------------------------------
        self.dec = torch.nn.ModuleDict()
        top = num_levels - 1
        for level in range(top, -1, -1):
            mult = channel_mult[level]
            if level == top:
                self.dec[f"l{level}_in0"] = UNetBlock3D(cout, cout, attention=bottleneck_attention, **block)
                self.dec[f"l{level}_in1"] = UNetBlock3D(cout, cout, **block)
            else:
                self.dec[f"l{level}_up"] = UNetBlock3D(cout, cout, up=True, **block)
            for idx in range(num_blocks + 1):
                cin, cout = cout + skips.pop(), model_channels * mult
                self.dec[f"l{level}_block{idx}"] = UNetBlock3D(cin, cout, attention=(idx == num_blocks and level in attention_levels),
                                                               **block)
            if decoder_type == "skip" or level == 0:
                if decoder_type == "skip" and level < top:
                    self.dec[f"l{level}_aux_up"] = Conv3D(x_channels, x_channels, kernel=0, up=True, resample_filter=resample_filter)
                self.dec[f"l{level}_aux_norm"] = GroupNorm3D(num_channels=cout, eps=1e-6)
                self.dec[f"l{level}_aux_conv"] = Conv3D(cout, x_channels, kernel=3, **init_zero)

    # ------------------------------------------------------------------------------------------------------------
    def _validate(self, x, t, vector, volume, keys):
        if x.ndim != 5:
            raise ValueError(f"Expected x to be a 5D tensor, got {x.ndim}D tensor with shape {tuple(x.shape)}")
        B, C, D, H, W = x.shape
        if C != self.x_channels:
            raise ValueError(f"Expected x to have {self.x_channels} channels (x_channels), got {C}")
        m = self._input_shape_mult
        for d in (D, H, W):
            pow2 = d > 0 and d & (d - 1) == 0
            if not ((pow2 and d < m) or d % m == 0):
                raise ValueError(f"Input spatial dimensions (D, H, W)={(D, H, W)} must be powers of 2 or multiples of "
                                 f"2**(num_levels-1)={m}")
        if t.shape != (B,):
            raise ValueError(f"Expected t to have shape ({B},), got {tuple(t.shape)}")
        extra = set(keys) - {"vector", "volume"}
        if extra:
            raise ValueError(f"Unexpected condition keys: {extra}. Allowed keys: {{'vector', 'volume'}}")
        if vector is not None:
            if self.embedding_type == "zero":
                raise ValueError("condition['vector'] cannot be used with embedding_type='zero'.")
            if self.vec_cond_dim == 0:
                raise ValueError("condition['vector'] provided but vec_cond_dim=0")
            if vector.shape != (B, self.vec_cond_dim):
                raise ValueError(f"Expected condition['vector'] to have shape {(B, self.vec_cond_dim)}, got {tuple(vector.shape)}")
        if volume is not None:
            if self.vol_cond_channels == 0:
                raise ValueError("condition['volume'] provided but vol_cond_channels=0")
            if volume.shape != (B, self.vol_cond_channels, D, H, W):
                raise ValueError(f"Expected condition['volume'] to have shape {(B, self.vol_cond_channels, D, H, W)}, "
                                 f"got {tuple(volume.shape)}")

    def _embedding(self, t: torch.Tensor, vector: Optional[torch.Tensor]) -> torch.Tensor:
        if self.embedding_type == "zero":
            return self.zero_emb.expand(t.shape[0], -1)
        emb = self.map_noise(t)
        half = emb.shape[1] // 2
        emb = torch.cat([emb[:, half:], emb[:, :half]], dim=1)            # [cos, sin] -> [sin, cos]
        if self.map_condition is not None and vector is not None:
            emb = emb + self.map_condition(vector * np.sqrt(self.map_condition.in_features))
        return silu(self.map_layer1(silu(self.map_layer0(emb))))

    def forward(self, x: torch.Tensor, t: torch.Tensor, condition: Optional[Mapping[str, torch.Tensor]] = None) -> torch.Tensor:
        vector = condition.get("vector", None) if condition is not None else None
        volume = condition.get("volume", None) if condition is not None else None
        if not torch.compiler.is_compiling():
            self._validate(x, t, vector, volume, condition.keys() if condition is not None else ())
        if volume is not None:
            x = torch.cat([x, volume], dim=1)
        emb = self._embedding(t, vector)

        def extent(v):
            return max(v.shape[-3:])

        threshold = (extent(x) >> self.checkpoint_level) + 1
        run = lambda blk, v, big: checkpoint(blk, v, emb, use_reentrant=False) if big else blk(v, emb)  # noqa: E731

        skips, aux = [], x
        for name, blk in self.enc.items():
            if "aux_down" in name:
                aux = blk(aux)
            elif "aux_skip" in name:
                x = skips[-1] = x + blk(aux)
            elif "aux_residual" in name:
                x = skips[-1] = aux = (x + blk(aux)) / np.sqrt(2)
            elif name.endswith("_conv"):
                x = blk(x)
                skips.append(x)
            else:
                x = run(blk, x, extent(x) > threshold)
                skips.append(x)

        out, tmp = None, None
        for name, blk in self.dec.items():
            if "aux_up" in name:
                out = blk(out)
            elif "aux_norm" in name:
                tmp = blk(x)
            elif "aux_conv" in name:
                tmp = blk(silu(tmp))
                out = tmp if out is None else tmp + out
            else:
                if x.shape[1] != blk.in_channels:
                    x = torch.cat([x, skips.pop()], dim=1)
                e = extent(x)
                x = run(blk, x, (e > threshold and "_block" in name) or (e > threshold / 2 and "_up" in name))
        return out

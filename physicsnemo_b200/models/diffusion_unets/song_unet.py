"""SongUNet (DDPM++ / NCSN++ U-Net of the EDM family) and its positional-embedding variants.

Parity: ``physicsnemo/models/diffusion_unets/song_unet.py`` — ``SongUNet`` (``:65-703``),
``SongUNetPosEmbd`` (``:711-1412``), ``SongUNetPosLtEmbd`` (``:1415-``).  Constructor arguments,
module-dict key scheme (``enc["{res}x{res}_conv|_down|_block{i}|_aux_*"]``,
``dec["{res}x{res}_in0|_in1|_up|_block{i}|_aux_up|_aux_norm|_aux_conv"]``) and therefore the
state-dict keys are the reference's.  Activation checkpointing above the resolution
threshold follows ``:351-354, 659-666, 691-702``.
"""
from __future__ import annotations

import math
import warnings
from dataclasses import dataclass
from typing import Callable, List, Literal, Set, Union

import numpy as np
import torch
from torch.nn.functional import silu
from torch.utils.checkpoint import checkpoint

from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.conv_layers import Conv2d
from ...nn.module.embedding_layers import FourierEmbedding, PositionalEmbedding
from ...nn.module.fully_connected_layers import Linear
from ...nn.module.group_norm import get_group_norm
from ...nn.module.unet_layers import UNetBlock
from ...nn.module.utils.utils import _recursive_property


@dataclass
class MetaData(ModelMetaData):
    jit: bool = False
    cuda_graphs: bool = False
    amp_cpu: bool = False
    amp_gpu: bool = True
    torch_fx: bool = False
    bf16: bool = True
    onnx: bool = False
    func_torch: bool = False
    auto_grad: bool = False


class SongUNet(Module):
    """U-Net backbone of score-based / EDM diffusion models and of regression U-Nets.

    Forward: ``x`` (B, C_in, H, W), ``noise_labels`` (B,) or (1,), optional ``class_labels``
    (B, label_dim) and ``augment_labels`` (B, augment_dim) → (B, C_out, H, W).
    """

    _overridable_args: Set[str] = {"use_apex_gn", "act"}

    def __init__(self, img_resolution: Union[List[int], int], in_channels: int, out_channels: int,
                 label_dim: int = 0, augment_dim: int = 0, model_channels: int = 128,
                 channel_mult: List[int] = [1, 2, 2, 2], channel_mult_emb: int = 4, num_blocks: int = 4,
                 attn_resolutions: List[int] = [16], dropout: float = 0.10, label_dropout: float = 0.0,
                 embedding_type: Literal["fourier", "positional", "zero"] = "positional", channel_mult_noise: int = 1,
                 encoder_type: Literal["standard", "skip", "residual"] = "standard",
                 decoder_type: Literal["standard", "skip"] = "standard", resample_filter: List[int] = [1, 1],
                 checkpoint_level: int = 0, additive_pos_embed: bool = False, bottleneck_attention: bool = True,
                 use_apex_gn: bool = False, act: str = "silu", profile_mode: bool = False, amp_mode: bool = False):
        for value, valid, what in ((embedding_type, ["fourier", "positional", "zero"], "embedding_type"),
                                   (encoder_type, ["standard", "skip", "residual"], "encoder_type"),
                                   (decoder_type, ["standard", "skip"], "decoder_type")):
            if value not in valid:
                raise ValueError(f"Invalid {what}: {value}. Must be one of {valid}.")
        super().__init__(meta=MetaData())
        self.label_dim, self.augment_dim, self.label_dropout = label_dim, augment_dim, label_dropout
        self.embedding_type = embedding_type
        emb_channels = model_channels * channel_mult_emb
        self.emb_channels = emb_channels
        noise_channels = model_channels * channel_mult_noise
        init = dict(init_mode="xavier_uniform")
        init_zero = dict(init_mode="xavier_uniform", init_weight=1e-5)
        init_attn = dict(init_mode="xavier_uniform", init_weight=np.sqrt(0.2))
        block_kwargs = dict(emb_channels=emb_channels, num_heads=1, dropout=dropout, skip_scale=0.7071067811865476,
                            eps=1e-6, resample_filter=resample_filter, resample_proj=True, adaptive_scale=False,
                            init=init, init_zero=init_zero, init_attn=init_attn, use_apex_gn=use_apex_gn, act=act,
                            fused_conv_bias=True, profile_mode=profile_mode, amp_mode=amp_mode)
        self.use_apex_gn = use_apex_gn
        self.img_resolution = img_resolution
        if isinstance(img_resolution, int):
            self.img_shape_y = self.img_shape_x = img_resolution
        else:
            self.img_shape_y, self.img_shape_x = img_resolution[0], img_resolution[1]
        self._num_levels = len(channel_mult)
        self._input_shape_mult = 2 ** (self._num_levels - 1)
        self.checkpoint_threshold = (math.floor(math.sqrt(self.img_shape_x * self.img_shape_y)) >> checkpoint_level) + 1
        self.additive_pos_embed = additive_pos_embed
        if additive_pos_embed:
            self.spatial_emb = torch.nn.Parameter(torch.randn(1, model_channels, self.img_shape_y, self.img_shape_x))
            torch.nn.init.trunc_normal_(self.spatial_emb, std=0.02)

        if embedding_type != "zero":
            self.map_noise = (PositionalEmbedding(num_channels=noise_channels, endpoint=True, amp_mode=amp_mode)
                              if embedding_type == "positional"
                              else FourierEmbedding(num_channels=noise_channels, amp_mode=amp_mode))
            self.map_label = Linear(in_features=label_dim, out_features=noise_channels, amp_mode=amp_mode, **init) if label_dim else None
            self.map_augment = Linear(in_features=augment_dim, out_features=noise_channels, bias=False, amp_mode=amp_mode, **init) if augment_dim else None
            self.map_layer0 = Linear(in_features=noise_channels, out_features=emb_channels, amp_mode=amp_mode, **init)
            self.map_layer1 = Linear(in_features=emb_channels, out_features=emb_channels, amp_mode=amp_mode, **init)
        else:
            self.register_buffer("zero_emb", torch.zeros(1, emb_channels), persistent=False)

        # ---- encoder
        self.enc = torch.nn.ModuleDict()
        cout = caux = in_channels
        for level, mult in enumerate(channel_mult):
            res = self.img_shape_y >> level
            if level == 0:
                cin, cout = cout, model_channels
                self.enc[f"{res}x{res}_conv"] = Conv2d(in_channels=cin, out_channels=cout, kernel=3,
                                                       fused_conv_bias=True, amp_mode=amp_mode, **init)
            else:
                self.enc[f"{res}x{res}_down"] = UNetBlock(in_channels=cout, out_channels=cout, down=True, **block_kwargs)
                if encoder_type == "skip":
                    self.enc[f"{res}x{res}_aux_down"] = Conv2d(in_channels=caux, out_channels=caux, kernel=0, down=True,
                                                               resample_filter=resample_filter, amp_mode=amp_mode)
                    self.enc[f"{res}x{res}_aux_skip"] = Conv2d(in_channels=caux, out_channels=cout, kernel=1,
                                                               fused_conv_bias=True, amp_mode=amp_mode, **init)
                if encoder_type == "residual":
                    self.enc[f"{res}x{res}_aux_residual"] = Conv2d(in_channels=caux, out_channels=cout, kernel=3,
                                                                   down=True, resample_filter=resample_filter,
                                                                   fused_resample=True, fused_conv_bias=True,
                                                                   amp_mode=amp_mode, **init)
                    caux = cout
            for idx in range(num_blocks):
                cin, cout = cout, model_channels * mult
                self.enc[f"{res}x{res}_block{idx}"] = UNetBlock(in_channels=cin, out_channels=cout,
                                                                attention=res in attn_resolutions, **block_kwargs)
        skips = [block.out_channels for name, block in self.enc.items() if "aux" not in name]

        # ---- decoder
        self.dec = torch.nn.ModuleDict()
        for level, mult in reversed(list(enumerate(channel_mult))):
            res = self.img_shape_y >> level
            if level == len(channel_mult) - 1:
                self.dec[f"{res}x{res}_in0"] = UNetBlock(in_channels=cout, out_channels=cout,
                                                         attention=bottleneck_attention, **block_kwargs)
                self.dec[f"{res}x{res}_in1"] = UNetBlock(in_channels=cout, out_channels=cout, **block_kwargs)
            else:
                self.dec[f"{res}x{res}_up"] = UNetBlock(in_channels=cout, out_channels=cout, up=True, **block_kwargs)
            for idx in range(num_blocks + 1):
                cin = cout + skips.pop()
                cout = model_channels * mult
                attn = idx == num_blocks and res in attn_resolutions
                self.dec[f"{res}x{res}_block{idx}"] = UNetBlock(in_channels=cin, out_channels=cout, attention=attn,
                                                                **block_kwargs)
            if decoder_type == "skip" or level == 0:
                if decoder_type == "skip" and level < len(channel_mult) - 1:
                    self.dec[f"{res}x{res}_aux_up"] = Conv2d(in_channels=out_channels, out_channels=out_channels,
                                                             kernel=0, up=True, resample_filter=resample_filter,
                                                             amp_mode=amp_mode)
                self.dec[f"{res}x{res}_aux_norm"] = get_group_norm(num_channels=cout, eps=1e-6,
                                                                   use_apex_gn=use_apex_gn, amp_mode=amp_mode)
                self.dec[f"{res}x{res}_aux_conv"] = Conv2d(in_channels=cout, out_channels=out_channels, kernel=3,
                                                           fused_conv_bias=True, amp_mode=amp_mode, **init_zero)
        self.profile_mode = profile_mode
        self.amp_mode = amp_mode

    profile_mode = _recursive_property("profile_mode", bool, "Should be set to ``True`` to enable profiling.")
    amp_mode = _recursive_property("amp_mode", bool, "Should be set to ``True`` to enable automatic mixed precision.")

    # ------------------------------------------------------------------ pieces
    def _validate(self, x, noise_labels, class_labels, augment_labels):
        b = x.shape[0]
        if x.ndim != 4:
            raise ValueError(f"Expected 'x' to be a 4D tensor, got {x.ndim}D tensor with shape {tuple(x.shape)}")
        for d in x.shape[-2:]:
            pow2 = (d & (d - 1)) == 0 and d > 0
            if not ((pow2 and d < self._input_shape_mult) or (d % self._input_shape_mult == 0)):
                raise ValueError(
                    f"Input spatial dimensions ({x.shape[-2:]}) must be either powers of 2 or multiples of 2**(N-1) "
                    f"where N (={self._num_levels}) is the number of levels in the U-Net."
                )
        if noise_labels.ndim != 1 or noise_labels.shape[0] not in (b, 1):
            raise ValueError(f"Expected 'noise_labels' shape ({b},) or (1,), got {tuple(noise_labels.shape)}")
        if self.label_dim > 0 and class_labels is not None and class_labels.shape != (b, self.label_dim):
            raise ValueError(f"Expected 'class_labels' shape ({b}, {self.label_dim}), got {tuple(class_labels.shape)}")
        if self.augment_dim > 0 and augment_labels is not None and augment_labels.shape != (b, self.augment_dim):
            raise ValueError(f"Expected 'augment_labels' shape ({b}, {self.augment_dim}), got {tuple(augment_labels.shape)}")

    def conditioning_embedding(self, x, noise_labels, class_labels=None, augment_labels=None):
        """Noise / class / augmentation conditioning vector (B, emb_channels)."""
        if self.embedding_type == "zero":
            return self.zero_emb.repeat(noise_labels.shape[0], 1)
        extra = None
        if self.map_label is not None:
            tmp = class_labels
            if self.training and self.label_dropout:
                tmp = tmp * (torch.rand([x.shape[0], 1], device=x.device) >= self.label_dropout).to(tmp.dtype)
            extra = self.map_label(tmp * np.sqrt(self.map_label.in_features))
        if self.map_augment is not None and augment_labels is not None:
            aug = self.map_augment(augment_labels)
            extra = aug if extra is None else extra + aug
        if self._fused_conditioning_ok(noise_labels):
            # one launch: [sin, cos] embedding (+ extra) -> Linear + SiLU -> Linear + SiLU
            from ...ops import conditioning as _cond

            out = _cond.edm_conditioning(noise_labels, self.map_noise.freqs, self.map_layer0.weight, self.map_layer0.bias,
                                         self.map_layer1.weight, self.map_layer1.bias, extra)
            return out.to(x.dtype) if self.map_layer0.amp_mode or x.dtype != torch.float32 else out
        emb = self.map_noise(noise_labels)
        shape = emb.shape
        emb = emb.reshape(shape[0], 2, -1)  # swap the sin / cos halves
        emb = torch.concat([emb[:, 1:], emb[:, :1]], dim=1).reshape(*shape)
        if extra is not None:
            emb = emb + extra
        emb = silu(self.map_layer0(emb))
        return silu(self.map_layer1(emb))

    def _fused_conditioning_ok(self, noise_labels) -> bool:
        mn = self.map_noise
        if not noise_labels.is_cuda or noise_labels.dim() != 1 or not isinstance(mn, PositionalEmbedding):
            return False
        if mn.learnable or mn.embed_fn != "cos_sin" or not hasattr(self.map_layer0, "weight"):
            return False
        from ...ops import conditioning as _cond

        return _cond.supported(noise_labels, mn.freqs, self.map_layer0.weight, self.map_layer1.weight)

    @staticmethod
    def _extent(x):
        return math.floor(math.sqrt(x.shape[-2] * x.shape[-1]))

    def forward(self, x, noise_labels, class_labels=None, augment_labels=None):
        if not torch.compiler.is_compiling():
            self._validate(x, noise_labels, class_labels, augment_labels)
        emb = self.conditioning_embedding(x, noise_labels, class_labels, augment_labels)
        skips = []
        aux = x
        for name, block in self.enc.items():
            if "aux_down" in name:
                aux = block(aux)
            elif "aux_skip" in name:
                x = skips[-1] = x + block(aux)
            elif "aux_residual" in name:
                x = skips[-1] = aux = (x + block(aux)) / np.sqrt(2)
            elif "_conv" in name:
                x = block(x)
                if self.additive_pos_embed:
                    x = x + self.spatial_emb.to(dtype=x.dtype)
                skips.append(x)
            else:
                if isinstance(block, UNetBlock):
                    if self._extent(x) > self.checkpoint_threshold:
                        x = checkpoint(block, x, emb, use_reentrant=False)
                    else:
                        x = block(x, emb)
                else:
                    x = block(x)
                skips.append(x)
        aux = tmp = None
        for name, block in self.dec.items():
            if "aux_up" in name:
                aux = block(aux)
            elif "aux_norm" in name:
                tmp = block(x)
            elif "aux_conv" in name:
                tmp = block(silu(tmp))
                aux = tmp if aux is None else tmp + aux
            else:
                if x.shape[1] != block.in_channels:
                    x = torch.cat([x, skips.pop()], dim=1)
                ext = self._extent(x)
                if (ext > self.checkpoint_threshold and "_block" in name) or (
                        ext > (self.checkpoint_threshold / 2) and "_up" in name):
                    x = checkpoint(block, x, emb, use_reentrant=False)
                else:
                    x = block(x, emb)
        return aux


class SongUNetPosEmbd(SongUNet):
    """``SongUNet`` whose input is augmented by a (fixed or learnable) positional-embedding grid.

    ``in_channels`` counts the ``N_grid_channels`` embedding channels.  ``forward`` accepts
    ``global_index`` (P, 2, H, W) to pick the embedding of each patch in patch-based
    (multi-diffusion) training, or an ``embedding_selector`` callable.
    """

    def __init__(self, img_resolution, in_channels, out_channels, label_dim=0, augment_dim=0, model_channels=128,
                 channel_mult=[1, 2, 2, 2], channel_mult_emb=4, num_blocks=4, attn_resolutions=[28], dropout=0.13,
                 label_dropout=0.0, embedding_type="positional", channel_mult_noise=1, encoder_type="standard",
                 decoder_type="standard", resample_filter=[1, 1], gridtype="sinusoidal", N_grid_channels=4,
                 checkpoint_level=0, additive_pos_embed=False, bottleneck_attention=True, use_apex_gn=False,
                 act="silu", profile_mode=False, amp_mode=False, lead_time_mode=False, lead_time_channels=None,
                 lead_time_steps=9, prob_channels=[]):
        if not getattr(self, "_is_song_unet_pos_lt_embd", False) and (lead_time_mode or lead_time_channels):
            raise ValueError(
                "For a model with lead-time embeddings, the recommended class is "
                "`SongUNetPosLtEmbd` instead of `SongUNetPosEmbd`."
            )
        super().__init__(img_resolution=img_resolution, in_channels=in_channels, out_channels=out_channels,
                         label_dim=label_dim, augment_dim=augment_dim, model_channels=model_channels,
                         channel_mult=channel_mult, channel_mult_emb=channel_mult_emb, num_blocks=num_blocks,
                         attn_resolutions=attn_resolutions, dropout=dropout, label_dropout=label_dropout,
                         embedding_type=embedding_type, channel_mult_noise=channel_mult_noise,
                         encoder_type=encoder_type, decoder_type=decoder_type, resample_filter=resample_filter,
                         checkpoint_level=checkpoint_level, additive_pos_embed=additive_pos_embed,
                         bottleneck_attention=bottleneck_attention, use_apex_gn=use_apex_gn, act=act,
                         profile_mode=profile_mode, amp_mode=amp_mode)
        self.gridtype, self.N_grid_channels = gridtype, N_grid_channels
        if gridtype == "learnable" or N_grid_channels == 0:
            self.pos_embd = self._get_positional_embedding()
        else:
            self.register_buffer("pos_embd", self._get_positional_embedding().float(), persistent=False)
        self.lead_time_mode = lead_time_mode
        if lead_time_mode:
            if lead_time_channels is None or lead_time_channels <= 0:
                raise ValueError("`lead_time_channels` must be >= 1 if `lead_time_mode` is enabled.")
            self.lead_time_channels, self.lead_time_steps = lead_time_channels, lead_time_steps
            self.lt_embd = self._get_lead_time_embedding()
            self.prob_channels = prob_channels
            if prob_channels:
                self.scalar = torch.nn.Parameter(torch.ones((1, len(prob_channels), 1, 1)))
        else:
            if lead_time_channels:
                raise ValueError("When `lead_time_mode` is disabled, `lead_time_channels` may not be set.")
            self.lt_embd = None
            self.prob_channels = []

    def forward(self, x, noise_labels, class_labels=None, global_index=None, embedding_selector=None,
                augment_labels=None, lead_time_label=None):
        if embedding_selector is not None and global_index is not None:
            raise ValueError("Cannot provide both embedding_selector and global_index.")
        if self.pos_embd is not None or self.lt_embd is not None:
            if embedding_selector is not None:
                sel = self.positional_embedding_selector(x, embedding_selector, lead_time_label=lead_time_label)
            else:
                sel = self.positional_embedding_indexing(x, global_index=global_index, lead_time_label=lead_time_label)
            x = torch.cat((x, sel.to(x.dtype)), dim=1)
        out = super().forward(x, noise_labels, class_labels, augment_labels)
        if self.lead_time_mode and self.prob_channels:
            scalar = self.scalar.to(out.dtype)
            probs = out[:, self.prob_channels] * scalar
            if not self.training:
                probs = probs.softmax(dim=1).to(out.dtype)
            out = out.clone()
            out[:, self.prob_channels] = probs
        return out

    def positional_embedding_indexing(self, x, global_index=None, lead_time_label=None):
        """Embedding grid for each batch element: whole grid, or the pixels named by ``global_index``."""
        pos = self.pos_embd.to(x.dtype) if self.pos_embd is not None else None
        lt = self.lt_embd.to(x.dtype) if self.lt_embd is not None else None
        if lt is not None and lead_time_label is None:
            raise ValueError("`lead_time_label` must be provided when `lt_embd` is not None.")
        parts = []
        if global_index is None:
            if pos is not None:
                parts.append(pos[None].expand((x.shape[0], -1, -1, -1)))
            if lt is not None:
                parts.append(lt[lead_time_label.int()].reshape(x.shape[0], self.lead_time_channels, self.img_shape_y,
                                                               self.img_shape_x))
        else:
            P, H, W = global_index.shape[0], global_index.shape[2], global_index.shape[3]
            B = x.shape[0] // P
            gi = global_index.permute(1, 0, 2, 3).reshape(2, -1)
            if pos is not None:
                s = pos[:, gi[0], gi[1]].reshape(pos.shape[0], P, H, W).permute(1, 0, 2, 3)
                parts.append(s.repeat(B, 1, 1, 1))
            if lt is not None:
                s = lt[lead_time_label.int()][:, :, gi[0], gi[1]]
                s = s.reshape(B, self.lead_time_channels, P, H, W).permute(0, 2, 1, 3, 4).contiguous()
                parts.append(s.reshape(B * P, self.lead_time_channels, H, W))
        if not parts:
            raise ValueError(
                "`positional_embedding_indexing` should not be called when neither lead-time nor positional embeddings are used."
            )
        return torch.cat(parts, dim=1)

    def positional_embedding_selector(self, x, embedding_selector: Callable, lead_time_label=None):
        """Apply a user selector (e.g. a patching object's ``apply``) to the embedding grids."""
        parts = []
        if self.pos_embd is not None:
            parts.append(embedding_selector(self.pos_embd.to(x.dtype)))
        if self.lt_embd is not None:
            if lead_time_label is None:
                raise ValueError("`lead_time_label` must be provided when `lt_embd` is not None.")
            lt = self.lt_embd.to(x.dtype)[lead_time_label.int()]  # (B, C_lt, H, W)
            sel = torch.stack([embedding_selector(lt[b]) for b in range(lt.shape[0])], dim=0)  # (B, P, C, h, w)
            sel = sel.reshape(-1, *sel.shape[2:])
            if parts:
                parts[0] = parts[0].repeat(lt.shape[0], 1, 1, 1)
            parts.append(sel)
        if not parts:
            raise ValueError(
                "`positional_embedding_selector` should not be called when neither lead-time nor positional embeddings are used."
            )
        return torch.cat(parts, dim=1)

    def _get_positional_embedding(self):
        ny, nx, n = self.img_shape_y, self.img_shape_x, self.N_grid_channels
        if n == 0:
            return None
        if self.gridtype == "learnable":
            return torch.nn.Parameter(torch.randn(n, ny, nx))
        if self.gridtype == "linear":
            if n != 2:
                raise ValueError("N_grid_channels must be set to 2 for gridtype linear")
            gy, gx = np.meshgrid(np.linspace(-1, 1, nx), np.linspace(-1, 1, ny))
            return torch.from_numpy(np.stack((gy, gx), axis=0))
        if self.gridtype in ("sinusoidal", "sinusoidal_octave"):
            if self.gridtype == "sinusoidal":
                warnings.warn(
                    'gridtype="sinusoidal" uses a legacy frequency-band formula that does not produce exact octave '
                    'doublings. Use "sinusoidal_octave" for new models. Only use "sinusoidal" when loading '
                    "pre-trained checkpoints.", FutureWarning, stacklevel=2)
                if n == 4:
                    x1, x2 = np.sin(np.linspace(0, 2 * np.pi, nx)), np.cos(np.linspace(0, 2 * np.pi, nx))
                    y1, y2 = np.sin(np.linspace(0, 2 * np.pi, ny)), np.cos(np.linspace(0, 2 * np.pi, ny))
                    gx1, gy1 = np.meshgrid(x1, y1)
                    gx2, gy2 = np.meshgrid(x2, y2)
                    return torch.from_numpy(np.stack((gx1, gy1, gx2, gy2), axis=0))
            if n % 4 != 0:
                raise ValueError("N_grid_channels must be a multiple of 4")
            num_freq = n // 4
            bands = 2.0 ** np.linspace(0.0, num_freq, num=num_freq) if self.gridtype == "sinusoidal" else 2.0 ** np.arange(num_freq)
            gx, gy = np.meshgrid(np.linspace(0, 2 * np.pi, nx), np.linspace(0, 2 * np.pi, ny))
            grids = []
            for f in bands:
                for fn in (np.sin, np.cos):
                    grids.append(fn(gx * f))
                    grids.append(fn(gy * f))
            return torch.from_numpy(np.stack(grids, axis=0))
        if self.gridtype == "test" and n == 2:
            my, mx = torch.meshgrid(torch.arange(ny), torch.arange(nx), indexing="ij")
            return torch.stack((my, mx), dim=0)
        raise ValueError("Gridtype not supported.")

    def _get_lead_time_embedding(self):
        if self.lead_time_steps is None or self.lead_time_channels is None:
            return None
        return torch.nn.Parameter(torch.randn(self.lead_time_steps, self.lead_time_channels, self.img_shape_y,
                                              self.img_shape_x))


class SongUNetPosLtEmbd(SongUNetPosEmbd):
    """``SongUNetPosEmbd`` with a learnable lead-time embedding grid and optional probability channels."""

    _is_song_unet_pos_lt_embd = True

    def __init__(self, img_resolution, in_channels, out_channels, label_dim=0, augment_dim=0, model_channels=128,
                 channel_mult=[1, 2, 2, 2], channel_mult_emb=4, num_blocks=4, attn_resolutions=[28], dropout=0.13,
                 label_dropout=0.0, embedding_type="positional", channel_mult_noise=1, encoder_type="standard",
                 decoder_type="standard", resample_filter=[1, 1], gridtype="sinusoidal", N_grid_channels=4,
                 lead_time_channels=None, lead_time_steps=9, prob_channels=[], checkpoint_level=0,
                 additive_pos_embed=False, bottleneck_attention=True, use_apex_gn=False, act="silu",
                 profile_mode=False, amp_mode=False):
        super().__init__(img_resolution, in_channels, out_channels, label_dim, augment_dim, model_channels,
                         channel_mult, channel_mult_emb, num_blocks, attn_resolutions, dropout, label_dropout,
                         embedding_type, channel_mult_noise, encoder_type, decoder_type, resample_filter, gridtype,
                         N_grid_channels, checkpoint_level, additive_pos_embed, bottleneck_attention, use_apex_gn,
                         act, profile_mode, amp_mode, True, lead_time_channels, lead_time_steps, prob_channels)

    def forward(self, x, noise_labels, class_labels=None, lead_time_label=None, global_index=None,
                embedding_selector=None, augment_labels=None):
        return super().forward(x=x, noise_labels=noise_labels, class_labels=class_labels, global_index=global_index,
                               embedding_selector=embedding_selector, augment_labels=augment_labels,
                               lead_time_label=lead_time_label)

"""TopoDiff: constraint-conditioned diffusion U-Net for topology optimisation, plus its classifier / regressor encoder.

Parity: ``physicsnemo/models/topodiff/topodiff.py`` — ``TopoDiff.forward(x, cons, timesteps)`` concatenates the
noisy topology with the physical constraint fields and runs an EDM-style U-Net (``enc`` / ``dec`` ModuleDicts keyed
``"{res}x{res}_conv|_down|_block{i}|_in0|_in1|_up"``); ``UNetEncoder`` is the time-conditioned encoder used for the
guidance classifier / compliance regressor.
"""
from dataclasses import dataclass
from typing import List

import numpy as np
import torch
import torch.nn as nn
from torch.nn.functional import silu

from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.conv_layers import Conv2d
from ...nn.module.embedding_layers import PositionalEmbedding
from ...nn.module.fully_connected_layers import Linear
from ...nn.module.group_norm import GroupNorm
from ...nn.module.unet_layers import UNetBlock
from ..diffusion_unets._adm_layout import Stage as _Stage
from ..diffusion_unets._adm_layout import unet_layout as _unet_layout


@dataclass
class MetaData(ModelMetaData):
    jit: bool = False
    cuda_graphs: bool = False
    amp_cpu: bool = False
    amp_gpu: bool = True
    onnx: bool = True
    var_dim: int = 1
    func_torch: bool = False
    auto_grad: bool = False


class TopoDiff(Module):
    """``forward(x, cons, timesteps)``: noisy topology ``x`` and constraint fields ``cons`` (same batch and grid) are
    concatenated along channels; ``timesteps`` ``[N]`` condition every block through the embedding MLP."""

    def __init__(self, img_resolution: int, in_channels: int, out_channels: int, label_dim: int = 0, augment_dim: int = 0,
                 model_channels: int = 128, channel_mult: List[int] = [1, 1, 1, 1], channel_mult_emb: int = 4,
                 num_blocks: int = 2, attn_resolutions: List[int] = [16, 8], dropout: float = 0.10,
                 label_dropout: float = 0.0):
        super().__init__(meta=MetaData())
        self.label_dropout = label_dropout
        width_emb = channel_mult_emb * model_channels
        third = float(np.sqrt(1 / 3))
        uniform = {"init_mode": "kaiming_uniform", "init_weight": third, "init_bias": third}
        zeros = {"init_mode": "kaiming_uniform", "init_weight": 0, "init_bias": 0}
        # time embedding: sinusoidal features -> two linear layers; optional augmentation / label maps (checkpoint keys)
        self.map_noise = PositionalEmbedding(num_channels=model_channels)
        self.map_augment = Linear(augment_dim, model_channels, bias=False, **zeros) if augment_dim else None
        self.map_layer0 = Linear(model_channels, width_emb, **uniform)
        self.map_layer1 = Linear(width_emb, width_emb, **uniform)
        self.map_label = None
        if label_dim:
            self.map_label = Linear(label_dim, width_emb, bias=False, init_mode="kaiming_normal", init_weight=np.sqrt(label_dim))
        encoder, decoder, width_last = _unet_layout(img_resolution, in_channels, model_channels, channel_mult, num_blocks,
                                                    attn_resolutions)

        def build(stage: _Stage) -> nn.Module:
            if stage.kind == "conv":
                return Conv2d(in_channels=stage.width_in, out_channels=stage.width_out, kernel=3, **uniform)
            return UNetBlock(in_channels=stage.width_in, out_channels=stage.width_out, emb_channels=width_emb, dropout=dropout,
                             channels_per_head=64, init=uniform, init_zero=zeros, **dict(stage.options))

        self.enc = nn.ModuleDict({stage.key: build(stage) for stage in encoder})
        self.dec = nn.ModuleDict({stage.key: build(stage) for stage in decoder})
        self.out_norm = GroupNorm(num_channels=width_last)
        self.out_conv = Conv2d(in_channels=width_last, out_channels=out_channels, kernel=3, **zeros)

    @staticmethod
    def _check_inputs(x, cons, timesteps) -> None:
        if x.ndim != 4 or cons.ndim != 4:
            raise ValueError(f"x and cons must be [N, C, H, W] images; their shapes are {tuple(x.shape)} and {tuple(cons.shape)}")
        same_batch, same_grid = x.shape[0] == cons.shape[0], x.shape[2:] == cons.shape[2:]
        if not (same_batch and same_grid):
            raise ValueError(f"x {tuple(x.shape)} and cons {tuple(cons.shape)} must agree in batch size and grid")
        if tuple(timesteps.shape) != (x.shape[0],):
            raise ValueError(f"one timestep per sample is needed ([{x.shape[0]}]), timesteps has shape {tuple(timesteps.shape)}")

    def forward(self, x, cons, timesteps):
        if not torch.compiler.is_compiling():
            self._check_inputs(x, cons, timesteps)
        emb = self.map_noise(timesteps)
        for layer in (self.map_layer0, self.map_layer1):
            emb = silu(layer(emb))
        h = torch.cat((x, cons), dim=1)
        stack = []
        for stage in self.enc.values():
            h = stage(h, emb) if isinstance(stage, UNetBlock) else stage(h)
            stack.append(h)
        for stage in self.dec.values():
            if stage.in_channels != h.shape[1]:            # this block takes a skip connection
                h = torch.cat((h, stack.pop()), dim=1)
            h = stage(h, emb)
        return self.out_conv(silu(self.out_norm(h)))


class UNetEncoder(Module):
    """Time-conditioned encoder → global mean → MLP head (classifier when ``output_prob`` else regressor)."""

    def __init__(self, in_channels: int, out_channels: int, model_channels: int = 128, num_res_blocks: int = 4,
                 channel_mult: tuple = (1, 1, 1, 1), channel_mult_emb: int = 4, attention_resolutions: tuple = (16, 8),
                 dropout=0, output_prob=False):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.dropout, self.output_prob = dropout, output_prob
        width_emb = channel_mult_emb * model_channels
        widths = [int(m * model_channels) for m in channel_mult]
        self.map_noise = PositionalEmbedding(num_channels=model_channels)
        self.conv = Conv2d(in_channels=in_channels, out_channels=widths[0], kernel=3)
        self.time_embed = nn.Sequential(Linear(model_channels, width_emb), nn.SiLU(), Linear(width_emb, width_emb))
        # every level: num_res_blocks blocks, the last of which halves the resolution (except at the coarsest level);
        # attention where the accumulated down-sampling factor is listed in attention_resolutions
        self.encoder = nn.ModuleList()
        current, last_level = widths[0], len(widths) - 1
        for level, target in enumerate(widths):
            factor = 2 ** level
            for i in range(num_res_blocks):
                shrink = level < last_level and i + 1 == num_res_blocks
                self.encoder.append(UNetBlock(in_channels=current, out_channels=target, emb_channels=width_emb,
                                              attention=factor in attention_resolutions, down=shrink))
                current = target
        self.middle = nn.ModuleList(UNetBlock(in_channels=current, out_channels=current, emb_channels=width_emb, attention=flag)
                                    for flag in (True, False))
        head = [Linear(current, 2048), GroupNorm(num_channels=2048), nn.ReLU(), nn.Dropout(p=dropout), nn.Linear(2048, out_channels)]
        if output_prob:
            head.append(nn.Sigmoid())
        self.out = nn.Sequential(*head)

    def forward(self, x, time_steps):
        if not torch.compiler.is_compiling():
            if x.ndim != 4:
                raise ValueError(f"the encoder takes [N, C, H, W] images, got a tensor of shape {tuple(x.shape)}")
            if tuple(time_steps.shape) != (x.shape[0],):
                raise ValueError(f"one time step per sample is needed ([{x.shape[0]}]), got shape {tuple(time_steps.shape)}")
        emb = self.time_embed(self.map_noise(time_steps))
        h = self.conv(x)
        for block in (*self.encoder, *self.middle):
            h = block(h, emb)
        return self.out(h.mean(dim=(2, 3)))

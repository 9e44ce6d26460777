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
    def __init__(self, img_resolution: int, in_channels: int, out_channels: int, label_dim: int = 0, augment_dim: int = 0,
                 model_channels: int = 128, channel_mult: List[int] = [1, 1, 1, 1], channel_mult_emb: int = 4,
                 num_blocks: int = 2, attn_resolutions: List[int] = [16, 8], dropout: float = 0.10,
                 label_dropout: float = 0.0):
        super().__init__(meta=MetaData())
        self.label_dropout = label_dropout
        emb_channels = model_channels * channel_mult_emb
        init = dict(init_mode="kaiming_uniform", init_weight=np.sqrt(1 / 3), init_bias=np.sqrt(1 / 3))
        init_zero = dict(init_mode="kaiming_uniform", init_weight=0, init_bias=0)
        blk = dict(emb_channels=emb_channels, channels_per_head=64, dropout=dropout, init=init, init_zero=init_zero)
        self.map_noise = PositionalEmbedding(num_channels=model_channels)
        self.map_augment = Linear(in_features=augment_dim, out_features=model_channels, bias=False, **init_zero) if augment_dim else None
        self.map_layer0 = Linear(in_features=model_channels, out_features=emb_channels, **init)
        self.map_layer1 = Linear(in_features=emb_channels, out_features=emb_channels, **init)
        self.map_label = Linear(in_features=label_dim, out_features=emb_channels, bias=False, init_mode="kaiming_normal",
                                init_weight=np.sqrt(label_dim)) if label_dim else None
        self.enc = torch.nn.ModuleDict()
        cout = in_channels
        for level, mult in enumerate(channel_mult):
            res = img_resolution >> level
            if level == 0:
                cin, cout = cout, model_channels * mult
                self.enc[f"{res}x{res}_conv"] = Conv2d(in_channels=cin, out_channels=cout, kernel=3, **init)
            else:
                self.enc[f"{res}x{res}_down"] = UNetBlock(in_channels=cout, out_channels=cout, down=True, **blk)
            for idx in range(num_blocks):
                cin, cout = cout, model_channels * mult
                self.enc[f"{res}x{res}_block{idx}"] = UNetBlock(in_channels=cin, out_channels=cout,
                                                                attention=(res in attn_resolutions), **blk)
        skips = [b.out_channels for b in self.enc.values()]
        self.dec = torch.nn.ModuleDict()
        for level, mult in reversed(list(enumerate(channel_mult))):
            res = img_resolution >> level
            if level == len(channel_mult) - 1:
                self.dec[f"{res}x{res}_in0"] = UNetBlock(in_channels=cout, out_channels=cout, attention=True, **blk)
                self.dec[f"{res}x{res}_in1"] = UNetBlock(in_channels=cout, out_channels=cout, **blk)
            else:
                self.dec[f"{res}x{res}_up"] = UNetBlock(in_channels=cout, out_channels=cout, up=True, **blk)
            for idx in range(num_blocks + 1):
                cin, cout = cout + skips.pop(), model_channels * mult
                self.dec[f"{res}x{res}_block{idx}"] = UNetBlock(in_channels=cin, out_channels=cout,
                                                                attention=(res in attn_resolutions), **blk)
        self.out_norm = GroupNorm(num_channels=cout)
        self.out_conv = Conv2d(in_channels=cout, out_channels=out_channels, kernel=3, **init_zero)

    def forward(self, x, cons, timesteps):
        if not torch.compiler.is_compiling():
            if x.ndim != 4 or cons.ndim != 4:
                raise ValueError(f"Expected 4D tensors for x and cons, got {tuple(x.shape)} and {tuple(cons.shape)}")
            if x.shape[0] != cons.shape[0] or x.shape[2:] != cons.shape[2:]:
                raise ValueError(f"x and cons must have matching batch and spatial dims (got x{tuple(x.shape)}, cons{tuple(cons.shape)})")
            if timesteps.ndim != 1 or timesteps.shape[0] != x.shape[0]:
                raise ValueError(f"Expected timesteps of shape (N,), got {tuple(timesteps.shape)}")
        emb = silu(self.map_layer1(silu(self.map_layer0(self.map_noise(timesteps)))))
        x = torch.cat([x, cons], dim=1)
        skips = []
        for block in self.enc.values():
            x = block(x, emb) if isinstance(block, UNetBlock) else block(x)
            skips.append(x)
        for block in self.dec.values():
            if x.shape[1] != block.in_channels:
                x = torch.cat([x, skips.pop()], dim=1)
            x = block(x, emb)
        return self.out_conv(silu(self.out_norm(x)))


class UNetEncoder(Module):
    """Time-conditioned encoder → global mean → MLP head (classifier when ``output_prob`` else regressor)."""

    def __init__(self, in_channels: int, out_channels: int, model_channels: int = 128, num_res_blocks: int = 4,
                 channel_mult: tuple = (1, 1, 1, 1), channel_mult_emb: int = 4, attention_resolutions: tuple = (16, 8),
                 dropout=0, output_prob=False):
        super().__init__()
        self.in_channels, self.out_channels, self.dropout, self.output_prob = in_channels, out_channels, dropout, output_prob
        self.map_noise = PositionalEmbedding(num_channels=model_channels)
        ch = int(model_channels * channel_mult[0])
        self.conv = Conv2d(in_channels=in_channels, out_channels=ch, kernel=3)
        emb_channels = model_channels * channel_mult_emb
        self.time_embed = nn.Sequential(Linear(in_features=model_channels, out_features=emb_channels), nn.SiLU(),
                                        Linear(in_features=emb_channels, out_features=emb_channels))
        ds = 1
        self.encoder = nn.ModuleList()
        for level, mult in enumerate(channel_mult):
            for i in range(num_res_blocks):
                down = i == num_res_blocks - 1 and level != len(channel_mult) - 1
                self.encoder.append(UNetBlock(in_channels=ch, out_channels=int(mult * model_channels),
                                              emb_channels=emb_channels, down=down, attention=ds in attention_resolutions))
                ch = int(mult * model_channels)
            ds *= 2
        self.middle = nn.ModuleList([UNetBlock(in_channels=ch, out_channels=ch, emb_channels=emb_channels, attention=True),
                                     UNetBlock(in_channels=ch, out_channels=ch, emb_channels=emb_channels, attention=False)])
        self.out = nn.Sequential(Linear(in_features=ch, out_features=2048), GroupNorm(num_channels=2048), nn.ReLU(),
                                 nn.Dropout(p=dropout), nn.Linear(in_features=2048, out_features=self.out_channels))
        if self.output_prob:
            self.out.append(nn.Sigmoid())

    def forward(self, x, time_steps):
        if not torch.compiler.is_compiling():
            if x.ndim != 4:
                raise ValueError(f"Expected 4D input tensor, got {tuple(x.shape)}")
            if time_steps.ndim != 1 or time_steps.shape[0] != x.shape[0]:
                raise ValueError(f"Expected time_steps of shape (N,), got {tuple(time_steps.shape)}")
        emb = self.time_embed(self.map_noise(time_steps))
        h = self.conv(x)
        for m in list(self.encoder) + list(self.middle):
            h = m(h, emb)
        return self.out(h.mean(dim=(2, 3)))

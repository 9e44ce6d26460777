"""ADM ("Dhariwal") diffusion U-Net.

Parity: ``physicsnemo/models/diffusion_unets/dhariwal_unet.py`` — sinusoidal noise embedding (+ augment / class
label maps with label dropout) → two-layer SiLU MLP; encoder / decoder ModuleDicts of ``UNetBlock`` keyed
``"{res}x{res}_conv|_down|_block{i}|_in0|_in1|_up"`` with attention at ``attn_resolutions``; GroupNorm → SiLU →
zero-initialised output conv.
"""
from dataclasses import dataclass
from typing import List

import numpy as np
import torch
from torch.nn.functional import silu

from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.conv_layers import Conv2d
from ...nn.module.embedding_layers import PositionalEmbedding
from ...nn.module.fully_connected_layers import Linear
from ...nn.module.group_norm import get_group_norm
from ...nn.module.unet_layers import UNetBlock
from ...nn.module.utils.utils import _recursive_property
from ._adm_layout import Stage, unet_layout


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


class DhariwalUNet(Module):
    """``forward(x, noise_labels, class_labels=None, augment_labels=None)`` → ``[B, out_channels, H, W]``."""

    def __init__(self, img_resolution: int, in_channels: int, out_channels: int, label_dim: int = 0, augment_dim: int = 0,
                 model_channels: int = 192, channel_mult: List[int] = [1, 2, 3, 4], channel_mult_emb: int = 4,
                 num_blocks: int = 3, attn_resolutions: List[int] = [32, 16, 8], dropout: float = 0.10,
                 label_dropout: float = 0.0):
        super().__init__(meta=MetaData())
        self.label_dim, self.augment_dim, self.label_dropout = label_dim, augment_dim, label_dropout
        width_emb = channel_mult_emb * model_channels
        third = float(np.sqrt(1 / 3))
        uniform = {"init_mode": "kaiming_uniform", "init_weight": third, "init_bias": third}
        zeros = {"init_mode": "kaiming_uniform", "init_weight": 0, "init_bias": 0}
        # embedding path (all names are checkpoint keys): noise features (+ augmentation map) -> 2-layer MLP (+ label map)
        self.map_noise = PositionalEmbedding(num_channels=model_channels)
        self.map_augment = Linear(augment_dim, model_channels, bias=False, **zeros) if augment_dim else None
        self.map_layer0 = Linear(model_channels, width_emb, **uniform)
        self.map_layer1 = Linear(width_emb, width_emb, **uniform)
        self.map_label = None
        if label_dim:
            self.map_label = Linear(label_dim, width_emb, bias=False, init_mode="kaiming_normal", init_weight=np.sqrt(label_dim))
        encoder, decoder, width_last = unet_layout(img_resolution, in_channels, model_channels, channel_mult, num_blocks,
                                                   attn_resolutions)

        def build(stage: Stage) -> torch.nn.Module:
            if stage.kind == "conv":
                return Conv2d(in_channels=stage.width_in, out_channels=stage.width_out, kernel=3, **uniform)
            return UNetBlock(in_channels=stage.width_in, out_channels=stage.width_out, emb_channels=width_emb, dropout=dropout,
                             channels_per_head=64, init=uniform, init_zero=zeros, **dict(stage.options))

        self.enc = torch.nn.ModuleDict({stage.key: build(stage) for stage in encoder})
        self.dec = torch.nn.ModuleDict({stage.key: build(stage) for stage in decoder})
        self.out_norm = get_group_norm(num_channels=width_last)
        self.out_conv = Conv2d(in_channels=width_last, out_channels=out_channels, kernel=3, **zeros)
        self.profile_mode = False
        self.amp_mode = False

    profile_mode = _recursive_property("profile_mode", bool, "Should be set to ``True`` to enable profiling.")
    amp_mode = _recursive_property("amp_mode", bool, "Should be set to ``True`` to enable automatic mixed precision.")

    def _check_inputs(self, x, noise_labels, class_labels, augment_labels) -> None:
        if x.ndim != 4:
            raise ValueError(f"'x' must be a batch of images [B, C_in, H, W]; got shape {tuple(x.shape)}")
        batch = x.shape[0]
        if noise_labels.ndim != 1 or noise_labels.shape[0] not in (1, batch):
            raise ValueError(f"'noise_labels' must hold one level per sample ([{batch}]) or a single level ([1]); "
                             f"got shape {tuple(noise_labels.shape)}")
        for name, labels, width in (("class_labels", class_labels, self.label_dim),
                                    ("augment_labels", augment_labels, self.augment_dim)):
            if width > 0 and labels is not None and tuple(labels.shape) != (batch, width):
                raise ValueError(f"'{name}' must have shape ({batch}, {width}); got {tuple(labels.shape)}")

    def _embedding(self, batch, device, noise_labels, class_labels, augment_labels):
        emb = self.map_noise(noise_labels)
        if augment_labels is not None and self.map_augment is not None:
            emb = emb + self.map_augment(augment_labels)
        emb = self.map_layer1(silu(self.map_layer0(emb)))
        if self.map_label is not None:
            labels = class_labels
            if self.label_dropout and self.training:       # drop whole label vectors (classifier-free guidance)
                dropped = torch.rand([batch, 1], device=device) < self.label_dropout
                labels = labels.masked_fill(dropped, 0)
            emb = emb + self.map_label(labels)
        return silu(emb)

    def forward(self, x, noise_labels, class_labels=None, augment_labels=None):
        if not torch.compiler.is_compiling():
            self._check_inputs(x, noise_labels, class_labels, augment_labels)
        emb = self._embedding(x.shape[0], x.device, noise_labels, class_labels, augment_labels)
        h, stack = x, []
        for stage in self.enc.values():
            h = stage(h, emb) if isinstance(stage, UNetBlock) else stage(h)
            stack.append(h)
        for stage in self.dec.values():
            if stage.in_channels != h.shape[1]:            # this block takes a skip connection
                h = torch.cat((h, stack.pop()), dim=1)
            h = stage(h, emb)
        return self.out_conv(silu(self.out_norm(h)))

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
    def __init__(self, img_resolution: int, in_channels: int, out_channels: int, label_dim: int = 0, augment_dim: int = 0,
                 model_channels: int = 192, channel_mult: List[int] = [1, 2, 3, 4], channel_mult_emb: int = 4,
                 num_blocks: int = 3, attn_resolutions: List[int] = [32, 16, 8], dropout: float = 0.10,
                 label_dropout: float = 0.0):
        super().__init__(meta=MetaData())
        self.label_dim, self.augment_dim, self.label_dropout = label_dim, augment_dim, label_dropout
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
        self.out_norm = get_group_norm(num_channels=cout)
        self.out_conv = Conv2d(in_channels=cout, out_channels=out_channels, kernel=3, **init_zero)
        self.profile_mode = False
        self.amp_mode = False

    profile_mode = _recursive_property("profile_mode", bool, "Should be set to ``True`` to enable profiling.")
    amp_mode = _recursive_property("amp_mode", bool, "Should be set to ``True`` to enable automatic mixed precision.")

    def forward(self, x, noise_labels, class_labels=None, augment_labels=None):
        if not torch.compiler.is_compiling():
            B = x.shape[0]
            if x.ndim != 4:
                raise ValueError(f"Expected 'x' to be a 4D tensor (B, C_in, H, W), got {x.ndim}D tensor with shape {tuple(x.shape)}")
            if noise_labels.ndim != 1 or noise_labels.shape[0] not in (B, 1):
                raise ValueError(f"Expected 'noise_labels' shape ({B},) or (1,), got {tuple(noise_labels.shape)}")
            if self.label_dim > 0 and class_labels is not None and tuple(class_labels.shape) != (B, self.label_dim):
                raise ValueError(f"Expected 'class_labels' shape ({B}, {self.label_dim}), got {tuple(class_labels.shape)}")
            if self.augment_dim > 0 and augment_labels is not None and tuple(augment_labels.shape) != (B, self.augment_dim):
                raise ValueError(f"Expected 'augment_labels' shape ({B}, {self.augment_dim}), got {tuple(augment_labels.shape)}")
        emb = self.map_noise(noise_labels)
        if self.map_augment is not None and augment_labels is not None:
            emb = emb + self.map_augment(augment_labels)
        emb = self.map_layer1(silu(self.map_layer0(emb)))
        if self.map_label is not None:
            lab = class_labels
            if self.training and self.label_dropout:
                lab = lab * (torch.rand([x.shape[0], 1], device=x.device) >= self.label_dropout).to(lab.dtype)
            emb = emb + self.map_label(lab)
        emb = silu(emb)
        skips = []
        for block in self.enc.values():
            x = block(x, emb) if isinstance(block, UNetBlock) else block(x)
            skips.append(x)
        for block in self.dec.values():
            if x.shape[1] != block.in_channels:
                x = torch.cat([x, skips.pop()], dim=1)
            x = block(x, emb)
        return self.out_conv(silu(self.out_norm(x)))

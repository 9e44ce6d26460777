"""Pix2Pix U-Net generator built from nested skip-connection blocks.

Parity: ``physicsnemo/models/pix2pix/pix2pixunet.py`` — ``UnetSkipConnectionBlock`` (down conv → submodule → up
conv, output concatenated with its input), ``UnetGenerator`` (innermost block wrapped ``n_downsampling − 5``
times at 8× filters, then 4×/2×/1× and the outermost Tanh block), ``Pix2PixUnet`` wrapper with
``load_networks`` for raw generator checkpoints.
"""
import functools
from dataclasses import dataclass
from typing import List

import torch
import torch.nn as nn
from torch.nn import init

from ...core.meta import ModelMetaData
from ...core.module import Module


def init_weights(net, init_type="normal", init_gain=0.02):
    """Initialise conv / linear weights (``normal | xavier | kaiming | orthogonal``) and BatchNorm2d affine terms."""
    fill = {"normal": lambda w: init.normal_(w, 0.0, init_gain), "xavier": lambda w: init.xavier_normal_(w, gain=init_gain),
            "kaiming": lambda w: init.kaiming_normal_(w, a=0, mode="fan_in"),
            "orthogonal": lambda w: init.orthogonal_(w, gain=init_gain)}

    def fn(m):
        name = type(m).__name__
        if hasattr(m, "weight") and ("Conv" in name or "Linear" in name):
            if init_type not in fill:
                raise NotImplementedError("initialization method [%s] is not implemented" % init_type)
            fill[init_type](m.weight.data)
            if getattr(m, "bias", None) is not None:
                init.constant_(m.bias.data, 0.0)
        elif "BatchNorm2d" in name:
            init.normal_(m.weight.data, 1.0, init_gain)
            init.constant_(m.bias.data, 0.0)

    net.apply(fn)


@dataclass
class MetaData(ModelMetaData):
    jit: bool = True
    cuda_graphs: bool = True
    amp_cpu: bool = False
    amp_gpu: bool = True
    onnx: bool = True
    var_dim: int = 1
    func_torch: bool = True
    auto_grad: bool = True


class UnetSkipConnectionBlock(nn.Module):
    def __init__(self, outer_nc: int, inner_nc: int, input_nc: int = None, submodule: nn.Module = None,
                 outermost: bool = False, innermost: bool = False, norm_layer=nn.BatchNorm2d, use_dropout: bool = False):
        super().__init__()
        self.outermost = outermost
        base = norm_layer.func if isinstance(norm_layer, functools.partial) else norm_layer
        bias = base == nn.InstanceNorm2d
        input_nc = outer_nc if input_nc is None else input_nc
        down = nn.Conv2d(input_nc, inner_nc, kernel_size=4, stride=2, padding=1, bias=bias)
        lrelu, relu = nn.LeakyReLU(0.2, True), nn.ReLU(True)
        dnorm, unorm = norm_layer(inner_nc), norm_layer(outer_nc)
        if outermost:
            up = nn.ConvTranspose2d(inner_nc * 2, outer_nc, kernel_size=4, stride=2, padding=1)
            layers = [down, submodule, relu, up, nn.Tanh()]
        elif innermost:
            up = nn.ConvTranspose2d(inner_nc, outer_nc, kernel_size=4, stride=2, padding=1, bias=bias)
            layers = [lrelu, down, relu, up, unorm]
        else:
            up = nn.ConvTranspose2d(inner_nc * 2, outer_nc, kernel_size=4, stride=2, padding=1, bias=bias)
            layers = [lrelu, down, dnorm, submodule, relu, up, unorm] + ([nn.Dropout(0.5)] if use_dropout else [])
        self.model = nn.Sequential(*layers)

    def forward(self, x):
        return self.model(x) if self.outermost else torch.cat([x, self.model(x)], 1)


class UnetGenerator(nn.Module):
    def __init__(self, in_channels: int, out_channels: int, n_downsampling: int, filter_size: int = 64,
                 norm_layer=nn.BatchNorm2d, use_dropout: bool = False):
        super().__init__()
        f = filter_size
        block = UnetSkipConnectionBlock(f * 8, f * 8, submodule=None, norm_layer=norm_layer, innermost=True)
        for _ in range(n_downsampling - 5):
            block = UnetSkipConnectionBlock(f * 8, f * 8, submodule=block, norm_layer=norm_layer, use_dropout=use_dropout)
        for outer, inner in ((f * 4, f * 8), (f * 2, f * 4), (f, f * 2)):
            block = UnetSkipConnectionBlock(outer, inner, submodule=block, norm_layer=norm_layer)
        self.model = UnetSkipConnectionBlock(out_channels, f, input_nc=in_channels, submodule=block, outermost=True,
                                             norm_layer=norm_layer)

    def forward(self, input):
        return self.model(input)


class Pix2PixUnet(Module):
    def __init__(self, in_channels: int, out_channels: int, n_downsampling: int, filter_size: int = 64,
                 norm_layer=nn.BatchNorm2d, use_dropout: bool = False, gpu_ids: List = []):
        if not (filter_size > 0 and n_downsampling >= 0):
            raise ValueError("Invalid arch params")
        super().__init__(meta=MetaData())
        self.gpu_ids = gpu_ids
        self.model_device = torch.device(f"cuda:{gpu_ids[0]}") if gpu_ids else torch.device("cpu")
        net = UnetGenerator(in_channels, out_channels, n_downsampling, filter_size, norm_layer, use_dropout)
        if gpu_ids:
            net = torch.nn.DataParallel(net.to(gpu_ids[0]), gpu_ids)
        self.netG = net

    @staticmethod
    def _drop_instance_norm_stats(state_dict, root):
        """InstanceNorm layers saved by old PyTorch carry running statistics that current modules do not expect."""
        for key in list(state_dict):
            *path, leaf = key.split(".")
            mod = root
            for p in path:
                mod = getattr(mod, p)
            if type(mod).__name__.startswith("InstanceNorm"):
                if leaf in ("running_mean", "running_var") and getattr(mod, leaf) is None:
                    state_dict.pop(key)
                elif leaf == "num_batches_tracked":
                    state_dict.pop(key)

    def load_networks(self, model_path: str) -> None:
        net = self.netG.module if isinstance(self.netG, torch.nn.DataParallel) else self.netG
        state = torch.load(model_path, map_location=str(self.model_device))
        if hasattr(state, "_metadata"):
            del state._metadata
        self._drop_instance_norm_stats(state, net)
        net.load_state_dict(state)

    def test(self, input):
        with torch.no_grad():
            return self.forward(input)

    def forward(self, input):
        return self.netG(input)

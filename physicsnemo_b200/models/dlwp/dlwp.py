"""DLWP: U-Net on the cubed sphere.

Parity: ``physicsnemo/models/dlwp/dlwp.py`` — six faces ``[B, C, 6, H, H]`` (0–3 equatorial, 4 / 5 polar); every
3×3 convolution sees a halo copied from the neighbouring faces (with the rotations that align their axes), the
equatorial faces share one set of weights and the polar faces another (face 5 mirrored).  Here the halo is
assembled once per layer for all faces and the shared-weight faces are folded into the batch, so a layer costs
two convolution launches instead of six.
"""
import math
from dataclasses import dataclass
from typing import Tuple, Union

import torch
import torch.nn as nn

from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.activations import get_activation


def _get_same_padding(x: int, k: int, s: int) -> int:
    return max(s * math.ceil(x / s) - s - x + k, 0)


def _pad_equatorial(main, left, right, top, bottom, nr_rot: int, size: int):
    if nr_rot:
        top = torch.rot90(top, k=nr_rot, dims=(-2, -1))
        bottom = torch.rot90(bottom, k=nr_rot, dims=(-1, -2))
    middle = torch.cat((left[..., :, -size:], main, right[..., :, :size]), dim=-1)
    widen = lambda f: torch.cat((f[..., :, :size], f, f[..., :, -size:]), dim=-1)  # noqa: E731  (corner filler)
    return torch.cat((widen(bottom)[..., -size:, :], middle, widen(top)[..., :size, :]), dim=-2)


def _pad_polar(main, left, right, top, bottom, rot_left, rot_right, size: int):
    left, right = torch.rot90(left, dims=rot_left), torch.rot90(right, dims=rot_right)
    middle = torch.cat((bottom[..., -size:, :], main, top[..., :size, :]), dim=-2)
    heighten = lambda f: torch.cat((f[..., :size, :], f, f[..., -size:, :]), dim=-2)  # noqa: E731
    return torch.cat((heighten(left)[..., :, -size:], middle, heighten(right)[..., :, :size]), dim=-1)


def _cubed_conv(faces, equator_conv: nn.Conv2d, polar_conv: nn.Conv2d):
    """``faces``: list of six ``[B, C, H, W]`` tensors → list of six outputs."""
    size = _get_same_padding(faces[0].size(-1), equator_conv.kernel_size[0], equator_conv.stride[0]) // 2
    f = faces
    if size:
        eq = [_pad_equatorial(f[i], f[(i - 1) % 4], f[(i + 1) % 4], f[5], f[4], nr_rot=i, size=size) for i in range(4)]
        north = _pad_polar(f[4], f[3], f[1], f[0], f[5], (-1, -2), (-2, -1), size)
        south = _pad_polar(f[5], f[3], f[1], f[4], f[0], (-2, -1), (-1, -2), size)
    else:
        eq, north, south = list(f[:4]), f[4], f[5]
    B = f[0].shape[0]
    eq_out = equator_conv(torch.cat(eq, dim=0)).split(B, dim=0)
    polar_out = polar_conv(torch.cat([north, torch.flip(south, [-1])], dim=0)).split(B, dim=0)
    return [*eq_out, polar_out[0], torch.flip(polar_out[1], [-1])]


@dataclass
class MetaData(ModelMetaData):
    jit: bool = False
    cuda_graphs: bool = True
    amp_cpu: bool = True
    amp_gpu: bool = True
    onnx: bool = False
    var_dim: int = 1
    func_torch: bool = False
    auto_grad: bool = False


class DLWP(Module):
    def __init__(self, nr_input_channels: int, nr_output_channels: int, nr_initial_channels: int = 64,
                 activation_fn: str = "leaky_relu", depth: int = 2,
                 clamp_activation: Tuple[Union[float, int, None], Union[float, int, None]] = (None, 10.0)) -> None:
        super().__init__(meta=MetaData())
        self.nr_input_channels, self.nr_output_channels = nr_input_channels, nr_output_channels
        self.nr_initial_channels, self.depth = nr_initial_channels, depth
        self.activation_fn = get_activation(activation_fn)
        self.clamp_activation = clamp_activation
        self.avg_pool = nn.AvgPool2d(2)
        self.upsample_layer = nn.Upsample(scale_factor=2)
        w0 = nr_initial_channels
        down, mid, up = [], [], []
        outs = w0
        for i in range(depth):
            ins = nr_input_channels if i == 0 else w0 * 2 ** (i - 1)
            outs = w0 * 2 ** i
            down += [(ins, outs), (outs, outs)]
        mid = [(outs, outs * 2), (outs * 2, outs)]
        for i in range(depth - 1, -1, -1):
            outs = w0 if i == 0 else w0 * 2 ** i
            final = outs if i == 0 else outs // 2
            up += [(outs * 2, outs), (outs, final)]
            outs = final
        pair = lambda spec: nn.ModuleList([nn.Conv2d(a, b, kernel_size=3) for a, b in spec])  # noqa: E731
        self.equatorial_downsample, self.polar_downsample = pair(down), pair(down)
        self.equatorial_mid_layers, self.polar_mid_layers = pair(mid), pair(mid)
        self.equatorial_upsample, self.polar_upsample = pair(up), pair(up)
        self.equatorial_last = nn.Conv2d(outs, nr_output_channels, kernel_size=1)
        self.polar_last = nn.Conv2d(outs, nr_output_channels, kernel_size=1)

    def activation(self, x):
        x = self.activation_fn(x)
        if any(isinstance(c, (float, int)) for c in self.clamp_activation):
            x = torch.clamp(x, min=self.clamp_activation[0], max=self.clamp_activation[1])
        return x

    def forward(self, cubed_sphere_input):
        if not torch.compiler.is_compiling():
            if cubed_sphere_input.ndim != 5:
                raise ValueError(f"Expected input tensor of shape (B, C, F, H, W) but got tensor of shape {tuple(cubed_sphere_input.shape)}")
            _, ch, nf, h, w = cubed_sphere_input.shape
            if ch != self.nr_input_channels:
                raise ValueError(f"Expected input tensor with {self.nr_input_channels} channels but got {ch} channels")
            if nf != 6:
                raise ValueError(f"Expected input tensor of shape (B, C, 6, H, W) but got tensor of shape {tuple(cubed_sphere_input.shape)}")
            if h != w:
                raise ValueError(f"Expected input tensor of shape (B, C, F, H, H) but got tensor of shape {tuple(cubed_sphere_input.shape)}")
        faces = list(cubed_sphere_input.unbind(dim=2))
        each = lambda fn, fs: [fn(t) for t in fs]  # noqa: E731
        skips = []
        for i, (eq, po) in enumerate(zip(self.equatorial_downsample, self.polar_downsample)):
            faces = each(self.activation, _cubed_conv(faces, eq, po))
            if i % 2:
                skips.append(faces)
                faces = each(self.avg_pool, faces)
        for eq, po in zip(self.equatorial_mid_layers, self.polar_mid_layers):
            faces = each(self.activation, _cubed_conv(faces, eq, po))
        for i, (eq, po) in enumerate(zip(self.equatorial_upsample, self.polar_upsample)):
            if i % 2 == 0:
                faces = [torch.cat((a, b), dim=1) for a, b in zip(each(self.upsample_layer, faces), skips.pop())]
            faces = each(self.activation, _cubed_conv(faces, eq, po))
        return torch.stack(_cubed_conv(faces, self.equatorial_last, self.polar_last), dim=2)

"""Channel-parallel (tensor-parallel) AFNO layers over the process group named ``"model_parallel"``.

Parity: ``physicsnemo/models/afno/distributed/layers.py`` (``DropPath``, ``DistributedMLP`` with 1×1-conv
weights ``w1 [hidden/P, in, 1, 1]``, ``w2 [out, hidden/P, 1, 1]`` and one all-reduce after the second
product; ``DistributedPatchEmbed`` producing ``embed_dim / P`` channels per rank; ``DistributedAFNO2D``
holding ``num_blocks / P`` spectral blocks per rank, FFT local per channel; parameters that see every
spatial position carry ``is_shared_spatial``).

The spectral mixing runs as complex batched products on the retained mode window only and is placed
back with one ``F.pad``; soft-shrinkage acts on that window (it maps the zeros outside it to zeros).
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ....core.module import Module
from ....distributed.manager import DistributedManager
from ....distributed.mappings import (copy_to_parallel_region, gather_from_parallel_region, reduce_from_parallel_region,
                                      scatter_to_parallel_region)
from ....distributed.utils import compute_split_shapes

_GROUP = "model_parallel"


def _group_size() -> int:
    return DistributedManager().group_size(_GROUP)


def drop_path(x: Tensor, drop_prob: float = 0.0, training: bool = False) -> Tensor:
    if drop_prob == 0.0 or not training:
        return x
    keep = 1.0 - drop_prob
    mask = (keep + torch.rand((x.shape[0],) + (1,) * (x.ndim - 1), dtype=x.dtype, device=x.device)).floor_()
    return x.div(keep) * mask


class DropPath(Module):
    def __init__(self, drop_prob: float = None):
        super().__init__()
        self.drop_prob = drop_prob

    def forward(self, x: Tensor) -> Tensor:
        return drop_path(x, self.drop_prob, self.training)


class DistributedMLP(Module):
    """Column-parallel first layer, row-parallel second layer: one all-reduce per call."""

    def __init__(self, in_features: int, hidden_features: int | None = None, out_features: int | None = None,
                 act_layer: type = nn.GELU, drop: float = 0.0, input_is_matmul_parallel: bool = False,
                 output_is_matmul_parallel: bool = False):
        super().__init__()
        out_features = out_features or in_features
        hidden_features = hidden_features or in_features
        self.input_is_matmul_parallel, self.output_is_matmul_parallel = input_is_matmul_parallel, output_is_matmul_parallel
        p = _group_size()
        if hidden_features % p != 0:
            raise ValueError("Error, hidden_features needs to be divisible by matmul_parallel_size")
        local = hidden_features // p
        self.w1 = nn.Parameter(torch.ones(local, in_features, 1, 1))
        self.b1 = nn.Parameter(torch.zeros(local))
        self.w2 = nn.Parameter(torch.ones(out_features, local, 1, 1))
        self.b2 = nn.Parameter(torch.zeros(out_features))
        self.act = act_layer()
        self.drop = nn.Dropout(drop) if drop > 0.0 else nn.Identity()
        if input_is_matmul_parallel:
            self.gather_shapes = compute_split_shapes(in_features, p)
        self._init_weights()

    def _init_weights(self) -> None:
        torch.nn.init.trunc_normal_(self.w1, std=0.02)
        nn.init.constant_(self.b1, 0.0)
        torch.nn.init.trunc_normal_(self.w2, std=0.02)
        nn.init.constant_(self.b2, 0.0)

    def forward(self, x: Tensor) -> Tensor:
        if self.input_is_matmul_parallel:
            x = gather_from_parallel_region(x, dim=1, shapes=self.gather_shapes, group=_GROUP)
        x = copy_to_parallel_region(x, group=_GROUP)
        x = self.drop(self.act(F.conv2d(x, self.w1, bias=self.b1)))
        x = reduce_from_parallel_region(F.conv2d(x, self.w2, bias=None), group=_GROUP)
        x = self.drop(x + self.b2.reshape(1, -1, 1, 1))
        if self.output_is_matmul_parallel:
            x = scatter_to_parallel_region(x, dim=1, group=_GROUP)
        return x


class DistributedPatchEmbed(Module):
    def __init__(self, inp_shape: Tuple[int, int] = (224, 224), patch_size: Tuple[int, int] = (16, 16), in_chans: int = 3,
                 embed_dim: int = 768, input_is_matmul_parallel: bool = False, output_is_matmul_parallel: bool = True):
        super().__init__()
        self.input_parallel, self.output_parallel = input_is_matmul_parallel, output_is_matmul_parallel
        p = _group_size()
        self.inp_shape = (inp_shape[0], inp_shape[1])
        self.patch_size = patch_size
        self.num_patches = (inp_shape[1] // patch_size[1]) * (inp_shape[0] // patch_size[0])
        if self.input_parallel:
            if in_chans % p != 0:
                raise ValueError("Error, the in_chans needs to be divisible by matmul_parallel_size")
            self.in_shapes = compute_split_shapes(in_chans, p)
        if self.output_parallel and embed_dim % p != 0:
            raise ValueError("Error, the embed_dim needs to be divisible by matmul_parallel_size")
        self.proj = nn.Conv2d(in_chans, embed_dim // p if self.output_parallel else embed_dim, kernel_size=patch_size,
                              stride=patch_size)
        self.proj.weight.is_shared_spatial = True
        self.proj.bias.is_shared_spatial = True

    def forward(self, x: Tensor) -> Tensor:
        if self.input_parallel:
            x = gather_from_parallel_region(x, dim=1, shapes=self.in_shapes, group=_GROUP)
        if self.output_parallel:
            x = copy_to_parallel_region(x, group=_GROUP)
        if not torch.compiler.is_compiling():
            if x.ndim != 4 or x.shape[1] != self.proj.in_channels or tuple(x.shape[2:]) != self.inp_shape:
                raise ValueError(f"Expected input shape (B, {self.proj.in_channels}, {self.inp_shape[0]}, {self.inp_shape[1]}), "
                                 f"got {tuple(x.shape)}")
        return self.proj(x).flatten(2)


def _compl_mul_add_fwd(a: Tensor, b: Tensor, c: Tensor) -> Tensor:
    """``a [B, K, I, X, Y, 2] · b [K, I, O, 2] + c [K, O, 1, 1, 2]`` as complex numbers stored in a trailing pair."""
    out = torch.einsum("bkixy,kio->bkoxy", torch.view_as_complex(a.contiguous()), torch.view_as_complex(b.contiguous()))
    return torch.view_as_real(out + torch.view_as_complex(c.contiguous()))


_compl_mul_add_fwd_c = _compl_mul_add_fwd


class DistributedAFNO2D(Module):
    def __init__(self, hidden_size: int, num_blocks: int = 8, sparsity_threshold: float = 0.01,
                 hard_thresholding_fraction: float = 1, hidden_size_factor: int = 1, input_is_matmul_parallel: bool = False,
                 output_is_matmul_parallel: bool = False):
        super().__init__()
        if hidden_size % num_blocks != 0:
            raise ValueError(f"hidden_size {hidden_size} should be divisible by num_blocks {num_blocks}")
        p = _group_size()
        if num_blocks % p != 0:
            raise ValueError("Error, num_blocks needs to be divisible by matmul_parallel_size")
        self.fft_handle, self.ifft_handle = torch.fft.rfft2, torch.fft.irfft2
        self.hidden_size, self.sparsity_threshold, self.num_blocks = hidden_size, sparsity_threshold, num_blocks
        self.num_blocks_local = num_blocks // p
        self.block_size = hidden_size // num_blocks
        self.hard_thresholding_fraction, self.hidden_size_factor, self.scale = hard_thresholding_fraction, hidden_size_factor, 0.02
        self._mult_handle = _compl_mul_add_fwd
        self.input_is_matmul_parallel, self.output_is_matmul_parallel = input_is_matmul_parallel, output_is_matmul_parallel
        nb, bs, f = self.num_blocks_local, self.block_size, hidden_size_factor
        self.w1 = nn.Parameter(self.scale * torch.randn(nb, bs, bs * f, 2))
        self.b1 = nn.Parameter(self.scale * torch.randn(nb, bs * f, 1, 1, 2))
        self.w2 = nn.Parameter(self.scale * torch.randn(nb, bs * f, bs, 2))
        self.b2 = nn.Parameter(self.scale * torch.randn(nb, bs, 1, 1, 2))
        for prm in (self.w1, self.b1, self.w2, self.b2):
            prm.is_shared_spatial = True

    def forward(self, x: Tensor) -> Tensor:
        if not self.input_is_matmul_parallel:
            num_chans = x.shape[1]
            x = scatter_to_parallel_region(x, dim=1, group=_GROUP)
        bias, dtype = x, x.dtype
        B, C, H, W = x.shape
        total = H // 2 + 1
        kept = int(total * self.hard_thresholding_fraction)
        xf = self.fft_handle(x.float(), (H, W), (-2, -1), "ortho").reshape(B, self.num_blocks_local, self.block_size, H, W // 2 + 1)
        lo, hi = total - kept, min(total + kept, H)
        win = torch.view_as_real(xf[:, :, :, lo:hi, :kept])
        o1 = F.relu(self._mult_handle(win, self.w1, self.b1))
        o2 = F.softshrink(self._mult_handle(o1, self.w2, self.b2), lambd=self.sparsity_threshold)
        o2 = F.pad(o2, [0, 0, 0, W // 2 + 1 - kept, lo, H - hi])
        y = self.ifft_handle(torch.view_as_complex(o2).reshape(B, C, H, W // 2 + 1), (H, W), (-2, -1), "ortho")
        y = y.type(dtype) + bias
        if not self.output_is_matmul_parallel:
            y = gather_from_parallel_region(y, dim=1, shapes=compute_split_shapes(num_chans, _group_size()), group=_GROUP)
        return y

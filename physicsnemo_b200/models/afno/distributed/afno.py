"""Channel-parallel AFNO (FourCastNet-style) over the ``"model_parallel"`` process group.

Parity: ``physicsnemo/models/afno/distributed/afno.py`` (``DistributedBlock``, ``DistributedAFNONet``,
``DistributedAFNO``): activations stay split over channels between blocks; the last block gathers; the
head (replicated, broadcast once from rank 0) and the un-patchify permutation run on full channels.
"""
from __future__ import annotations

from functools import partial
from typing import Tuple, Union

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor

from ....core.module import Module
from ....distributed.manager import DistributedManager
from ....distributed.mappings import copy_to_parallel_region, gather_from_parallel_region, scatter_to_parallel_region
from ....distributed.utils import compute_split_shapes
from ....nn.module.layer_norm import get_layer_norm_class
from .layers import DistributedAFNO2D, DistributedMLP, DistributedPatchEmbed, DropPath

_LayerNormClass = get_layer_norm_class()
_GROUP = "model_parallel"


class DistributedBlock(Module):
    def __init__(self, h: int, w: int, dim: int, mlp_ratio: float = 4.0, drop: float = 0.0, drop_path: float = 0.0,
                 act_layer: type = nn.GELU, norm_layer: Union[type, None] = None, double_skip: bool = True,
                 num_blocks: int = 8, sparsity_threshold: float = 0.01, hard_thresholding_fraction: float = 1.0,
                 input_is_matmul_parallel: bool = False, output_is_matmul_parallel: bool = False):
        super().__init__()
        norm_layer = norm_layer or partial(_LayerNormClass, eps=1e-6)
        self.input_is_matmul_parallel, self.output_is_matmul_parallel = input_is_matmul_parallel, output_is_matmul_parallel
        self.norm1 = norm_layer((h, w))
        self.filter = DistributedAFNO2D(dim, num_blocks, sparsity_threshold, hard_thresholding_fraction,
                                        input_is_matmul_parallel=True, output_is_matmul_parallel=True)
        self.drop_path = DropPath(drop_path) if drop_path > 0.0 else nn.Identity()
        self.norm2 = norm_layer((h, w))
        self.mlp = DistributedMLP(in_features=dim, hidden_features=int(dim * mlp_ratio), act_layer=act_layer, drop=drop,
                                  input_is_matmul_parallel=True, output_is_matmul_parallel=True)
        self.double_skip = double_skip

    def forward(self, x: Tensor) -> Tensor:
        if not self.input_is_matmul_parallel:
            shapes = compute_split_shapes(x.shape[1], DistributedManager().group_size(_GROUP))
            x = scatter_to_parallel_region(x, dim=1, group=_GROUP)
        residual = x
        x = self.filter(self.norm1(x))
        if self.double_skip:
            x = x + residual
            residual = x
        x = self.drop_path(self.mlp(self.norm2(x))) + residual
        if not self.output_is_matmul_parallel:
            if self.input_is_matmul_parallel:
                shapes = compute_split_shapes(x.shape[1] * DistributedManager().group_size(_GROUP),
                                              DistributedManager().group_size(_GROUP))
            x = gather_from_parallel_region(x, dim=1, shapes=shapes, group=_GROUP)
        return x


class DistributedAFNONet(Module):
    def __init__(self, inp_shape: Tuple[int, int] = (720, 1440), patch_size: Tuple[int, int] = (16, 16), in_chans: int = 2,
                 out_chans: int = 2, embed_dim: int = 768, depth: int = 12, mlp_ratio: float = 4.0, drop_rate: float = 0.0,
                 drop_path_rate: float = 0.0, num_blocks: int = 16, sparsity_threshold: float = 0.01,
                 hard_thresholding_fraction: float = 1.0, input_is_matmul_parallel: bool = False,
                 output_is_matmul_parallel: bool = False):
        super().__init__()
        p = DistributedManager().group_size(_GROUP)
        self.inp_shape, self.patch_size, self.in_chans, self.out_chans = inp_shape, patch_size, in_chans, out_chans
        self.num_features = self.embed_dim = embed_dim
        self.num_blocks = num_blocks
        self.input_is_matmul_parallel, self.output_is_matmul_parallel = input_is_matmul_parallel, output_is_matmul_parallel
        norm_layer = partial(_LayerNormClass, eps=1e-6)
        self.patch_embed = DistributedPatchEmbed(inp_shape=inp_shape, patch_size=patch_size, in_chans=in_chans,
                                                 embed_dim=embed_dim, input_is_matmul_parallel=input_is_matmul_parallel,
                                                 output_is_matmul_parallel=True)
        self.embed_dim_local = embed_dim // p
        self.pos_embed = nn.Parameter(torch.zeros(1, self.embed_dim_local, self.patch_embed.num_patches))
        self.pos_drop = nn.Dropout(p=drop_rate)
        dpr = [v.item() for v in torch.linspace(0, drop_path_rate, depth)]
        self.h, self.w = inp_shape[0] // patch_size[0], inp_shape[1] // patch_size[1]
        self.blocks = nn.ModuleList([
            DistributedBlock(h=self.h, w=self.w, dim=embed_dim, mlp_ratio=mlp_ratio, drop=drop_rate, drop_path=dpr[i],
                             norm_layer=norm_layer, num_blocks=num_blocks, sparsity_threshold=sparsity_threshold,
                             hard_thresholding_fraction=hard_thresholding_fraction, input_is_matmul_parallel=True,
                             output_is_matmul_parallel=i < depth - 1) for i in range(depth)])
        self.out_chans_local = (out_chans + p - 1) // p if output_is_matmul_parallel else out_chans
        self.head = nn.Conv2d(embed_dim, self.out_chans_local * patch_size[0] * patch_size[1], 1, bias=False)
        self.synchronized_head = False
        torch.nn.init.trunc_normal_(self.pos_embed, std=0.02)
        self.apply(self._init_weights)

    def _init_weights(self, m: nn.Module) -> None:
        if isinstance(m, (nn.Linear, nn.Conv2d)):
            torch.nn.init.trunc_normal_(m.weight, std=0.02)
            if m.bias is not None:
                nn.init.constant_(m.bias, 0)
        elif isinstance(m, _LayerNormClass):
            nn.init.constant_(m.bias, 0)
            nn.init.constant_(m.weight, 1.0)

    def _no_weight_decay(self) -> set:
        return {"pos_embed", "cls_token"}

    def _forward_features(self, x: Tensor) -> Tensor:
        B = x.shape[0]
        x = self.pos_drop(self.patch_embed(x) + self.pos_embed).reshape(B, self.embed_dim_local, self.h, self.w)
        for blk in self.blocks:
            x = blk(x)
        return x

    def forward(self, x: Tensor) -> Tensor:
        x = self._forward_features(x)
        if self.output_is_matmul_parallel:
            x = copy_to_parallel_region(x, group=_GROUP)
        elif not self.synchronized_head:
            group = DistributedManager().group(_GROUP)
            if dist.is_initialized() and DistributedManager().group_size(_GROUP) > 1:
                src = dist.get_global_rank(group, 0) if group is not None else 0
                for param in self.head.parameters():
                    dist.broadcast(param.data, src, group=group)
            self.synchronized_head = True
        x = self.head(x)
        b, (ph, pw) = x.shape[0], self.patch_size
        x = x.reshape(b, ph, pw, -1, self.h, self.w).permute(0, 3, 4, 1, 5, 2)
        return x.reshape(b, -1, self.h * ph, self.w * pw)


class DistributedAFNO(Module):
    """``forward(x [B, C_in, H, W]) -> [B, C_out, H, W]``; needs a process group named ``"model_parallel"``."""

    def __init__(self, inp_shape: Tuple[int, int], in_channels: int, out_channels: Union[int, None] = None, patch_size: int = 16,
                 embed_dim: int = 256, depth: int = 4, num_blocks: int = 4, channel_parallel_inputs: bool = False,
                 channel_parallel_outputs: bool = False) -> None:
        super().__init__()
        out_channels = out_channels or in_channels
        try:
            group = DistributedManager().group(_GROUP)
        except Exception:  # noqa: BLE001
            group = None
        if group is None:
            raise RuntimeError("Distributed AFNO needs to have model parallel group created first. "
                               "Check the MODEL_PARALLEL_SIZE environment variable")
        if channel_parallel_inputs and in_channels % DistributedManager().group_size(_GROUP) != 0:
            raise ValueError("Error, in_channels needs to be divisible by model_parallel size")
        self.inp_shape, self.in_channels, self.out_channels = inp_shape, in_channels, out_channels
        self._impl = DistributedAFNONet(inp_shape=inp_shape, patch_size=(patch_size, patch_size), in_chans=in_channels,
                                        out_chans=out_channels, embed_dim=embed_dim, depth=depth, num_blocks=num_blocks,
                                        input_is_matmul_parallel=False, output_is_matmul_parallel=False)

    def forward(self, in_vars: Tensor) -> Tensor:
        if not torch.compiler.is_compiling():
            want = (self.in_channels, self.inp_shape[0], self.inp_shape[1])
            if in_vars.ndim != 4 or tuple(in_vars.shape[1:]) != want:
                raise ValueError(f"Expected input shape (B, {want[0]}, {want[1]}, {want[2]}), got {tuple(in_vars.shape)}")
        return self._impl(in_vars)

"""GroupNorm with optional fused activation.

Parity: ``physicsnemo/nn/module/group_norm.py`` — ``get_group_norm`` (``:72-141``) and ``GroupNorm``
(``:144-288``): groups = ``min(num_groups, num_channels // min_channels_per_group)``; training uses
``F.group_norm``, evaluation the explicit mean / (unbiased) variance form; activation by name.
The Apex NHWC kernel of the reference (``use_apex_gn``) is replaced by this package's
GroupNorm(+SiLU) kernels (``ops/group_norm.py``), used for every CUDA bf16 / fp32 input they cover in
either memory format, so ``use_apex_gn=True`` is accepted and maps to the same class.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ...ops import group_norm as _gn
from .utils.utils import _validate_amp


def _compute_groupnorm_groups(num_channels: int, num_groups: int = 32, min_channels_per_group: int = 4) -> int:
    groups = min(num_groups, num_channels // min_channels_per_group)
    groups = max(groups, 1)
    if num_channels % groups != 0:
        raise ValueError(
            f"num_channels ({num_channels}) must be divisible by the number of groups ({groups})"
        )
    return groups


_ACTS = {"silu": F.silu, "relu": F.relu, "leaky_relu": F.leaky_relu, "sigmoid": torch.sigmoid, "tanh": torch.tanh,
         "gelu": F.gelu, "elu": F.elu}


class GroupNorm(torch.nn.Module):
    """Group normalisation over (B, C, H, W) with ``weight`` / ``bias`` of size C."""

    def __init__(self, num_channels: int, num_groups: int = 32, min_channels_per_group: int = 4, eps: float = 1e-5,
                 use_apex_gn: bool = False, fused_act: bool = False, act: str | None = None, amp_mode: bool = False):
        super().__init__()
        if use_apex_gn:
            raise ValueError("'use_apex_gn' is deprecated. Please use 'get_group_norm' to enable Apex-based group norm.")
        if fused_act:
            raise ValueError(
                "'fused_act' is deprecated and only supported for Apex-based group norm. "
                "Please use `get_group_norm` to enable fused activations."
            )
        self.num_groups = _compute_groupnorm_groups(num_channels, num_groups, min_channels_per_group)
        self.eps = eps
        self.weight = torch.nn.Parameter(torch.ones(num_channels))
        self.bias = torch.nn.Parameter(torch.zeros(num_channels))
        self.act = act.lower() if act else act
        self.act_fn = self.get_activation_function() if self.act is not None else None
        self.amp_mode = amp_mode

    def get_activation_function(self):
        fn = _ACTS.get(self.act)
        if fn is None:
            raise ValueError(f"Unknown activation function: {self.act}")
        return fn

    def forward(self, x):
        weight, bias = self.weight, self.bias
        _validate_amp(self.amp_mode)
        if not self.amp_mode:
            if weight.dtype != x.dtype:
                weight = weight.to(x.dtype)
            if bias.dtype != x.dtype:
                bias = bias.to(x.dtype)
        if type(x) is not torch.Tensor:
            from ...parallel.shard_tensor import ShardTensor

            if isinstance(x, ShardTensor):   # moments over all shards, fused with the activation where the kernels cover it
                from ...parallel.patches.norm import group_norm_act

                return group_norm_act(x, self.num_groups, self.weight, self.bias, self.eps, self.act)
        if type(x) is torch.Tensor and x.is_cuda and _gn.supported(x, self.num_groups):
            # one kernel pair for norm + affine (+ SiLU); same arithmetic in training and evaluation
            fuse = self.act == "silu"
            x = _gn.group_norm(x, self.num_groups, self.weight, self.bias, self.eps, silu=fuse)
            return x if fuse or self.act_fn is None else self.act_fn(x)
        if self.training:
            x = F.group_norm(x, num_groups=self.num_groups, weight=weight, bias=bias, eps=self.eps)
        else:
            b, c = x.shape[:2]
            xg = x.reshape(b, self.num_groups, c // self.num_groups, *x.shape[2:])
            dims = list(range(2, xg.dim()))
            mean = xg.mean(dim=dims, keepdim=True)
            var = xg.var(dim=dims, keepdim=True)
            xg = (xg - mean) * (var + self.eps).rsqrt()
            shape = [1, c] + [1] * (x.dim() - 2)
            x = xg.reshape(x.shape) * weight.reshape(shape) + bias.reshape(shape)
        if self.act_fn is not None:
            x = self.act_fn(x)
        return x


def get_group_norm(num_channels: int, num_groups: int = 32, min_channels_per_group: int = 4, eps: float = 1e-5,
                   use_apex_gn: bool = False, act: str | None = None, amp_mode: bool = False) -> torch.nn.Module:
    """Factory used by the U-Net layers; ``use_apex_gn`` selects the same class here."""
    return GroupNorm(num_channels=num_channels, num_groups=num_groups, min_channels_per_group=min_channels_per_group,
                     eps=eps, act=act.lower() if act else act, amp_mode=amp_mode)

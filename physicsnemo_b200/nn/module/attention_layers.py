"""Attention layers for image models.

Parity: ``physicsnemo/nn/module/attention_layers.py`` — ``AttentionOp`` (fp32 softmax with an
explicit backward, ``:29-66``) and ``UNetAttention`` (``:69-178``: GroupNorm → 1×1 ``qkv`` conv →
(B, heads, HW, 3, C/heads) → SDPA with ``scale = 1/sqrt(d)`` → 1×1 ``proj`` + residual).
"""
from __future__ import annotations

import math
from typing import Any, Dict

import numpy as np
import torch

from .conv_layers import Conv2d
from .group_norm import get_group_norm


class AttentionOp(torch.autograd.Function):
    """``softmax(q^T k / sqrt(d))`` computed in fp32 with a hand-written backward."""

    @staticmethod
    def forward(ctx, q, k):
        w = (
            torch.einsum("ncq,nck->nqk", q.to(torch.float32), (k / np.sqrt(k.shape[1])).to(torch.float32))
            .softmax(dim=2)
            .to(q.dtype)
        )
        ctx.save_for_backward(q, k, w)
        return w

    @staticmethod
    def backward(ctx, dw):
        q, k, w = ctx.saved_tensors
        db = torch._softmax_backward_data(grad_output=dw.to(torch.float32), output=w.to(torch.float32), dim=2,
                                          input_dtype=torch.float32)
        dq = torch.einsum("nck,nqk->ncq", k.to(torch.float32), db).to(q.dtype) / np.sqrt(k.shape[1])
        dk = torch.einsum("ncq,nqk->nck", q.to(torch.float32), db).to(k.dtype) / np.sqrt(k.shape[1])
        return dq, dk


def _wide_head_gemm_attention(q: torch.Tensor) -> bool:
    """Plain CUDA 16-bit tensors with a head wider than the flash kernels take (the 512-wide single head of the
    SongUNet bottleneck): attention as two tcgen05 GEMMs around the library's row softmax (``ops/gemm_attention.py``)."""
    if type(q) is not torch.Tensor or not q.is_cuda or q.dtype not in (torch.bfloat16, torch.float16):
        return False
    if q.shape[-1] <= 128 or q.shape[-1] % 8 or q.shape[-2] % 8 or q.shape[0] * q.shape[1] > 16:
        return False
    from ...ops import _lib

    return _lib.available()


class UNetAttention(torch.nn.Module):
    """Self-attention over the pixels of a feature map (keys ``norm``, ``qkv``, ``proj``)."""

    def __init__(self, *, out_channels: int, num_heads: int, eps: float = 1e-5,
                 init_zero: Dict[str, Any] = dict(init_weight=0), init_attn: Any = None,
                 init: Dict[str, Any] = dict(), use_apex_gn: bool = False, amp_mode: bool = False,
                 fused_conv_bias: bool = False) -> None:
        super().__init__()
        if not isinstance(num_heads, int) or num_heads <= 0:
            raise ValueError(f"`num_heads` must be a positive integer, but got {num_heads}")
        if out_channels % num_heads != 0:
            raise ValueError(
                f"`out_channels` must be divisible by `num_heads`, but got {out_channels} and {num_heads}"
            )
        self.num_heads = num_heads
        self.norm = get_group_norm(num_channels=out_channels, eps=eps, use_apex_gn=use_apex_gn, amp_mode=amp_mode)
        self.qkv = Conv2d(in_channels=out_channels, out_channels=out_channels * 3, kernel=1,
                          fused_conv_bias=fused_conv_bias, amp_mode=amp_mode,
                          **(init_attn if init_attn is not None else init))
        self.proj = Conv2d(in_channels=out_channels, out_channels=out_channels, kernel=1,
                           fused_conv_bias=fused_conv_bias, amp_mode=amp_mode, **init_zero)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x1 = self.qkv(self.norm(x))
        qkv = x1.reshape(x.shape[0], self.num_heads, x.shape[1] // self.num_heads, 3, -1).permute(0, 1, 4, 3, 2)
        q, k, v = (qkv[..., i, :] for i in range(3))
        if _wide_head_gemm_attention(q):
            from ...ops.gemm_attention import gemm_attention

            attn = gemm_attention(q, k, v, 1 / math.sqrt(k.shape[-1]))
        else:
            attn = torch.nn.functional.scaled_dot_product_attention(q, k, v, scale=1 / math.sqrt(k.shape[-1]))
        attn = attn.transpose(-1, -2)
        return self.proj(attn.reshape(*x.shape)) + x


class _EarthAttention(torch.nn.Module):
    """Window attention with the earth-specific position bias of Pangu-Weather.

    Parity: ``physicsnemo/nn/module/attention_layers.py:181-394`` (``EarthAttention3D`` / ``EarthAttention2D``).
    Input ``[B·n_lon, n_windows, N, C]``; the bias table holds one entry per (absolute pressure / latitude pair,
    relative longitude) and per *type of window* (pressure–latitude window position).  Bias and the
    shifted-window mask are folded into one additive mask of a single fused scaled-dot-product call.
    """

    _ndim = 3

    def __init__(self, dim, input_resolution, window_size, num_heads, qkv_bias=True, qk_scale=None, attn_drop=0.0,
                 proj_drop=0.0):
        super().__init__()
        from .utils import get_earth_position_index

        self.dim, self.window_size, self.num_heads = dim, window_size, num_heads
        self.scale = qk_scale or (dim // num_heads) ** -0.5
        *abs_w, w_lon = window_size
        self.type_of_windows, table = 1, 2 * w_lon - 1
        for n, w in zip(input_resolution, abs_w):
            self.type_of_windows *= n // w
            table *= w * w
        self.earth_position_bias_table = torch.nn.Parameter(torch.zeros(table, self.type_of_windows, num_heads))
        self.register_buffer("earth_position_index", get_earth_position_index(window_size, ndim=self._ndim))
        self.qkv = torch.nn.Linear(dim, dim * 3, bias=qkv_bias)
        self.attn_drop = torch.nn.Dropout(attn_drop)
        self.proj = torch.nn.Linear(dim, dim)
        self.proj_drop = torch.nn.Dropout(proj_drop)
        torch.nn.init.trunc_normal_(self.earth_position_bias_table, std=0.02)
        self.softmax = torch.nn.Softmax(dim=-1)

    def forward(self, x: torch.Tensor, mask=None):
        B_, nW, N, C = x.shape
        H = self.num_heads
        q, k, v = self.qkv(x).reshape(B_, nW, N, 3, H, C // H).permute(3, 0, 4, 1, 2, 5)      # [B_, H, nW, N, d]
        bias = self.earth_position_bias_table[self.earth_position_index.view(-1)].view(N, N, self.type_of_windows, H)
        bias = bias.permute(3, 2, 0, 1).unsqueeze(0)                                           # [1, H, nW, N, N]
        if mask is not None:
            n_lon = mask.shape[0]
            bias = (bias.unsqueeze(1) + mask[None, :, None]).expand(B_ // n_lon, -1, -1, -1, -1, -1).reshape(B_, H, nW, N, N)
        out = torch.nn.functional.scaled_dot_product_attention(
            q, k, v, attn_mask=bias.to(q.dtype), dropout_p=self.attn_drop.p if self.training else 0.0, scale=self.scale)
        out = out.permute(0, 2, 3, 1, 4).reshape(B_, nW, N, C)
        return self.proj_drop(self.proj(out))


class EarthAttention3D(_EarthAttention):
    _ndim = 3


class EarthAttention2D(_EarthAttention):
    _ndim = 2

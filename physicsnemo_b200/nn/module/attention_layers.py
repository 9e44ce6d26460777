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
        attn = torch.nn.functional.scaled_dot_product_attention(q, k, v, scale=1 / math.sqrt(k.shape[-1]))
        attn = attn.transpose(-1, -2)
        return self.proj(attn.reshape(*x.shape)) + x

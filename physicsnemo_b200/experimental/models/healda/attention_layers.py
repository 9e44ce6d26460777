"""Attention layers of the HealDA assimilation models: attention along the time axis of every grid pixel, and cross
attention from grid pixels to their packed observation tokens.

Counterpart of ``physicsnemo/experimental/models/healda/attention_layers.py`` (``mask_causal`` :44, ``TemporalAttention``
:78, ``CrossAttentionModuleBase`` :205, ``_pixel_attention_reference`` :243, ``PixelCrossAttention`` :298); parameter
names are the same.  The cross attention runs on ``ops.pixel_attention`` (projections re-associated to the pixel side,
one variable-length kernel in token space) on every device; there is no separate slow path.
"""

from __future__ import annotations

import math
from typing import Any, Optional

import torch
import torch.nn as nn

from ....nn.module.rope import apply_rotary_pos_emb
from ....ops.pixel_attention import pixel_attention
from .obs_context import PixelGroupMap

__all__ = ["mask_causal", "TemporalAttention", "CrossAttentionModuleBase", "PixelCrossAttention"]


def mask_causal(attn: torch.Tensor, linear: bool = True, window: Optional[int] = None) -> torch.Tensor:
    """Mask ``[B, Tq, Tk, X, H]`` scores so step ``q`` sees steps ``k <= q`` (and ``k > q - window``); masked entries become
    0 for linear attention and ``-inf`` before a softmax."""
    tq, tk = attn.shape[1], attn.shape[2]
    hide = torch.ones(tq, tk, dtype=torch.bool, device=attn.device).triu(diagonal=1)
    if window is not None:
        hide = hide | torch.ones(tq, tk, dtype=torch.bool, device=attn.device).tril(diagonal=-window)
    return attn.masked_fill(hide.view(1, tq, tk, 1, 1), 0.0 if linear else float("-inf"))


class TemporalAttention(nn.Module):
    """Attention over the time axis of ``[B, T, X, C]``, independently for every pixel; linear (no softmax) by default."""

    def __init__(self, *, hidden_size: int, num_heads: int, use_rope: bool = True, is_causal: bool = False,
                 linear_attention: bool = True, causal_window: Optional[int] = None):
        if causal_window is not None and not is_causal:
            raise ValueError("causal_window was set but is_causal=False")
        super().__init__()
        self.hidden_size, self.num_heads, self.head_dim = hidden_size, num_heads, hidden_size // num_heads
        self.use_rope, self.is_causal, self.linear_attention, self.causal_window = use_rope, is_causal, linear_attention, causal_window
        self._time_parallel_group = None
        self.qkv = nn.Linear(hidden_size, hidden_size * 3)
        self.proj = nn.Linear(hidden_size, hidden_size)

    def forward(self, x: torch.Tensor, rope_cos: Optional[torch.Tensor] = None, rope_sin: Optional[torch.Tensor] = None) -> torch.Tensor:
        if not torch.compiler.is_compiling():
            if x.ndim != 4:
                raise ValueError(f"Expected 4D input (B, T, X, C), got {x.ndim}D tensor with shape {tuple(x.shape)}")
            if x.shape[-1] != self.hidden_size:
                raise ValueError(f"Expected hidden_size {self.hidden_size}, got {x.shape[-1]} channels")
            if self.use_rope and (rope_cos is None or rope_sin is None):
                raise ValueError("use_rope=True but rope_cos/rope_sin were not provided")
        B, T, X, _ = x.shape
        q, k, v = self.qkv(x).view(B, T, X, 3, self.num_heads, self.head_dim).unbind(3)       # [B, T, X, H, c]
        if self.use_rope:
            cos, sin = rope_cos.view(1, T, 1, 1, -1), rope_sin.view(1, T, 1, 1, -1)
            q, k = apply_rotary_pos_emb(q, cos, sin), apply_rotary_pos_emb(k, cos, sin)
        attn = torch.einsum("bqxhc,bkxhc->bqkxh", q, k / math.sqrt(self.head_dim))
        if self.is_causal:
            attn = mask_causal(attn, linear=self.linear_attention, window=self.causal_window)
        if not self.linear_attention:
            attn = attn.softmax(2)
        out = torch.einsum("bqkxh,bkxhc->bqxhc", attn, v).reshape(B, T, X, self.hidden_size)
        return self.proj(out)


class CrossAttentionModuleBase(nn.Module):
    """Interface of the cross-attention modules a HealDA block can host: ``forward(hidden_states, **kwargs)``."""

    def forward(self, hidden_states: torch.Tensor, **cross_attn_kwargs: Any) -> torch.Tensor:   # pragma: no cover - interface
        raise NotImplementedError


class PixelCrossAttention(CrossAttentionModuleBase):
    """Grouped-query cross attention of every ``(batch, time, pixel)`` site over its own observation tokens."""

    def __init__(self, hidden_size: int, token_dim: int, n_q_heads: int, n_kv_heads: int, d_head: int, use_proj_bias: bool = False):
        super().__init__()
        if n_kv_heads < 1 or (n_kv_heads > 2 and n_kv_heads % 2 != 0):
            raise ValueError(f"PixelCrossAttention requires n_kv_heads=1,2 or an even number, got {n_kv_heads}")
        if n_q_heads % n_kv_heads != 0:
            raise ValueError(f"n_q_heads={n_q_heads} must be divisible by n_kv_heads={n_kv_heads}")
        self.hidden_size, self.token_dim, self.n_q_heads, self.n_kv_heads, self.d_head = hidden_size, token_dim, n_q_heads, n_kv_heads, d_head
        self.attn_dim = n_q_heads * d_head
        self.scale = 1.0 / math.sqrt(d_head)
        self.q_proj = nn.Linear(hidden_size, self.attn_dim, bias=use_proj_bias)
        self.k_proj = nn.Linear(token_dim, n_kv_heads * d_head, bias=False)
        self.v_proj = nn.Linear(token_dim, n_kv_heads * d_head, bias=use_proj_bias)
        self.out_proj = nn.Linear(self.attn_dim, hidden_size, bias=use_proj_bias)

    def forward(self, hidden_states: torch.Tensor, tokens: torch.Tensor, cu_seqlens_k: torch.Tensor, max_seqlen_k: int = 0,
                group_map: Optional[PixelGroupMap] = None) -> torch.Tensor:
        if not torch.compiler.is_compiling():
            if tokens is None:
                raise ValueError("tokens must be set before PixelCrossAttention forward")
            if hidden_states.ndim != 4:
                raise ValueError(f"Expected hidden_states of shape (B, T, X, C), got {hidden_states.ndim}D tensor with shape "
                                 f"{tuple(hidden_states.shape)}")
            if hidden_states.shape[-1] != self.hidden_size:
                raise ValueError(f"Expected hidden_size {self.hidden_size}, got {hidden_states.shape[-1]} channels")
        b, t, x, _ = hidden_states.shape
        P = b * t * x
        if not torch.compiler.is_compiling():
            if cu_seqlens_k.numel() != P + 1:
                raise ValueError(f"Expected cu_seqlens_k length {P + 1} (B*T*X+1), got {cu_seqlens_k.numel()}")
            if int(cu_seqlens_k[-1]) != tokens.shape[0]:
                raise ValueError(f"Expected {tokens.shape[0]} packed tokens, but cu_seqlens_k ends at {int(cu_seqlens_k[-1])}")
        Q = self.q_proj(hidden_states.reshape(P, self.hidden_size)).view(P, self.n_q_heads, self.d_head)
        attn = pixel_attention(Q, tokens, self.k_proj.weight, self.v_proj.weight, cu_seqlens_k, max_seqlen_k, n_kv_heads=self.n_kv_heads,
                               scale=self.scale, B_v=self.v_proj.bias, group_map=group_map)
        return self.out_proj(attn.reshape(P, self.attn_dim)).view(b, t, x, self.hidden_size)

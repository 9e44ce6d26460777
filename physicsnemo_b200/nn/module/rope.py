"""Rotary position embeddings: 1-D and axial 2-D tables and their application.

Parity: ``physicsnemo/nn/module/rope.py`` — interleaved-pair convention (channels ``2i, 2i+1`` rotate
together), ``θ^{-k/d}`` frequencies; the 2-D variant spends the first half of the head on the row index and
the second half on the column index.  Tables are non-persistent buffers rebuilt when the latent size changes.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ...core import Module


def _pair_tables(pos: torch.Tensor, n_channels: int, theta: float):
    k = torch.arange(0, n_channels, 2, dtype=torch.float32, device=pos.device)
    ang = pos[:, None] * theta ** (-k / n_channels)[None, :]
    return ang.cos().repeat_interleave(2, dim=-1), ang.sin().repeat_interleave(2, dim=-1)


def build_rope_cos_sin_1d(seq_len: int, head_dim: int, theta: float = 10000.0, device=None):
    if head_dim % 2 != 0:
        raise ValueError(f"head_dim={head_dim} must be even for 1D RoPE (rotation acts on adjacent channel pairs).")
    cos, sin = _pair_tables(torch.arange(seq_len, dtype=torch.float32, device=device), head_dim, theta)
    return cos.contiguous(), sin.contiguous()


def build_axial_rope_cos_sin_2d(h: int, w: int, head_dim: int, theta: float = 10000.0, device=None):
    if head_dim % 4 != 0:
        raise ValueError(f"head_dim={head_dim} must be divisible by 4 for axial 2D RoPE "
                         "(half per axis, then adjacent pairs within each half).")
    half = head_dim // 2
    cr, sr = _pair_tables(torch.arange(h, dtype=torch.float32, device=device), half, theta)
    cc, sc = _pair_tables(torch.arange(w, dtype=torch.float32, device=device), half, theta)
    cos = torch.cat([cr[:, None].expand(h, w, half), cc[None].expand(h, w, half)], dim=-1)
    sin = torch.cat([sr[:, None].expand(h, w, half), sc[None].expand(h, w, half)], dim=-1)
    return cos.contiguous(), sin.contiguous()


def apply_rotary_pos_emb(x, cos, sin):
    """Rotate adjacent channel pairs of ``x`` (computed in fp32, returned in the input dtype)."""
    dt = x.dtype
    x = x.float()
    rot = torch.stack((-x[..., 1::2], x[..., 0::2]), dim=-1).flatten(-2)
    return (x * cos + rot * sin).to(dt)


class RotaryEmbedding2DTables(Module):
    def __init__(self, head_dim: int, latent_hw: Tuple[int, int], theta: float = 10000.0):
        super().__init__()
        if head_dim % 4 != 0:
            raise ValueError(f"head_dim={head_dim} must be divisible by 4 for axial 2D RoPE.")
        self.head_dim, self.theta = int(head_dim), float(theta)
        self._latent_hw = (int(latent_hw[0]), int(latent_hw[1]))
        cos, sin = build_axial_rope_cos_sin_2d(*self._latent_hw, self.head_dim, theta=self.theta)
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)

    def _maybe_rebuild(self, h: int, w: int) -> None:
        if (int(h), int(w)) == self._latent_hw:
            return
        dt, dev = self.rope_cos.dtype, self.rope_cos.device
        cos, sin = build_axial_rope_cos_sin_2d(h, w, self.head_dim, theta=self.theta, device=dev)
        self.register_buffer("rope_cos", cos.to(dt), persistent=False)
        self.register_buffer("rope_sin", sin.to(dt), persistent=False)
        self._latent_hw = (int(h), int(w))

    def forward(self, latent_hw: Optional[Tuple[int, int]] = None):
        if latent_hw is not None:
            self._maybe_rebuild(int(latent_hw[0]), int(latent_hw[1]))
        return self.rope_cos, self.rope_sin


class RotaryEmbedding1DTables(Module):
    def __init__(self, head_dim: int, max_seq_len: int, theta: float = 10000.0):
        super().__init__()
        if head_dim % 2 != 0:
            raise ValueError(f"head_dim={head_dim} must be even for 1D RoPE.")
        self.head_dim, self.theta, self.max_seq_len = int(head_dim), float(theta), int(max_seq_len)
        cos, sin = build_rope_cos_sin_1d(self.max_seq_len, self.head_dim, theta=self.theta)
        self.register_buffer("cos", cos, persistent=False)
        self.register_buffer("sin", sin, persistent=False)

    def forward(self, seq_len: Optional[int] = None):
        if seq_len is None:
            return self.cos, self.sin
        if not torch.compiler.is_compiling() and seq_len > self.max_seq_len:
            raise ValueError(f"sequence length {seq_len} exceeds max_seq_len={self.max_seq_len}")
        return self.cos[:seq_len], self.sin[:seq_len]

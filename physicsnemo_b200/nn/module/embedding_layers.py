"""Embedding layers for diffusion / transformer models.

Parity: ``physicsnemo/nn/module/embedding_layers.py`` — ``FourierEmbedding`` (``:29``),
``PositionalEmbedding`` (``:67-152``: ``freqs`` buffer, ``cos_sin`` / ``np_sin_cos``
ordering, optional learnable MLP), ``SinusoidalTimestepEmbedding``, ``OneHotEmbedding``.
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn as nn


class FourierEmbedding(nn.Module):
    """Random Fourier features of a scalar (noise level) input."""

    def __init__(self, num_channels: int, scale: int = 16, amp_mode: bool = False):
        super().__init__()
        self.register_buffer("freqs", torch.randn(num_channels // 2) * scale)
        self.amp_mode = amp_mode

    def forward(self, x):
        freqs = self.freqs
        if not self.amp_mode and x.dtype != freqs.dtype:
            freqs = freqs.to(x.dtype)
        x = x.ger(2 * np.pi * freqs)
        return torch.cat([x.cos(), x.sin()], dim=1)


class PositionalEmbedding(nn.Module):
    """Sinusoidal embedding ``[cos(x f), sin(x f)]`` with ``f_i = max_positions^(-i/(C/2))``."""

    def __init__(self, num_channels: int, max_positions: int = 10000, endpoint: bool = False,
                 amp_mode: bool = False, learnable: bool = False, freq_embed_dim: int | None = None,
                 mlp_hidden_dim: int | None = None, embed_fn: str = "cos_sin"):
        super().__init__()
        self.num_channels = num_channels
        self.max_positions = max_positions
        self.endpoint = endpoint
        self.amp_mode = amp_mode
        self.learnable = learnable
        self.embed_fn = embed_fn
        if embed_fn not in ("cos_sin", "np_sin_cos"):
            raise ValueError(f"embed_fn must be 'cos_sin' or 'np_sin_cos', got {embed_fn}")
        if learnable:
            self.freq_embed_dim = freq_embed_dim or num_channels
            self.mlp_hidden_dim = mlp_hidden_dim or 2 * num_channels
            self.mlp = nn.Sequential(
                nn.Linear(self.freq_embed_dim, self.mlp_hidden_dim, bias=True), nn.SiLU(),
                nn.Linear(self.mlp_hidden_dim, num_channels, bias=True),
            )
            n = self.freq_embed_dim // 2
        else:
            n = num_channels // 2
        freqs = torch.arange(start=0, end=n, dtype=torch.float32)
        freqs = freqs / (n - (1 if endpoint else 0))
        freqs = (1 / max_positions) ** freqs
        self.register_buffer("freqs", freqs, persistent=True)
        self._register_load_state_dict_pre_hook(self._fill_missing_freqs, with_module=False)

    def _fill_missing_freqs(self, state_dict, prefix, *args):
        # checkpoints written before ``freqs`` became a persistent buffer lack the key
        key = prefix + "freqs"
        if key not in state_dict:
            state_dict[key] = self.freqs.detach().clone()

    def forward(self, x):
        freqs = self.freqs
        if not self.amp_mode and x.dtype != freqs.dtype:
            freqs = freqs.to(x.dtype)
        x = x.ger(freqs)
        if self.embed_fn == "cos_sin":
            x = torch.cat([x.cos(), x.sin()], dim=1)
        else:
            x = torch.cat([x.sin(), x.cos()], dim=1)
        if self.learnable:
            x = self.mlp(x)
        return x


class SinusoidalTimestepEmbedding(nn.Module):
    """Embedding of a scalar in [0, 1]: ``cat(cos(pi k t), sin(pi k t))`` for ``k = 1 .. num_channels // 2``.

    Parity: ``physicsnemo/nn/module/embedding_layers.py`` (``SinusoidalTimestepEmbedding``; persistent buffer ``freqs``).
    """

    def __init__(self, num_channels: int):
        super().__init__()
        self.num_channels = num_channels
        self.register_buffer("freqs", torch.pi * torch.arange(1, num_channels // 2 + 1, dtype=torch.float32))

    def forward(self, t):
        arg = t.reshape(-1).outer(self.freqs.to(t.dtype))
        return torch.cat([arg.cos(), arg.sin()], dim=1)


class OneHotEmbedding(nn.Module):
    """Soft one-hot embedding of ``t`` in [0, 1] over ``num_channels`` bins."""

    def __init__(self, num_channels: int):
        super().__init__()
        self.num_channels = num_channels
        ind = torch.arange(num_channels).view(1, -1)
        self.register_buffer("indices", ind)

    def forward(self, t):
        ind = t * (self.num_channels - 1)
        return torch.clamp(1 - torch.abs(ind - self.indices), min=0)


class FourierPositionalEmbedding(nn.Module):
    """Parameter-free per-axis Fourier features of coordinates (the encoding of implicit decoders).

    Every coordinate ``x_a`` becomes ``[sin(f_0 x_a) … sin(f_{F-1} x_a), cos(f_0 x_a) … cos(f_{F-1} x_a)]``
    with ``f_i = base_freq · freq_scale^i`` (or an explicit ``freqs`` vector); the axes follow one another and
    the raw coordinates come first when ``include_input``.  Parity:
    ``physicsnemo/nn/module/embedding_layers.py:263`` (persistent ``freqs`` buffer, ``out_dim`` property).
    """

    def __init__(self, in_dim: int = 3, num_bands: int = 10, include_input: bool = True, base_freq: float = math.pi,
                 freq_scale: float = 2.0, freqs: torch.Tensor | None = None):
        super().__init__()
        if in_dim < 1:
            raise ValueError(f"in_dim must be >= 1, got {in_dim}")
        if freqs is None:
            if num_bands < 1:
                raise ValueError(f"num_bands must be >= 1, got {num_bands}")
            table = base_freq * freq_scale ** torch.arange(num_bands, dtype=torch.float32)
        else:
            table = torch.as_tensor(freqs, dtype=torch.float32)
            if table.ndim != 1 or table.numel() < 1:
                raise ValueError(f"freqs must be a 1-D tensor of shape (F,) with F >= 1, got shape {tuple(table.shape)}.")
        self.in_dim, self.include_input = int(in_dim), bool(include_input)
        self.register_buffer("freqs", table)

    @property
    def num_bands(self) -> int:
        return self.freqs.numel()

    @property
    def out_dim(self) -> int:
        return self.in_dim * (2 * self.num_bands + int(self.include_input))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[-1] != self.in_dim:
            raise ValueError(f"Expected tensor with last dim {self.in_dim}, got tensor of shape {tuple(x.shape)}")
        phase = x[..., None] * self.freqs.to(x.dtype)
        waves = torch.cat([phase.sin(), phase.cos()], dim=-1).flatten(-2)
        return torch.cat([x, waves], dim=-1) if self.include_input else waves

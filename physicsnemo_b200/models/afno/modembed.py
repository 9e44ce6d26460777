"""Embedding network of the modulation input (a lead time) of ``ModAFNO``.

Parity: ``physicsnemo/models/afno/modembed.py:33-`` — the time, scaled by ``max_time``, is embedded sinusoidally or as a
soft one-hot vector and passed through ``depth`` Linear + activation layers (keys ``mlp.{2i}.weight|bias``).
"""
from __future__ import annotations

from typing import Type

import torch
import torch.nn as nn

from ...core.module import Module
from ...nn.module.embedding_layers import OneHotEmbedding, SinusoidalTimestepEmbedding


class ModEmbedNet(Module):
    """``t`` of shape (B,) or (B, 1) → embedding (B, dim)."""

    def __init__(self, max_time: float = 1.0, dim: int = 64, depth: int = 1, activation_fn: Type[nn.Module] = nn.GELU,
                 method: str = "sinusoidal"):
        super().__init__()
        self.max_time, self.method, self.dim = max_time, method, dim
        if method == "onehot":
            self.onehot_embed = OneHotEmbedding(dim)
        elif method == "sinusoidal":
            self.sinusoid_embed = SinusoidalTimestepEmbedding(dim)
        else:
            raise ValueError(f"modulation embedding method must be 'sinusoidal' or 'onehot', got '{method}'")
        layers = []
        for _ in range(depth):
            layers += [nn.Linear(dim, dim), activation_fn()]
        self.mlp = nn.Sequential(*layers)

    def forward(self, t: torch.Tensor) -> torch.Tensor:
        t = t / self.max_time
        if self.method == "onehot":
            emb = self.onehot_embed(t.reshape(-1, 1))
        else:
            emb = self.sinusoid_embed(t.reshape(-1))
        return self.mlp(emb)

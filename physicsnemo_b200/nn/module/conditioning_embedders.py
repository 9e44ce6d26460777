"""Conditioning embedders for diffusion backbones (parity: ``physicsnemo/nn/module/conditioning_embedders.py``)."""
import math
from enum import Enum
from typing import Any, Protocol, runtime_checkable

import torch
import torch.nn as nn

from ...core import Module
from .embedding_layers import PositionalEmbedding
from .fully_connected_layers import Linear


@runtime_checkable
class ConditioningEmbedder(Protocol):
    """``forward(t, **kwargs) -> [batch, output_dim]``."""

    @property
    def output_dim(self) -> int: ...

    def forward(self, t, **kwargs): ...


class ZeroConditioningEmbedder(Module):
    """Emits an empty ``[batch, 0]`` embedding (unconditional backbones)."""

    def __init__(self):
        super().__init__()
        self._output_dim = 0

    @property
    def output_dim(self) -> int:
        return self._output_dim

    def forward(self, t, **kwargs):
        return torch.empty(t.shape[0], 0, device=t.device, dtype=t.dtype)


class DiTConditionEmbedder(Module):
    """Learnable sinusoidal timestep embedding plus an optional zero-initialised linear map of the condition."""

    def __init__(self, hidden_size: int, condition_dim: int = 0, amp_mode: bool = False, **timestep_embed_kwargs: Any):
        super().__init__()
        self._output_dim = hidden_size
        self.t_embedder = PositionalEmbedding(num_channels=hidden_size, amp_mode=amp_mode, learnable=True,
                                              **timestep_embed_kwargs)
        self.cond_embedder = Linear(in_features=condition_dim, out_features=hidden_size, bias=False, amp_mode=amp_mode,
                                    init_mode="kaiming_uniform", init_weight=0, init_bias=0) if condition_dim else None

    @property
    def output_dim(self) -> int:
        return self._output_dim

    def forward(self, t, condition=None, **kwargs):
        c = self.t_embedder(t)
        if self.cond_embedder is not None and condition is not None:
            c = c + self.cond_embedder(condition)
        return c


class EDMConditionEmbedder(Module):
    """EDM noise embedding: sin/cos positional features (+ scaled condition map, with train-time condition
    dropout) → Linear → SiLU → Linear."""

    def __init__(self, emb_channels: int, noise_channels: int, condition_dim: int = 0, condition_dropout: float = 0.0,
                 legacy_condition_bias: bool = False, max_positions: int = 10000, **kwargs):
        super().__init__()
        self._output_dim = emb_channels
        self.condition_dropout = condition_dropout
        self.legacy_condition_bias = legacy_condition_bias
        self.map_noise = PositionalEmbedding(num_channels=noise_channels, max_positions=max_positions, endpoint=True,
                                             learnable=False, embed_fn="np_sin_cos")
        self.map_condition = nn.Linear(condition_dim, noise_channels) if (condition_dim > 0 or legacy_condition_bias) else None
        self.map_layer0 = nn.Linear(noise_channels, emb_channels)
        self.map_layer1 = nn.Linear(emb_channels, emb_channels)

    @property
    def output_dim(self) -> int:
        return self._output_dim

    def forward(self, t, condition=None, **kwargs):
        emb = self.map_noise(t)
        if self.map_condition is not None and condition is not None:
            c = condition
            if self.training and self.condition_dropout:
                keep = torch.rand([t.shape[0], 1], device=c.device) >= self.condition_dropout
                c = c * keep.to(c.dtype)
            emb = emb + self.map_condition(c * math.sqrt(self.map_condition.in_features))
        return self.map_layer1(torch.nn.functional.silu(self.map_layer0(emb)))


class ConditioningEmbedderType(Enum):
    DIT = DiTConditionEmbedder
    EDM = EDMConditionEmbedder
    ZERO = ZeroConditioningEmbedder


def get_conditioning_embedder(conditioning_embedder: ConditioningEmbedderType = ConditioningEmbedderType.DIT,
                              **kwargs: Any) -> ConditioningEmbedder:
    cls = conditioning_embedder.value
    return cls() if conditioning_embedder is ConditioningEmbedderType.ZERO else cls(**kwargs)

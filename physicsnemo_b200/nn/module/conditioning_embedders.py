"""Conditioning embedders for diffusion backbones (parity: ``physicsnemo/nn/module/conditioning_embedders.py``).

An embedder turns the diffusion time (and optionally a per-sample condition vector) into the ``[batch, output_dim]``
vector that modulates every block of a DiT / EDM backbone.  Sub-module names (``t_embedder``, ``cond_embedder``,
``map_noise``, ``map_condition``, ``map_layer0/1``) are checkpoint keys.
"""
import math
from enum import Enum
from typing import Any, Protocol, runtime_checkable

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...core import Module
from .embedding_layers import PositionalEmbedding
from .fully_connected_layers import Linear


@runtime_checkable
class ConditioningEmbedder(Protocol):
    """``forward(t, **kwargs) -> [batch, output_dim]``."""

    @property
    def output_dim(self) -> int: ...

    def forward(self, t, **kwargs): ...


class _Embedder(Module):
    """Shared bookkeeping: the width of the produced embedding."""

    def __init__(self, width: int):
        super().__init__()
        self._output_dim = int(width)

    @property
    def output_dim(self) -> int:
        return self._output_dim


class ZeroConditioningEmbedder(_Embedder):
    """Emits an empty ``[batch, 0]`` embedding (unconditional backbones)."""

    def __init__(self):
        super().__init__(0)

    def forward(self, t, **kwargs):
        return t.new_empty((t.shape[0], 0))


class DiTConditionEmbedder(_Embedder):
    """Learnable sinusoidal timestep embedding plus an optional zero-initialised linear map of the condition."""

    def __init__(self, hidden_size: int, condition_dim: int = 0, amp_mode: bool = False, **timestep_embed_kwargs: Any):
        super().__init__(hidden_size)
        self.t_embedder = PositionalEmbedding(num_channels=hidden_size, learnable=True, amp_mode=amp_mode, **timestep_embed_kwargs)
        self.cond_embedder = None
        if condition_dim:
            # starts at zero: an untrained model ignores the condition
            self.cond_embedder = Linear(condition_dim, hidden_size, bias=False, init_mode="kaiming_uniform", init_weight=0,
                                        init_bias=0, amp_mode=amp_mode)

    def forward(self, t, condition=None, **kwargs):
        out = self.t_embedder(t)
        use_condition = condition is not None and self.cond_embedder is not None
        return out + self.cond_embedder(condition) if use_condition else out


class EDMConditionEmbedder(_Embedder):
    """EDM noise embedding: sin/cos positional features (+ scaled condition map, with train-time condition
    dropout) → Linear → SiLU → Linear."""

    def __init__(self, emb_channels: int, noise_channels: int, condition_dim: int = 0, condition_dropout: float = 0.0,
                 legacy_condition_bias: bool = False, max_positions: int = 10000, **kwargs):
        super().__init__(emb_channels)
        self.condition_dropout, self.legacy_condition_bias = condition_dropout, legacy_condition_bias
        self.map_noise = PositionalEmbedding(num_channels=noise_channels, embed_fn="np_sin_cos", endpoint=True, learnable=False,
                                             max_positions=max_positions)
        wants_condition_map = legacy_condition_bias or condition_dim > 0
        self.map_condition = nn.Linear(condition_dim, noise_channels) if wants_condition_map else None
        self.map_layer0, self.map_layer1 = nn.Linear(noise_channels, emb_channels), nn.Linear(emb_channels, emb_channels)

    def _condition_features(self, condition: torch.Tensor) -> torch.Tensor:
        """``map_condition(√d · c)``; whole conditions are dropped per sample with probability ``condition_dropout``
        while training (classifier-free guidance)."""
        if self.training and self.condition_dropout:
            dropped = torch.rand([condition.shape[0], 1], device=condition.device) < self.condition_dropout
            condition = condition.masked_fill(dropped, 0)
        return self.map_condition(math.sqrt(self.map_condition.in_features) * condition)

    def forward(self, t, condition=None, **kwargs):
        features = self.map_noise(t)
        if condition is not None and self.map_condition is not None:
            features = features + self._condition_features(condition)
        return self.map_layer1(F.silu(self.map_layer0(features)))


class ConditioningEmbedderType(Enum):
    DIT = DiTConditionEmbedder
    EDM = EDMConditionEmbedder
    ZERO = ZeroConditioningEmbedder


def get_conditioning_embedder(conditioning_embedder: ConditioningEmbedderType = ConditioningEmbedderType.DIT,
                              **kwargs: Any) -> ConditioningEmbedder:
    """Instantiate the embedder behind an enum member (the ``ZERO`` embedder takes no arguments)."""
    factory = conditioning_embedder.value
    if factory is ZeroConditioningEmbedder:
        return factory()
    return factory(**kwargs)

"""Protocols of the diffusion tool-kit (parity: ``physicsnemo/diffusion/base.py:37-316``).

``DiffusionModel(x, t, condition=None, **kw)`` — a trainable network;
``Predictor(x, t)`` — anything returning a prediction (x0, score, epsilon) for a noisy state;
``Denoiser(x, t)`` — the right-hand side used by a solver (``dx/dt``).
"""
from __future__ import annotations

from typing import Any, Protocol, runtime_checkable

from torch import Tensor


@runtime_checkable
class DiffusionModel(Protocol):
    def __call__(self, x: Tensor, t: Tensor, condition: Any = None, **model_kwargs: Any) -> Tensor: ...


@runtime_checkable
class Predictor(Protocol):
    def __call__(self, x: Tensor, t: Tensor) -> Tensor: ...


@runtime_checkable
class Denoiser(Protocol):
    def __call__(self, x: Tensor, t: Tensor) -> Tensor: ...

"""Adapters between network signatures and the ``DiffusionModel`` protocol
(parity: ``physicsnemo/diffusion/utils/model_wrappers.py``)."""
from __future__ import annotations

from typing import Any

import torch

from ...core.module import Module


class ConcatConditionWrapper(Module):
    """Wraps ``net(x, noise_labels, ...)``: an image-like ``condition`` is concatenated to ``x`` along
    channels; a dict condition is passed as keyword arguments (``image`` key concatenated)."""

    def __init__(self, model: Module):
        super().__init__()
        self.model = model

    def forward(self, x: torch.Tensor, t: torch.Tensor, condition: Any = None, **model_kwargs: Any) -> torch.Tensor:
        if condition is None:
            return self.model(x, t, **model_kwargs)
        if isinstance(condition, torch.Tensor):
            return self.model(torch.cat([x, condition.to(x.dtype)], dim=1), t, **model_kwargs)
        cond = dict(condition)
        img = cond.pop("image", None)
        if img is not None:
            x = torch.cat([x, img.to(x.dtype)], dim=1)
        return self.model(x, t, **cond, **model_kwargs)

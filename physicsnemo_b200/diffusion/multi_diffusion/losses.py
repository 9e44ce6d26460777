"""Denoising score-matching losses on random patches of a ``MultiDiffusionModel2D``.

Parity: ``physicsnemo/diffusion/multi_diffusion/losses.py`` (``MultiDiffusionMSEDSMLoss``,
``MultiDiffusionWeightedMSEDSMLoss``): draw fresh patch positions, patch the clean data once, noise the *patches* with one
diffusion time per patch, run the model on the pre-patched input, convert its prediction to ``x0`` and return the
loss-weighted squared error.
"""
from __future__ import annotations

from typing import Any, Callable

import torch
from torch import Tensor

from ..utils.utils import apply_loss_weight
from .models import MultiDiffusionModel2D


def _unwrap_module(model, target_cls):
    """Peel ``DistributedDataParallel`` (``.module``) and ``torch.compile`` (``._orig_mod``) wrappers."""
    m: Any = model
    while not isinstance(m, target_cls):
        if hasattr(m, "module"):
            m = m.module
        elif hasattr(m, "_orig_mod"):
            m = m._orig_mod
        else:
            raise TypeError(f"expected a (possibly wrapped) {target_cls.__name__}, got {type(model).__name__}")
    return m


def _x0_converter(prediction_type, score_to_x0_fn, epsilon_to_x0_fn) -> Callable[[Tensor, Tensor, Tensor], Tensor]:
    if prediction_type == "x0":
        return lambda prediction, x_t, t: prediction
    if prediction_type == "score":
        if score_to_x0_fn is None:
            raise ValueError("score_to_x0_fn is required for prediction_type='score'")
        return score_to_x0_fn
    if prediction_type == "epsilon":
        if epsilon_to_x0_fn is None:
            raise ValueError("epsilon_to_x0_fn is required for prediction_type='epsilon'")
        return epsilon_to_x0_fn
    raise ValueError(f"prediction_type must be 'x0', 'score' or 'epsilon', got {prediction_type!r}")


_REDUCTIONS = {"none": lambda x: x, "mean": lambda x: x.mean(), "sum": lambda x: x.sum()}


class MultiDiffusionMSEDSMLoss:
    def __init__(self, model, noise_scheduler, prediction_type: str = "x0", score_to_x0_fn=None, epsilon_to_x0_fn=None, reduction: str = "mean"):
        self.model, self.noise_scheduler = model, noise_scheduler
        self._md_model = _unwrap_module(model, MultiDiffusionModel2D)
        self._to_x0 = _x0_converter(prediction_type, score_to_x0_fn, epsilon_to_x0_fn)
        if reduction not in _REDUCTIONS:
            raise ValueError(f"reduction must be one of {sorted(_REDUCTIONS)}, got {reduction!r}")
        self._reduce = _REDUCTIONS[reduction]

    def _patched_error(self, x0, condition, reset_patch_indices, t, model_kwargs):
        if reset_patch_indices:
            self._md_model.reset_patch_indices()
        x0_p = self._md_model.patch_x(x0)
        if t is None:
            t = self.noise_scheduler.sample_time(x0_p.shape[0], device=x0.device, dtype=x0.dtype)
        x_t = self.noise_scheduler.add_noise(x0_p, t)
        pred = self.model(x_t, t, condition=condition, x_is_patched=True, t_is_patched=True, **model_kwargs)
        err = (self._to_x0(pred, x_t, t) - x0_p) ** 2
        return err, apply_loss_weight(self.noise_scheduler.loss_weight(t), x0_p.ndim)

    def __call__(self, x0: Tensor, condition=None, reset_patch_indices: bool = True, t: Tensor | None = None, **model_kwargs: Any) -> Tensor:
        err, w = self._patched_error(x0, condition, reset_patch_indices, t, model_kwargs)
        return self._reduce(w * err)


class MultiDiffusionWeightedMSEDSMLoss(MultiDiffusionMSEDSMLoss):
    """Same, with a per-element weight map that is patched at the same positions as the data."""

    def __call__(self, x0: Tensor, weight: Tensor, condition=None, reset_patch_indices: bool = True, t: Tensor | None = None,
                 **model_kwargs: Any) -> Tensor:
        if weight.shape != x0.shape:
            raise ValueError(f"weight must have the shape of x0, got {tuple(weight.shape)} and {tuple(x0.shape)}")
        err, w = self._patched_error(x0, condition, reset_patch_indices, t, model_kwargs)
        return self._reduce(w * self._md_model.patch_x(weight) * err)

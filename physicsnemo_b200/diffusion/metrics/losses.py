"""Denoising score matching losses.

Parity: ``physicsnemo/diffusion/metrics/losses.py`` — ``MSEDSMLoss`` (``:96-446``): draw ``t`` from
the scheduler, perturb ``x0``, run the model, convert the prediction to ``x0``, weight
``(x̂0 − x0)²`` by ``loss_weight(t)`` and reduce; ``WeightedMSEDSMLoss`` (``:449-646``) adds an
element-wise weight.  Works on plain tensors and on ``ShardTensor`` inputs (the mean over a
sharded tensor is a Partial value resolved in ``backward``).
"""
from __future__ import annotations

from typing import Any, Callable, Literal, Optional

import torch
from torch import Tensor

from ..utils.utils import apply_loss_weight


def _converters(prediction_type, score_to_x0_fn, epsilon_to_x0_fn):
    if prediction_type == "x0":
        return lambda prediction, x_t, t: prediction
    if prediction_type == "score":
        if score_to_x0_fn is None:
            raise ValueError("score_to_x0_fn must be provided when prediction_type='score'.")
        return score_to_x0_fn
    if prediction_type == "epsilon":
        if epsilon_to_x0_fn is None:
            raise ValueError("epsilon_to_x0_fn must be provided when prediction_type='epsilon'.")
        return epsilon_to_x0_fn
    raise ValueError(f"prediction_type must be 'x0', 'score', or 'epsilon', got '{prediction_type}'.")


_REDUCTIONS = {"none": lambda x: x, "mean": lambda x: x.mean(), "sum": lambda x: x.sum()}


def _check_domain_parallel(x0, scheduler):
    from ...parallel import ShardTensor
    from ..noise_schedulers import DomainParallelNoiseScheduler

    if isinstance(x0, ShardTensor) and x0.spec.sharded_tensor_dims() and not isinstance(scheduler, DomainParallelNoiseScheduler):
        raise ValueError(
            "x0 is a sharded ShardTensor: wrap the noise scheduler in DomainParallelNoiseScheduler so that all "
            "shards of a sample share one noise level")


class MSEDSMLoss:
    def __init__(self, model, noise_scheduler, prediction_type: str = "x0", score_to_x0_fn: Optional[Callable] = None,
                 epsilon_to_x0_fn: Optional[Callable] = None, reduction: Literal["none", "mean", "sum"] = "mean"):
        self.model, self.noise_scheduler = model, noise_scheduler
        self._to_x0 = _converters(prediction_type, score_to_x0_fn, epsilon_to_x0_fn)
        if reduction not in _REDUCTIONS:
            raise ValueError(f"reduction must be 'none', 'mean', or 'sum', got '{reduction}'.")
        self._reduce = _REDUCTIONS[reduction]

    def _weighted(self, x0, t, condition, extra_weight, model_kwargs):
        _check_domain_parallel(x0, self.noise_scheduler)
        if t is None:
            t = self.noise_scheduler.sample_time(x0.shape[0], device=x0.device, dtype=x0.dtype)
        x_t = self.noise_scheduler.add_noise(x0, t)
        prediction = self.model(x_t, t, condition=condition, **model_kwargs)
        x0_pred = self._to_x0(prediction, x_t, t)
        loss = (x0_pred - x0) ** 2
        if extra_weight is not None:
            loss = extra_weight * loss
        w = apply_loss_weight(self.noise_scheduler.loss_weight(t), x0.ndim)
        return self._reduce(w * loss)

    def __call__(self, x0: Tensor, t: Optional[Tensor] = None, condition: Any = None, **model_kwargs: Any) -> Tensor:
        return self._weighted(x0, t, condition, None, model_kwargs)


class WeightedMSEDSMLoss(MSEDSMLoss):
    def __call__(self, x0: Tensor, weight: Tensor, t: Optional[Tensor] = None, condition: Any = None,
                 **model_kwargs: Any) -> Tensor:
        return self._weighted(x0, t, condition, weight, model_kwargs)

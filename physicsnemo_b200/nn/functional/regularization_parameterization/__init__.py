"""Stochastic depth and weight factorisation as functionals.

Parity: ``physicsnemo/nn/functional/regularization_parameterization`` (``drop_path``, ``weight_fact``).
"""
import torch

from ....core.function_spec import FunctionSpec


class DropPath(FunctionSpec):
    """Zero whole samples with probability ``drop_prob`` (rescaling the survivors by ``1/keep``)."""

    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(x, drop_prob: float = 0.0, training: bool = False, scale_by_keep: bool = True):
        if drop_prob == 0.0 or not training:
            return x
        keep = 1.0 - drop_prob
        mask = x.new_empty((x.shape[0],) + (1,) * (x.ndim - 1)).bernoulli_(keep)
        if keep > 0.0 and scale_by_keep:
            mask.div_(keep)
        return x * mask


class WeightFact(FunctionSpec):
    """Random factorisation ``w = g · v`` with per-row scale ``g = exp(N(mean, stddev))``."""

    @FunctionSpec.register(name="torch", rank=0, baseline=True)
    def torch_forward(w, mean: float = 1.0, stddev: float = 0.1):
        g = torch.exp(torch.normal(mean, stddev, size=(w.shape[0], 1), device=w.device))
        return g, w / g


drop_path = DropPath.make_function("drop_path")
weight_fact = WeightFact.make_function("weight_fact")

__all__ = ["DropPath", "drop_path", "WeightFact", "weight_fact"]

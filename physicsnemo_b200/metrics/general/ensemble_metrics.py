"""Streaming ensemble statistics, summed across ranks when a process group is live.

Parity: ``physicsnemo/metrics/general/ensemble_metrics.py`` — ``EnsembleMetrics`` base, ``Mean``
(``:110-200``) and ``Variance`` (``:230-378``, pairwise / Chan update of the centred second moment).
"""
from __future__ import annotations

from abc import ABC
from typing import List, Tuple, Union

import torch
import torch.distributed as dist
from torch import Tensor


def _live() -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


class EnsembleMetrics(ABC):
    def __init__(self, input_shape: Union[Tuple[int, ...], List[int]], device: Union[str, torch.device] = "cpu",
                 dtype: torch.dtype = torch.float32):
        self.input_shape = list(input_shape)
        self.device = torch.device(device)
        self.dtype = dtype

    def _check_shape(self, inputs: Tensor) -> None:
        if list(inputs.shape[1:]) != self.input_shape:
            raise ValueError(f"Expected new input to have compatible shape with existing shapes but got "
                             f"{list(inputs.shape)} and {self.input_shape}.")

    def _check_device(self, inputs: Tensor) -> None:
        if inputs.device != self.device:
            raise AssertionError(f"Input device, {inputs.device}, and Module device, {self.device}, must be the same.")

    def __call__(self, *args):
        raise NotImplementedError("Class member must implement a __call__ method.")

    def update(self, *args):
        raise NotImplementedError("Class member must implement an update method.")

    def finalize(self, *args):
        raise NotImplementedError("Class member must implement a finalize method.")


def _update_mean(old_sum, old_n, inputs, batch_dim=0):
    if batch_dim is None:
        inputs, batch_dim = inputs.unsqueeze(0), 0
    return old_sum + inputs.sum(dim=batch_dim), old_n + inputs.shape[batch_dim]


class Mean(EnsembleMetrics):
    def __init__(self, input_shape, **kwargs):
        super().__init__(input_shape, **kwargs)
        self.sum = torch.zeros(self.input_shape, dtype=self.dtype, device=self.device)
        self.n = torch.zeros([1], dtype=torch.int32, device=self.device)

    def _totals(self, inputs, dim):
        s = inputs.sum(dim=dim)
        n = torch.as_tensor([inputs.shape[dim]], device=self.device, dtype=torch.int32)
        if _live():
            dist.all_reduce(s)
            dist.all_reduce(n)
        return s, n

    def __call__(self, inputs: Tensor, dim: int = 0) -> Tensor:
        self._check_device(inputs)
        self.sum, self.n = self._totals(inputs, dim)
        return self.sum / self.n

    def update(self, inputs: Tensor, dim: int = 0) -> Tensor:
        self._check_shape(inputs)
        self._check_device(inputs)
        s, n = self._totals(inputs, dim)
        self.sum = self.sum + s
        self.n = self.n + n
        return self.sum / self.n

    def finalize(self) -> Tensor:
        self.mean = self.sum / self.n
        return self.mean


def _update_var(old_sum, old_sum2, old_n, inputs, batch_dim=0):
    if batch_dim is None:
        inputs, batch_dim = inputs.unsqueeze(0), 0
    n = inputs.shape[batch_dim]
    s = inputs.sum(dim=batch_dim)
    s2 = ((inputs - s / n) ** 2).sum(dim=batch_dim)
    delta = old_sum * n / old_n - s
    return old_sum + s, old_sum2 + s2 + old_n / n / (old_n + n) * delta ** 2, old_n + n


class Variance(EnsembleMetrics):
    def __init__(self, input_shape, **kwargs):
        super().__init__(input_shape, **kwargs)
        self.n = torch.zeros([1], dtype=torch.int32, device=self.device)
        self.sum = torch.zeros(self.input_shape, dtype=self.dtype, device=self.device)
        self.sum2 = torch.zeros(self.input_shape, dtype=self.dtype, device=self.device)

    def _moments(self, inputs, dim=0):
        n = torch.as_tensor([inputs.shape[dim]], device=self.device, dtype=torch.int32)
        s = inputs.sum(dim=dim)
        if _live():
            dist.all_reduce(n)
            dist.all_reduce(s)
        s2 = ((inputs - s / n) ** 2).sum(dim=dim)
        if _live():
            dist.all_reduce(s2)
        return n, s, s2

    def _value(self):
        return self.sum2 if self.n < 2.0 else self.sum2 / (self.n - 1.0)

    def __call__(self, inputs: Tensor, dim: int = 0) -> Tensor:
        self._check_device(inputs)
        self.n, self.sum, self.sum2 = self._moments(inputs, dim)
        return self._value()

    def update(self, inputs: Tensor) -> Tensor:
        self._check_shape(inputs)
        self._check_device(inputs)
        n, s, s2 = self._moments(inputs, 0)
        if int(self.n) == 0:
            self.n, self.sum, self.sum2 = n, s, s2
            return self._value()
        delta = self.sum * n / self.n - s
        self.sum2 = self.sum2 + s2 + self.n / n / (self.n + n) * delta ** 2
        self.sum = self.sum + s
        self.n = self.n + n
        return self._value()

    @property
    def mean(self) -> Tensor:
        return self.sum / self.n

    def finalize(self, std: bool = False):
        if not (self.n > 1.0):
            raise ValueError("Error! In order to finalize, there needs to be at least 2 samples.")
        self.var = self.sum2 / (self.n - 1.0)
        if std:
            self.std = torch.sqrt(self.var)
            return self.std
        return self.var

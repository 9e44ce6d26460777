"""Couplers: how one component model (atmosphere) receives the fields of another (ocean) during training and roll-out.

Parity: ``physicsnemo/datapipes/healpix/couplers.py`` (``ConstantCoupler``, ``TrailingAverageCoupler``).  For every
model integration step ``i`` and every requested lead time the coupler supplies the coupled variables as extra input
channels (``len(variables) * len(input_times)`` of them).  While training they are read from the data at fixed offsets
from the sample's start (index tables built once by ``compute_coupled_indices``); in a coupled forecast the other
model's output replaces the data (``set_coupled_fields``) — held constant (``ConstantCoupler``) or averaged over the
window that ends at each lead time (``TrailingAverageCoupler``).  Data handed to a coupler is expected to be prepared:
each time step already holds the average over the window ending there.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from .timeseries_dataset import ArrayStore, to_timedelta


class _CouplerBase:
    def __init__(self, dataset, batch_size: int, variables: Sequence[str], presteps: int = 0, input_time_dim: int = 2,
                 output_time_dim: int = 2, input_times: Sequence = ("24h", "48h"), prepared_coupled_data: bool = True):
        self.ds = dataset if isinstance(dataset, ArrayStore) else ArrayStore(dataset)
        self.batch_size, self.variables, self.presteps = batch_size, list(variables), presteps
        self.input_time_dim, self.output_time_dim = input_time_dim, output_time_dim
        self.input_times = [to_timedelta(t) for t in input_times]
        self.spatial_dims = tuple(self.ds.inputs.shape[2:])
        self.coupled_integration_dim = presteps + max(output_time_dim // input_time_dim, 1)
        self.timevar_dim = self.output_channels = len(self.input_times) * len(self.variables)
        if not prepared_coupled_data:
            raise NotImplementedError("coupled data must be prepared: every step holds the average of the window ending there")
        names = self.ds.channel_in or []
        missing = [v for v in self.variables if v not in names]
        if missing:
            raise KeyError(f"the coupled dataset has no variables {missing}")
        self._var_index = [names.index(v) for v in self.variables]
        self._coupled_offsets: Optional[np.ndarray] = None
        self.coupled_scaling = {"mean": 0.0, "std": 1.0}
        self.reset_coupler()

    def _lead(self, i: int, interval: int) -> int:
        raise NotImplementedError

    def compute_coupled_indices(self, interval: int, data_time_step) -> None:
        """``offsets[b, i, k]``: data index (relative to the batch's first time) of lead time k at integration step i."""
        dt = to_timedelta(data_time_step)
        leads = np.array([int(t / dt) for t in self.input_times])
        b = np.arange(self.batch_size)[:, None, None]
        i = np.array([self._lead(j, interval) for j in range(self.coupled_integration_dim)])[None, :, None]
        self._coupled_offsets = (b + i + leads[None, None, :]).astype(int)

    def set_scaling(self, scaling: dict) -> None:
        """``scaling``: ``{variable: {"mean", "std"}}``."""
        mean = np.array([scaling[v]["mean"] for v in self.variables], np.float32).reshape(1, -1, 1, 1, 1)
        std = np.array([scaling[v]["std"] for v in self.variables], np.float32).reshape(1, -1, 1, 1, 1)
        self.coupled_scaling = {"mean": mean, "std": std}

    def reset_coupler(self) -> None:
        self.coupled_mode = False
        self.integrated_couplings = None
        self.preset_coupled_fields = None

    def setup_coupling(self, coupled_module) -> None:
        """Which of the other model's output channels feed this coupler (names may carry a ``-suffix``)."""
        outputs = list(coupled_module.output_variables)
        self.coupled_channel_indices = [i for i, name in enumerate(outputs) for v in self.variables if name == v.split("-")[0]]

    def construct_integrated_couplings(self, batch=None, bsize: Optional[int] = None):
        """``[integration steps, B, variables * lead times, F, H, W]`` for the batch starting at ``batch["time"].start``."""
        if self.coupled_mode:
            return self.preset_coupled_fields
        start = batch["time"].start
        last = int(self._coupled_offsets[:bsize].max())
        slab = ArrayStore.slab(self.ds.inputs, start, start + last + 1)[:, self._var_index]
        slab = (slab - self.coupled_scaling["mean"]) / self.coupled_scaling["std"]
        picked = slab[self._coupled_offsets[:bsize]]                       # [B, I, lead, var, F, H, W]
        B, I = picked.shape[:2]
        picked = picked.reshape(B, I, self.timevar_dim, *self.spatial_dims)
        self.integrated_couplings = picked
        return np.ascontiguousarray(picked.transpose(1, 0, 2, 3, 4, 5)).astype(np.float32)


class ConstantCoupler(_CouplerBase):
    """The coupled field at the integration time forces the model unchanged through the whole step."""

    def _lead(self, i: int, interval: int) -> int:
        return 0

    def set_coupled_fields(self, coupled_fields: torch.Tensor) -> None:
        """``coupled_fields``: the other model's output ``[B, F, T, C, H, W]``; its first time step is used for all
        integration steps and lead times."""
        f = coupled_fields[:, :, :1, self.coupled_channel_indices].permute(2, 0, 3, 1, 4, 5)      # [1, B, C, F, H, W]
        f = f.repeat(1, 1, len(self.input_times), 1, 1, 1)
        self.preset_coupled_fields = f.expand(self.coupled_integration_dim, -1, -1, -1, -1, -1).clone()
        self.coupled_mode = True


class TrailingAverageCoupler(_CouplerBase):
    """Each lead time receives the average over the ``averaging_window`` that ends at it."""

    def __init__(self, dataset, batch_size: int, variables: Sequence[str], presteps: int = 0, input_time_dim: int = 2,
                 output_time_dim: int = 2, averaging_window: str = "24h", input_times: Sequence = ("24h", "48h"),
                 prepared_coupled_data: bool = True):
        self.averaging_window = to_timedelta(averaging_window)
        super().__init__(dataset, batch_size, variables, presteps, input_time_dim, output_time_dim, input_times, prepared_coupled_data)
        dt = self.ds.time[1] - self.ds.time[0]
        if any(int(t / np.timedelta64(1, "s")) % int(dt / np.timedelta64(1, "s")) for t in self.input_times):
            raise ValueError(f"coupled lead times {self.input_times} are not multiples of the data step {dt}")
        self.averaging_slices: List[List[slice]] = []

    def _lead(self, i: int, interval: int) -> int:
        return (self.input_time_dim * i + 1) * interval

    def setup_coupling(self, coupled_module) -> None:
        super().setup_coupling(coupled_module)
        step = to_timedelta(coupled_module.time_step)
        ends = [int(t / step) for t in self.input_times]
        stride = ends[0]
        self.averaging_slices = [[slice(self.input_time_dim * j * stride + k * stride, self.input_time_dim * j * stride + end)
                                  for k, end in enumerate(ends)] for j in range(self.coupled_integration_dim)]

    def set_coupled_fields(self, coupled_fields: torch.Tensor) -> None:
        f = coupled_fields[:, :, :, self.coupled_channel_indices]
        per_step = []
        for windows in self.averaging_slices:
            means = [f[:, :, w].mean(dim=2, keepdim=True) for w in windows]            # each [B, F, 1, C, H, W]
            per_step.append(torch.cat(means, dim=3))
        self.preset_coupled_fields = torch.cat(per_step, dim=2).permute(2, 0, 3, 1, 4, 5)
        self.coupled_mode = True

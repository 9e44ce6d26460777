"""Time-series samples with coupled fields from another component model.

Parity: ``physicsnemo/datapipes/healpix/coupledtimeseries_dataset.py`` (``CoupledTimeSeriesDataset``): a
``TimeSeriesDataset`` restricted to ``input_variables`` / ``output_variables`` whose items additionally carry the
couplers' integrated fields (appended after the constants), optional Gaussian training noise on inputs and couplings,
and ``next_integration`` to assemble the inputs of the following roll-out step from the model's own outputs.
"""
from __future__ import annotations

from typing import Mapping, Optional, Sequence

import numpy as np
import torch

from ...utils.insolation import insolation
from . import couplers as _couplers
from .timeseries_dataset import ArrayStore, TimeSeriesDataset, TimeStep


class CoupledTimeSeriesDataset(TimeSeriesDataset):
    def __init__(self, dataset, input_variables: Sequence[str], output_variables: Optional[Sequence[str]] = None,
                 scaling: Optional[Mapping] = None, input_time_dim: int = 1, presteps: int = 0, output_time_dim: int = 1,
                 data_time_step: TimeStep = "3h", time_step: TimeStep = "6h", gap: Optional[TimeStep] = None, batch_size: int = 32,
                 drop_last: bool = False, add_insolation: bool = False, forecast_init_times: Optional[Sequence] = None,
                 couplings: Sequence = (), add_train_noise: bool = False, train_noise_params: Optional[Mapping] = None,
                 train_noise_seed: int = 42, meta=None):
        store = dataset if isinstance(dataset, ArrayStore) else ArrayStore(dataset)
        self.input_variables = list(input_variables)
        self.output_variables = list(output_variables) if output_variables is not None else list(input_variables)
        names_in, names_out = store.channel_in or [], store.channel_out or []
        self._in_index = [names_in.index(v) for v in self.input_variables]
        self._out_index = [names_out.index(v) for v in self.output_variables]
        self.presteps = presteps
        self.add_train_noise, self.train_noise_params = add_train_noise, dict(train_noise_params or {})
        self.rng = np.random.default_rng(train_noise_seed)
        super().__init__(store, scaling, input_time_dim, output_time_dim, data_time_step, time_step, gap, batch_size, drop_last,
                         add_insolation, forecast_init_times, meta)
        self.couplings = []
        for spec in couplings:
            if isinstance(spec, Mapping):                       # {"coupler": class name, "params": {...}} as in the configs
                cls = getattr(_couplers, spec["coupler"])
                params = {k: v for k, v in spec.get("params", {}).items() if k != "batch_size"}     # the dataset's own is used
                spec = cls(store, self.batch_size, **dict(params, presteps=presteps, input_time_dim=input_time_dim,
                                                          output_time_dim=output_time_dim))
            spec.compute_coupled_indices(self.interval, self.data_time_step)
            if self.scaling:
                spec.set_scaling(self.scaling)
            self.couplings.append(spec)
        self.integration_step, self.curr_item = 1, None

    def _get_scaling_da(self) -> None:
        self.input_scaling = self._scale_vectors(self.input_variables, len(self.input_variables))
        self.target_scaling = self._scale_vectors(self.output_variables, len(self.output_variables))

    def __getitem__(self, item: int):
        if item < 0:
            item += len(self)
        if not 0 <= item < len(self):
            raise IndexError(f"item {item} outside a dataset of {len(self)} batches")
        self.curr_item, self.integration_step = item, 1
        (start, stop), size = self._get_time_index(item)
        x = ArrayStore.slab(self.ds.inputs, start, stop)[:, self._in_index]
        x = (x - self.input_scaling["mean"]) / self.input_scaling["std"]
        inputs = x[self._input_indices[:size]]
        coupled = None
        if self.couplings:
            coupled = np.concatenate([c.construct_integrated_couplings({"time": slice(start, stop)}, size) for c in self.couplings], axis=2)
        if self.add_train_noise and not self.forecast_mode:
            for i, v in enumerate(self.input_variables):
                std = self.train_noise_params.get("inputs", {}).get(v, {}).get("std", 0.0)
                if std:
                    inputs[:, :, i] += self.rng.normal(0, std, inputs[:, :, i].shape).astype(np.float32)
            at = 0
            for c in self.couplings:
                for v in c.variables:
                    std = self.train_noise_params.get("couplings", {}).get(v, {}).get("std", 0.0)
                    for k in range(len(c.input_times)):
                        if std:
                            coupled[:, :, at] += self.rng.normal(0, std, coupled[:, :, at].shape).astype(np.float32)
                        at += 1
        out = [np.ascontiguousarray(np.transpose(inputs, (0, 3, 1, 2, 4, 5)))]
        if self.add_insolation:
            sol = insolation(self._get_forecast_sol_times(item), self.ds.lat, self.ds.lon)[:, None].astype(np.float32)
            both = np.concatenate([self._input_indices[:size], self._output_indices[:size]], axis=1)
            out.append(np.ascontiguousarray(np.transpose(sol[both], (0, 3, 1, 2, 4, 5))))
        if self.constants is not None:
            out.append(self.constants)
        if coupled is not None:
            out.append(coupled)
        if self.forecast_mode:
            return out
        y = ArrayStore.slab(self.ds.targets, start, stop)[:, self._out_index]
        y = (y - self.target_scaling["mean"]) / self.target_scaling["std"]
        return out, np.ascontiguousarray(np.transpose(y[self._output_indices[:size]], (0, 3, 1, 2, 4, 5)))

    def next_integration(self, model_outputs: torch.Tensor, constants):
        """Inputs of the next roll-out step (forecast mode): the last ``input_time_dim`` outputs, the insolation of the
        following window, the constants, and the couplers' current fields."""
        n_in = self.input_time_dim
        out = [model_outputs[:, :, -n_in:]]
        if self.add_insolation:
            shift = self.time_step * self.output_time_dim * self.integration_step
            times = self._get_forecast_sol_times(self.curr_item)
            idx = np.concatenate([self._input_indices[0], self._output_indices[0]])
            sol = insolation(times[idx] + shift, self.ds.lat, self.ds.lon)[:, None].astype(np.float32)      # [T, 1, F, H, W]
            out.append(torch.as_tensor(np.ascontiguousarray(sol[None].transpose(0, 3, 1, 2, 4, 5))))
        out.append(constants)
        self.integration_step += 1
        if self.couplings:
            fields = [c.construct_integrated_couplings() for c in self.couplings]
            out.append(torch.cat([torch.as_tensor(f) for f in fields], dim=2))
        return out

"""Per-channel MSE losses on HEALPix tensors ``[B, T, F, C, H, W]`` (parity:
``physicsnemo/metrics/climate/healpix_loss.py``): plain, channel-weighted, and ocean-masked
variants whose land-sea mask comes from an xarray dataset."""
from typing import Sequence

import numpy as np
import torch as th

_CHANNEL_AXES = (0, 1, 2, 4, 5)


def _need_6d(prediction, target):
    if not (prediction.ndim == 6 and target.ndim == 6):
        raise AssertionError("Expected predictions to have 6 dimensions")


class BaseMSE(th.nn.MSELoss):
    def __init__(self):
        super().__init__()
        self.device = None

    def setup(self, trainer):
        pass

    def _per_channel(self, prediction, target):
        _need_6d(prediction, target)
        return ((target - prediction) ** 2).mean(dim=_CHANNEL_AXES)

    def forward(self, prediction, target, average_channels=True):
        d = self._per_channel(prediction, target)
        return d.mean() if average_channels else d


class WeightedMSE(BaseMSE):
    def __init__(self, weights: Sequence = ()):
        super().__init__()
        self.loss_weights = th.tensor(list(weights))

    def setup(self, trainer):
        if len(trainer.output_variables) != len(self.loss_weights):
            raise ValueError("Length of outputs and loss_weights is not the same!")
        self.loss_weights = self.loss_weights.to(device=trainer.device)

    def forward(self, prediction, target, average_channels=True):
        d = self._per_channel(prediction, target) * self.loss_weights
        return d.mean() if average_channels else d


class OceanMSE(th.nn.MSELoss):
    """Squared error counted over ocean cells only (``1 − lsm``)."""

    def __init__(self, lsm_file: str, open_dict: dict = None, selection_dict: dict = None):
        super().__init__()
        self.device = None
        self.lsm_file = lsm_file
        self.open_dict = {"engine": "zarr"} if open_dict is None else open_dict
        self.selection_dict = {"channel_c": "lsm"} if selection_dict is None else selection_dict
        self.lsm_ds = None
        self.lsm_tensor = None
        self.lsm_sum_calculated = False
        self.lsm_sum = None
        self.lsm_var_sum = None
        self.loss_weights = None

    def _load_mask(self, trainer):
        from ...core.version_check import OptionalImport

        xr = OptionalImport("xarray")
        self.lsm_ds = xr.open_dataset(self.lsm_file, **self.open_dict).constants.sel(self.selection_dict)
        self.lsm_tensor = 1 - th.tensor(np.expand_dims(self.lsm_ds.values, (0, 2, 3))).to(trainer.device)

    def setup(self, trainer):
        self._load_mask(trainer)

    def forward(self, prediction, target, average_channels=True):
        if not self.lsm_sum_calculated:
            full = th.broadcast_to(self.lsm_tensor, target.shape)
            self.lsm_sum, self.lsm_var_sum = full.sum(), full.sum(dim=_CHANNEL_AXES)
            self.lsm_sum_calculated = True
        err = (((target - prediction) ** 2) * self.lsm_tensor).sum(dim=_CHANNEL_AXES)
        if self.loss_weights is not None:
            err = err * self.loss_weights
        return err.sum() / self.lsm_sum if average_channels else err / self.lsm_var_sum


class WeightedOceanMSE(OceanMSE):
    def __init__(self, lsm_file: str, open_dict: dict = None, selection_dict: dict = None, weights: Sequence = ()):
        super().__init__(lsm_file, open_dict, selection_dict)
        self.loss_weights = th.tensor(list(weights))

    def setup(self, trainer):
        self._load_mask(trainer)
        if len(trainer.output_variables) != len(self.loss_weights):
            raise ValueError("Length of outputs and loss_weights is not the same!")
        self.loss_weights = self.loss_weights.to(device=trainer.device)

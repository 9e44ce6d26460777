"""Cell-area weighted losses of the GraphCast recipe (parity: ``physicsnemo/metrics/climate/graphcast_loss.py``)."""
import json
import math
from collections import defaultdict

import numpy as np
import torch
import torch.nn as nn
from torch.autograd.function import once_differentiable


class CellAreaWeightedLossFunction(nn.Module):
    """Mean over (T, C) of the squared error, weighted by ``area`` (H, W), then averaged."""

    def __init__(self, area):
        super().__init__()
        self.area = area

    def forward(self, invar, outvar):
        return (((invar - outvar) ** 2).mean(dim=(0, 1)) * self.area).mean()


class CustomCellAreaWeightedLossAutogradFunction(torch.autograd.Function):
    """Same loss with the gradient formed in the forward pass (one saved tensor, no graph)."""

    @staticmethod
    def forward(ctx, invar, outvar, area):
        diff = invar - outvar
        loss = ((diff * diff).mean(dim=(0, 1)) * area).mean()
        ctx.save_for_backward(diff * area[None, None] * (2.0 / math.prod(invar.shape)))
        return loss

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_loss):
        (g,) = ctx.saved_tensors
        return g * grad_loss, None, None


class CustomCellAreaWeightedLossFunction(CellAreaWeightedLossFunction):
    def forward(self, invar, outvar):
        return CustomCellAreaWeightedLossAutogradFunction.apply(invar, outvar, self.area)


class GraphCastLossFunction(nn.Module):
    """Area weights × per-variable weights (surface 0.1, ``t2m`` 1, pressure levels ∝ level) /
    time-difference variance."""

    def __init__(self, area, channels_list, dataset_metadata_path, time_diff_std_path):
        super().__init__()
        self.area = area
        self.channel_dict = self.get_channel_dict(dataset_metadata_path, channels_list)
        self.variable_weights = self.assign_variable_weights()
        self.time_diff_std = self.get_time_diff_std(time_diff_std_path, channels_list)

    def forward(self, invar, outvar):
        err = (invar - outvar) ** 2
        err = err / torch.square(self.time_diff_std.view(1, -1, 1, 1).to(err.device))
        err = err * self.variable_weights.view(1, -1, 1, 1).to(err.device)
        return (err.mean(dim=(0, 1)) * self.area).mean()

    def get_time_diff_std(self, time_diff_std_path, channels_list):
        if time_diff_std_path is None:
            return torch.tensor([1.0], dtype=torch.float)
        return torch.FloatTensor(np.load(time_diff_std_path)[:, channels_list, ...])

    def get_channel_dict(self, dataset_metadata_path, channels_list):
        with open(dataset_metadata_path, "r") as f:
            names = json.load(f)["coords"]["channel"]
        out = {"surface": [], "atmosphere": []}
        for c in channels_list:
            name = names[c]
            out["atmosphere" if name[-1].isdigit() else "surface"].append(name)
        return out

    def parse_variable(self, variable_list):
        for i, ch in enumerate(variable_list):
            if ch.isdigit():
                return variable_list[:i], int(variable_list[i:])

    def calculate_linear_weights(self, variables):
        by_var = defaultdict(list)
        for v in variables:
            stem, level = self.parse_variable(v)
            by_var[stem].append((v, level))
        weights = {}
        for members in by_var.values():
            total = sum(level for _, level in members)
            weights.update({v: level / total for v, level in members})
        return weights

    def assign_surface_weights(self):
        w = {name: 0.1 for name in self.channel_dict["surface"]}
        if "t2m" in w:
            w["t2m"] = 1
        return w

    def assign_atmosphere_weights(self):
        return self.calculate_linear_weights(self.channel_dict["atmosphere"])

    def assign_variable_weights(self):
        vals = list(self.assign_surface_weights().values()) + list(self.assign_atmosphere_weights().values())
        return torch.FloatTensor(vals)

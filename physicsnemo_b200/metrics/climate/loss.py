"""SSIM and the MSE+DSSIM loss on HEALPix face tensors (parity: ``physicsnemo/metrics/climate/loss.py``)."""
import numpy as np
import torch
from torch.nn import functional as F


class SSIM(torch.nn.Module):
    """Structural similarity with a Gaussian window; input ``[B, C, F, H, W]`` (or with a leading
    time dim when ``time_series_forecasting``), faces folded into channels."""

    def __init__(self, window_size: int = 11, time_series_forecasting: bool = False, padding_mode: str = "constant",
                 mse: bool = False, mse_epochs: int = 0):
        super().__init__()
        self.window_size = window_size
        self.time_series_forecasting = time_series_forecasting
        self.padding_mode = padding_mode
        self.mse = torch.nn.MSELoss() if mse else None
        self.mse_epochs = mse_epochs
        self.c1, self.c2 = 0.01 ** 2, 0.03 ** 2
        self.register_buffer("window", self._create_window(window_size), persistent=False)

    @staticmethod
    def _gaussian(window_size: int, sigma: float) -> torch.Tensor:
        x = torch.arange(window_size) - window_size // 2
        g = torch.exp(-((x / (2 * sigma)) ** 2))
        return g / g.sum()

    def _create_window(self, window_size: int, sigma: float = 1.5) -> torch.Tensor:
        g = self._gaussian(window_size, sigma)
        return torch.outer(g, g)[None, None]

    def forward(self, predicted: torch.Tensor, target: torch.Tensor, mask: torch.Tensor = None, epoch: int = 0):
        if predicted.ndim != target.ndim:
            raise AssertionError("Predicted and target tensor need to have the same number of dimensions")
        ok = (5, 6) if self.time_series_forecasting else (4, 5)
        if predicted.ndim not in ok:
            raise AssertionError("Need 5 or 6 dimensions when using time series forecasting" if self.time_series_forecasting
                                 else "Need 4 or 5 dimensions when not using time series forecasting")
        predicted, target = predicted.transpose(2, 3), target.transpose(2, 3)
        if self.time_series_forecasting:
            predicted, target = predicted.flatten(0, 2), target.flatten(0, 2)
        window = self.window.expand(predicted.shape[1], -1, -1, -1).to(dtype=predicted.dtype)
        return self._ssim(predicted, target, window, mask, epoch)

    def _ssim(self, predicted, target, window, mask=None, epoch: int = 0):
        if epoch < self.mse_epochs:
            return F.mse_loss(predicted, target)
        ch, k = window.shape[0], window.shape[2]
        window = window.to(predicted.device)
        lo, hi = (k - 1) // 2, (k - 1) // 2 + (k - 1) % 2

        pad = lambda t: F.pad(t, [lo, hi, lo, hi], mode=self.padding_mode)  # noqa: E731
        pp, tp = pad(predicted), pad(target)
        conv = lambda t: F.conv2d(t, window, groups=ch)  # noqa: E731
        m1, m2 = conv(pp), conv(tp)
        v1 = conv(pp * pp) - m1 * m1
        v2 = conv(tp * tp) - m2 * m2
        cov = conv(pp * tp) - m1 * m2
        smap = ((2 * m1 * m2 + self.c1) * (2 * cov + self.c2)) / ((m1 * m1 + m2 * m2 + self.c1) * (v1 + v2 + self.c2))
        if mask is not None:
            smap, predicted, target = smap[..., mask], predicted[..., mask], target[..., mask]
        out = smap.mean().abs()
        if self.mse:
            out = out + self.mse(predicted, target)
        return out


class MSE_SSIM(torch.nn.Module):
    """Per-variable MSE, blended with ``min(1, mse)·(1 − SSIM)`` for the variables in ``ssim_variables``."""

    def __init__(self, mse_params=None, ssim_params=None, ssim_variables=("ttr1h", "tcwv0"), weights=(0.5, 0.5)):
        super().__init__()
        self.ssim = SSIM(**(ssim_params or {}))
        self.mse = torch.nn.MSELoss(**(mse_params or {}))
        if np.sum(weights) != 1:
            raise ValueError("Weights passed to MSE_SSIM loss must sum to 1")
        self.mse_dssim_weights = list(weights)
        self.ssim_variables = list(ssim_variables)

    def forward(self, prediction: torch.Tensor, targets: torch.Tensor, model: torch.nn.Module):
        if prediction.shape[-1] != prediction.shape[-2]:
            raise AssertionError(f"Spatial dims H and W must match: got {prediction.shape[-2]} and {prediction.shape[-1]}")
        if prediction.shape[3] != 12:
            raise AssertionError(f"Spatial dim F must be 12: got {prediction.shape[3]}")
        if prediction.shape[2] != model.output_channels:
            raise AssertionError(f"model output channels and prediction output channels don't match: got {model.output_channels} for model and {prediction.shape[2]} for input")
        if prediction.shape[1] not in (model.output_time_dim, model.output_time_dim // model.input_time_dim):
            raise AssertionError("Number of time steps in prediction must equal to model output time dim, or model output time dime divided by model input time dim")
        w_mse, w_dssim = self.mse_dssim_weights
        per_var = []
        for i, name in enumerate(model.output_variables):
            p, t = prediction[:, :, i:i + 1], targets[:, :, i:i + 1]
            e = self.mse(p, t)
            if name in self.ssim_variables:
                dssim = min(1.0, float(e)) * (1 - self.ssim(p, t))
                e = w_mse * e + w_dssim * dssim
            per_var.append(e)
        return torch.stack(per_var).mean()

"""Heavy-tailed (Student-t) EDM for super-resolution diffusion: preconditioner and residual loss.

Parity: ``physicsnemo/experimental/models/diffusion/preconditioning.py`` (``tEDMPrecondSuperRes``) and
``physicsnemo/experimental/metrics/diffusion/loss.py`` (``tEDMResidualLoss``): the noise is ``n = z σ / sqrt(κ)`` with
``κ ~ χ²(ν)/ν`` (a Student-t with ``ν`` degrees of freedom), and the network / loss weight see the variance-matched noise level
``σ sqrt(ν / (ν − 2))``.
"""
from __future__ import annotations

import math

import torch

from ...diffusion.metrics.legacy_losses import ResidualLoss
from ...diffusion.preconditioners.legacy import EDMPrecondSuperResolution


class tEDMPrecondSuperRes(EDMPrecondSuperResolution):
    def __init__(self, img_resolution, img_in_channels: int, img_out_channels: int, use_fp16: bool = False, model_type: str = "SongUNetPosEmbd",
                 sigma_data: float = 0.5, sigma_min=0.0, sigma_max=float("inf"), nu: int = 10, **model_kwargs):
        if nu <= 2:
            raise ValueError(f"Expected nu > 2, but got {nu}.")
        super().__init__(img_resolution=img_resolution, img_in_channels=img_in_channels, img_out_channels=img_out_channels, use_fp16=use_fp16,
                         model_type=model_type, sigma_data=sigma_data, sigma_min=sigma_min, sigma_max=sigma_max, **model_kwargs)
        self.nu = nu

    def forward(self, x, img_lr, sigma, force_fp32: bool = False, **model_kwargs):
        return super().forward(x, img_lr, sigma * math.sqrt(self.nu / (self.nu - 2)), force_fp32, **model_kwargs)


class tEDMResidualLoss(ResidualLoss):
    def __init__(self, regression_net, P_mean: float = 0.0, P_std: float = 1.2, sigma_data: float = 0.5, hr_mean_conditioning: bool = False,
                 nu: int = 10):
        if nu <= 2:
            raise ValueError(f"Expected nu > 2, but got {nu}.")
        super().__init__(regression_net, P_mean=P_mean, P_std=P_std, sigma_data=sigma_data, hr_mean_conditioning=hr_mean_conditioning)
        self.nu = nu
        self.chi_dist = torch.distributions.Chi2(float(nu))

    def get_noise_params(self, y: torch.Tensor):
        sigma = (torch.randn([y.shape[0], 1, 1, 1], device=y.device) * self.P_std + self.P_mean).exp()
        scaled = sigma * math.sqrt(self.nu / (self.nu - 2))
        weight = (scaled ** 2 + self.sigma_data ** 2) / (scaled * self.sigma_data) ** 2
        kappa = (self.chi_dist.sample((y.shape[0],)).to(y.device) / self.nu).view(-1, 1, 1, 1)
        return torch.randn_like(y) / torch.sqrt(kappa) * sigma, sigma, weight

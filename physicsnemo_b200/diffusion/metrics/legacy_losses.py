"""Loss callables with the pre-v2 signatures ``loss(net, images, ...)`` returning per-pixel losses.

Parity: ``physicsnemo/diffusion/metrics/legacy_losses.py`` — ``VPLoss`` (``:42``), ``VELoss`` (``:142``),
``EDMLoss`` (``:208``), ``EDMLossLogUniform`` (``:327``), ``EDMLossSR`` (``:360``), ``RegressionLoss``
(``:437``), ``ResidualLoss`` (``:556``; CorrDiff: diffusion on the residual of a regression net,
optional patching), ``RegressionLossCE`` (``:1023``).
"""
from __future__ import annotations

import math
from typing import Callable, Optional, Tuple

import torch
from torch import Tensor


def _augment(pipe, images):
    return pipe(images) if pipe is not None else (images, None)


class VPLoss:
    def __init__(self, beta_d: float = 19.9, beta_min: float = 0.1, epsilon_t: float = 1e-5):
        self.beta_d, self.beta_min, self.epsilon_t = beta_d, beta_min, epsilon_t

    def sigma(self, t):
        t = torch.as_tensor(t)
        return ((0.5 * self.beta_d * (t ** 2) + self.beta_min * t).exp() - 1).sqrt()

    def __call__(self, net, images, labels, augment_pipe=None):
        rnd = torch.rand([images.shape[0], 1, 1, 1], device=images.device)
        sigma = self.sigma(1 + rnd * (self.epsilon_t - 1))
        y, aug = _augment(augment_pipe, images)
        D_yn = net(y + torch.randn_like(y) * sigma, sigma, labels, augment_labels=aug)
        return (1 / sigma ** 2) * ((D_yn - y) ** 2)


class VELoss:
    def __init__(self, sigma_min: float = 0.02, sigma_max: float = 100.0):
        self.sigma_min, self.sigma_max = sigma_min, sigma_max

    def __call__(self, net, images, labels, augment_pipe=None):
        rnd = torch.rand([images.shape[0], 1, 1, 1], device=images.device)
        sigma = self.sigma_min * ((self.sigma_max / self.sigma_min) ** rnd)
        y, aug = _augment(augment_pipe, images)
        D_yn = net(y + torch.randn_like(y) * sigma, sigma, labels, augment_labels=aug)
        return (1 / sigma ** 2) * ((D_yn - y) ** 2)


class EDMLoss:
    def __init__(self, P_mean: float = -1.2, P_std: float = 1.2, sigma_data=0.5):
        self.P_mean, self.P_std, self.sigma_data = P_mean, P_std, sigma_data

    def get_noise_level(self, y: Tensor) -> Tensor:
        return (torch.randn((y.shape[0], 1, 1, 1), device=y.device) * self.P_std + self.P_mean).exp()

    def get_loss_weight(self, y: Tensor, sigma: Tensor) -> Tensor:
        return (sigma ** 2 + self.sigma_data ** 2) / (sigma * self.sigma_data) ** 2

    def sample_noise(self, y: Tensor, sigma: Tensor) -> Tensor:
        return torch.randn_like(y) * sigma

    def __call__(self, net, images, condition=None, labels=None, augment_pipe=None, lead_time_label=None):
        y, aug = _augment(augment_pipe, images)
        sigma = self.get_noise_level(y)
        weight = self.get_loss_weight(y, sigma)
        n = self.sample_noise(y, sigma)
        opt = {k: v for k, v in {"augment_labels": aug, "lead_time_label": lead_time_label}.items() if v is not None}
        if condition is not None:
            D_yn = net(y + n, sigma, condition=condition, class_labels=labels, **opt)
        else:
            D_yn = net(y + n, sigma, labels, **opt)
        return weight * ((D_yn - y) ** 2)


class EDMLossLogUniform(EDMLoss):
    def __init__(self, sigma_min: float = 0.02, sigma_max: float = 1000, sigma_data=0.5):
        self.sigma_data, self.sigma_min, self.sigma_max = sigma_data, sigma_min, sigma_max

    def get_noise_level(self, y: Tensor) -> Tensor:
        u = torch.rand((y.shape[0], 1, 1, 1), device=y.device)
        lo, hi = math.log(self.sigma_min), math.log(self.sigma_max)
        return (lo + u * (hi - lo)).exp()


class EDMLossSR:
    def __init__(self, P_mean: float = -1.2, P_std: float = 1.2, sigma_data: float = 0.5):
        self.P_mean, self.P_std, self.sigma_data = P_mean, P_std, sigma_data

    def __call__(self, net, img_clean, img_lr, labels=None, augment_pipe=None):
        sigma = (torch.randn([img_clean.shape[0], 1, 1, 1], device=img_clean.device) * self.P_std + self.P_mean).exp()
        weight = (sigma ** 2 + self.sigma_data ** 2) / (sigma * self.sigma_data) ** 2
        y_tot, aug = _augment(augment_pipe, torch.cat((img_clean, img_lr), dim=1))
        y, y_lr = y_tot[:, : img_clean.shape[1]], y_tot[:, img_clean.shape[1]:]
        D_yn = net(y + torch.randn_like(y) * sigma, y_lr, sigma, labels, augment_labels=aug)
        return weight * ((D_yn - y) ** 2)


class RegressionLoss:
    """Deterministic regression through a preconditioned U-Net: input is zeros + the conditioning image."""

    def __init__(self):
        pass

    def __call__(self, net, img_clean, img_lr, augment_pipe=None, lead_time_label=None):
        y_tot, aug = _augment(augment_pipe, torch.cat((img_clean, img_lr), dim=1))
        y, y_lr = y_tot[:, : img_clean.shape[1]], y_tot[:, img_clean.shape[1]:]
        kw = {"lead_time_label": lead_time_label} if lead_time_label is not None else {}
        D_yn = net(torch.zeros_like(y), y_lr, force_fp32=False, augment_labels=aug, **kw)
        return (D_yn - y) ** 2


class ResidualLoss:
    """CorrDiff: EDM loss on ``y − regression_net(y_lr)``, optionally on random patches."""

    def __init__(self, regression_net, P_mean: float = 0.0, P_std: float = 1.2, sigma_data: float = 0.5,
                 hr_mean_conditioning: bool = False):
        self.regression_net = regression_net
        self.P_mean, self.P_std, self.sigma_data = P_mean, P_std, sigma_data
        self.hr_mean_conditioning = hr_mean_conditioning
        self.y_mean = None

    def get_noise_params(self, y: Tensor):
        sigma = (torch.randn([y.shape[0], 1, 1, 1], device=y.device) * self.P_std + self.P_mean).exp()
        weight = (sigma ** 2 + self.sigma_data ** 2) / (sigma * self.sigma_data) ** 2
        return torch.randn_like(y) * sigma, sigma, weight

    def __call__(self, net, img_clean, img_lr, patching=None, lead_time_label=None, augment_pipe=None,
                 use_patch_grad_acc: bool = False):
        from ..multi_diffusion.patching import RandomPatching2D

        if patching and not isinstance(patching, RandomPatching2D):
            raise ValueError("patching must be a 'RandomPatching2D' object.")
        if img_clean.shape[0] != img_lr.shape[0] or img_clean.shape[2:] != img_lr.shape[2:]:
            raise ValueError(
                f"Shape mismatch between img_clean {img_clean.shape} and img_lr {img_lr.shape}. "
                f"Batch size, height and width must match.")
        y_tot, aug = _augment(augment_pipe, torch.cat((img_clean, img_lr), dim=1))
        y, y_lr = y_tot[:, : img_clean.shape[1]], y_tot[:, img_clean.shape[1]:]
        batch_size = y.shape[0]
        kw = {"lead_time_label": lead_time_label} if lead_time_label is not None else {}
        if not use_patch_grad_acc or self.y_mean is None:
            self.y_mean = self.regression_net(torch.zeros_like(y), y_lr, augment_labels=aug, **kw)
        y = y - self.y_mean
        if self.hr_mean_conditioning:
            y_lr = torch.cat((self.y_mean, y_lr), dim=1)
        if patching:
            y, y_lr = patching.apply(input=y), patching.apply(input=y_lr, additional_input=img_lr)
        n, sigma, weight = self.get_noise_params(y)
        gi = patching.global_index(batch_size, img_clean.device) if patching is not None else None
        D_yn = net(y + n, y_lr, sigma, embedding_selector=None, global_index=gi, augment_labels=aug, **kw)
        return weight * ((D_yn - y) ** 2)


class RegressionLossCE:
    """Regression loss with cross-entropy on probability channels (lead-time aware models)."""

    def __init__(self, P_mean: float = -1.2, P_std: float = 1.2, sigma_data: float = 0.5, prob_channels=(4, 5, 6, 7, 8)):
        self.P_mean, self.P_std, self.sigma_data = P_mean, P_std, sigma_data
        self.entropy = torch.nn.CrossEntropyLoss(reduction="none")
        self.prob_channels = list(prob_channels)

    def __call__(self, net, img_clean, img_lr, lead_time_label=None, augment_pipe=None):
        all_ch = list(range(img_clean.shape[1]))
        scalar_ch = [c for c in all_ch if c not in self.prob_channels]
        y_tot, aug = _augment(augment_pipe, torch.cat((img_clean, img_lr), dim=1))
        y, y_lr = y_tot[:, : img_clean.shape[1]], y_tot[:, img_clean.shape[1]:]
        kw = {"lead_time_label": lead_time_label} if lead_time_label is not None else {}
        D_yn = net(torch.zeros_like(y), y_lr, force_fp32=False, augment_labels=aug, **kw)
        loss1 = (D_yn[:, scalar_ch] - y[:, scalar_ch]) ** 2
        ce = self.entropy(D_yn[:, self.prob_channels], torch.argmax(y[:, self.prob_channels], dim=1))
        return torch.cat((loss1, ce[:, None]), dim=1)

"""Samplers with the pre-v2 call signature ``sampler(net, latents, img_lr, ...)``.

Parity: ``physicsnemo/diffusion/samplers/legacy_stochastic_sampler.py`` (EDM stochastic Heun
sampler with optional grid patching: every denoiser call runs on patches that are fused back)
and ``legacy_deterministic_sampler.py`` (the EDM "ablation" sampler: Euler / Heun-alpha solvers,
VP / VE / iDDPM / EDM time discretisations, VP / VE / linear noise schedules, VP / no scaling).
"""
from __future__ import annotations

from typing import Callable, Optional

import numpy as np
import torch
from torch import Tensor

from ..multi_diffusion.patching import GridPatching2D


def _call_net(net, x, x_lr, t, class_labels, optional_args):
    from ..preconditioners.legacy import EDMPrecond

    if isinstance(net, EDMPrecond):
        return net(x, t, condition=x_lr, class_labels=class_labels, **optional_args)
    return net(x, x_lr, t, class_labels, **optional_args)


def _prepare(net, latents, img_lr, patching, mean_hr, lead_time_label):
    if patching is not None and not isinstance(patching, GridPatching2D):
        raise ValueError("patching must be an instance of GridPatching2D.")
    if patching and img_lr.shape[-2:] != latents.shape[-2:]:
        raise ValueError(f"img_lr and latents must have the same height and width, but found "
                         f"{img_lr.shape[-2:]} vs {latents.shape[-2:]}. ")
    if img_lr.shape[0] != latents.shape[0]:
        raise ValueError(f"img_lr and latents must have the same batch size, but found "
                         f"{img_lr.shape[0]} vs {latents.shape[0]}.")
    batch_size = img_lr.shape[0]
    x_lr = img_lr
    if mean_hr is not None:
        if mean_hr.shape[-2:] != img_lr.shape[-2:]:
            raise ValueError(f"mean_hr and img_lr must have the same height and width, but found "
                             f"{mean_hr.shape[-2:]} vs {img_lr.shape[-2:]}.")
        x_lr = torch.cat((mean_hr.expand(x_lr.shape[0], -1, -1, -1), x_lr), dim=1)
    optional_args = {}
    if lead_time_label is not None:
        optional_args["lead_time_label"] = lead_time_label
    if patching:
        x_lr = patching.apply(input=x_lr, additional_input=img_lr)
        optional_args["embedding_selector"] = lambda emb: patching.apply(emb.expand(batch_size, -1, -1, -1))
    return x_lr, optional_args, batch_size


def stochastic_sampler(net, latents: Tensor, img_lr: Tensor, class_labels: Optional[Tensor] = None,
                       randn_like: Callable = torch.randn_like, patching: Optional[GridPatching2D] = None,
                       mean_hr: Optional[Tensor] = None, lead_time_label: Optional[Tensor] = None,
                       num_steps: int = 18, sigma_min: float = 0.002, sigma_max: float = 800, rho: float = 7,
                       S_churn: float = 0, S_min: float = 0, S_max: float = float("inf"), S_noise: float = 1) -> Tensor:
    """EDM stochastic sampler (Heun with churn) conditioned on ``img_lr``."""
    sigma_min, sigma_max = max(sigma_min, net.sigma_min), min(sigma_max, net.sigma_max)
    x_lr, optional_args, batch_size = _prepare(net, latents, img_lr, patching, mean_hr, lead_time_label)
    i = torch.arange(num_steps, device=latents.device)
    t_steps = (sigma_max ** (1 / rho) + i / (num_steps - 1) * (sigma_min ** (1 / rho) - sigma_max ** (1 / rho))) ** rho
    t_steps = torch.cat([net.round_sigma(t_steps), torch.zeros_like(t_steps[:1])])

    def denoise(x, t):
        xb = patching.apply(input=x) if patching else x
        d = _call_net(net, xb.to(latents.device), x_lr.to(latents.device), t, class_labels, optional_args)
        return patching.fuse(input=d, batch_size=batch_size) if patching else d

    x_next = latents * t_steps[0]
    for k, (t_cur, t_next) in enumerate(zip(t_steps[:-1], t_steps[1:])):
        gamma = S_churn / num_steps if S_min <= t_cur <= S_max else 0
        t_hat = net.round_sigma(t_cur + gamma * t_cur)
        x_hat = x_next + (t_hat ** 2 - t_cur ** 2).sqrt() * S_noise * randn_like(x_next)
        d_cur = (x_hat - denoise(x_hat, t_hat)) / t_hat
        x_next = x_hat + (t_next - t_hat) * d_cur
        if k < num_steps - 1:
            d_prime = (x_next - denoise(x_next, t_next)) / t_next
            x_next = x_hat + (t_next - t_hat) * (0.5 * d_cur + 0.5 * d_prime)
    return x_next


def deterministic_sampler(net, latents: Tensor, img_lr: Tensor, class_labels: Optional[Tensor] = None,
                          randn_like: Callable = torch.randn_like, patching: Optional[GridPatching2D] = None,
                          mean_hr: Optional[Tensor] = None, lead_time_label: Optional[Tensor] = None,
                          num_steps: int = 18, sigma_min: Optional[float] = None, sigma_max: Optional[float] = None,
                          rho: float = 7.0, solver: str = "heun", discretization: str = "edm",
                          schedule: str = "linear", scaling: str = "none", epsilon_s: float = 1e-3,
                          C_1: float = 0.001, C_2: float = 0.008, M: int = 1000, alpha: float = 1.0,
                          S_churn: int = 0, S_min: float = 0.0, S_max: float = float("inf"), S_noise: float = 1.0,
                          dtype: torch.dtype = torch.float64) -> Tensor:
    """Generalised deterministic / stochastic sampler over the design space of EDM (table 1)."""
    if solver not in ("euler", "heun"):
        raise ValueError(f"Unknown solver {solver}")
    if discretization not in ("vp", "ve", "iddpm", "edm"):
        raise ValueError(f"Unknown discretization {discretization}")
    if schedule not in ("vp", "ve", "linear"):
        raise ValueError(f"Unknown schedule {schedule}")
    if scaling not in ("vp", "none"):
        raise ValueError(f"Unknown scaling {scaling}")
    x_lr, optional_args, batch_size = _prepare(net, latents, img_lr, patching, mean_hr, lead_time_label)
    # helper functions of the VP and VE formulations
    vp_sigma = lambda beta_d, beta_min: lambda t: (np.e ** (0.5 * beta_d * (t ** 2) + beta_min * t) - 1) ** 0.5  # noqa: E731
    vp_sigma_deriv = lambda beta_d, beta_min: lambda t: 0.5 * (beta_min + beta_d * t) * (sigma(t) + 1 / sigma(t))  # noqa: E731
    vp_sigma_inv = lambda beta_d, beta_min: lambda s: ((beta_min ** 2 + 2 * beta_d * (s ** 2 + 1).log()).sqrt() - beta_min) / beta_d  # noqa: E731
    ve_sigma = lambda t: t.sqrt()  # noqa: E731
    ve_sigma_deriv = lambda t: 0.5 / t.sqrt()  # noqa: E731
    ve_sigma_inv = lambda s: s ** 2  # noqa: E731
    if sigma_min is None:
        sigma_min = {"vp": vp_sigma(19.9, 0.1)(epsilon_s), "ve": 0.02, "iddpm": 0.002, "edm": 0.002}[discretization]
    if sigma_max is None:
        sigma_max = {"vp": vp_sigma(19.9, 0.1)(1), "ve": 100, "iddpm": 81, "edm": 80}[discretization]
    sigma_min, sigma_max = max(sigma_min, net.sigma_min), min(sigma_max, net.sigma_max)
    vp_beta_d = 2 * (np.log(sigma_min ** 2 + 1) / epsilon_s - np.log(sigma_max ** 2 + 1)) / (epsilon_s - 1)
    vp_beta_min = np.log(sigma_max ** 2 + 1) - 0.5 * vp_beta_d
    step_indices = torch.arange(num_steps, dtype=dtype, device=latents.device)
    if discretization == "vp":
        orig_t = 1 + step_indices / (num_steps - 1) * (epsilon_s - 1)
        sigma_steps = vp_sigma(vp_beta_d, vp_beta_min)(orig_t)
    elif discretization == "ve":
        orig_t = (sigma_max ** 2) * ((sigma_min ** 2 / sigma_max ** 2) ** (step_indices / (num_steps - 1)))
        sigma_steps = ve_sigma(orig_t)
    elif discretization == "iddpm":
        u = torch.zeros(M + 1, dtype=dtype, device=latents.device)
        alpha_bar = lambda j: (0.5 * np.pi * j / M / (C_2 + 1)).sin() ** 2  # noqa: E731
        for j in torch.arange(M, 0, -1, device=latents.device):
            u[j - 1] = ((u[j] ** 2 + 1) / (alpha_bar(j - 1) / alpha_bar(j)).clip(min=C_1) - 1).sqrt()
        u_filtered = u[torch.logical_and(u >= sigma_min, u <= sigma_max)]
        sigma_steps = u_filtered[((len(u_filtered) - 1) / (num_steps - 1) * step_indices).round().to(torch.int64)]
    else:
        sigma_steps = (sigma_max ** (1 / rho) + step_indices / (num_steps - 1) *
                       (sigma_min ** (1 / rho) - sigma_max ** (1 / rho))) ** rho
    if schedule == "vp":
        sigma, sigma_deriv, sigma_inv = (vp_sigma(vp_beta_d, vp_beta_min), vp_sigma_deriv(vp_beta_d, vp_beta_min),
                                         vp_sigma_inv(vp_beta_d, vp_beta_min))
    elif schedule == "ve":
        sigma, sigma_deriv, sigma_inv = ve_sigma, ve_sigma_deriv, ve_sigma_inv
    else:
        sigma, sigma_deriv, sigma_inv = (lambda t: t), (lambda t: 1), (lambda s: s)
    if scaling == "vp":
        s = lambda t: 1 / (1 + sigma(t) ** 2).sqrt()  # noqa: E731
        s_deriv = lambda t: -sigma(t) * sigma_deriv(t) * (s(t) ** 3)  # noqa: E731
    else:
        s, s_deriv = (lambda t: 1), (lambda t: 0)
    t_steps = sigma_inv(net.round_sigma(sigma_steps))
    t_steps = torch.cat([t_steps, torch.zeros_like(t_steps[:1])])

    def denoise(x, sig):
        xb = patching.apply(input=x) if patching else x
        d = _call_net(net, xb, x_lr, sig, class_labels, optional_args).to(dtype)
        return patching.fuse(input=d, batch_size=batch_size) if patching else d

    t_next = t_steps[0]
    x_next = latents.to(dtype) * (sigma(t_next) * s(t_next))
    for i, (t_cur, t_next) in enumerate(zip(t_steps[:-1], t_steps[1:])):
        x_cur = x_next
        gamma = min(S_churn / num_steps, np.sqrt(2) - 1) if S_min <= sigma(t_cur) <= S_max else 0
        t_hat = sigma_inv(net.round_sigma(sigma(t_cur) + gamma * sigma(t_cur)))
        x_hat = s(t_hat) / s(t_cur) * x_cur + (sigma(t_hat) ** 2 - sigma(t_cur) ** 2).clip(min=0).sqrt() * s(t_hat) * \
            S_noise * randn_like(x_cur)
        h = t_next - t_hat
        denoised = denoise(x_hat / s(t_hat), sigma(t_hat))
        d_cur = (sigma_deriv(t_hat) / sigma(t_hat) + s_deriv(t_hat) / s(t_hat)) * x_hat - \
            sigma_deriv(t_hat) * s(t_hat) / sigma(t_hat) * denoised
        x_prime = x_hat + alpha * h * d_cur
        t_prime = t_hat + alpha * h
        if solver == "euler" or i == num_steps - 1:
            x_next = x_hat + h * d_cur
        else:
            denoised = denoise(x_prime / s(t_prime), sigma(t_prime))
            d_prime = (sigma_deriv(t_prime) / sigma(t_prime) + s_deriv(t_prime) / s(t_prime)) * x_prime - \
                sigma_deriv(t_prime) * s(t_prime) / sigma(t_prime) * denoised
            x_next = x_hat + h * ((1 - 1 / (2 * alpha)) * d_cur + 1 / (2 * alpha) * d_prime)
    return x_next

"""CorrDiff-style two-stage generation helpers: a deterministic regression pass and seeded diffusion sampling.

Parity: ``physicsnemo/diffusion/generate/legacy_generate.py`` (``regression_step``, ``diffusion_step``).
"""
from __future__ import annotations

import warnings
from typing import Callable, Literal, Optional, Sequence

import torch

from ..utils import StackedRandomGenerator


def regression_step(net: torch.nn.Module, img_lr: torch.Tensor, latents_shape, lead_time_label: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Mean prediction of the regression network for one conditioning image, repeated to ``latents_shape[0]`` samples."""
    if img_lr.shape[0] > 1:
        raise ValueError(f"Expected img_lr to have a batch size of 1, but found {img_lr.shape[0]}.")
    device = getattr(net, "device", img_lr.device)
    x_hat = torch.zeros(tuple(latents_shape), dtype=torch.float64, device=device)
    kw = {"lead_time_label": lead_time_label} if lead_time_label is not None else {}
    with torch.inference_mode():
        x = net(x=x_hat[0:1], img_lr=img_lr, **kw)
    if x_hat.shape[0] > 1:
        x = x.repeat([d if i == 0 else 1 for i, d in enumerate(x_hat.shape)])
    return x


def diffusion_step(net: torch.nn.Module, sampler_fn: Callable, img_shape: Sequence[int], img_out_channels: int, rank_batches: list,
                   img_lr: torch.Tensor, rank: int, device, mean_hr: torch.Tensor = None, lead_time_label: torch.Tensor = None,
                   distribution: Literal["normal", "student_t"] = "normal", nu: Optional[int] = None) -> torch.Tensor:
    """Sample one image per seed of every batch in ``rank_batches`` (each sample owns an independent generator)."""
    if tuple(img_lr.shape[2:]) != tuple(img_shape):
        raise ValueError(f"img_lr shape {img_lr.shape[2:]} does not match expected shape img_shape {img_shape}")
    if mean_hr is not None:
        if tuple(mean_hr.shape[2:]) != tuple(img_shape):
            raise ValueError(f"mean_hr shape {mean_hr.shape[2:]} does not match expected shape img_shape {img_shape}")
        if mean_hr.shape[0] != 1:
            raise ValueError(f"mean_hr must have batch size 1, got {mean_hr.shape[0]}")
    if distribution not in ("normal", "student_t"):
        raise ValueError(f"Invalid distribution: {distribution}")
    if distribution == "student_t":
        if nu is None:
            raise ValueError("nu must be provided for student_t distribution")
        if nu <= 2:
            raise ValueError(f"Expected nu > 2 for student_t distribution, but got {nu}.")
        warnings.warn("Student-t distribution is an experimental feature under active development and APIs may change without notice.")
    img_lr = img_lr.to(memory_format=torch.channels_last)
    extra = {}
    if mean_hr is not None:
        extra["mean_hr"] = mean_hr
    if lead_time_label is not None:
        extra["lead_time_label"] = lead_time_label
    images = []
    for seeds in rank_batches:
        if len(seeds) == 0:
            continue
        rnd = StackedRandomGenerator(device, seeds)
        shape = [img_lr.shape[0], img_out_channels, img_shape[0], img_shape[1]]
        latents = rnd.randn(shape, device=device) if distribution == "normal" else rnd.randt(nu, shape, device=device)
        with torch.inference_mode():
            images.append(sampler_fn(net, latents.to(memory_format=torch.channels_last), img_lr, randn_like=rnd.randn_like, **extra))
    return torch.cat(images)

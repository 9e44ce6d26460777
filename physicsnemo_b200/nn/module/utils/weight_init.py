"""Weight initialisation helpers.

Parity: ``physicsnemo/nn/module/utils/weight_init.py`` — ``_weight_init`` (``:302-346``) and
``shrink_and_perturb_`` (``:112-300``).
"""
from __future__ import annotations

from typing import Callable, Optional, Union

import numpy as np
import torch


def _weight_init(shape, mode: str, fan_in: int, fan_out: int) -> torch.Tensor:
    """Draw a tensor of ``shape`` by Xavier / Kaiming uniform or normal rules."""
    if mode == "xavier_uniform":
        return np.sqrt(6 / (fan_in + fan_out)) * (torch.rand(*shape) * 2 - 1)
    if mode == "xavier_normal":
        return np.sqrt(2 / (fan_in + fan_out)) * torch.randn(*shape)
    if mode == "kaiming_uniform":
        return np.sqrt(3 / fan_in) * (torch.rand(*shape) * 2 - 1)
    if mode == "kaiming_normal":
        return np.sqrt(1 / fan_in) * torch.randn(*shape)
    raise ValueError(f'Invalid init mode "{mode}"')


@torch.no_grad()
def shrink_and_perturb_(module: torch.nn.Module, shrink: float = 0.5, perturb: float = 0.1, *,
                        noise: Union[str, Callable[[torch.Tensor], torch.Tensor]] = "scaled_normal",
                        include: Optional[Callable[[str, torch.Tensor], bool]] = None,
                        generator: Optional[torch.Generator] = None) -> torch.nn.Module:
    """In-place ``p <- shrink * p + perturb * eps`` for every (selected) floating parameter.

    ``noise="scaled_normal"`` draws ``eps ~ N(0, std(p)^2)`` (no noise for single-element
    tensors), ``"normal"`` draws ``N(0, 1)``, a callable receives an empty tensor like ``p``.
    """
    if not 0.0 <= shrink <= 1.0:
        raise ValueError(f"shrink must be in [0, 1], got {shrink}")
    if perturb < 0:
        raise ValueError(f"perturb must be non-negative, got {perturb}")
    if not callable(noise) and noise not in ("scaled_normal", "normal"):
        raise ValueError(f'Invalid noise "{noise}"; expected a callable or one of ("scaled_normal", "normal")')
    for name, p in module.named_parameters():
        if not p.is_floating_point() and not p.is_complex():
            continue
        if include is not None and not include(name, p):
            continue
        if callable(noise):
            eps = noise(torch.empty_like(p))
            if eps.shape != p.shape:
                raise ValueError(f"noise for parameter '{name}' returned shape {tuple(eps.shape)}, expected {tuple(p.shape)}")
        elif noise == "scaled_normal":
            if p.numel() < 2:
                eps = torch.zeros_like(p)
            else:
                eps = torch.empty_like(p).normal_(generator=generator).mul_(p.detach().std())
        else:
            eps = torch.empty_like(p).normal_(generator=generator)
        p.mul_(shrink).add_(eps, alpha=perturb)
    return module

"""Preconditioners with the pre-v2 constructor signatures (they build the network themselves).

Parity: ``physicsnemo/diffusion/preconditioners/legacy.py`` — ``VPPrecond`` (``:74``), ``VEPrecond``
(``:263``), ``iDDPMPrecond`` (``:396``), ``EDMPrecond`` (``:566``), ``EDMPrecondSuperResolution``
(``:737``) and its alias ``EDMPrecondSR``.  ``forward(x, sigma, ...)`` takes the noise level
directly; ``round_sigma`` maps noise levels onto the supported set.
"""
from __future__ import annotations

from typing import Any, List, Tuple, Union

import numpy as np
import torch

from ...core.module import Module
from .preconditioners import EDMPreconditioner, IDDPMPreconditioner, VEPreconditioner, VPPreconditioner


def _network(model_type: str):
    from ...models import diffusion_unets

    if not hasattr(diffusion_unets, model_type):
        raise ValueError(f"Model type '{model_type}' is not available in physicsnemo_b200.models.diffusion_unets")
    return getattr(diffusion_unets, model_type)


def _build(model_type, img_resolution, in_ch, out_ch, label_dim, model_kwargs):
    return _network(model_type)(img_resolution=img_resolution, in_channels=in_ch, out_channels=out_ch,
                                label_dim=label_dim, **model_kwargs)


class _LegacyMixin:
    def _labels(self, class_labels, x):
        if self.label_dim == 0:
            return None
        if class_labels is None:
            return torch.zeros([1, self.label_dim], device=x.device)
        return class_labels.to(torch.float32).reshape(-1, self.label_dim)

    def _dtype(self, x, force_fp32):
        return torch.float16 if (self.use_fp16 and not force_fp32 and x.device.type == "cuda") else torch.float32

    def _legacy_forward(self, x, sigma, condition=None, class_labels=None, force_fp32=False, **model_kwargs):
        x = x.to(torch.float32)
        sigma = sigma.to(torch.float32).reshape(-1, 1, 1, 1)
        dtype = self._dtype(x, force_fp32)
        c_in, c_noise, c_out, c_skip = self.compute_coefficients(sigma)
        arg = c_in * x
        if condition is not None:
            arg = torch.cat([arg, condition], dim=1)
        F_x = self.model(arg.to(dtype), c_noise.flatten(), class_labels=self._labels(class_labels, x), **model_kwargs)
        if F_x.dtype != dtype and not torch.is_autocast_enabled():
            raise ValueError(f"Expected the dtype to be {dtype}, but got {F_x.dtype} instead.")
        return c_skip * x + c_out * F_x.to(torch.float32)


class VPPrecond(_LegacyMixin, VPPreconditioner):
    def __init__(self, img_resolution, img_channels, label_dim=0, use_fp16=False, beta_d=19.9, beta_min=0.1,
                 M=1000, epsilon_t=1e-5, model_type="SongUNet", **model_kwargs):
        model = _build(model_type, img_resolution, img_channels, img_channels, label_dim, model_kwargs)
        super().__init__(model=model, beta_d=beta_d, beta_min=beta_min, M=M)
        self.img_resolution, self.img_channels, self.label_dim, self.use_fp16 = img_resolution, img_channels, label_dim, use_fp16
        self.epsilon_t = epsilon_t
        self.sigma_min = float(self.sigma(torch.tensor(epsilon_t)))
        self.sigma_max = float(self.sigma(torch.tensor(1.0)))

    def forward(self, x, sigma, class_labels=None, force_fp32=False, **model_kwargs):
        return self._legacy_forward(x, sigma, None, class_labels, force_fp32, **model_kwargs)

    def sigma_inv(self, sigma):
        sigma = torch.as_tensor(sigma)
        return ((self.beta_min ** 2 + 2 * self.beta_d * (1 + sigma ** 2).log()).sqrt() - self.beta_min) / self.beta_d

    def round_sigma(self, sigma):
        return torch.as_tensor(sigma)


class VEPrecond(_LegacyMixin, VEPreconditioner):
    def __init__(self, img_resolution, img_channels, label_dim=0, use_fp16=False, sigma_min=0.02, sigma_max=100.0,
                 model_type="SongUNet", **model_kwargs):
        super().__init__(model=_build(model_type, img_resolution, img_channels, img_channels, label_dim, model_kwargs))
        self.img_resolution, self.img_channels, self.label_dim, self.use_fp16 = img_resolution, img_channels, label_dim, use_fp16
        self.sigma_min, self.sigma_max = sigma_min, sigma_max

    def forward(self, x, sigma, class_labels=None, force_fp32=False, **model_kwargs):
        return self._legacy_forward(x, sigma, None, class_labels, force_fp32, **model_kwargs)

    def round_sigma(self, sigma):
        return torch.as_tensor(sigma)


class iDDPMPrecond(_LegacyMixin, IDDPMPreconditioner):
    def __init__(self, img_resolution, img_channels, label_dim=0, use_fp16=False, C_1=0.001, C_2=0.008, M=1000,
                 model_type="DhariwalUNet", **model_kwargs):
        model = _network(model_type)(img_resolution=img_resolution, in_channels=img_channels,
                                     out_channels=img_channels * 2, label_dim=label_dim, **model_kwargs)
        super().__init__(model=model, C_1=C_1, C_2=C_2, M=M)
        self.img_resolution, self.img_channels, self.label_dim, self.use_fp16 = img_resolution, img_channels, label_dim, use_fp16
        self.sigma_min, self.sigma_max = float(self.u[M - 1]), float(self.u[0])

    def forward(self, x, sigma, class_labels=None, force_fp32=False, **model_kwargs):
        x = x.to(torch.float32)
        sigma = sigma.to(torch.float32).reshape(-1, 1, 1, 1)
        dtype = self._dtype(x, force_fp32)
        c_in, c_noise, c_out, c_skip = self.compute_coefficients(sigma)
        F_x = self.model((c_in * x).to(dtype), c_noise.flatten(), class_labels=self._labels(class_labels, x), **model_kwargs)
        return c_skip * x + c_out * F_x[:, : self.img_channels].to(torch.float32)

    def alpha_bar(self, j):
        j = torch.as_tensor(j)
        return (0.5 * np.pi * j / self.M / (self.C_2 + 1)).sin() ** 2

    def round_sigma(self, sigma, return_index=False):
        sigma = torch.as_tensor(sigma)
        index = torch.cdist(sigma.to(self.u.device).to(torch.float32).reshape(1, -1, 1),
                            self.u.reshape(1, -1, 1)).argmin(2)
        result = index if return_index else self.u[index.flatten()].to(sigma.dtype)
        return result.reshape(sigma.shape).to(sigma.device)


class EDMPrecond(_LegacyMixin, EDMPreconditioner):
    def __init__(self, img_resolution, img_channels, label_dim=0, use_fp16=False, sigma_min=0.0,
                 sigma_max=float("inf"), sigma_data=0.5, model_type="DhariwalUNet", img_in_channels=None,
                 img_out_channels=None, **model_kwargs):
        in_ch = img_channels if img_in_channels is None else img_in_channels
        out_ch = img_channels if img_out_channels is None else img_out_channels
        super().__init__(model=_build(model_type, img_resolution, in_ch, out_ch, label_dim, model_kwargs),
                         sigma_data=sigma_data)
        self.img_resolution, self.label_dim, self.use_fp16 = img_resolution, label_dim, use_fp16
        self.sigma_min, self.sigma_max = sigma_min, sigma_max

    def forward(self, x, sigma, condition=None, class_labels=None, force_fp32=False, **model_kwargs):
        return self._legacy_forward(x, sigma, condition, class_labels, force_fp32, **model_kwargs)

    @staticmethod
    def round_sigma(sigma):
        return torch.as_tensor(sigma)


class EDMPrecondSuperResolution(Module):
    """EDM preconditioning of a super-resolution network: the low-resolution image is concatenated
    (unscaled) to the scaled noisy state."""

    _wrapped_classes = {"SongUNetPosEmbd", "SongUNetPosLtEmbd", "SongUNet", "DhariwalUNet"}

    def __init__(self, img_resolution: Union[int, Tuple[int, int]], img_in_channels: int, img_out_channels: int,
                 use_fp16: bool = False, model_type: str = "SongUNetPosEmbd", sigma_data: float = 0.5, sigma_min=0.0,
                 sigma_max=float("inf"), **model_kwargs: Any):
        super().__init__()
        if model_type not in self._wrapped_classes:
            raise ValueError(f"Model type '{model_type}' is not supported. Must be one of: {', '.join(sorted(self._wrapped_classes))}")
        self.img_resolution, self.img_in_channels, self.img_out_channels = img_resolution, img_in_channels, img_out_channels
        self.sigma_data, self.sigma_min, self.sigma_max = sigma_data, sigma_min, sigma_max
        self.model = _network(model_type)(img_resolution=img_resolution, in_channels=img_in_channels + img_out_channels,
                                          out_channels=img_out_channels, **model_kwargs)
        self.scaling_fn = self._scaling_fn
        self.use_fp16 = use_fp16

    @property
    def use_fp16(self):
        return self._use_fp16

    @use_fp16.setter
    def use_fp16(self, value):
        if not (isinstance(value, bool) or value in [0, 1]):
            raise ValueError(f"`use_fp16` must be a boolean, but got {type(value).__name__}.")
        self._use_fp16 = value
        self.to(torch.float16 if value else torch.float32)

    @property
    def amp_mode(self):
        return getattr(self.model, "amp_mode", False)

    @amp_mode.setter
    def amp_mode(self, value):
        self.model.amp_mode = value

    @property
    def profile_mode(self):
        return getattr(self.model, "profile_mode", False)

    @profile_mode.setter
    def profile_mode(self, value):
        self.model.profile_mode = value

    @staticmethod
    def _scaling_fn(x, img_lr, c_in):
        return torch.cat([c_in * x, img_lr.to(x.dtype)], dim=1)

    def forward(self, x, img_lr, sigma, force_fp32: bool = False, **model_kwargs: Any):
        x = x.to(torch.float32)
        sigma = sigma.to(torch.float32).reshape(-1, 1, 1, 1)
        dtype = torch.float16 if (self.use_fp16 and not force_fp32 and x.device.type == "cuda") else torch.float32
        sd = self.sigma_data
        c_skip = sd ** 2 / (sigma ** 2 + sd ** 2)
        c_out = sigma * sd / (sigma ** 2 + sd ** 2).sqrt()
        c_in = 1 / (sd ** 2 + sigma ** 2).sqrt()
        c_noise = sigma.log() / 4
        arg = c_in * x if img_lr is None else self.scaling_fn(x, img_lr, c_in)
        F_x = self.model(arg.to(dtype), c_noise.flatten(), class_labels=None, **model_kwargs)
        if F_x.dtype != dtype and not torch.is_autocast_enabled():
            raise ValueError(f"Expected the dtype to be {dtype}, but got {F_x.dtype} instead.")
        return c_skip * x + c_out * F_x.to(torch.float32)

    @staticmethod
    def round_sigma(sigma):
        return torch.as_tensor(sigma)


EDMPrecondSR = EDMPrecondSuperResolution

"""Thin wrappers that run a diffusion U-Net backbone as a deterministic regression / forecasting network.

Parity: ``physicsnemo/models/diffusion_unets/unet.py`` — ``CorrDiffRegressionUNet`` (input = latent ⊕ low-resolution
image, zero noise label, output cast to fp32; deprecated alias ``UNet``) and ``StormCastUNet``.
"""
import warnings
from dataclasses import dataclass
from typing import Any, Dict, List, Set, Tuple, Union

import torch

from ...core.meta import ModelMetaData
from ...core.module import Module


def _wrapped_property(name: str, inner: str, doc: str):
    def get(self):
        return getattr(getattr(self, inner), name)

    def set_(self, value):
        setattr(getattr(self, inner), name, value)

    return property(get, set_, doc=doc)


def _backbone(model_type: str):
    from . import dhariwal_unet, song_unet

    table = {"SongUNet": song_unet.SongUNet, "SongUNetPosEmbd": song_unet.SongUNetPosEmbd,
             "SongUNetPosLtEmbd": song_unet.SongUNetPosLtEmbd, "DhariwalUNet": dhariwal_unet.DhariwalUNet}
    return table[model_type]


@dataclass
class MetaData(ModelMetaData):
    jit: bool = False
    cuda_graphs: bool = False
    amp_cpu: bool = False
    amp_gpu: bool = True
    torch_fx: bool = False
    bf16: bool = True
    onnx: bool = False
    func_torch: bool = False
    auto_grad: bool = False


def _run(self, x, dtype, noise_dtype, model_kwargs):
    out = self.model(x.to(dtype), torch.zeros(x.shape[0], dtype=noise_dtype, device=x.device), class_labels=None,
                     **model_kwargs)
    if out.dtype != dtype and not torch.is_autocast_enabled():
        raise ValueError(f"Expected the dtype to be {dtype}, but got {out.dtype} instead.")
    return out.to(torch.float32)


class CorrDiffRegressionUNet(Module):
    __model_checkpoint_version__ = "0.2.0"
    __supported_model_checkpoint_version__ = {
        "0.1.0": "Loading CorrDiffRegressionUNet checkpoint from older version 0.1.0 (current version is 0.2.0). This "
                 "version is still supported, but consider re-saving the model to upgrade to version 0.2.0 and remove "
                 "this warning."
    }
    _wrapped_classes: Set[str] = {"SongUNetPosEmbd", "SongUNetPosLtEmbd", "SongUNet", "DhariwalUNet"}
    _overridable_args: Set[str] = {"use_apex_gn", "act", "profile_mode", "amp_mode"}

    @classmethod
    def _backward_compat_arg_mapper(cls, version: str, args: Dict[str, Any]) -> Dict[str, Any]:
        args = super()._backward_compat_arg_mapper(version, args)
        if version == "0.1.0":
            for stale in ("img_channels", "sigma_min", "sigma_max", "sigma_data"):
                args.pop(stale, None)
        return args

    def __init__(self, img_resolution: Union[int, Tuple[int, int]], img_in_channels: int, img_out_channels: int,
                 use_fp16: bool = False, model_type: str = "SongUNetPosEmbd", **model_kwargs: dict):
        super().__init__(meta=MetaData)
        if model_type not in self._wrapped_classes:
            raise ValueError(f"Model type '{model_type}' is not supported. Must be one of: {', '.join(self._wrapped_classes)}")
        if isinstance(img_resolution, int):
            self.img_shape_x = self.img_shape_y = img_resolution
        else:
            self.img_shape_y, self.img_shape_x = img_resolution[0], img_resolution[1]
        self.img_in_channels, self.img_out_channels = img_in_channels, img_out_channels
        self.model = _backbone(model_type)(img_resolution=img_resolution, in_channels=img_in_channels + img_out_channels,
                                           out_channels=img_out_channels, **model_kwargs)
        self.use_fp16 = use_fp16

    amp_mode = _wrapped_property("amp_mode", "model", "Set to ``True`` when using automatic mixed precision.")
    profile_mode = _wrapped_property("profile_mode", "model", "Set to ``True`` to enable profiling of the wrapped model.")

    @property
    def use_fp16(self):
        return self._use_fp16

    @use_fp16.setter
    def use_fp16(self, value: bool):
        if not (isinstance(value, bool) or value in (0, 1)):
            raise ValueError(f"`use_fp16` must be a boolean, but got {type(value).__name__}.")
        self._use_fp16 = value
        self.to(torch.float16 if value else torch.float32)

    def forward(self, x, img_lr=None, force_fp32: bool = False, **model_kwargs: dict):
        if not torch.compiler.is_compiling():
            if x.ndim != 4:
                raise ValueError(f"Expected 'x' to be a 4D tensor (B, C, H, W), got {x.ndim}D tensor with shape {tuple(x.shape)}")
            if img_lr is not None:
                if img_lr.ndim != 4:
                    raise ValueError(f"Expected 'img_lr' to be a 4D tensor (B, C, H, W), got {img_lr.ndim}D tensor with shape {tuple(img_lr.shape)}")
                if img_lr.shape[0] != x.shape[0] or img_lr.shape[2:] != x.shape[2:]:
                    raise ValueError(f"Expected 'img_lr' spatial dimensions to match 'x': x has shape {tuple(x.shape)}, but img_lr has shape {tuple(img_lr.shape)}")
        if img_lr is not None:
            x = torch.cat((x, img_lr), dim=1)
        dtype = torch.float16 if (self.use_fp16 and not force_fp32 and x.device.type == "cuda") else torch.float32
        return _run(self, x, dtype, dtype, model_kwargs)

    def round_sigma(self, sigma: Union[float, List, torch.Tensor]) -> torch.Tensor:
        return torch.as_tensor(sigma)


class UNet(CorrDiffRegressionUNet):
    def __init__(self, img_resolution, img_in_channels: int, img_out_channels: int, use_fp16: bool = False,
                 model_type: str = "SongUNetPosEmbd", **model_kwargs: dict):
        warnings.warn("UNet is deprecated and will be removed in a future version. Please use CorrDiffRegressionUNet instead.",
                      DeprecationWarning, stacklevel=2)
        super().__init__(img_resolution=img_resolution, img_in_channels=img_in_channels, img_out_channels=img_out_channels,
                         use_fp16=use_fp16, model_type=model_type, **model_kwargs)


class StormCastUNet(Module):
    def __init__(self, img_resolution, img_in_channels, img_out_channels, use_fp16=False, sigma_min=0,
                 sigma_max=float("inf"), sigma_data=0.5, model_type="SongUNet", **model_kwargs):
        super().__init__(meta=MetaData("StormCastUNet"))
        if isinstance(img_resolution, int):
            self.img_shape_x = self.img_shape_y = img_resolution
        else:
            self.img_shape_x, self.img_shape_y = img_resolution[0], img_resolution[1]
        self.img_in_channels, self.img_out_channels = img_in_channels, img_out_channels
        self.use_fp16 = use_fp16
        self.sigma_min, self.sigma_max, self.sigma_data = sigma_min, sigma_max, sigma_data
        self.model = _backbone(model_type)(img_resolution=img_resolution, in_channels=img_in_channels,
                                           out_channels=img_out_channels, **model_kwargs)

    amp_mode = _wrapped_property("amp_mode", "model", "Set to ``True`` when using automatic mixed precision.")
    profile_mode = _wrapped_property("profile_mode", "model", "Set to ``True`` to enable profiling of the wrapped model.")

    def forward(self, x, force_fp32: bool = False, **model_kwargs: dict):
        if not torch.compiler.is_compiling() and x.ndim != 4:
            raise ValueError(f"Expected 'x' to be a 4D tensor (B, C, H, W), got {x.ndim}D tensor with shape {tuple(x.shape)}")
        x = x.to(torch.float32)
        dtype = torch.float16 if (self.use_fp16 and not force_fp32 and x.device.type == "cuda") else torch.float32
        return _run(self, x, dtype, x.dtype, model_kwargs)

"""Building blocks of the DLWP-HEALPix U-Nets: config instantiation, conv / ConvNeXt / GRU blocks, encoder, decoder,
conditional layer norm and output constraints.

Parity: ``physicsnemo/models/dlwp_healpix/layers/`` (``healpix_blocks.py``, ``healpix_encoder.py``,
``healpix_decoder.py``, ``normalization.py``, ``healpix_constraints.py``).  Module attribute names and the positions
inside ``Sequential`` / ``ModuleList`` containers follow the reference so state dicts carry over.

The reference builds its sub-modules with ``hydra.utils.instantiate``; ``build`` here is a dependency-free equivalent for
the subset those configs use: a mapping with ``_target_`` (dotted path or a bare class name from this package / ``torch.nn``;
every reference spelling of the HEALPix layer paths is accepted), optional ``_partial_``, nested mappings built
recursively unless ``_recursive_`` is false, plus keyword overrides.  Classes, ``functools.partial`` objects and ready modules are accepted in place of
a mapping.
"""
from __future__ import annotations

import copy
import functools
import importlib
from typing import Any, Mapping, Sequence

import torch
from torch.utils.checkpoint import checkpoint

from ...nn.module.hpx import HEALPixAvgPool, HEALPixLayer, HEALPixMaxPool, HEALPixPadding

_ALIASES = {"AvgPool": "HEALPixAvgPool", "MaxPool": "HEALPixMaxPool"}


def _resolve(target: str):
    name = target.rsplit(".", 1)[-1]
    name = _ALIASES.get(name, name)
    if target.startswith("torch."):
        mod, _, attr = target.rpartition(".")
        return getattr(importlib.import_module(mod), attr)
    here = globals()
    if name in here:
        return here[name]
    from ...nn.module import activations as _act

    for space in (_act, torch.nn):
        if hasattr(space, name):
            return getattr(space, name)
    if "." in target:
        mod, _, attr = target.rpartition(".")
        return getattr(importlib.import_module(mod), attr)
    raise ValueError(f"cannot resolve target {target!r}")


def _is_config(obj) -> bool:
    return isinstance(obj, Mapping) or (hasattr(obj, "keys") and hasattr(obj, "__getitem__") and not isinstance(obj, torch.nn.Module))


def build(config: Any, **overrides):
    """Instantiate ``config`` (see the module docstring) with keyword ``overrides``."""
    if config is None:
        return None
    if _is_config(config):
        cfg = {k: config[k] for k in config.keys()}
        if "_target_" not in cfg:
            return {k: build(v) if _is_config(v) else v for k, v in cfg.items()}
        target = cfg.pop("_target_")
        partial = bool(cfg.pop("_partial_", False))
        recursive = bool(cfg.pop("_recursive_", True))   # False: nested configs reach the constructor unbuilt
        cfg.pop("_convert_", None)
        cfg.update(overrides)
        kwargs = {k: (build(v) if recursive and _is_config(v) and "_target_" in v.keys() else v) for k, v in cfg.items()}
        fn = _resolve(target) if isinstance(target, str) else target
        return functools.partial(fn, **kwargs) if partial else fn(**kwargs)
    if isinstance(config, torch.nn.Module):
        if overrides:
            raise TypeError("a ready module cannot take constructor overrides; pass a class, a partial or a config mapping")
        return config
    if callable(config):
        return config(**overrides)
    raise TypeError(f"cannot instantiate from {type(config).__name__}")


def _cfg_copy(config):
    return copy.copy(config) if not _is_config(config) else {k: config[k] for k in config.keys()}


def _strip_cln(config, keep: bool):
    if keep:
        return config
    if _is_config(config) and "conditional_layer_norm" in config.keys() and config["conditional_layer_norm"] is not None:
        config = _cfg_copy(config)
        config["conditional_layer_norm"] = None
    elif isinstance(config, functools.partial) and config.keywords.get("conditional_layer_norm") is not None:
        config = functools.partial(config.func, *config.args, **{**config.keywords, "conditional_layer_norm": None})
    return config


# ---- normalisation and constraints -----------------------------------------------------------------------------------
class ConditionalLayerNorm(torch.nn.Module):
    """Channel LayerNorm whose scale and shift come from an MLP of per-sample conditions ``[B, condition_shape]``; the
    per-sample affine is broadcast over the ``n_faces`` faces folded into the batch axis."""

    def __init__(self, condition_shape: int, channel_depth: int, mlp_hidden_dims: Sequence[int] = (128, 128), activation=None,
                 n_faces: int = 12, norm_op: str = "torch", init_cln_to_zero: bool = False, scale_center: float = 1.0):
        super().__init__()
        self.condition_shape, self.channel_depth, self.hidden_dims = condition_shape, channel_depth, list(mlp_hidden_dims)
        self.activation = activation if activation is not None else torch.nn.Identity()
        layers, d = [], condition_shape
        for h in self.hidden_dims:
            layers += [torch.nn.Linear(d, 2 * h), self.activation]
            d = 2 * h
        layers.append(torch.nn.Linear(d, 2 * channel_depth))
        self.gamma_beta_mlp = torch.nn.Sequential(*layers)
        self.n_faces, self.scale_center = n_faces, scale_center
        if init_cln_to_zero:
            torch.nn.init.zeros_(self.gamma_beta_mlp[-1].weight)
            torch.nn.init.zeros_(self.gamma_beta_mlp[-1].bias)
        if norm_op not in ("torch", "apex"):
            raise ValueError(f"norm_op must be 'torch' or 'apex', got {norm_op!r}")
        self.norm = torch.nn.LayerNorm(channel_depth, elementwise_affine=False)

    def forward(self, x: torch.Tensor, conditions: torch.Tensor) -> torch.Tensor:
        channels_last = x.is_contiguous(memory_format=torch.channels_last)
        xn = self.norm(x.permute(0, 2, 3, 1))
        gamma, beta = self.gamma_beta_mlp(conditions).chunk(2, dim=-1)
        C = gamma.shape[-1]
        gamma = (self.scale_center + gamma).unsqueeze(1).expand(-1, self.n_faces, -1).reshape(-1, 1, 1, C)
        beta = beta.unsqueeze(1).expand(-1, self.n_faces, -1).reshape(-1, 1, 1, C)
        out = (gamma * xn + beta).permute(0, 3, 1, 2)
        return out.contiguous(memory_format=torch.channels_last) if channels_last else out


class NonnegativeConstraint(torch.nn.Module):
    """Clamp the named output variables of ``[B, F, T, C, H, W]`` at physical zero (``-mean/std`` in scaled units)."""

    def __init__(self, variables, channels, scaling):
        super().__init__()
        self.channels, self.scaling = channels, scaling
        self.variables = [v for v in variables if v in channels]
        self.register_buffer("var_indices", torch.tensor([channels.index(v) for v in self.variables], dtype=torch.long), persistent=False)
        self.var_means = torch.tensor([scaling[v]["mean"] for v in self.variables])
        self.var_stds = torch.tensor([scaling[v]["std"] for v in self.variables])
        self.register_buffer("thresholds", ((0.0 - self.var_means) / self.var_stds).view(1, 1, 1, -1, 1, 1), persistent=False)

    def forward(self, x):
        sel = torch.index_select(x, 3, self.var_indices)
        x.index_copy_(3, self.var_indices, torch.maximum(sel, self.thresholds).to(x.dtype))
        return x


# ---- blocks ----------------------------------------------------------------------------------------------------------
def _geo_conv(geometry_layer, cin, cout, k, dilation, nhwc, pad):
    return geometry_layer(layer=torch.nn.Conv2d, in_channels=cin, out_channels=cout, kernel_size=k, dilation=dilation,
                          enable_nhwc=nhwc, enable_healpixpad=pad)


def _run(layers, x, conditions_cln):
    for layer in layers:
        x = layer(x, conditions=conditions_cln) if isinstance(layer, ConditionalLayerNorm) else layer(x)
    return x


def _skip(geometry_layer, cin, cout, nhwc, pad):
    if cin == cout:
        return lambda x: x
    return geometry_layer(layer=torch.nn.Conv2d, in_channels=cin, out_channels=cout, kernel_size=1, enable_nhwc=nhwc, enable_healpixpad=pad)


class ConvGRUBlock(torch.nn.Module):
    """Convolutional GRU cell with a residual connection; the hidden state lives on the module until ``reset``."""

    def __init__(self, geometry_layer=HEALPixLayer, in_channels: int = 3, kernel_size: int = 1, enable_nhwc: bool = False,
                 enable_healpixpad: bool = False):
        super().__init__()
        self.channels = in_channels
        mk = lambda cout: geometry_layer(layer=torch.nn.Conv2d, in_channels=2 * in_channels, out_channels=cout, kernel_size=kernel_size,  # noqa: E731
                                         padding="same", enable_nhwc=enable_nhwc, enable_healpixpad=enable_healpixpad)
        self.conv_gates = mk(2 * in_channels)
        self.conv_can = mk(in_channels)
        self.h = torch.zeros(1, 1, 1, 1)

    def forward(self, inputs):
        if inputs.shape != self.h.shape or inputs.device != self.h.device or inputs.dtype != self.h.dtype:
            self.h = torch.zeros_like(inputs)
        gamma, beta = torch.split(self.conv_gates(torch.cat([inputs, self.h], dim=1)), self.channels, dim=1)
        reset_gate, update_gate = torch.sigmoid(gamma), torch.sigmoid(beta)
        cand = torch.tanh(self.conv_can(torch.cat([inputs, reset_gate * self.h], dim=1)))
        self.h = (1 - update_gate) * self.h + update_gate * cand
        return inputs + self.h

    def reset(self):
        self.h = torch.zeros_like(self.h)


class BasicConvBlock(torch.nn.Module):
    def __init__(self, geometry_layer=HEALPixLayer, in_channels: int = 3, out_channels: int = 1, kernel_size: int = 3, dilation: int = 1,
                 n_layers: int = 1, latent_channels: int = None, activation=None, enable_nhwc: bool = False, enable_healpixpad: bool = False):
        super().__init__()
        latent = max(in_channels, out_channels) if latent_channels is None else latent_channels
        mods = []
        for n in range(n_layers):
            mods.append(_geo_conv(geometry_layer, in_channels if n == 0 else latent, out_channels if n == n_layers - 1 else latent,
                                  kernel_size, dilation, enable_nhwc, enable_healpixpad))
            if activation is not None:
                mods.append(activation)
        self.convblock = torch.nn.Sequential(*mods)

    def forward(self, x):
        return self.convblock(x)


class ConvNeXtBlock(torch.nn.Module):
    """k×k → k×k → 1×1 with a widened middle and a (projected) skip connection."""

    def __init__(self, geometry_layer=HEALPixLayer, in_channels: int = 3, latent_channels: int = 1, out_channels: int = 1, kernel_size: int = 3,
                 dilation: int = 1, n_layers: int = 1, upscale_factor: int = 4, activation=None, enable_nhwc: bool = False,
                 enable_healpixpad: bool = False):
        super().__init__()
        self.skip_module = _skip(geometry_layer, in_channels, out_channels, enable_nhwc, enable_healpixpad)
        wide = int(latent_channels * upscale_factor)
        mods = []
        for cin, cout, k in ((in_channels, wide, kernel_size), (wide, wide, kernel_size)):
            mods.append(_geo_conv(geometry_layer, cin, cout, k, dilation, enable_nhwc, enable_healpixpad))
            if activation is not None:
                mods.append(activation)
        mods.append(geometry_layer(layer=torch.nn.Conv2d, in_channels=wide, out_channels=out_channels, kernel_size=1,
                                   enable_nhwc=enable_nhwc, enable_healpixpad=enable_healpixpad))
        self.convblock = torch.nn.Sequential(*mods)

    def forward(self, x):
        return self.skip_module(x) + self.convblock(x)


def _cln_stack(geometry_layer, plan, dilation, activation, dropout, conditional_layer_norm, nhwc, pad):
    """Conv stack of ``plan = [(cin, cout, kernel, with_norm)]``; each conv is followed by [CLN] [activation] [dropout]."""
    mods = []
    for cin, cout, k, with_norm in plan:
        mods.append(_geo_conv(geometry_layer, cin, cout, k, dilation, nhwc, pad))
        if with_norm and conditional_layer_norm is not None:
            mods.append(conditional_layer_norm(channel_depth=cout))
        if activation is not None:
            mods.append(activation)
        if dropout > 0.0:
            mods.append(torch.nn.Dropout2d(p=dropout))
    return torch.nn.ModuleList(mods)


class DoubleConvNeXtBlock(torch.nn.Module):
    """Two inverted-bottleneck stages (k×k → 1×1 wide → 1×1), each with its own skip connection."""

    def __init__(self, geometry_layer=HEALPixLayer, in_channels: int = 3, out_channels: int = 1, kernel_size: int = 3, dilation: int = 1,
                 n_layers: int = 1, upscale_factor: int = 4, latent_channels: int = 1, activation=None, enable_nhwc: bool = False,
                 enable_healpixpad: bool = False, dropout: float = 0.0, conditional_layer_norm=None):
        super().__init__()
        self.cln_enabled = conditional_layer_norm is not None
        lat, wide = int(latent_channels), int(latent_channels * upscale_factor)
        self.skip_module1 = _skip(geometry_layer, in_channels, lat, enable_nhwc, enable_healpixpad)
        self.skip_module2 = _skip(geometry_layer, lat, out_channels, enable_nhwc, enable_healpixpad)
        args = (dilation, activation, dropout, conditional_layer_norm, enable_nhwc, enable_healpixpad)
        self.convblock1 = _cln_stack(geometry_layer, [(in_channels, lat, kernel_size, True), (lat, wide, 1, True), (wide, lat, 1, False)], *args)
        self.convblock2 = _cln_stack(geometry_layer, [(lat, lat, kernel_size, True), (lat, wide, 1, True), (wide, out_channels, 1, False)], *args)

    def forward(self, x, conditions_cln=None):
        x1 = self.skip_module1(x) + _run(self.convblock1, x, conditions_cln)
        return self.skip_module2(x1) + _run(self.convblock2, x1, conditions_cln)


class SymmetricConvNeXtBlock(torch.nn.Module):
    """k×k → 1×1 wide → 1×1 → k×k with an optional block-level skip connection."""

    def __init__(self, geometry_layer=HEALPixLayer, in_channels: int = 3, latent_channels: int = 1, out_channels: int = 1, kernel_size: int = 3,
                 dilation: int = 1, n_layers: int = 1, upscale_factor: int = 4, activation=None, enable_nhwc: bool = False,
                 enable_healpixpad: bool = False, dropout: float = 0.0, conditional_layer_norm=None, use_block_skip_connection: bool = True):
        super().__init__()
        self.use_block_skip_connection, self.activation, self.dropout = use_block_skip_connection, activation, dropout > 0.0
        self.cln_enabled = conditional_layer_norm is not None
        if use_block_skip_connection:
            self.skip_module = _skip(geometry_layer, in_channels, int(out_channels), enable_nhwc, enable_healpixpad)
        lat, wide = int(latent_channels), int(latent_channels * upscale_factor)
        self.convblock = _cln_stack(geometry_layer, [(in_channels, lat, kernel_size, True), (lat, wide, 1, True), (wide, lat, 1, True),
                                                     (lat, out_channels, kernel_size, False)],
                                    dilation, activation, dropout, conditional_layer_norm, enable_nhwc, enable_healpixpad)

    def forward(self, x, conditions_cln=None):
        residual = self.skip_module(x) if self.use_block_skip_connection else 0
        return _run(self.convblock, x, conditions_cln) + residual


class Multi_SymmetricConvNeXtBlock(torch.nn.Module):
    """``n_layers`` symmetric ConvNeXt blocks in sequence."""

    def __init__(self, geometry_layer=HEALPixLayer, in_channels: int = 3, latent_channels: int = 1, out_channels: int = 1, kernel_size: int = 3,
                 dilation: int = 1, upscale_factor: int = 4, n_layers: int = 1, activation=None, enable_nhwc: bool = False,
                 enable_healpixpad: bool = False, dropout: float = 0.0, conditional_layer_norm=None, use_block_skip_connection: bool = True):
        super().__init__()
        self.cln_enabled = conditional_layer_norm is not None
        self.blocks = torch.nn.ModuleList([
            SymmetricConvNeXtBlock(geometry_layer=geometry_layer, in_channels=in_channels if i == 0 else out_channels,
                                   latent_channels=latent_channels, out_channels=out_channels, kernel_size=kernel_size, dilation=dilation,
                                   upscale_factor=upscale_factor, activation=activation, enable_nhwc=enable_nhwc,
                                   enable_healpixpad=enable_healpixpad, dropout=dropout, conditional_layer_norm=conditional_layer_norm,
                                   use_block_skip_connection=use_block_skip_connection) for i in range(n_layers)])

    def forward(self, x, conditions_cln=None):
        for block in self.blocks:
            x = block(x, conditions_cln=conditions_cln)
        return x


class TransposedConvUpsample(torch.nn.Module):
    def __init__(self, geometry_layer=HEALPixLayer, in_channels: int = 3, out_channels: int = 1, upsampling: int = 2, activation=None,
                 enable_nhwc: bool = False, enable_healpixpad: bool = False):
        super().__init__()
        mods = [geometry_layer(layer=torch.nn.ConvTranspose2d, in_channels=in_channels, out_channels=out_channels, kernel_size=upsampling,
                               stride=upsampling, padding=0, enable_nhwc=enable_nhwc, enable_healpixpad=enable_healpixpad)]
        if activation is not None:
            mods.append(activation)
        self.upsampler = torch.nn.Sequential(*mods)

    def forward(self, x):
        return self.upsampler(x)


class Interpolate(torch.nn.Module):
    def __init__(self, scale_factor, mode: str = "nearest"):
        super().__init__()
        self.scale_factor, self.mode = scale_factor, mode

    def forward(self, inputs):
        return torch.nn.functional.interpolate(inputs, scale_factor=self.scale_factor, mode=self.mode)


# ---- encoder / decoder -----------------------------------------------------------------------------------------------
def _per_level(values, n, name, default):
    if values is None:
        return [default] * n
    if len(values) != n:
        raise ValueError(f"{name} must be a list of booleans of the same length as n_channels. Got {len(values)} for {name} and {n} for n_channels")
    return list(values)


def _call_block(layer, x, conditions_cln):
    if getattr(layer, "cln_enabled", False):
        if conditions_cln is None:
            raise ValueError("Conditional inputs are required for layers with cln_enabled=True")
        return layer(x, conditions_cln=conditions_cln)
    return layer(x)


class UNetEncoder(torch.nn.Module):
    """Levels of [downsample →] conv block; returns the activations of every level, finest first."""

    def __init__(self, conv_block, down_sampling_block, recurrent_block=None, input_channels: int = 3, n_channels: Sequence = (16, 32, 64),
                 n_layers: Sequence = (2, 2, 1), dilations: list = None, enable_nhwc: bool = False, enable_healpixpad: bool = False,
                 per_level_cln: Sequence[bool] = None, per_level_checkpointing: Sequence[bool] = None):
        super().__init__()
        self.n_channels = n_channels
        cln = _per_level(per_level_cln, len(n_channels), "per_level_cln", True)
        self.per_level_checkpointing = _per_level(per_level_checkpointing, len(n_channels), "per_level_checkpointing", False)
        dilations = dilations if dilations is not None else [1] * len(n_channels)
        levels, old = [], input_channels
        for n, ch in enumerate(n_channels):
            mods = []
            if n > 0:
                mods.append(build(down_sampling_block, enable_nhwc=enable_nhwc, enable_healpixpad=enable_healpixpad))
            mods.append(build(_strip_cln(conv_block, cln[n]), in_channels=old, latent_channels=ch, out_channels=ch, dilation=dilations[n],
                              n_layers=n_layers[n], enable_nhwc=enable_nhwc, enable_healpixpad=enable_healpixpad))
            old = ch
            levels.append(torch.nn.Sequential(*mods))
        self.encoder = torch.nn.ModuleList(levels)

    @staticmethod
    def _forward_layer_pass(group, x, conditions_cln=None):
        for layer in group:
            x = _call_block(layer, x, conditions_cln)
        return x

    def forward(self, inputs, conditions_cln=None):
        outputs, x = [], inputs
        for n, group in enumerate(self.encoder):
            if self.per_level_checkpointing[n]:
                x = checkpoint(self._forward_layer_pass, group, x, conditions_cln, use_reentrant=False)
            else:
                x = self._forward_layer_pass(group, x, conditions_cln)
            outputs.append(x)
        return outputs

    def reset(self):
        pass


class UNetDecoder(torch.nn.Module):
    """Levels of [upsample + skip concat →] conv block [→ recurrent block], coarsest first, then the output layer."""

    def __init__(self, conv_block, up_sampling_block, output_layer, recurrent_block=None, n_channels: Sequence = (64, 32, 16),
                 n_layers: Sequence = (1, 2, 2), output_channels: int = 1, dilations: list = None, enable_nhwc: bool = False,
                 enable_healpixpad: bool = False, per_level_cln: Sequence[bool] = None, per_level_checkpointing: Sequence[bool] = None):
        super().__init__()
        self.channel_dim = 1
        cln = _per_level(per_level_cln, len(n_channels), "per_level_cln", True)
        self.per_level_checkpointing = _per_level(per_level_checkpointing, len(n_channels), "per_level_checkpointing", False)
        dilations = dilations if dilations is not None else [1] * len(n_channels)
        levels = []
        for n, ch in enumerate(n_channels):
            up = None if n == 0 else build(up_sampling_block, in_channels=ch, out_channels=ch, enable_nhwc=enable_nhwc,
                                           enable_healpixpad=enable_healpixpad)
            nxt = n_channels[n + 1] if n < len(n_channels) - 1 else n_channels[-1]
            conv = build(_strip_cln(conv_block, cln[n]), in_channels=ch * 2 if n > 0 else ch, latent_channels=ch, out_channels=nxt,
                         dilation=dilations[n], n_layers=n_layers[n], enable_nhwc=enable_nhwc, enable_healpixpad=enable_healpixpad)
            rec = build(recurrent_block, in_channels=nxt, enable_healpixpad=enable_healpixpad) if recurrent_block is not None else None
            levels.append(torch.nn.ModuleDict({"upsamp": up, "conv": conv, "recurrent": rec}))
        self.decoder = torch.nn.ModuleList(levels)
        self.output_layer = build(output_layer, in_channels=n_channels[-1], out_channels=output_channels, dilation=dilations[-1],
                                  enable_nhwc=enable_nhwc, enable_healpixpad=enable_healpixpad)

    def _forward_layer_pass(self, layer, x, skip_connection=None, conditions_cln=None):
        if layer["upsamp"] is not None:
            x = torch.cat([layer["upsamp"](x), skip_connection], dim=self.channel_dim)
        return _call_block(layer["conv"], x, conditions_cln)

    def forward(self, inputs, conditions_cln=None):
        x = inputs[-1]
        for n, layer in enumerate(self.decoder):
            skip = inputs[-1 - n] if layer["upsamp"] is not None else None
            if self.per_level_checkpointing[n]:
                x = checkpoint(self._forward_layer_pass, layer, x, skip, conditions_cln, use_reentrant=False)
            else:
                x = self._forward_layer_pass(layer, x, skip, conditions_cln)
            if layer["recurrent"] is not None:
                x = layer["recurrent"](x)
        return self.output_layer(x)

    def reset(self):
        for layer in self.decoder:
            if layer["recurrent"] is not None:
                layer["recurrent"].reset()


AvgPool, MaxPool = HEALPixAvgPool, HEALPixMaxPool

__all__ = ["AvgPool", "BasicConvBlock", "ConditionalLayerNorm", "ConvGRUBlock", "ConvNeXtBlock", "DoubleConvNeXtBlock", "HEALPixAvgPool",
           "HEALPixLayer", "HEALPixMaxPool", "HEALPixPadding", "Interpolate", "MaxPool", "Multi_SymmetricConvNeXtBlock",
           "NonnegativeConstraint", "SymmetricConvNeXtBlock", "TransposedConvUpsample", "UNetDecoder", "UNetEncoder", "build"]

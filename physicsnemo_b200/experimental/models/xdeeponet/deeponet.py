"""Extended DeepONet: one or two branch networks, an optional trunk, and a decoder on their product.

Counterpart of ``physicsnemo/experimental/models/xdeeponet/deeponet.py`` (``DeepONet`` :97).  Covers the same
variants by composition: DeepONet / U-DeepONet / Fourier-DeepONet (spatial ``branch1`` + trunk), MIONet (two
branches), TNO (temporal-projection decoder), and trunkless xFNO-style operators.

Calling conventions
-------------------
* core mode (``auto_pad=False``): ``model(x_branch1, x_time[, x_branch2])`` or, without a trunk, ``model(x_branch1)``.
* packed mode (``auto_pad=True``): ``model(x[, x_branch2], target_times=...)`` where ``x`` is ``[B, *S, T, C]`` whose
  last channels hold the grid coordinates and the time; the spatial axes are right-padded (replicate) to a multiple
  of 8 with at least ``padding`` cells, and the output is cropped back.

Memory layout: the branch field ``[B, *S, W]`` and the trunk table ``[T, W]`` are multiplied straight into the output
order ``[B, *S, T, W]`` so the pointwise MLP decoder writes ``[B, *S, T, C_out]`` with no trailing permutation; only
the convolutional decoder needs a channels-first view (``[B*T, W, *S]``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Literal, Optional

import torch
import torch.nn as nn
from torch import Tensor

from ....core.meta import ModelMetaData
from ....core.module import Module
from ....models.mlp import FullyConnected
from ....nn.module.activations import get_activation
from ....nn.module.fully_connected_layers import Conv2dFCLayer, Conv3dFCLayer
from ._padding import compute_right_pad_to_multiple, pad_spatial_right
from .branches import SpatialBranch

__all__ = ["DeepONet"]

_DECODERS = ("mlp", "conv", "temporal_projection")


@dataclass
class _MetaData(ModelMetaData):
    pass


class DeepONet(Module):
    """``decoder(branch1(u) * branch2(v) * trunk(t))`` with the variants described in the module docstring."""

    def __init__(self, branch1: nn.Module, *, trunk: Optional[nn.Module] = None, branch2: Optional[nn.Module] = None,
                 dimension: Literal[2, 3] = 2, width: int = 64, out_channels: int = 1,
                 decoder_type: Literal["mlp", "conv", "temporal_projection"] = "mlp", decoder_width: int = 128,
                 decoder_layers: int = 2, decoder_activation_fn: str = "relu", output_window: Optional[int] = None,
                 auto_pad: bool = False, padding: int = 8, trunk_input: Literal["time", "grid"] = "time",
                 time_modes: Optional[int] = None):
        super().__init__(meta=_MetaData())
        if dimension not in (2, 3):
            raise ValueError(f"DeepONet only supports dimension=2 or dimension=3, got dimension={dimension!r}.")
        if out_channels < 1:
            raise ValueError(f"out_channels must be >= 1, got {out_channels}.")
        kind = decoder_type.lower()
        if kind not in _DECODERS:
            raise ValueError(f"Unknown decoder_type: {decoder_type!r}. Valid: {sorted(_DECODERS)}.")
        if trunk_input not in ("time", "grid"):
            raise ValueError(f"trunk_input must be 'time' or 'grid', got {trunk_input!r}.")
        if padding < 0:
            raise ValueError(f"padding must be non-negative, got {padding}.")
        if time_modes is not None:
            if trunk is not None:
                raise ValueError("time_modes is only meaningful when trunk is None (xFNO-style trunkless operators).  "
                                 "Drop time_modes, or set trunk=None.")
            if not auto_pad:
                raise ValueError("time_modes requires auto_pad=True; the time-axis-extend feature is part of the "
                                 "packed-input forward path.")
            if time_modes < 1:
                raise ValueError(f"time_modes must be >= 1, got {time_modes}.")
        b1_vector = not isinstance(branch1, SpatialBranch)
        b2_vector = branch2 is not None and not isinstance(branch2, SpatialBranch)
        if trunk is None and kind == "temporal_projection":
            raise ValueError("decoder_type='temporal_projection' requires a trunk; use decoder_type='mlp' or 'conv' for "
                             "trunkless operators.")
        if b1_vector and kind != "mlp":
            raise ValueError(f"decoder_type={kind!r} is not supported with MLP branches.  Use decoder_type='mlp', or "
                             "pass a SpatialBranch as branch1.")
        if branch2 is not None and b1_vector and not b2_vector:
            raise ValueError("When branch1 is an MLP branch, branch2 must also be an MLP branch (i.e. produce a 2D "
                             "(B, width) output).  Swap branch1 and branch2, or pass a SpatialBranch as branch1.")
        if b1_vector and auto_pad:
            raise ValueError("auto_pad=True requires a SpatialBranch branch1 (the packed-input forward path operates on "
                             "spatial dims).  Use auto_pad=False with an MLP branch.")
        if output_window is not None and kind == "temporal_projection" and output_window < 1:
            raise ValueError(f"output_window must be a positive integer, got {output_window}")

        self.dimension, self.out_channels, self.width = dimension, out_channels, width
        self.decoder_type, self.decoder_activation_fn, self.trunk_input = kind, decoder_activation_fn, trunk_input
        self.auto_pad, self.padding, self.time_modes = auto_pad, -(-padding // 8) * 8, time_modes
        self.has_branch2 = branch2 is not None
        self.branch1 = branch1
        if branch2 is not None:
            self.branch2 = branch2
        self.trunk = trunk
        self._temporal_projection = kind == "temporal_projection"
        if self._temporal_projection:
            self.decoder = self._make_decoder(width, width, decoder_layers, decoder_width, "mlp", decoder_activation_fn)
            self.temporal_head = nn.Linear(width, output_window * out_channels) if output_window is not None else None
        else:
            self.decoder = self._make_decoder(width, out_channels, decoder_layers, decoder_width, kind, decoder_activation_fn)

    # ----------------------------------------------------------------------------------------------------------
    @property
    def has_temporal_projection(self) -> bool:
        return self._temporal_projection

    def set_output_window(self, K: int) -> None:
        """(Re)create the temporal head for ``K`` output steps (temporal-projection decoder only)."""
        if self._temporal_projection:
            self.temporal_head = nn.Linear(self.width, K * self.out_channels).to(next(self.parameters()).device)

    def _make_decoder(self, width, out_channels, num_layers, hidden, kind, act) -> nn.Module:
        if kind == "mlp":
            return nn.Linear(width, out_channels) if num_layers == 0 else FullyConnected(width, hidden, out_channels, num_layers, act)
        if kind != "conv":
            raise ValueError(f"Unknown decoder_type: {kind}")
        pointwise = Conv2dFCLayer if self.dimension == 2 else Conv3dFCLayer
        if num_layers == 0:
            return pointwise(width, out_channels)
        layers, cin = [], width
        for _ in range(num_layers):
            layers += [pointwise(cin, hidden), get_activation(act)]
            cin = hidden
        return nn.Sequential(*layers, pointwise(hidden, out_channels))

    # ---------------------------------------------------------------------------------------------- dispatch
    def forward(self, *args: Tensor, x_branch2: Optional[Tensor] = None, target_times: Optional[Tensor] = None) -> Tensor:
        trunkless = self.trunk is None
        if trunkless:
            mode = "packed" if self.auto_pad else "core"
            if len(args) != 1:
                raise TypeError(f"In trunkless {mode}{'-input' if self.auto_pad else ''} mode (auto_pad={self.auto_pad}, "
                                f"trunk=None), forward expects exactly 1 positional tensor, got {len(args)}.")
            if x_branch2 is not None:
                raise TypeError("x_branch2 is not supported in trunkless mode.")
        if not self.auto_pad and target_times is not None:
            raise TypeError("target_times is only valid in packed-input mode (construct DeepONet with auto_pad=True).")
        if trunkless:
            return self._packed_trunkless(args[0], target_times) if self.auto_pad else self._core(args[0], None, None)
        lo = 1 if self.auto_pad else 2
        if not lo <= len(args) <= lo + 1:
            what = "((x,) or (x, x_branch2))" if self.auto_pad else "((x_branch1, x_time) or (x_branch1, x_time, x_branch2))"
            raise TypeError(f"In trunked {'packed-input' if self.auto_pad else 'core'} mode (auto_pad={self.auto_pad}, "
                            f"trunk!=None), forward expects {lo} or {lo + 1} positional tensors {what}, got {len(args)}.")
        if len(args) == lo + 1:
            if x_branch2 is not None:
                raise TypeError("x_branch2 supplied both positionally and as a keyword argument.")
            x_branch2 = args[lo]
        if self.auto_pad:
            return self._packed(args[0], x_branch2, target_times)
        return self._core(args[0], args[1], x_branch2)

    # ------------------------------------------------------------------------------------------- packed input
    @staticmethod
    def _check_times(target_times):
        if target_times is not None and target_times.ndim not in (1, 2):
            raise ValueError(f"Expected target_times to be 1D (K,) or 2D (K, 1), got {target_times.ndim}D tensor with "
                             f"shape {tuple(target_times.shape)}.")

    def _spatial_pad(self, x: Tensor, like_shape=None) -> Tensor:
        shape = x.shape[1:1 + self.dimension] if like_shape is None else like_shape
        pads = compute_right_pad_to_multiple(shape, multiple=8, min_right_pad=self.padding)
        return pad_spatial_right(x, spatial_ndim=self.dimension, right_pad=pads, mode="replicate")

    def _packed(self, x: Tensor, x_branch2: Optional[Tensor], target_times: Optional[Tensor]) -> Tensor:
        d = self.dimension
        if not torch.compiler.is_compiling():
            if x.ndim != d + 3:
                raise ValueError(f"Packed-input mode (trunked) expects {d + 3}D input (B, {'H, W' if d == 2 else 'X, Y, Z'}, "
                                 f"T, C), got {x.ndim}D tensor with shape {tuple(x.shape)}.")
            self._check_times(target_times)
        space = tuple(x.shape[1:1 + d])
        if self.padding > 0:
            x = self._spatial_pad(x, space)
            if x_branch2 is not None and x_branch2.dim() > 2:
                x_branch2 = self._spatial_pad(x_branch2, space)
        first_step = (slice(None),) * (1 + d) + (0,)
        origin = (0,) * (1 + d)                      # sample 0, first grid cell: where the coordinates are read
        if x_branch2 is not None and x_branch2.ndim == d + 3:
            x_branch2 = x_branch2[first_step]
        if target_times is not None:
            t = target_times.reshape(-1, 1)
            if self.trunk_input == "grid":
                here = x[origin + (0, slice(-(d + 1), -1))]
                t = torch.cat([here.expand(t.shape[0], -1), t], dim=-1)
        elif self.trunk_input == "grid":
            t = x[origin + (slice(None), slice(-(d + 1), None))]
        else:
            t = x[origin + (slice(None), slice(-1, None))]
        out = self._core(x[first_step], t, x_branch2)
        if self.padding > 0:
            out = out[(slice(None),) + tuple(slice(0, s) for s in space)]
        return out

    def _packed_trunkless(self, x: Tensor, target_times: Optional[Tensor]) -> Tensor:
        d = self.dimension
        if not torch.compiler.is_compiling():
            if x.ndim != d + 2:
                raise ValueError(f"Packed-input mode (trunkless) expects {d + 2}D input (B, {'H, W' if d == 2 else 'X, Y, Z'}, "
                                 f"C), got {x.ndim}D tensor with shape {tuple(x.shape)}.")
            if target_times is not None and self.time_modes is None:
                raise ValueError("target_times provided but the model was constructed without time_modes; nothing to "
                                 "extend.  Either pass time_modes=N at construction (xFNO-style autoregressive bundling) "
                                 "or omit target_times.")
            self._check_times(target_times)
        space = tuple(x.shape[1:1 + d])
        t_in, k_future = space[-1], None
        if self.time_modes is not None and target_times is not None and target_times.shape[0] != t_in:
            # the last spatial axis is time: extend it (replicate) so that the K future steps fit and the spectral
            # layers still see at least 2 * time_modes cells
            k_future = target_times.shape[0]
            extra = max(t_in + k_future, 2 * self.time_modes) - t_in
            x = pad_spatial_right(x, spatial_ndim=d, right_pad=(0,) * (d - 1) + (extra,), mode="replicate")
        if self.padding > 0:
            x = self._spatial_pad(x)
        out = self._core(x, None, None)
        last = slice(t_in, t_in + k_future) if k_future is not None else slice(0, t_in)
        return out[(slice(None),) + tuple(slice(0, s) for s in space[:-1]) + (last,)]

    # --------------------------------------------------------------------------------------------------- core
    def _core(self, x_branch1: Tensor, x_time: Optional[Tensor], x_branch2: Optional[Tensor]) -> Tensor:
        d, nd = self.dimension, self.dimension + 2
        if not torch.compiler.is_compiling():
            if x_branch1.ndim not in (2, nd):
                raise ValueError(f"Expected x_branch1 to be 2D (B, D_in) for MLP branches or {nd}D "
                                 f"{'(B, H, W, C)' if d == 2 else '(B, X, Y, Z, C)'} for spatial branches, got "
                                 f"{x_branch1.ndim}D tensor with shape {tuple(x_branch1.shape)}")
            if x_time is not None and x_time.ndim not in (1, 2):
                raise ValueError(f"Expected x_time to be 1D (T,) or 2D (T, D), got {x_time.ndim}D tensor with shape "
                                 f"{tuple(x_time.shape)}")
            if self.has_branch2 and x_branch2 is None:
                raise ValueError("branch2 is configured but x_branch2 was not provided to forward().")
        u = self.branch1(x_branch1)
        v = self.branch2(x_branch2) if self.has_branch2 else None
        spatial = u.dim() == nd
        if v is not None and spatial and v.dim() != nd:
            v = v.reshape(v.shape[0], *(1,) * d, v.shape[-1])            # vector branch against a field
        uv = u if v is None else u * v

        if self.trunk is None:
            if spatial and self.decoder_type == "conv":
                return self.decoder(uv.movedim(-1, 1)).movedim(1, -1)
            return self.decoder(uv)

        tau = self.trunk(x_time.reshape(-1, 1) if x_time.dim() == 1 else x_time)      # [T, W]
        if not spatial:
            return self.decoder(uv.unsqueeze(1) * tau)                                   # [B, T, C_out]
        if self._temporal_projection:
            if self.temporal_head is None:
                raise RuntimeError("decoder_type='temporal_projection' requires either output_window to be provided at "
                                   "construction time, or set_output_window(K) to be called before forward.")
            y = self.temporal_head(self.decoder(uv * tau[0]))
            return y.reshape(*y.shape[:-1], -1, self.out_channels)
        z = uv.unsqueeze(-2) * tau                                                        # [B, *S, T, W]
        if self.decoder_type == "mlp":
            return self.decoder(z)
        B, T, S = z.shape[0], z.shape[-2], z.shape[1:-2]
        y = self.decoder(z.permute(0, d + 1, d + 2, *range(1, d + 1)).reshape(B * T, self.width, *S))
        return y.reshape(B, T, self.out_channels, *S).permute(0, *range(3, d + 3), 1, 2)

"""Channels-last wrapper of the 4-D (x, y, z, t) Fourier neural operator with autoregressive time extension.

Counterpart of ``physicsnemo/experimental/models/xdeeponet/fno4d.py`` (``FNO4DWrapper`` :46).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Union

import torch
from torch import Tensor

from ....core.meta import ModelMetaData
from ....core.module import Module
from ....models.fno import FNO
from ._padding import pad_spatial_right

__all__ = ["FNO4DWrapper"]


@dataclass
class _MetaData(ModelMetaData):
    pass


class FNO4DWrapper(Module):
    """``[B, X, Y, Z, T, C_in] -> [B, X, Y, Z, T or K, C_out]`` (the channel axis is dropped when ``C_out == 1``).

    With ``target_times`` of length ``K != T`` the time axis is right-extended by replication to
    ``max(T + K, 2 * time_modes)`` cells and the output is the slice ``[T, T + K)``.
    """

    def __init__(self, in_channels: int, out_channels: int = 1, latent_channels: int = 32, num_fno_layers: int = 4,
                 num_fno_modes: Union[int, List[int]] = 16, padding: int = 8, padding_type: str = "constant",
                 activation_fn: str = "gelu", decoder_layers: int = 1, decoder_layer_size: int = 32,
                 decoder_activation_fn: str = "silu", coord_features: bool = True):
        super().__init__(meta=_MetaData())
        self.time_modes = int(num_fno_modes[-1] if isinstance(num_fno_modes, (list, tuple)) else num_fno_modes)
        self.fno = FNO(in_channels=in_channels, out_channels=out_channels, dimension=4, latent_channels=latent_channels,
                       num_fno_layers=num_fno_layers, num_fno_modes=num_fno_modes, padding=padding, padding_type=padding_type,
                       activation_fn=activation_fn, decoder_layers=decoder_layers, decoder_layer_size=decoder_layer_size,
                       decoder_activation_fn=decoder_activation_fn, coord_features=coord_features)

    def forward(self, x: Tensor, target_times: Optional[Tensor] = None) -> Tensor:
        if not torch.compiler.is_compiling() and x.ndim != 6:
            raise ValueError(f"Expected x to be 6D (B, X, Y, Z, T, C_in), got {x.ndim}D tensor with shape {tuple(x.shape)}.")
        t_in = x.shape[4]
        window = slice(0, t_in)
        if target_times is not None and target_times.shape[0] != t_in:
            k = target_times.shape[0]
            extra = max(t_in + k, 2 * self.time_modes) - t_in
            x = pad_spatial_right(x, spatial_ndim=4, right_pad=(0, 0, 0, extra), mode="replicate")
            window = slice(t_in, t_in + k)
        y = self.fno(x.movedim(-1, 1)).movedim(1, -1)
        return y[:, :, :, :, window].squeeze(-1)

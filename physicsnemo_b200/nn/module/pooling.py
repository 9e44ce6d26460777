"""Point-cloud pooling heads (parity: ``physicsnemo/nn/module/pooling.py``)."""
from __future__ import annotations

import torch
import torch.nn as nn

from .activations import get_activation


def _maybe_spectral_norm(layer: nn.Module, enable: bool) -> nn.Module:
    return torch.nn.utils.parametrizations.spectral_norm(layer) if enable else layer


def _finish(out, normalize, scale):
    return nn.functional.normalize(out, dim=-1) * scale if normalize else out


class AttentionPooling(nn.Module):
    """Softmax-attention weighted mean over points, then an MLP projector (Linear → act → LayerNorm blocks)."""

    def __init__(self, feat_dim: int = 256, embed_dim: int = 32, hidden: int = 128,
                 projector_hidden: list[int] | None = None, activation: str = "relu", spectral_norm: bool = False,
                 normalize: bool = False, target_scale: float = 1.0) -> None:
        super().__init__()
        widths = [256, 128] if projector_hidden is None else projector_hidden
        sn = spectral_norm
        self.attention = nn.Sequential(_maybe_spectral_norm(nn.Linear(feat_dim, hidden), sn), nn.Tanh(),
                                       _maybe_spectral_norm(nn.Linear(hidden, 1), sn))
        layers, d = [], feat_dim
        for h in widths:
            layers += [_maybe_spectral_norm(nn.Linear(d, h), sn), get_activation(activation), nn.LayerNorm(h)]
            d = h
        layers.append(_maybe_spectral_norm(nn.Linear(d, embed_dim), sn))
        self.projector = nn.Sequential(*layers)
        self.normalize, self.target_scale = normalize, target_scale

    def forward(self, point_feats: torch.Tensor) -> torch.Tensor:
        w = torch.softmax(self.attention(point_feats), dim=1)
        return _finish(self.projector((w * point_feats).sum(dim=1)), self.normalize, self.target_scale)


class MeanPooling(nn.Module):
    def __init__(self, feat_dim: int = 256, embed_dim: int = 32, spectral_norm: bool = False, normalize: bool = False,
                 target_scale: float = 1.0) -> None:
        super().__init__()
        self.projector = _maybe_spectral_norm(nn.Linear(feat_dim, embed_dim), spectral_norm)
        self.normalize, self.target_scale = normalize, target_scale

    def forward(self, point_feats: torch.Tensor) -> torch.Tensor:
        return _finish(self.projector(point_feats.mean(dim=1)), self.normalize, self.target_scale)

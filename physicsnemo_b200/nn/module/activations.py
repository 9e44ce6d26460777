"""Activation modules and the name → module table.

Parity: ``physicsnemo/nn/module/activations.py`` (``Identity``, ``Stan``,
``SquarePlus``, ``CappedLeakyReLU``, ``CappedGELU``, ``Sin``, ``ACT2FN`` and
``get_activation`` at ``:188-243``).
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor


class Identity(nn.Module):
    """Returns its input (placeholder that removes an activation)."""

    def forward(self, x: Tensor) -> Tensor:
        return x


class Sin(nn.Module):
    """Sine activation."""

    def forward(self, x: Tensor) -> Tensor:
        return x.sin()


class Stan(nn.Module):
    """Self-scalable tanh: ``tanh(x) * (1 + beta * x)`` with one learnable ``beta`` per feature."""

    def __init__(self, out_features: int = 1):
        super().__init__()
        self.beta = nn.Parameter(torch.ones(out_features))

    def forward(self, x: Tensor) -> Tensor:
        width = self.beta.numel()
        if x.size(-1) != width:
            raise ValueError(f"Stan holds {width} slopes, so the input's last dimension must be {width}; got {tuple(x.shape)}")
        squashed = torch.tanh(x)
        return torch.addcmul(squashed, squashed, self.beta * x)


class SquarePlus(nn.Module):
    """``0.5 * (x + sqrt(x^2 + b))`` with ``b = 4``: a smooth ReLU without exponentials."""

    def __init__(self):
        super().__init__()
        self.b = 4

    def forward(self, x: Tensor) -> Tensor:
        return (x + (x.square() + self.b).sqrt()) / 2


class _Capped(nn.Module):
    """``min(inner(x), cap)``; the inner activation is registered under ``slot`` (a state-dict key of checkpoints)."""

    slot: str = ""
    inner_type: type = nn.Identity

    def __init__(self, cap_value=1.0, **kwargs):
        super().__init__()
        setattr(self, self.slot, self.inner_type(**kwargs))
        self.register_buffer("cap", torch.tensor(cap_value, dtype=torch.float32))

    def forward(self, inputs):
        return torch.minimum(getattr(self, self.slot)(inputs), self.cap.to(inputs.dtype))


class CappedLeakyReLU(_Capped):
    """Leaky ReLU clamped from above at ``cap_value``."""

    slot, inner_type = "leaky_relu", nn.LeakyReLU


class CappedGELU(_Capped):
    """GELU clamped from above at ``cap_value``."""

    slot, inner_type = "gelu", nn.GELU


# name -> class, or (class, constructor arguments) where the reference fixes arguments
_TORCH_BY_NAME = {name.lower(): getattr(nn, name) for name in (
    "ELU", "GELU", "Hardtanh", "LogSigmoid", "PReLU", "ReLU", "ReLU6", "SELU", "SiLU", "Sigmoid", "Softplus", "Softshrink",
    "Softsign", "Tanh", "Tanhshrink")}
_WITH_ARGUMENTS = {
    "celu": (nn.CELU, {"alpha": 1.0}),
    "leaky_relu": (nn.LeakyReLU, {"negative_slope": 0.1}),
    "threshold": (nn.Threshold, {"threshold": 1.0, "value": 1.0}),
}
_OWN = {"identity": Identity, "sin": Sin, "stan": Stan, "squareplus": SquarePlus, "capped_gelu": CappedGELU,
        "capped_leaky_relu": CappedLeakyReLU, "cappek_leaky_relu": CappedLeakyReLU}   # the misspelt key is a published alias
ACT2FN = {**_TORCH_BY_NAME, **_WITH_ARGUMENTS, **_OWN}


def get_activation(activation: str) -> nn.Module:
    """A new instance of the activation registered under ``activation`` (case-insensitive)."""
    entry = ACT2FN.get(activation.lower())
    if entry is None:
        raise KeyError(f"no activation is registered as {activation!r}; known names: {sorted(ACT2FN)}")
    cls, kwargs = entry if isinstance(entry, tuple) else (entry, {})
    return cls(**kwargs)


_EPILOGUE_CODES = ((nn.SiLU, 2), (nn.ReLU, 3))


def activation_code(act) -> int | None:
    """Epilogue code of the fused GEMM kernel for ``act`` or ``None`` if unfusable.

    0 = identity, 1 = GELU (erf), 2 = SiLU, 3 = ReLU.
    """
    if act is None or isinstance(act, (Identity, nn.Identity)):
        return 0
    if isinstance(act, nn.GELU):
        return 1 if getattr(act, "approximate", "none") == "none" else None
    for kind, code in _EPILOGUE_CODES:
        if isinstance(act, kind):
            return code
    return None

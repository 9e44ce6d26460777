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


class Stan(nn.Module):
    """Self-scalable tanh: ``tanh(x) * (1 + beta * x)`` with learnable ``beta``."""

    def __init__(self, out_features: int = 1):
        super().__init__()
        self.beta = nn.Parameter(torch.ones(out_features))

    def forward(self, x: Tensor) -> Tensor:
        if x.shape[-1] != self.beta.shape[-1]:
            raise ValueError(
                f"The last dimension of the input must be equal to the dimension of Stan parameters. Got inputs: {x.shape}, params: {self.beta.shape}"
            )
        return torch.tanh(x) * (1.0 + self.beta * x)


class SquarePlus(nn.Module):
    """``0.5 * (x + sqrt(x^2 + b))`` with ``b = 4``."""

    def __init__(self):
        super().__init__()
        self.b = 4

    def forward(self, x: Tensor) -> Tensor:
        return 0.5 * (x + torch.sqrt(x * x + self.b))


class CappedLeakyReLU(nn.Module):
    """Leaky ReLU clamped from above at ``cap_value``."""

    def __init__(self, cap_value=1.0, **kwargs):
        super().__init__()
        self.add_module("leaky_relu", nn.LeakyReLU(**kwargs))
        self.register_buffer("cap", torch.tensor(cap_value, dtype=torch.float32))

    def forward(self, inputs):
        return torch.clamp(self.leaky_relu(inputs), max=self.cap)


class CappedGELU(nn.Module):
    """GELU clamped from above at ``cap_value``."""

    def __init__(self, cap_value=1.0, **kwargs):
        super().__init__()
        self.add_module("gelu", nn.GELU(**kwargs))
        self.register_buffer("cap", torch.tensor(cap_value, dtype=torch.float32))

    def forward(self, inputs):
        return torch.clamp(self.gelu(inputs), max=self.cap)


class Sin(nn.Module):
    """Sine activation."""

    def forward(self, x: Tensor) -> Tensor:
        return torch.sin(x)


ACT2FN = {
    "relu": nn.ReLU,
    "leaky_relu": (nn.LeakyReLU, {"negative_slope": 0.1}),
    "prelu": nn.PReLU,
    "relu6": nn.ReLU6,
    "elu": nn.ELU,
    "celu": (nn.CELU, {"alpha": 1.0}),
    "selu": nn.SELU,
    "silu": nn.SiLU,
    "gelu": nn.GELU,
    "sin": Sin,
    "sigmoid": nn.Sigmoid,
    "logsigmoid": nn.LogSigmoid,
    "softplus": nn.Softplus,
    "softshrink": nn.Softshrink,
    "softsign": nn.Softsign,
    "tanh": nn.Tanh,
    "tanhshrink": nn.Tanhshrink,
    "threshold": (nn.Threshold, {"threshold": 1.0, "value": 1.0}),
    "hardtanh": nn.Hardtanh,
    "identity": Identity,
    "stan": Stan,
    "squareplus": SquarePlus,
    "cappek_leaky_relu": CappedLeakyReLU,
    "capped_leaky_relu": CappedLeakyReLU,
    "capped_gelu": CappedGELU,
}


def get_activation(activation: str) -> nn.Module:
    """Instantiate the activation registered under ``activation``."""
    try:
        entry = ACT2FN[activation.lower()]
    except KeyError:
        raise KeyError(
            f"Activation function {activation} not found. Available options are: {list(ACT2FN.keys())}"
        )
    if isinstance(entry, tuple):
        return entry[0](**entry[1])
    return entry()


def activation_code(act) -> int | None:
    """Epilogue code of the fused GEMM kernel for ``act`` or ``None`` if unfusable.

    0 = identity, 1 = GELU (erf), 2 = SiLU, 3 = ReLU.
    """
    if act is None or isinstance(act, (Identity, nn.Identity)):
        return 0
    if isinstance(act, nn.GELU) and getattr(act, "approximate", "none") == "none":
        return 1
    if isinstance(act, nn.SiLU):
        return 2
    if isinstance(act, nn.ReLU):
        return 3
    return None

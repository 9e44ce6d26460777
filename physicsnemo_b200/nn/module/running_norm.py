"""Scale normalisation by a running geometric-mean magnitude (parity: ``physicsnemo/nn/module/running_norm.py``)."""
from typing import Literal, Sequence

import torch
import torch.nn as nn

from ...core.module import Module


class RunningNorm(Module):
    r"""``y = x · exp(−m)`` where ``m`` tracks ``log mean|x|`` (zeros ignored) with momentum; ``shape`` gives the
    statistic's shape, size-1 axes are averaged over.  Optional affine weight / bias."""

    def __init__(self, shape: torch.Size | Sequence[int] = tuple(), momentum: float = 0.99, affine: bool = False,
                 bias: bool = True, initialization_behavior: Literal["no_op", "first_batch"] = "no_op",
                 disable: bool = False):
        if not (0.0 <= momentum < 1.0):
            raise ValueError(f"{momentum= } must satisfy 0 <= momentum < 1")
        super().__init__()
        self.shape, self.momentum, self.affine = shape, momentum, affine
        self.initialization_behavior, self.disable = initialization_behavior, disable
        if not disable and affine:
            self.weight = nn.Parameter(torch.ones(shape))
            if bias:
                self.bias = nn.Parameter(torch.zeros(shape))
            else:
                self.register_parameter("bias", None)
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)
        self.register_buffer("ln_running_mean", torch.zeros(shape))
        self.register_buffer("_initialized", torch.tensor(False, dtype=torch.bool))

    def __repr__(self) -> str:
        return f"RunningNorm(shape={tuple(self.shape)}, affine={self.affine})"

    def forward(self, x):
        if self.disable:
            return x
        if not torch.compiler.is_compiling() and len(self.shape) != x.ndim:
            raise ValueError(f"Expected input with {len(self.shape)} dimensions matching {self.shape=!r}, "
                             f"got tensor with shape {tuple(x.shape)}")
        if self.training:
            if self.initialization_behavior not in ("first_batch", "no_op"):
                raise ValueError(f"Invalid {self.initialization_behavior=!r}")
            mag = x.detach().abs()
            mag = torch.where(mag == 0.0, torch.nan, mag)
            for d, (want, have) in enumerate(zip(self.shape, x.shape)):
                if want != have:
                    if want != 1:
                        raise ValueError(f"Shape mismatch for dim={d!r}: desired_size={want!r} != actual_size={have!r}")
                    mag = torch.nanmean(mag, dim=d, keepdim=True)
            ln_batch = torch.nan_to_num(mag, nan=0.0).log()
            first = ln_batch if self.initialization_behavior == "first_batch" else self.ln_running_mean
            blended = self.momentum * self.ln_running_mean + (1.0 - self.momentum) * ln_batch
            self.ln_running_mean.copy_(torch.where(self._initialized, blended, first))
            self._initialized.fill_(True)
        x = x * torch.exp(-self.ln_running_mean)
        if self.weight is not None:
            x = x * self.weight
        if self.bias is not None:
            x = x + self.bias
        return x

"""Weight-normalised linear layer (parity: ``physicsnemo/nn/module/weight_norm.py``)."""
import torch
import torch.nn as nn
import torch.nn.functional as F


class WeightNormLinear(nn.Module):
    """``y = x (g * v / ||v||_row)^T + b`` with parameters ``weight`` (v), ``weight_g``, ``bias``."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.weight_g = nn.Parameter(torch.empty(out_features, 1))
        self.bias = nn.Parameter(torch.empty(out_features)) if bias else None
        self.reset_parameters()

    def reset_parameters(self):
        nn.init.xavier_uniform_(self.weight)
        nn.init.constant_(self.weight_g, 1.0)
        if self.bias is not None:
            nn.init.constant_(self.bias, 0.0)

    def forward(self, x):
        norm = self.weight.norm(dim=1, p=2, keepdim=True)
        return F.linear(x, self.weight_g * self.weight / norm, self.bias)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"

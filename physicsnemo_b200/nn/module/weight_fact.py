"""Weight-factorised linear layer (parity: ``physicsnemo/nn/module/weight_fact.py``).

``W = diag(g) V`` with ``g = exp(N(mean, stddev))`` drawn at initialisation and ``V = W0 / g``.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F


class WeightFactLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, mean: float = 1.0, stddev: float = 0.1):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.mean, self.stddev = mean, stddev
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.weight_g = nn.Parameter(torch.empty(out_features, 1))
        self.bias = nn.Parameter(torch.empty(out_features)) if bias else None
        self.reset_parameters()

    def reset_parameters(self):
        w = torch.empty(self.out_features, self.in_features)
        nn.init.xavier_uniform_(w)
        g = torch.exp(torch.randn(self.out_features, 1) * self.stddev + self.mean)
        with torch.no_grad():
            self.weight.copy_(w / g)
            self.weight_g.copy_(g)
            if self.bias is not None:
                self.bias.zero_()

    def forward(self, x):
        return F.linear(x, self.weight_g * self.weight, self.bias)

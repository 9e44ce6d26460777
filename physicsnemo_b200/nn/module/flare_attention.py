"""FLARE: low-rank attention through learned global queries (parity: ``physicsnemo/nn/module/flare_attention.py``).

``z = softmax(G Kᵀ) V`` gathers the N tokens into M global slots, ``y = softmax(K Gᵀ) z`` scatters them
back: cost O(N·M) instead of O(N²).  Keys / values are per-head linear maps of the projected input.
``use_te`` is accepted for signature parity; the SDPA path is always used.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


def _flare_self_attention(x_mid, q_global, self_k, self_v, scale: float):
    G = q_global.to(dtype=x_mid.dtype).expand(x_mid.shape[0], -1, -1, -1)
    k, v = self_k(x_mid), self_v(x_mid)
    z = F.scaled_dot_product_attention(G, k, v, scale=scale)
    return F.scaled_dot_product_attention(k, G, z, scale=scale)


class FLARE(nn.Module):
    def __init__(self, dim, heads: int = 8, dim_head: int = 64, dropout: float = 0.0, n_global_queries: int = 64,
                 use_te: bool = False):
        super().__init__()
        self.use_te = False
        self.heads, self.dim_head, self.scale = heads, dim_head, 1.0
        inner = dim_head * heads
        self.q_global = nn.Parameter(torch.randn(1, heads, n_global_queries, dim_head))
        self.in_project_x = nn.Linear(dim, inner)
        self.self_k = nn.Linear(dim_head, dim_head)
        self.self_v = nn.Linear(dim_head, dim_head)
        self.out_linear = nn.Linear(inner, dim)
        self.out_dropout = nn.Dropout(dropout)

    def forward(self, x):
        B, N, _ = x.shape
        x_mid = self.in_project_x(x).reshape(B, N, self.heads, self.dim_head).permute(0, 2, 1, 3)
        y = _flare_self_attention(x_mid, self.q_global, self.self_k, self.self_v, self.scale)
        return self.out_dropout(self.out_linear(y.permute(0, 2, 1, 3).reshape(B, N, -1)))

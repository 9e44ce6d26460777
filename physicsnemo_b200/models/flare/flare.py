"""FLARE model: the Transolver trunk with FLARE (global-query low-rank) attention blocks.

Parity: ``physicsnemo/models/flare/flare.py`` — same constructor as ``Transolver`` (``slice_num`` becomes the
number of global queries); pre-norm blocks ``x + FLARE(LN x)``, ``x + MLP(LN x)`` and an output head on the last.
The MLP branch runs through the fused LayerNorm / GEMM-chain kernels on CUDA bf16 inputs.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ... import ops
from ...nn.module.flare_attention import FLARE as FLAREAttention
from ...nn.module.layer_norm import LayerNorm
from ..transolver import Transolver as CoreTransolver
from ..transolver.transolver import _TransolverMlp


class _FLAREBlock(nn.Module):
    def __init__(self, num_heads: int, hidden_dim: int, dropout: float, act: str = "gelu", mlp_ratio: int = 4,
                 last_layer: bool = False, out_dim: int = 1, n_global_queries: int = 32, use_te: bool = False) -> None:
        super().__init__()
        self.last_layer = last_layer
        self.ln_1 = LayerNorm(hidden_dim)
        self.Attn = FLAREAttention(dim=hidden_dim, heads=num_heads, dim_head=hidden_dim // num_heads, dropout=dropout,
                                   n_global_queries=n_global_queries, use_te=False)
        self.ln_mlp1 = nn.Sequential(LayerNorm(hidden_dim),
                                     _TransolverMlp(in_features=hidden_dim, hidden_features=hidden_dim * mlp_ratio,
                                                    out_features=hidden_dim, act_layer=act, use_te=False))
        if last_layer:
            self.ln_mlp2 = nn.Sequential(LayerNorm(hidden_dim), nn.Linear(hidden_dim, out_dim))

    def forward(self, fx):
        fx = self.Attn(self.ln_1(fx)) + fx
        ln = self.ln_mlp1[0]
        xn, skip = ops.layer_norm(fx, ln.weight, ln.bias, ln.eps, return_residual=True)
        fx = self.ln_mlp1[1](xn, residual=skip)
        return self.ln_mlp2(fx) if self.last_layer else fx


class FLARE(CoreTransolver):
    def __init__(self, functional_dim: int, out_dim: int, embedding_dim: int | None = None, n_layers: int = 4,
                 n_hidden: int = 256, dropout: float = 0.0, n_head: int = 8, act: str = "gelu", mlp_ratio: int = 4,
                 slice_num: int = 32, unified_pos: bool = False, ref: int = 8, structured_shape=None,
                 time_input: bool = False, use_te: bool = False) -> None:
        super().__init__(functional_dim=functional_dim, out_dim=out_dim, embedding_dim=embedding_dim, n_layers=n_layers,
                         n_hidden=n_hidden, dropout=dropout, n_head=n_head, act=act, mlp_ratio=mlp_ratio,
                         slice_num=slice_num, unified_pos=unified_pos, ref=ref, structured_shape=structured_shape,
                         use_te=use_te, time_input=time_input, plus=False)
        self.blocks = nn.ModuleList([
            _FLAREBlock(num_heads=n_head, hidden_dim=n_hidden, dropout=dropout, act=act, mlp_ratio=mlp_ratio,
                        last_layer=(i == n_layers - 1), out_dim=out_dim, n_global_queries=slice_num, use_te=False)
            for i in range(n_layers)])
        self.initialize_weights()

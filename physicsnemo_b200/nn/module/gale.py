"""GALE: geometry-aware slice attention — physics attention whose slice tokens also attend to a context.

Parity: ``physicsnemo/nn/module/gale.py`` (``GALE``, ``GALEStructuredMesh2D/3D``, ``GALE_FA``,
``GALEBlock``; cross-attention parameters ``cross_q / cross_k / cross_v``; mixing of self- and
cross-attended slice tokens by a learned sigmoid weight (``state_mixing``) or by
``concat_project``).  All variants take a tuple of token tensors that share the weights (e.g.
surface and volume points) and return one output per input.

Several inputs are processed as one batch where shapes allow it: slice tokens of all inputs are
stacked so that the slice self-attention, the cross-attention projections and the mixing each run
once per block instead of once per input.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .concrete_dropout import ConcreteDropout
from .flare_attention import _flare_self_attention
from .mlp_layers import Mlp
from .physics_attention import (PhysicsAttentionIrregularMesh, PhysicsAttentionStructuredMesh2D,
                                PhysicsAttentionStructuredMesh3D, _project_input)


def _mix_self_and_cross(self_attn, cross_attn, mode: str, state_mixing=None, concat_project=None):
    if mode == "weighted":
        w = torch.sigmoid(state_mixing)
        return w * self_attn + (1 - w) * cross_attn
    if mode == "concat_project":
        return concat_project(torch.cat([self_attn, cross_attn], dim=-1))
    raise ValueError(f"Invalid state_mixing_mode: {mode!r}")


def _replicated(t):
    if hasattr(t, "redistribute"):
        from ...parallel import Replicate

        return t.redistribute(placements=[Replicate()])
    return t


def _gale_cross_init(self: nn.Module, dim_head: int, context_dim: int, use_te: bool, state_mixing_mode: str = "weighted") -> None:
    self.cross_q = nn.Linear(dim_head, dim_head)
    self.cross_k = nn.Linear(context_dim, dim_head)
    self.cross_v = nn.Linear(context_dim, dim_head)
    self.state_mixing_mode = state_mixing_mode
    if state_mixing_mode == "weighted":
        self.state_mixing = nn.Parameter(torch.tensor(0.0))
    elif state_mixing_mode == "concat_project":
        self.concat_project = nn.Sequential(nn.Linear(2 * dim_head, dim_head), nn.GELU())
    else:
        raise ValueError(f"Invalid state_mixing_mode: {state_mixing_mode!r}. Expected 'weighted' or 'concat_project'.")


def _gale_compute_slice_attention_cross(module, slice_tokens, context):
    """Slice tokens (queries, concatenated along the slice axis) attend to the context tokens."""
    q = module.cross_q(_replicated(torch.cat(slice_tokens, dim=-2)))
    context = _replicated(context)
    out = F.scaled_dot_product_attention(q, module.cross_k(context), module.cross_v(context), is_causal=False)
    return list(torch.split(out, slice_tokens[0].shape[-2], dim=-2))


def _gale_forward_impl(module, x, context):
    if not torch.compiler.is_compiling():
        if len(x) == 0:
            raise ValueError("Expected non-empty tuple of input tensors")
        for i, t in enumerate(x):
            if t.ndim != 3:
                raise ValueError(f"Expected 3D input tensor (B, N, C) at index {i}, got {t.ndim}D tensor with shape {tuple(t.shape)}")
    if module.plus:
        x_mid = [module.project_input_onto_slices(t) for t in x]
        fx_mid = x_mid
    else:
        x_mid, fx_mid = zip(*[module.project_input_onto_slices(t) for t in x])
    weights, tokens = zip(*[module._compute_slices_from_projections(module.in_project_slice(xm), fm)
                            for xm, fm in zip(x_mid, fx_mid)])
    n = len(tokens)
    stacked = torch.cat(tokens, dim=0) if n > 1 else tokens[0]                 # [n B, H, S, D]: one pass for all inputs
    out = module._compute_slice_attention_sdpa(stacked)
    if context is not None:
        ctx = context if n == 1 else torch.cat([context] * n, dim=0)
        cross = module.compute_slice_attention_cross([stacked], ctx)[0]
        out = _mix_self_and_cross(out, cross, module.state_mixing_mode, getattr(module, "state_mixing", None),
                                  getattr(module, "concat_project", None))
    outs = out.chunk(n, dim=0) if n > 1 else (out,)
    return [module._project_attention_outputs(o, w) for o, w in zip(outs, weights)]


class GALE(PhysicsAttentionIrregularMesh):
    def __init__(self, dim: int, heads: int = 8, dim_head: int = 64, dropout: float = 0.0, slice_num: int = 64,
                 use_te: bool = False, plus: bool = False, context_dim: int = 0, concrete_dropout: bool = False,
                 state_mixing_mode: str = "weighted") -> None:
        super().__init__(dim, heads, dim_head, dropout, slice_num, use_te, plus)
        _gale_cross_init(self, dim_head, context_dim, use_te, state_mixing_mode)
        if concrete_dropout:
            self.out_dropout = ConcreteDropout(in_features=dim, init_p=max(dropout, 0.05))

    def compute_slice_attention_cross(self, slice_tokens, context):
        return _gale_compute_slice_attention_cross(self, slice_tokens, context)

    def forward(self, x, context=None):
        return _gale_forward_impl(self, x, context)


class _GALEStructuredForwardMixin:
    def compute_slice_attention_cross(self, slice_tokens, context):
        return _gale_compute_slice_attention_cross(self, slice_tokens, context)

    def forward(self, x, context=None):
        return _gale_forward_impl(self, x, context)


class GALEStructuredMesh2D(_GALEStructuredForwardMixin, PhysicsAttentionStructuredMesh2D):
    def __init__(self, dim: int, spatial_shape, heads: int = 8, dim_head: int = 64, dropout: float = 0.0, slice_num: int = 64,
                 kernel: int = 3, use_te: bool = False, plus: bool = False, context_dim: int = 0,
                 state_mixing_mode: str = "weighted") -> None:
        super().__init__(dim, spatial_shape, heads, dim_head, dropout, slice_num, kernel, use_te, plus)
        _gale_cross_init(self, dim_head, context_dim, use_te, state_mixing_mode)


class GALEStructuredMesh3D(_GALEStructuredForwardMixin, PhysicsAttentionStructuredMesh3D):
    def __init__(self, dim: int, spatial_shape, heads: int = 8, dim_head: int = 64, dropout: float = 0.0, slice_num: int = 64,
                 kernel: int = 3, use_te: bool = False, plus: bool = False, context_dim: int = 0,
                 state_mixing_mode: str = "weighted") -> None:
        super().__init__(dim, spatial_shape, heads, dim_head, dropout, slice_num, kernel, use_te, plus)
        _gale_cross_init(self, dim_head, context_dim, use_te, state_mixing_mode)


class GALE_FA(nn.Module):
    """FLARE-style variant: learned global queries summarise the tokens; points also attend to the context."""

    def __init__(self, dim, heads: int = 8, dim_head: int = 64, dropout: float = 0.0, n_global_queries: int = 64,
                 use_te: bool = False, context_dim: int = 0, concrete_dropout: bool = False,
                 state_mixing_mode: str = "weighted"):
        super().__init__()
        self.use_te = False
        self.heads, self.dim_head, self.scale = heads, dim_head, 1.0
        inner = dim_head * heads
        self.q_global = nn.Parameter(torch.randn(1, heads, n_global_queries, dim_head))
        self.in_project_x = nn.Linear(dim, inner)
        self.self_k = nn.Linear(dim_head, dim_head)
        self.self_v = nn.Linear(dim_head, dim_head)
        if context_dim > 0:
            _gale_cross_init(self, dim_head, context_dim, use_te, state_mixing_mode)
        self.out_linear = nn.Linear(inner, dim)
        self.out_dropout = (ConcreteDropout(in_features=dim, init_p=max(dropout, 0.05)) if concrete_dropout
                            else nn.Dropout(dropout))

    def forward(self, x, context=None):
        outs = []
        if context is not None:
            k, v = self.cross_k(context), self.cross_v(context)
        for t in x:
            xm = _project_input(t, self.in_project_x, self.heads, self.dim_head, False).permute(0, 2, 1, 3)   # [B, H, N, D]
            y = _flare_self_attention(xm, self.q_global, self.self_k, self.self_v, self.scale)
            if context is not None:
                cross = F.scaled_dot_product_attention(self.cross_q(xm), k, v, scale=self.scale)
                y = _mix_self_and_cross(y, cross, self.state_mixing_mode, getattr(self, "state_mixing", None),
                                        getattr(self, "concat_project", None))
            y = y.permute(0, 2, 1, 3)
            outs.append(self.out_dropout(self.out_linear(y.reshape(y.shape[0], y.shape[1], -1))))
        return outs


class GALEBlock(nn.Module):
    """Pre-norm transformer block around a GALE attention; inputs and outputs are lists of token tensors."""

    def __init__(self, num_heads: int, hidden_dim: int, dropout: float, act: str = "gelu", mlp_ratio: int = 4,
                 last_layer: bool = False, out_dim: int = 1, slice_num: int = 32, use_te: bool = False, plus: bool = False,
                 context_dim: int = 0, spatial_shape=None, attention_type: str = "GALE", concrete_dropout: bool = False,
                 state_mixing_mode: str = "weighted") -> None:
        super().__init__()
        self.last_layer = last_layer
        self.ln_1 = nn.LayerNorm(hidden_dim)
        dim_head = hidden_dim // num_heads
        common = dict(heads=num_heads, dim_head=dim_head, dropout=dropout, use_te=False, context_dim=context_dim,
                      state_mixing_mode=state_mixing_mode)
        if attention_type == "GALE":
            if spatial_shape is None:
                self.Attn = GALE(hidden_dim, slice_num=slice_num, plus=plus, concrete_dropout=concrete_dropout, **common)
            elif len(spatial_shape) == 2:
                self.Attn = GALEStructuredMesh2D(hidden_dim, spatial_shape=tuple(int(s) for s in spatial_shape),
                                                 slice_num=slice_num, plus=plus, **common)
            elif len(spatial_shape) == 3:
                self.Attn = GALEStructuredMesh3D(hidden_dim, spatial_shape=tuple(int(s) for s in spatial_shape),
                                                 slice_num=slice_num, plus=plus, **common)
            else:
                raise ValueError(f"spatial_shape must be None, length-2, or length-3; got {spatial_shape!r}")
        elif attention_type == "GALE_FA":
            self.Attn = GALE_FA(hidden_dim, n_global_queries=slice_num, concrete_dropout=concrete_dropout, **common)
        else:
            raise ValueError(f"Invalid attention type: {attention_type}. Expected 'GALE' or 'GALE_FA'.")
        self.ln_mlp1 = nn.Sequential(nn.LayerNorm(hidden_dim),
                                     Mlp(in_features=hidden_dim, hidden_features=hidden_dim * mlp_ratio,
                                         out_features=hidden_dim, act_layer=act, use_te=False))
        if concrete_dropout:
            self.attn_dropout = ConcreteDropout(in_features=hidden_dim, init_p=max(dropout, 0.05))
            self.ffn_dropout = ConcreteDropout(in_features=hidden_dim, init_p=max(dropout, 0.05))
        else:
            self.attn_dropout = self.ffn_dropout = None

    def forward(self, fx, global_context):
        if not torch.compiler.is_compiling():
            if len(fx) == 0:
                raise ValueError("Expected non-empty tuple of input tensors")
            for i, t in enumerate(fx):
                if t.ndim != 3:
                    raise ValueError(f"Expected 3D input tensor (B, N, C) at index {i}, got {t.ndim}D tensor with shape {tuple(t.shape)}")
        attn = self.Attn(tuple(self.ln_1(t) for t in fx), global_context)
        out = [a + t for a, t in zip(attn, fx)]
        if self.attn_dropout is not None:
            out = [self.attn_dropout(t) for t in out]
        out = [self.ln_mlp1(t) + t for t in out]
        if self.ffn_dropout is not None:
            out = [self.ffn_dropout(t) for t in out]
        return out

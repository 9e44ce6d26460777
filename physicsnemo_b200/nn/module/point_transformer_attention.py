"""Local vector attention over k-nearest neighbours of point clouds (Point-Transformer style), with adaLN conditioning.

Parity: ``physicsnemo/nn/module/point_transformer_attention.py`` (``AdaLNResidualMLP``, ``LocalPointTransformerBlock``,
``LocalTokenCrossAttentionBlock``; same attribute names, so state dicts carry over).  Every query gathers ``k``
(optionally dilated) neighbours found by the kNN functional, forms per-head logits from ``MLP(q − k + pos(rel))``,
softmaxes over the neighbours (masked to the same batch element when batch ids are given) and sums ``v + pos(rel)``.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ...core.module import Module
from ..functional.neighbors import knn
from .mlp_layers import Mlp


def _gather_rows(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    return x.index_select(0, idx.reshape(-1)).reshape(*idx.shape, x.shape[-1])


def _dilated_knn(*, query_coords, key_coords, k: int, dilation: int) -> torch.Tensor:
    """Every ``dilation``-th of the ``k · dilation`` nearest keys."""
    k_wide = min(int(k) * int(dilation), int(key_coords.shape[0]))
    idx = knn(key_coords.float(), query_coords.float(), k_wide)[0]
    if dilation > 1:
        idx = idx[:, ::int(dilation)]
    return idx[:, :max(1, k_wide // int(dilation))].long()


def _dilate_precomputed_idx(idx: torch.Tensor, *, k: int, dilation: int) -> torch.Tensor:
    if dilation > 1:
        idx = idx[:, ::int(dilation)]
    return idx[:, :min(int(k), int(idx.shape[1]))]


def _make_conditioning_mlp(cond_dim: int, out_dim: int) -> Mlp:
    mlp = Mlp(in_features=int(cond_dim), hidden_features=max(int(cond_dim), int(out_dim)), out_features=int(out_dim), act_layer=nn.SiLU, drop=0.0)
    nn.init.zeros_(mlp.layers[-1].weight)                      # conditioning starts as the identity modulation
    nn.init.zeros_(mlp.layers[-1].bias)
    return mlp


def _reshape_condition(cond: torch.Tensor) -> torch.Tensor:
    if cond.ndim == 1:
        return cond.unsqueeze(0)
    if cond.ndim != 2:
        raise ValueError(f"conditioning tensor must have shape [D], [1, D], or [N, D], got {tuple(cond.shape)}")
    return cond


def _masked_softmax(logits: torch.Tensor, neighbor_mask: torch.Tensor | None) -> torch.Tensor:
    if neighbor_mask is None:
        return torch.softmax(logits, dim=-1)
    mask = neighbor_mask.unsqueeze(1)
    attn = torch.softmax(logits.masked_fill(~mask, -1e9), dim=-1) * mask.to(logits.dtype)
    return attn / attn.sum(dim=-1, keepdim=True).clamp_min(1e-12)


class AdaLNResidualMLP(Module):
    """``x + gate · MLP(LN(x) · (1 + scale) + shift)`` with (shift, scale, gate) from the condition."""

    def __init__(self, dim: int, mlp_ratio: int, dropout: float, conditioning_dim: int | None = None, adaln_zero: bool = False, use_te: bool = False):
        super().__init__()
        self.dim = int(dim)
        self.norm = nn.LayerNorm(self.dim)
        self.conditioning = None if conditioning_dim is None else _make_conditioning_mlp(int(conditioning_dim), 3 * self.dim)
        self.adaln_zero = bool(adaln_zero)
        self.net = Mlp(in_features=self.dim, hidden_features=max(1, int(mlp_ratio)) * self.dim, out_features=self.dim, act_layer=nn.GELU,
                       drop=float(dropout), final_dropout=True)

    def forward(self, x, cond=None):
        if x.shape[-1] != self.dim:
            raise ValueError(f"Expected x with last dim {self.dim}, got tensor of shape {tuple(x.shape)}")
        h, gate = self.norm(x), None
        if self.conditioning is not None:
            if cond is None:
                raise ValueError("conditioning input must be provided for conditioned AdaLNResidualMLP.")
            shift, scale, gate = self.conditioning(_reshape_condition(cond)).chunk(3, dim=-1)
            h = h * (1.0 + scale) + shift
        out = self.net(h)
        if gate is not None:
            out = out * (gate if self.adaln_zero else 1.0 + gate)
        return x + out


class _LocalVectorAttentionBlock(Module):
    def __init__(self, *, dim, num_heads, neighbor_k, mlp_ratio, dropout, coord_dim, conditioning_dim, adaln_zero, num_cond_chunks, use_te=False):
        super().__init__()
        if int(dim) % int(num_heads):
            raise ValueError("dim must be divisible by num_heads.")
        self.dim, self.num_heads, self.head_dim = int(dim), int(num_heads), int(dim) // int(num_heads)
        self.neighbor_k, self.coord_dim, self.adaln_zero = int(neighbor_k), int(coord_dim), bool(adaln_zero)
        self.conditioning = None if conditioning_dim is None else _make_conditioning_mlp(int(conditioning_dim), int(num_cond_chunks) * self.dim)
        self.q_proj, self.k_proj, self.v_proj = nn.Linear(self.dim, self.dim), nn.Linear(self.dim, self.dim), nn.Linear(self.dim, self.dim)
        self.pos_proj = Mlp(in_features=self.coord_dim, hidden_features=self.dim, out_features=self.dim, act_layer=nn.GELU, drop=0.0)
        self.attn_proj = Mlp(in_features=self.dim, hidden_features=self.dim, out_features=self.num_heads, act_layer=nn.GELU, drop=0.0)
        self.out_proj = nn.Linear(self.dim, self.dim)
        self.dropout = nn.Dropout(float(dropout))
        self.ffn = AdaLNResidualMLP(dim=self.dim, mlp_ratio=int(mlp_ratio), dropout=float(dropout), conditioning_dim=conditioning_dim,
                                    adaln_zero=adaln_zero)

    def _attend(self, q_in, kv_in, query_coords, key_coords, idx, neighbor_mask):
        n, kk, H, D = q_in.shape[0], idx.shape[1], self.num_heads, self.head_dim
        q = self.q_proj(q_in).reshape(n, H, D)
        k = _gather_rows(self.k_proj(kv_in), idx).reshape(n, kk, H, D)
        v = _gather_rows(self.v_proj(kv_in), idx).reshape(n, kk, H, D)
        rel_bias = self.pos_proj(_gather_rows(key_coords, idx) - query_coords.unsqueeze(1)).reshape(n, kk, H, D)
        logits = self.attn_proj((q.unsqueeze(1) - k + rel_bias).reshape(n, kk, self.dim)).transpose(1, 2)     # [n, H, kk]
        attn = _masked_softmax(logits, neighbor_mask)
        out = (attn.unsqueeze(-1) * (v + rel_bias).permute(0, 2, 1, 3)).sum(dim=2).reshape(n, self.dim)
        return self.dropout(self.out_proj(out))

    def _gated(self, out, gate):
        return out if gate is None else out * (gate if self.adaln_zero else 1.0 + gate)


class LocalPointTransformerBlock(_LocalVectorAttentionBlock):
    """Self-attention of a point set over its own (dilated) k nearest neighbours, followed by the adaLN MLP."""

    def __init__(self, *, dim, num_heads, neighbor_k, dilation, mlp_ratio, dropout, coord_dim=3, conditioning_dim=None, adaln_zero=False, use_te=False):
        super().__init__(dim=dim, num_heads=num_heads, neighbor_k=neighbor_k, mlp_ratio=mlp_ratio, dropout=dropout, coord_dim=coord_dim,
                         conditioning_dim=conditioning_dim, adaln_zero=adaln_zero, num_cond_chunks=3)
        self.dilation = int(max(1, dilation))
        self.norm = nn.LayerNorm(self.dim)

    def forward(self, features, coords, cond=None, batch_ids=None, precomputed_idx=None):
        if features.ndim != 2 or features.shape[1] != self.dim:
            raise ValueError(f"Expected features of shape (N, {self.dim}), got tensor of shape {tuple(features.shape)}")
        if coords.ndim != 2 or coords.shape[1] != self.coord_dim:
            raise ValueError(f"Expected coords of shape (N, {self.coord_dim}), got tensor of shape {tuple(coords.shape)}")
        if coords.shape[0] != features.shape[0]:
            raise ValueError(f"features and coords must share the point count N, got {features.shape[0]} and {coords.shape[0]}")
        if features.shape[0] <= 1:
            return self.ffn(features, cond=cond)
        h, gate = self.norm(features), None
        if self.conditioning is not None:
            if cond is None:
                raise ValueError("conditioning input must be provided for conditioned LocalPointTransformerBlock.")
            shift, scale, gate = self.conditioning(_reshape_condition(cond)).chunk(3, dim=-1)
            h = h * (1.0 + scale) + shift
        k = min(self.neighbor_k, int(coords.shape[0]))
        idx = (_dilated_knn(query_coords=coords, key_coords=coords, k=k, dilation=self.dilation) if precomputed_idx is None
               else _dilate_precomputed_idx(precomputed_idx, k=k, dilation=self.dilation))
        mask = None if batch_ids is None else _gather_rows(batch_ids.unsqueeze(-1), idx).squeeze(-1) == batch_ids.unsqueeze(1)
        out = features + self._gated(self._attend(h, h, coords, coords, idx, mask), gate)
        return self.ffn(out, cond=cond)


class LocalTokenCrossAttentionBlock(_LocalVectorAttentionBlock):
    """Queries attend to their k nearest context tokens (e.g. points reading from latent tokens and back)."""

    def __init__(self, *, dim, num_heads, neighbor_k, mlp_ratio, dropout, coord_dim=3, conditioning_dim=None, adaln_zero=False, use_te=False):
        super().__init__(dim=dim, num_heads=num_heads, neighbor_k=neighbor_k, mlp_ratio=mlp_ratio, dropout=dropout, coord_dim=coord_dim,
                         conditioning_dim=conditioning_dim, adaln_zero=adaln_zero, num_cond_chunks=5)
        self.norm_q, self.norm_kv = nn.LayerNorm(self.dim), nn.LayerNorm(self.dim)

    def forward(self, query_features, query_coords, context_features, context_coords, cond=None, context_cond=None, query_batch_ids=None,
                context_batch_ids=None, precomputed_idx=None):
        for name, f, c in (("query", query_features, query_coords), ("context", context_features, context_coords)):
            if f.ndim != 2 or f.shape[1] != self.dim:
                raise ValueError(f"Expected {name}_features of shape (N, {self.dim}), got tensor of shape {tuple(f.shape)}")
            if c.ndim != 2 or c.shape[1] != self.coord_dim or c.shape[0] != f.shape[0]:
                raise ValueError(f"Expected {name}_coords of shape ({f.shape[0]}, {self.coord_dim}), got tensor of shape {tuple(c.shape)}")
        if query_features.shape[0] == 0 or context_features.shape[0] == 0:
            return query_features
        q_in, kv_in, gate = self.norm_q(query_features), self.norm_kv(context_features), None
        if self.conditioning is not None:
            if cond is None:
                raise ValueError("conditioning input must be provided for conditioned LocalTokenCrossAttentionBlock.")
            q_shift, q_scale, _, _, gate = self.conditioning(_reshape_condition(cond)).chunk(5, dim=-1)
            q_in = q_in * (1.0 + q_scale) + q_shift
            if context_cond is not None:
                kv_source = _reshape_condition(context_cond)
            else:
                kv_source = _reshape_condition(cond)
                if kv_source.shape[0] > 1:
                    kv_source = kv_source.mean(dim=0, keepdim=True)
            kv_shift, kv_scale = self.conditioning(kv_source).chunk(5, dim=-1)[2:4]
            kv_in = kv_in * (1.0 + kv_scale) + kv_shift
        k = min(self.neighbor_k, int(context_coords.shape[0]))
        idx = (_dilated_knn(query_coords=query_coords, key_coords=context_coords, k=k, dilation=1) if precomputed_idx is None
               else _dilate_precomputed_idx(precomputed_idx, k=k, dilation=1))
        mask = None
        if query_batch_ids is not None and context_batch_ids is not None:
            mask = _gather_rows(context_batch_ids.unsqueeze(-1), idx).squeeze(-1) == query_batch_ids.unsqueeze(1)
        out = query_features + self._gated(self._attend(q_in, kv_in, query_coords, context_coords, idx, mask), gate)
        return self.ffn(out, cond=cond)


__all__ = ["AdaLNResidualMLP", "LocalPointTransformerBlock", "LocalTokenCrossAttentionBlock"]

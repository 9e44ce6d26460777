"""JEPA predictor: field tokens at given target positions from geometry tokens and operating conditions.

Parity: ``physicsnemo/experimental/models/aerojepa/predictor.py`` (``PrototypeTokenJEPAHead`` ``:54``).
Queries start as a Fourier embedding of the target positions plus the projected condition, then
alternate local self-attention among the targets with local cross-attention into the context tokens.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from ....core.module import Module
from ....nn.functional.neighbors import knn
from ....nn.module.embedding_layers import FourierPositionalEmbedding
from ....nn.module.mlp_layers import Mlp
from ....nn.module.point_transformer_attention import LocalPointTransformerBlock, LocalTokenCrossAttentionBlock
from .tokens import FlatTokens, TokenSet, shared_offset_step


def _rows(name: str, t: torch.Tensor, batch: int) -> torch.Tensor:
    """Bring a per-item tensor ``(…)`` or ``(1 | B, …)`` to ``B`` leading rows."""
    if t.shape[0] == batch:
        return t
    if t.shape[0] == 1:
        return t.expand(batch, *t.shape[1:])
    raise ValueError(f"{name} batch ({t.shape[0]}) does not match context batch ({batch}).")


class PrototypeTokenJEPAHead(Module):
    """``forward(context_tokens, target_positions, cond)`` → predicted token features ``(T, C)`` or ``(B, T, C)``.

    ``target_positions`` is ``(T, 3)`` (shared by all items) or ``(B, T, 3)``; ``cond`` is ``(D,)``,
    ``(1, D)`` or ``(B, D)`` and required when ``cond_dim > 0``.
    """

    def __init__(self, *, token_dim: int, cond_dim: int, hidden_dim: Optional[int] = None, depth: int = 4, num_heads: int = 8,
                 neighbor_k: int = 24, query_pe_bands: int = 6, mlp_ratio: int = 4, dropout: float = 0.0, use_te: bool = False):
        super().__init__()
        self.token_dim, self.cond_dim = int(token_dim), int(cond_dim)
        self.hidden_dim = int(hidden_dim) if hidden_dim is not None else self.token_dim
        self.depth = max(1, int(depth))
        self.query_pos_enc = FourierPositionalEmbedding(in_dim=3, num_bands=int(query_pe_bands), include_input=True)
        self.query_in = nn.Linear(self.query_pos_enc.out_dim, self.hidden_dim)
        self.context_in = nn.Linear(self.token_dim, self.hidden_dim)
        self.cond_proj = None
        if self.cond_dim > 0:
            self.cond_proj = Mlp(in_features=self.cond_dim, hidden_features=self.hidden_dim, out_features=self.hidden_dim,
                                 act_layer=nn.SiLU, final_dropout=False)
        block = dict(dim=self.hidden_dim, num_heads=int(num_heads), neighbor_k=int(neighbor_k), mlp_ratio=int(mlp_ratio),
                     dropout=float(dropout), conditioning_dim=self.hidden_dim if self.cond_dim > 0 else None)
        self.self_blocks = nn.ModuleList(LocalPointTransformerBlock(dilation=1, **block) for _ in range(self.depth))
        self.cross_blocks = nn.ModuleList(LocalTokenCrossAttentionBlock(**block) for _ in range(self.depth))
        self.out_norm = nn.LayerNorm(self.hidden_dim)
        self.out_proj = nn.Linear(self.hidden_dim, self.token_dim)

    def _condition(self, cond: Optional[torch.Tensor], batch: int, like: torch.Tensor) -> torch.Tensor:
        if cond is not None:
            cond = cond.unsqueeze(0) if cond.ndim == 1 else cond
            if cond.ndim != 2:
                raise ValueError(f"cond must have shape [B, D] or [D], got {tuple(cond.shape)}")
            cond = _rows("cond", cond, batch)
        if self.cond_proj is None:
            return like.new_zeros(batch, self.hidden_dim)
        if cond is None:
            raise ValueError("cond must be provided when cond_dim > 0.")
        return self.cond_proj(cond)

    def forward(self, *, context_tokens: TokenSet, target_positions: torch.Tensor, cond: Optional[torch.Tensor] = None) -> torch.Tensor:
        single = not context_tokens.is_batched
        ctx_feat = context_tokens.features[None] if single else context_tokens.features
        ctx_pos = context_tokens.coords[None] if single else context_tokens.coords
        ctx_mask = None if single else context_tokens.mask
        B = ctx_feat.shape[0]
        if target_positions.ndim == 2:
            target_positions = target_positions[None]
        if target_positions.ndim != 3:
            raise ValueError(f"target_positions must have shape [T, 3] or [B, T, 3], got {tuple(target_positions.shape)}")
        tgt_pos = _rows("target_positions", target_positions, B)
        cond_embed = self._condition(cond, B, ctx_feat)

        step = shared_offset_step((tgt_pos, None), (ctx_pos, ctx_mask))
        tgt, ctx = FlatTokens.from_padded(tgt_pos, None, step), FlatTokens.from_padded(ctx_pos, ctx_mask, step)
        tgt_cond, ctx_cond = tgt.per_item(cond_embed), ctx.per_item(cond_embed)
        q = self.query_in(self.query_pos_enc(tgt.coords)) + tgt_cond
        kv = self.context_in(ctx.gather(ctx_feat))
        k_self = min(self.self_blocks[0].neighbor_k, tgt.search.shape[0])
        k_cross = min(self.cross_blocks[0].neighbor_k, ctx.search.shape[0])
        self_idx = knn(points=tgt.search.float(), queries=tgt.search.float(), k=k_self)[0].long()
        cross_idx = knn(points=ctx.search.float(), queries=tgt.search.float(), k=k_cross)[0].long()
        use_cond = self.cond_proj is not None
        for self_block, cross_block in zip(self.self_blocks, self.cross_blocks):
            q = self_block(q, tgt.search, cond=tgt_cond if use_cond else None, batch_ids=tgt.batch, precomputed_idx=self_idx)
            q = cross_block(q, tgt.search, kv, ctx.search, cond=tgt_cond if use_cond else None,
                            context_cond=ctx_cond if use_cond else None, query_batch_ids=tgt.batch,
                            context_batch_ids=ctx.batch, precomputed_idx=cross_idx)
        out = self.out_proj(self.out_norm(tgt.scatter(q)))
        return out[0] if single and out.shape[0] == 1 else out

"""Field decoder: continuous query points read from the latent tokens by local cross-attention.

Parity: ``physicsnemo/experimental/models/aerojepa/decoder.py`` (``SirenHead`` ``:56``,
``QueryTokenDecoder`` ``:120``).  A query is embedded from its Fourier-encoded position, optional
signed distance (with optional |sdf|, sign and 1/|sdf| extras) and the broadcast condition, attends to
its nearest tokens, and goes through an MLP trunk and output head.  Options: a sine-activated
refinement of the trunk output, separate velocity / pressure heads (pressure as MLP or SIREN), and a
wall gate ``σ(α · sdf)`` on the three velocity channels.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from ....core.module import Module
from ....nn.functional.neighbors import knn
from ....nn.module.embedding_layers import FourierPositionalEmbedding
from ....nn.module.mlp_layers import Mlp
from ....nn.module.point_transformer_attention import LocalTokenCrossAttentionBlock
from ....nn.module.siren_layers import SirenLayer, SirenLayerType
from ...nn.point_utils import counts_to_mask
from .tokens import FlatTokens, TokenSet, shared_offset_step


class SirenHead(nn.Module):
    """``num_layers`` sine layers followed by a linear SIREN output layer."""

    def __init__(self, *, in_dim: int, hidden_dim: int, out_dim: int, num_layers: int, omega_0: float = 30.0):
        super().__init__()
        n = max(1, int(num_layers))
        kinds = [SirenLayerType.FIRST] + [SirenLayerType.HIDDEN] * (n - 1)
        widths = [int(in_dim)] + [int(hidden_dim)] * n
        self.hidden = nn.Sequential(*(SirenLayer(widths[i], widths[i + 1], layer_type=kinds[i], omega_0=float(omega_0))
                                      for i in range(n)))
        self.out = SirenLayer(int(hidden_dim), int(out_dim), layer_type=SirenLayerType.LAST, omega_0=float(omega_0))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.out(self.hidden(x))


class QueryTokenDecoder(Module):
    """``forward`` decodes ``(Nq, 3)`` queries of one case, ``forward_batched`` a padded batch; both return ``(prediction, query embedding)``."""

    def __init__(self, *, token_dim: int, query_dim: int = 3, hidden_dim: int = 256, num_layers: int = 4, out_dim: int = 4,
                 use_sdf: bool = True, cond_dim: int = 0, pe_num_bands: int = 16, cross_attention_heads: int = 8,
                 cross_attention_layers: int = 2, cross_attention_k: int = 32, attention_mlp_ratio: int = 4, dropout: float = 0.0,
                 query_chunk_size: int = 4096, wall_velocity_gate_enabled: bool = False, wall_velocity_gate_alpha: float = 20.0,
                 pressure_split_head_enabled: bool = False, pressure_head_hidden_dim: Optional[int] = None,
                 pressure_head_style: str = "mlp", pressure_head_siren_layers: int = 2, pressure_head_siren_omega0: float = 30.0,
                 final_refinement_style: str = "none", final_refinement_siren_layers: int = 2,
                 final_refinement_siren_omega0: float = 30.0, extra_sdf_features_enabled: bool = False,
                 extra_sdf_inv_eps: float = 1e-3, use_te: bool = False):
        super().__init__()
        self.pressure_head_style, self.final_refinement_style = str(pressure_head_style).lower(), str(final_refinement_style).lower()
        if self.pressure_head_style not in ("mlp", "siren"):
            raise ValueError("pressure_head_style must be one of: 'mlp', 'siren'.")
        if self.final_refinement_style not in ("none", "siren"):
            raise ValueError("final_refinement_style must be one of: 'none', 'siren'.")
        token_dim, hidden_dim = int(token_dim), int(hidden_dim)
        self.use_sdf, self.cond_dim, self.query_chunk_size = bool(use_sdf), int(cond_dim), int(query_chunk_size)
        self.wall_velocity_gate_enabled, self.wall_velocity_gate_alpha = bool(wall_velocity_gate_enabled), float(wall_velocity_gate_alpha)
        self.pressure_split_head_enabled = bool(pressure_split_head_enabled)
        self.pressure_head_hidden_dim = int(pressure_head_hidden_dim) if pressure_head_hidden_dim is not None else hidden_dim
        self.extra_sdf_features_enabled, self.extra_sdf_inv_eps = bool(extra_sdf_features_enabled), float(extra_sdf_inv_eps)
        self.pe = FourierPositionalEmbedding(in_dim=int(query_dim), num_bands=int(pe_num_bands), include_input=True)
        width = self.pe.out_dim + int(self.use_sdf) + self.cond_dim + (3 if self.extra_sdf_features_enabled else 0)
        self.query_in = nn.Linear(width, token_dim)
        self.cross_blocks = nn.ModuleList(
            LocalTokenCrossAttentionBlock(dim=token_dim, num_heads=int(cross_attention_heads), neighbor_k=int(cross_attention_k),
                                          mlp_ratio=int(attention_mlp_ratio), dropout=float(dropout))
            for _ in range(int(cross_attention_layers)))
        layers = [nn.LayerNorm(token_dim), nn.Linear(token_dim, hidden_dim), nn.SiLU()]
        for _ in range(max(0, int(num_layers) - 1)):
            layers += [nn.Linear(hidden_dim, hidden_dim), nn.SiLU()]
        self.trunk = nn.Sequential(*layers)
        self.final_refinement = None
        if self.final_refinement_style == "siren":
            self.final_refinement = SirenHead(in_dim=hidden_dim, hidden_dim=hidden_dim, out_dim=hidden_dim,
                                              num_layers=int(final_refinement_siren_layers), omega_0=float(final_refinement_siren_omega0))
        self.out = self.vel_head = self.p_head = None
        if not self.pressure_split_head_enabled:
            self.out = nn.Linear(hidden_dim, int(out_dim))
        else:
            self.vel_head = nn.Linear(hidden_dim, 3)
            if self.pressure_head_style == "siren":
                self.p_head = SirenHead(in_dim=hidden_dim, hidden_dim=self.pressure_head_hidden_dim, out_dim=1,
                                        num_layers=int(pressure_head_siren_layers), omega_0=float(pressure_head_siren_omega0))
            else:
                self.p_head = Mlp(in_features=hidden_dim, hidden_features=self.pressure_head_hidden_dim, out_features=1,
                                  act_layer=nn.SiLU, final_dropout=False)

    # ----------------------------------------------------------------- pieces
    def _query_inputs(self, pos: torch.Tensor, sdf: Optional[torch.Tensor], cond: Optional[torch.Tensor]) -> torch.Tensor:
        parts = [self.pe(pos)]
        if self.use_sdf:
            if sdf is None:
                raise ValueError("query_sdf must be provided when use_sdf=True.")
            parts.append(sdf)
            if self.extra_sdf_features_enabled:
                mag = sdf.abs()
                parts += [mag, sdf.sign(), 1.0 / (mag + max(self.extra_sdf_inv_eps, 1e-12))]
        if self.cond_dim > 0:
            if cond is None:
                raise ValueError("cond must be provided when cond_dim > 0.")
            parts.append(cond)
        return torch.cat(parts, dim=-1)

    def _head(self, query_tokens: torch.Tensor, sdf: Optional[torch.Tensor]) -> torch.Tensor:
        h = self.trunk(query_tokens)
        if self.final_refinement is not None:
            h = h + self.final_refinement(h)
        pred = self.out(h) if self.out is not None else torch.cat([self.vel_head(h), self.p_head(h)], dim=-1)
        if self.wall_velocity_gate_enabled:
            if sdf is None:
                raise ValueError("query_sdf must be provided when wall_velocity_gate_enabled=True.")
            pred = torch.cat([pred[:, :3] * torch.sigmoid(self.wall_velocity_gate_alpha * sdf), pred[:, 3:]], dim=-1)
        return pred

    def _decode_flat(self, q_pos, q_search, q_batch, sdf, cond, tok_feat, tok_search, tok_batch):
        """Chunked decode of flat queries against flat tokens; batch ids are ``None`` for a single case."""
        preds, embeds = [], []
        k = min(self.cross_blocks[0].neighbor_k, tok_search.shape[0]) if len(self.cross_blocks) else 0
        for lo in range(0, q_pos.shape[0], self.query_chunk_size):
            hi = lo + self.query_chunk_size
            cut = lambda t: None if t is None else t[lo:hi]  # noqa: E731
            x = self.query_in(self._query_inputs(q_pos[lo:hi], cut(sdf), cut(cond)))
            idx = knn(points=tok_search.float(), queries=q_search[lo:hi].float(), k=k)[0].long() if k else None
            for block in self.cross_blocks:
                x = block(x, q_search[lo:hi], tok_feat, tok_search, query_batch_ids=cut(q_batch),
                          context_batch_ids=tok_batch, precomputed_idx=idx)
            preds.append(self._head(x, cut(sdf)))
            embeds.append(x)
        if not preds:
            x = self.query_in(self._query_inputs(q_pos, sdf, cond))
            return self._head(x, sdf), x
        return torch.cat(preds), torch.cat(embeds)

    # ---------------------------------------------------------------- forward
    def forward(self, *, query_pos: torch.Tensor, query_sdf: Optional[torch.Tensor], target_tokens: TokenSet,
                cond: Optional[torch.Tensor] = None):
        feats, coords = target_tokens.features, target_tokens.coords
        if target_tokens.mask is not None:
            feats, coords = feats[target_tokens.mask], coords[target_tokens.mask]
        if feats.shape[0] == 0:
            raise ValueError("target_tokens must contain at least one valid token.")
        return self._decode_flat(query_pos, query_pos, None, query_sdf, cond, feats, coords, None)

    def forward_batched(self, *, query_pos: torch.Tensor, query_sdf: Optional[torch.Tensor], query_counts: torch.Tensor,
                        target_tokens: TokenSet, cond: Optional[torch.Tensor] = None):
        if query_pos.ndim != 3:
            raise ValueError(f"forward_batched expects rank-3 query_pos, got {tuple(query_pos.shape)}")
        q_mask = counts_to_mask(query_counts, query_pos.shape[1])
        step = shared_offset_step((query_pos, q_mask), (target_tokens.coords, target_tokens.mask))
        q = FlatTokens.from_padded(query_pos, q_mask, step)
        t = FlatTokens.from_padded(target_tokens.coords, target_tokens.mask, step)
        pred, emb = self._decode_flat(q.coords, q.search, q.batch, None if query_sdf is None else q.gather(query_sdf),
                                      None if cond is None else q.per_item(cond), t.gather(target_tokens.features),
                                      t.search, t.batch)
        return q.scatter(pred), q.scatter(emb)

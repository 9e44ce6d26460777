"""Point-cloud transformer encoders of AeroJEPA: the shared trunk and its context / target wrappers.

Parity: ``physicsnemo/experimental/models/aerojepa/encoders/point.py`` (``build_geometry_features``
``:90``, ``PointClusterGraphPool`` ``:168``, ``PointTransformer`` ``:299``), ``encoders/context.py``
(``ContextTransformer`` ``:37``), ``encoders/target.py`` (``TargetTransformer`` ``:39``) and
``encoders/base.py``.  Submodule names (``tokenizer``, ``graph_pool``, ``feature_in``, ``pos_enc``,
``pos_proj``, ``gen_proj``, ``blocks``, ``out_norm``) match the reference so that state dicts map
one to one.  Both entry points (one cloud, padded batch) run the same flat-token code path.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
from torch import nn

from ....core.module import Module
from ....nn.functional.neighbors import knn
from ....nn.module.embedding_layers import FourierPositionalEmbedding
from ....nn.module.mlp_layers import Mlp
from ....nn.module.point_transformer_attention import LocalPointTransformerBlock
from ...nn.point_tokenizer import PointCloudTokenizer
from ...nn.point_utils import counts_to_mask, masked_mean
from .tokens import EncoderOutput, FlatTokens, TokenSet


def shared_neighbor_index(blocks, queries: torch.Tensor, keys: torch.Tensor) -> Optional[torch.Tensor]:
    """One k-NN table wide enough for every block (``neighbor_k · dilation``); blocks stride into it."""
    if len(blocks) == 0:
        return None
    width = max(min(int(b.neighbor_k) * int(getattr(b, "dilation", 1)), keys.shape[0]) for b in blocks)
    return knn(points=keys.float(), queries=queries.float(), k=max(1, width))[0].long()


def build_geometry_features(*, context_pos: torch.Tensor, context_feat: torch.Tensor, use_sdf: bool = False,
                            use_solid_normals: bool = False, use_solid_n_dot_uinf: bool = False) -> torch.Tensor:
    """Positions followed by the selected trailing channels of ``context_feat``.

    ``context_feat`` ends with ``[sdf (1)] [normals (3)] [n · u_inf (1)]`` for whichever of them the
    dataset provides, in that order.
    """
    widths = [(use_sdf, 1), (use_solid_normals, 3), (use_solid_n_dot_uinf, 1)]
    needed = sum(w for on, w in widths if on)
    if needed == 0:
        return context_pos
    if context_feat.shape[-1] < context_pos.shape[-1] + needed:
        raise ValueError("context_feat does not contain enough channels for configured geometry features.")
    tail = context_feat[..., context_feat.shape[-1] - needed:]
    return torch.cat([context_pos, tail], dim=-1)


class PointClusterGraphPool(nn.Module):
    """Learned pooling of a token's member points: gated messages over the (point → token) edges, then a residual update."""

    def __init__(self, *, point_feature_dim: int, coord_dim: int = 3, hidden_dim: int, num_layers: int, dropout: float,
                 use_te: bool = False):
        super().__init__()
        self.point_feature_dim, self.coord_dim = int(point_feature_dim), int(coord_dim)
        self.hidden_dim, self.num_layers = int(hidden_dim), max(1, int(num_layers))
        edge = 2 * self.point_feature_dim + self.coord_dim + 1

        def mlp(i, o, drop):
            return Mlp(in_features=i, hidden_features=self.hidden_dim, out_features=o, act_layer=nn.SiLU, drop=drop,
                       final_dropout=False)

        self.msg_mlps = nn.ModuleList(mlp(edge, self.point_feature_dim, float(dropout)) for _ in range(self.num_layers))
        self.gate_mlps = nn.ModuleList(mlp(edge, 1, 0.0) for _ in range(self.num_layers))
        self.update_mlps = nn.ModuleList(mlp(2 * self.point_feature_dim, self.point_feature_dim, float(dropout))
                                         for _ in range(self.num_layers))
        self.out_norm = nn.LayerNorm(self.point_feature_dim)

    def forward(self, *, point_positions, point_features, token_positions, token_features, cluster_idx):
        if token_positions.shape[0] == 0 or cluster_idx is None:
            return token_features
        rel = point_positions[cluster_idx] - token_positions[:, None, :]
        static = torch.cat([rel, torch.linalg.norm(rel, dim=-1, keepdim=True)], dim=-1)
        member = point_features[cluster_idx]
        h = token_features
        for msg, gate, update in zip(self.msg_mlps, self.gate_mlps, self.update_mlps):
            edge = torch.cat([member, h[:, None, :].expand(-1, cluster_idx.shape[1], -1), static], dim=-1)
            g = torch.sigmoid(gate(edge))
            pooled = (g * msg(edge)).sum(1) / g.sum(1).clamp_min(1e-6)
            h = h + update(torch.cat([h, pooled], dim=-1))
        return self.out_norm(h)


def _as_coord_tensor(coords) -> Optional[torch.Tensor]:
    if coords is None or isinstance(coords, torch.Tensor):
        return coords
    return torch.tensor(coords, dtype=torch.float32)


class PointTransformer(Module):
    """Tokenise a point cloud, embed the tokens, run dilated local-attention blocks, normalise.

    ``encode_single`` takes ``(N, 3)`` positions and ``(N, F)`` features; ``forward_batched`` takes
    padded ``(B, N, ·)`` tensors with per-item point counts.  The output tokens carry their mean as
    ``global_token``.  With ``use_gen_conditioning`` a projection of ``gen_params`` is added to the
    embedding and modulates every block.  ``tokenizer_cluster_pooling='graph'`` replaces the
    tokenizer's mean pooling by :class:`PointClusterGraphPool`.
    """

    supports_batched_forward = True

    def __init__(self, *, point_input_dim: int, token_dim: int, max_point_tokens: int, tokenizer_strategy: str,
                 tokenizer_deterministic_eval: bool, tokenizer_cluster_size: Optional[int], tokenizer_voxel_size,
                 tokenizer_prototype_coords, tokenizer_prototype_knn_k: Optional[int], tokenizer_knn_chunk_size: int,
                 point_pos_pe_bands: int, num_heads: int, num_layers: int, neighbor_k: int,
                 dilation_schedule: Optional[Sequence[int]], mlp_ratio: int, dropout: float, tokenizer_cluster_pooling: str,
                 tokenizer_graph_pool_hidden_dim: Optional[int], tokenizer_graph_pool_layers: int,
                 use_gen_conditioning: bool = False, gen_conditioning_dim: Optional[int] = None, use_te: bool = False):
        super().__init__()
        if isinstance(tokenizer_prototype_coords, torch.Tensor):        # keep the saved constructor arguments serialisable
            self._args["__args__"]["tokenizer_prototype_coords"] = tokenizer_prototype_coords.detach().cpu().tolist()
        self.tokenizer = PointCloudTokenizer(
            max_point_tokens=int(max_point_tokens), strategy=str(tokenizer_strategy).lower(),
            deterministic_eval=bool(tokenizer_deterministic_eval), cluster_size=tokenizer_cluster_size,
            knn_chunk_size=int(tokenizer_knn_chunk_size), voxel_size=tokenizer_voxel_size,
            prototype_coords=_as_coord_tensor(tokenizer_prototype_coords), prototype_knn_k=tokenizer_prototype_knn_k)
        self.tokenizer_cluster_pooling = str(tokenizer_cluster_pooling).lower()
        if self.tokenizer_cluster_pooling not in ("mean", "graph"):
            raise ValueError("tokenizer_cluster_pooling must be one of: 'mean', 'graph'.")
        self.graph_pool = None
        if self.tokenizer_cluster_pooling == "graph":
            if not self.tokenizer.uses_cluster_pooling:
                raise ValueError("tokenizer_cluster_pooling='graph' requires a cluster tokenizer strategy.")
            hidden = tokenizer_graph_pool_hidden_dim or max(4 * int(point_input_dim), int(token_dim) // 2, 32)
            self.graph_pool = PointClusterGraphPool(point_feature_dim=int(point_input_dim), coord_dim=3, hidden_dim=int(hidden),
                                                    num_layers=int(tokenizer_graph_pool_layers), dropout=float(dropout))
        self.feature_in = nn.Linear(int(point_input_dim), int(token_dim))
        self.pos_enc = FourierPositionalEmbedding(in_dim=3, num_bands=int(point_pos_pe_bands), include_input=True)
        self.pos_proj = nn.Linear(self.pos_enc.out_dim, int(token_dim))
        self.use_gen_conditioning = bool(use_gen_conditioning)
        self.gen_proj = None
        if self.use_gen_conditioning:
            if gen_conditioning_dim is None:
                raise ValueError("gen_conditioning_dim must be provided when use_gen_conditioning=True.")
            self.gen_proj = Mlp(in_features=int(gen_conditioning_dim), hidden_features=int(token_dim), out_features=int(token_dim),
                                act_layer=nn.SiLU, final_dropout=False)
        dilations = list(dilation_schedule) if dilation_schedule else [1]
        dilations += [dilations[-1]] * (int(num_layers) - len(dilations))
        self.blocks = nn.ModuleList(
            LocalPointTransformerBlock(dim=int(token_dim), num_heads=int(num_heads), neighbor_k=int(neighbor_k),
                                       dilation=int(dilations[i]), mlp_ratio=int(mlp_ratio), dropout=float(dropout),
                                       conditioning_dim=int(token_dim) if self.use_gen_conditioning else None)
            for i in range(int(num_layers)))
        self.out_norm = nn.LayerNorm(int(token_dim))

    # ---------------------------------------------------------------- tokens
    def _tokenize_single(self, *, point_positions: torch.Tensor, point_features: torch.Tensor):
        if self.graph_pool is None:
            return self.tokenizer(point_positions=point_positions, point_features=point_features)
        coords, feats, members = self.tokenizer.tokenize_with_clusters(point_positions=point_positions,
                                                                       point_features=point_features)
        if members is not None:
            feats = self.graph_pool(point_positions=point_positions, point_features=point_features,
                                    token_positions=coords, token_features=feats, cluster_idx=members)
        return coords, feats

    def _tokenize_batched(self, *, point_positions, point_features, point_counts):
        if self.graph_pool is None and not self.tokenizer.requires_per_sample_loop:
            return self.tokenizer.forward_batched(point_positions=point_positions, point_features=point_features,
                                                  point_counts=point_counts)
        per_item = [self._tokenize_single(point_positions=point_positions[b, :int(n)], point_features=point_features[b, :int(n)])
                    for b, n in enumerate(point_counts.tolist())]
        counts = torch.tensor([c.shape[0] for c, _ in per_item], device=point_positions.device, dtype=torch.long)
        T = int(counts.max()) if counts.numel() else 0
        coords = point_positions.new_zeros(len(per_item), T, point_positions.shape[-1])
        feats = point_features.new_zeros(len(per_item), T, point_features.shape[-1])
        for b, (c, f) in enumerate(per_item):
            coords[b, :c.shape[0]], feats[b, :f.shape[0]] = c, f
        return coords, feats, counts_to_mask(counts, T), counts

    # ------------------------------------------------------------- attention
    def _gen_embedding(self, gen_params: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        if self.gen_proj is None:
            return None
        if gen_params is None:
            raise ValueError("gen_params must be provided when use_gen_conditioning=True.")
        return self.gen_proj(gen_params)

    def _encode(self, coords: torch.Tensor, feats: torch.Tensor, mask: Optional[torch.Tensor], gen: Optional[torch.Tensor]):
        """``coords`` / ``feats`` padded ``(B, T, ·)``, ``gen`` ``(B, C)`` or ``None`` → padded output features and the token list."""
        flat = FlatTokens.from_padded(coords, mask)
        x = self.feature_in(flat.gather(feats)) + self.pos_proj(self.pos_enc(flat.coords))
        cond = None if gen is None else flat.per_item(gen)
        if cond is not None:
            x = x + cond
        table = shared_neighbor_index(self.blocks, flat.search, flat.search) if x.shape[0] else None
        many = flat.mask.shape[0] > 1
        for block in self.blocks:
            x = block(x, flat.search, cond=cond, batch_ids=flat.batch if many else None, precomputed_idx=table)
        return flat.scatter(self.out_norm(x)), flat

    def encode_single(self, *, point_positions: torch.Tensor, point_features: torch.Tensor,
                      gen_params: Optional[torch.Tensor]) -> EncoderOutput:
        coords, feats = self._tokenize_single(point_positions=point_positions, point_features=point_features)
        gen = self._gen_embedding(gen_params)
        out, _ = self._encode(coords[None], feats[None], None, None if gen is None else gen.reshape(1, -1))
        x = out[0]
        glob = masked_mean(x, None)
        return EncoderOutput(tokens=TokenSet(features=x, coords=coords, global_token=glob), global_token=glob,
                             aux={"point_token_count": int(x.shape[0])})

    def forward_batched(self, *, point_positions: torch.Tensor, point_features: torch.Tensor, point_counts: torch.Tensor,
                        gen_params: Optional[torch.Tensor]) -> EncoderOutput:
        coords, feats, mask, counts = self._tokenize_batched(point_positions=point_positions, point_features=point_features,
                                                             point_counts=point_counts)
        out, _ = self._encode(coords, feats, mask, self._gen_embedding(gen_params))
        glob = masked_mean(out, mask).squeeze(1)
        return EncoderOutput(tokens=TokenSet(features=out, coords=coords, mask=mask, global_token=glob), global_token=glob,
                             aux={"point_token_count": counts})


class BaseContextEncoder(Module):
    """Interface of a geometry (context) encoder: ``forward`` for one cloud, ``forward_batched`` for a padded batch."""

    supports_batched_forward = False

    def forward(self, *, context_pos: torch.Tensor, context_feat: torch.Tensor) -> EncoderOutput:
        raise NotImplementedError

    def forward_batched(self, *, context_pos, context_feat, context_pos_n) -> EncoderOutput:
        raise NotImplementedError(f"{type(self).__name__} has no batched path")


class BaseTargetEncoder(Module):
    """Interface of a flow-field (target) encoder over surface and volume samples."""

    supports_batched_forward = False

    def forward(self, *, surface_pos, surface_main_feat, volume_pos, volume_feat) -> EncoderOutput:
        raise NotImplementedError

    def forward_batched(self, *, surface_pos, surface_main_feat, surface_pos_n, volume_pos, volume_feat, volume_pos_n) -> EncoderOutput:
        raise NotImplementedError(f"{type(self).__name__} has no batched path")


def _point_transformer(kw: dict) -> PointTransformer:
    kw = dict(kw)
    kw["tokenizer_strategy"] = str(kw["tokenizer_strategy"]).lower()
    kw["tokenizer_cluster_pooling"] = str(kw["tokenizer_cluster_pooling"]).lower()
    return PointTransformer(use_gen_conditioning=False, gen_conditioning_dim=None, **kw)


class ContextTransformer(BaseContextEncoder):
    """Geometry encoder: positions plus the selected solid features through an unconditioned :class:`PointTransformer`."""

    supports_batched_forward = True

    def __init__(self, *, point_input_dim: int, token_dim: int, max_point_tokens: int, tokenizer_strategy: str = "voxel_fps_cluster",
                 tokenizer_deterministic_eval: bool = True, tokenizer_cluster_size: Optional[int] = None,
                 tokenizer_knn_chunk_size: int = 128, tokenizer_voxel_size=None, tokenizer_prototype_coords=None,
                 tokenizer_prototype_knn_k: Optional[int] = None, point_pos_pe_bands: int = 6, num_heads: int = 8,
                 num_layers: int = 6, neighbor_k: int = 24, dilation_schedule: Optional[Sequence[int]] = None, mlp_ratio: int = 4,
                 dropout: float = 0.0, tokenizer_cluster_pooling: str = "mean", tokenizer_graph_pool_hidden_dim: Optional[int] = None,
                 tokenizer_graph_pool_layers: int = 2, use_sdf: bool = False, use_solid_normals: bool = False,
                 use_solid_n_dot_uinf: bool = False, use_te: bool = False):
        super().__init__()
        if isinstance(tokenizer_prototype_coords, torch.Tensor):
            self._args["__args__"]["tokenizer_prototype_coords"] = tokenizer_prototype_coords.detach().cpu().tolist()
        self._feature_flags = dict(use_sdf=bool(use_sdf), use_solid_normals=bool(use_solid_normals),
                                   use_solid_n_dot_uinf=bool(use_solid_n_dot_uinf))
        self.use_sdf, self.use_solid_normals, self.use_solid_n_dot_uinf = self._feature_flags.values()
        args = {k: v for k, v in self._args["__args__"].items() if k not in self._feature_flags}
        args["tokenizer_prototype_coords"] = tokenizer_prototype_coords
        self.encoder = _point_transformer(args)

    def forward(self, *, context_pos: torch.Tensor, context_feat: torch.Tensor) -> EncoderOutput:
        feats = build_geometry_features(context_pos=context_pos, context_feat=context_feat, **self._feature_flags)
        return self.encoder.encode_single(point_positions=context_pos, point_features=feats, gen_params=None)

    def forward_batched(self, *, context_pos, context_feat, context_pos_n) -> EncoderOutput:
        feats = build_geometry_features(context_pos=context_pos, context_feat=context_feat, **self._feature_flags)
        return self.encoder.forward_batched(point_positions=context_pos, point_features=feats, point_counts=context_pos_n,
                                            gen_params=None)


class TargetTransformer(BaseTargetEncoder):
    """Flow-field encoder: surface and volume samples of one case form a single cloud for a :class:`PointTransformer`."""

    supports_batched_forward = True

    def __init__(self, *, point_input_dim: int, token_dim: int, max_point_tokens: int, tokenizer_strategy: str = "voxel_fps_cluster",
                 tokenizer_deterministic_eval: bool = True, tokenizer_cluster_size: Optional[int] = None,
                 tokenizer_knn_chunk_size: int = 128, tokenizer_voxel_size=None, tokenizer_prototype_coords=None,
                 tokenizer_prototype_knn_k: Optional[int] = None, point_pos_pe_bands: int = 6, num_heads: int = 8,
                 num_layers: int = 6, neighbor_k: int = 24, dilation_schedule: Optional[Sequence[int]] = None, mlp_ratio: int = 4,
                 dropout: float = 0.0, tokenizer_cluster_pooling: str = "mean", tokenizer_graph_pool_hidden_dim: Optional[int] = None,
                 tokenizer_graph_pool_layers: int = 2, use_te: bool = False):
        super().__init__()
        if isinstance(tokenizer_prototype_coords, torch.Tensor):
            self._args["__args__"]["tokenizer_prototype_coords"] = tokenizer_prototype_coords.detach().cpu().tolist()
        args = dict(self._args["__args__"])
        args["tokenizer_prototype_coords"] = tokenizer_prototype_coords
        self.encoder = _point_transformer(args)

    def forward(self, *, surface_pos, surface_main_feat, volume_pos, volume_feat) -> EncoderOutput:
        if surface_main_feat.shape[-1] != volume_feat.shape[-1]:
            raise ValueError("Target encoder requires matching feature dims for surface_main_feat and volume_feat.")
        return self.encoder.encode_single(point_positions=torch.cat([surface_pos, volume_pos], dim=0),
                                          point_features=torch.cat([surface_main_feat, volume_feat], dim=0), gen_params=None)

    def forward_batched(self, *, surface_pos, surface_main_feat, surface_pos_n, volume_pos, volume_feat, volume_pos_n) -> EncoderOutput:
        """Every item's valid surface rows followed by its valid volume rows, re-padded to the longest item."""
        counts = surface_pos_n + volume_pos_n
        B, width = surface_pos.shape[0], int(counts.max()) if counts.numel() else 0
        pos = surface_pos.new_zeros(B, width, surface_pos.shape[-1])
        feat = surface_main_feat.new_zeros(B, width, surface_main_feat.shape[-1])
        s_mask = counts_to_mask(surface_pos_n, surface_pos.shape[1])
        v_mask = counts_to_mask(volume_pos_n, volume_pos.shape[1])
        s_item, s_col = s_mask.nonzero(as_tuple=True)
        v_item, v_col = v_mask.nonzero(as_tuple=True)
        v_col = v_col + surface_pos_n[v_item]
        pos[s_item, s_col], feat[s_item, s_col] = surface_pos[s_mask], surface_main_feat[s_mask]
        pos[v_item, v_col], feat[v_item, v_col] = volume_pos[v_mask], volume_feat[v_mask]
        return self.encoder.forward_batched(point_positions=pos, point_features=feat, point_counts=counts, gen_params=None)

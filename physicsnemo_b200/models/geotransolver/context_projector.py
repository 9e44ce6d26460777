"""Context construction of GeoTransolver: geometry / global / multi-scale local features → context slice tokens.

Parity: ``physicsnemo/models/geotransolver/context_projector.py`` (``ContextProjector``,
``StructuredContextProjector``, ``GeometricFeatureProcessor``, ``MultiScaleFeatureExtractor``,
``GlobalContextBuilder``; parameter names ``in_project_x``, ``in_project_fx``, ``in_project_slice``,
``temperature``, ``proj_temperature``, ``processors``, ``tokenizers``, ``local_extractors``,
``geometry_tokenizer``, ``global_tokenizer``).  A projector maps tokens to per-head features, softly
assigns them to ``slice_num`` slices and returns the normalised slice sums ``[B, H, S, D]``; the
ball-query features use this package's radius-search kernels through ``BQWarp``.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ...nn.module.ball_query import BQWarp
from ...nn.module.concrete_dropout import ConcreteDropout
from ...nn.module.mlp_layers import Mlp
from ...nn.module.physics_attention import _compute_slices_from_projections, _project_input


def _structured_grid_to_conv_input(x, batch: int, tokens: int, channels: int, ndim: int, spatial_shape):
    n = 1
    for s in spatial_shape:
        n *= int(s)
    if tokens != n:
        raise ValueError(f"Expected N={n} tokens for {ndim}D grid, got N={tokens}")
    return x.reshape(batch, *spatial_shape, channels).movedim(-1, 1)


class _SliceToContextMixin:
    def _init_slice_components(self, dim_head: int, slice_num: int, heads: int, use_te: bool, plus: bool) -> None:
        self.in_project_slice = nn.Linear(dim_head, slice_num)
        self.temperature = nn.Parameter(torch.ones([1, 1, heads, 1]) * 0.5)
        if plus:
            self.proj_temperature = nn.Sequential(nn.Linear(dim_head, slice_num), nn.GELU(), nn.Linear(slice_num, 1), nn.GELU())

    def _compute_slices(self, slice_projections, fx):
        proj_temp = getattr(self, "proj_temperature", None) if self.plus else None
        return _compute_slices_from_projections(slice_projections, fx, self.temperature, self.plus, proj_temperature=proj_temp)

    def _tokens(self, projected):
        px, pf = (projected, projected) if self.plus else projected
        _, slice_tokens = self._compute_slices(self.in_project_slice(px), pf)
        return self.output_dropout(slice_tokens) if self.output_dropout is not None else slice_tokens


class ContextProjector(_SliceToContextMixin, nn.Module):
    def __init__(self, dim: int, heads: int = 8, dim_head: int = 64, dropout: float = 0.0, slice_num: int = 64,
                 use_te: bool = False, plus: bool = False, concrete_dropout: bool = False) -> None:
        super().__init__()
        inner = dim_head * heads
        self.dim_head, self.heads, self.plus, self.scale, self.use_te = dim_head, heads, plus, dim_head ** -0.5, False
        self.in_project_x = nn.Linear(dim, inner)
        if not plus:
            self.in_project_fx = nn.Linear(dim, inner)
        self.softmax = nn.Softmax(dim=-1)
        self._init_slice_components(dim_head, slice_num, heads, use_te, plus)
        self.output_dropout = ConcreteDropout(in_features=dim_head, init_p=max(dropout, 0.05)) if concrete_dropout else None

    def project_input_onto_slices(self, x):
        return _project_input(x, self.in_project_x, self.heads, self.dim_head, False,
                              project_fx=None if self.plus else self.in_project_fx)

    def forward(self, x):
        if not torch.compiler.is_compiling() and x.ndim != 3:
            raise ValueError(f"Expected 3D input tensor (B, N, C), got {x.ndim}D tensor with shape {tuple(x.shape)}")
        return self._tokens(self.project_input_onto_slices(x))


class StructuredContextProjector(_SliceToContextMixin, nn.Module):
    def __init__(self, dim: int, spatial_shape, heads: int = 8, dim_head: int = 64, dropout: float = 0.0, slice_num: int = 64,
                 kernel: int = 3, use_te: bool = False, plus: bool = False, concrete_dropout: bool = False) -> None:
        super().__init__()
        if len(spatial_shape) not in (2, 3):
            raise ValueError(f"StructuredContextProjector expects spatial_shape of length 2 or 3, got {spatial_shape!r}")
        inner = dim_head * heads
        self.dim_head, self.heads, self.plus, self.use_te = dim_head, heads, plus, False
        self.spatial_shape = tuple(int(s) for s in spatial_shape)
        self._nd = len(self.spatial_shape)
        conv = nn.Conv2d if self._nd == 2 else nn.Conv3d
        self.in_project_x = conv(dim, inner, kernel, 1, kernel // 2)
        if not plus:
            self.in_project_fx = conv(dim, inner, kernel, 1, kernel // 2)
        self.softmax = nn.Softmax(dim=-1)
        self.dropout = nn.Dropout(dropout)
        self._init_slice_components(dim_head, slice_num, heads, use_te, plus)
        self.output_dropout = ConcreteDropout(in_features=dim_head, init_p=max(dropout, 0.05)) if concrete_dropout else None

    def _grid_project(self, x):
        B, N, C = x.shape
        grid = _structured_grid_to_conv_input(x, B, N, C, self._nd, self.spatial_shape)
        return _project_input(grid, self.in_project_x, self.heads, self.dim_head, True,
                              project_fx=None if self.plus else self.in_project_fx)

    def forward(self, x):
        if not torch.compiler.is_compiling() and x.ndim != 3:
            raise ValueError(f"Expected 3D input (B, N, C), got {x.ndim}D shape {tuple(x.shape)}")
        return self._tokens(self._grid_project(x))


class GeometricFeatureProcessor(nn.Module):
    """Features of the ``neighbors_in_radius`` nearest keys within ``radius`` of every query, through an MLP."""

    def __init__(self, radius: float, neighbors_in_radius: int, feature_dim: int, hidden_dim: int) -> None:
        super().__init__()
        self.bq_warp = BQWarp(radius=radius, neighbors_in_radius=neighbors_in_radius)
        self.mlp = Mlp(in_features=feature_dim * neighbors_in_radius, hidden_features=[hidden_dim, hidden_dim // 2],
                       out_features=hidden_dim, act_layer=nn.GELU, drop=0.0)

    def forward(self, query_points, key_features):
        if not torch.compiler.is_compiling():
            if query_points.ndim != 3:
                raise ValueError(f"Expected 3D query_points tensor (B, N, 3), got {query_points.ndim}D tensor with shape {tuple(query_points.shape)}")
            if key_features.ndim != 3:
                raise ValueError(f"Expected 3D key_features tensor (B, N, C), got {key_features.ndim}D tensor with shape {tuple(key_features.shape)}")
        _, neighbors = self.bq_warp(query_points, key_features)
        return torch.tanh(self.mlp(neighbors.reshape(*neighbors.shape[:2], -1)))


class MultiScaleFeatureExtractor(nn.Module):
    def __init__(self, geometry_dim: int, radii, neighbors_in_radius, hidden_dim: int, n_head: int, dim_head: int,
                 dropout: float = 0.0, slice_num: int = 64, use_te: bool = False, plus: bool = False,
                 concrete_dropout: bool = False) -> None:
        super().__init__()
        self.num_scales = len(radii)
        self.processors = nn.ModuleList([GeometricFeatureProcessor(radii[i], neighbors_in_radius[i], geometry_dim, hidden_dim)
                                         for i in range(self.num_scales)])
        self.tokenizers = nn.ModuleList([ContextProjector(hidden_dim, n_head, dim_head, dropout, slice_num, use_te, plus,
                                                          concrete_dropout=concrete_dropout) for _ in range(self.num_scales)])

    def extract_context_features(self, spatial_coords, geometry):
        return [tok(proc(spatial_coords, geometry)) for proc, tok in zip(self.processors, self.tokenizers)]

    def extract_local_features(self, spatial_coords, geometry):
        return torch.cat([proc(geometry, spatial_coords) for proc in self.processors], dim=-1)


class GlobalContextBuilder(nn.Module):
    def __init__(self, functional_dims, geometry_dim=None, global_dim=None, radii=None, neighbors_in_radius=None,
                 n_hidden_local: int = 32, n_hidden: int = 256, n_head: int = 8, dropout: float = 0.0, slice_num: int = 32,
                 use_te: bool = False, plus: bool = False, include_local_features: bool = False, structured_shape=None,
                 concrete_dropout: bool = False) -> None:
        super().__init__()
        radii = [0.05, 0.25] if radii is None else radii
        neighbors_in_radius = [8, 32] if neighbors_in_radius is None else neighbors_in_radius
        dim_head = n_hidden // n_head
        context_dim = 0
        self.structured_shape = structured_shape
        if geometry_dim is not None and include_local_features and structured_shape is None:
            self.local_extractors = nn.ModuleList([
                MultiScaleFeatureExtractor(geometry_dim, radii, neighbors_in_radius, n_hidden_local, n_head, dim_head, dropout,
                                           slice_num, use_te, plus, concrete_dropout=concrete_dropout)
                for _ in functional_dims])
            context_dim += dim_head * len(radii) * len(functional_dims)
        else:
            self.local_extractors = None
        if geometry_dim is not None:
            if structured_shape is not None:
                self.geometry_tokenizer = StructuredContextProjector(geometry_dim, structured_shape, n_head, dim_head, dropout,
                                                                     slice_num, use_te=use_te, plus=plus,
                                                                     concrete_dropout=concrete_dropout)
            else:
                self.geometry_tokenizer = ContextProjector(geometry_dim, n_head, dim_head, dropout, slice_num, use_te,
                                                           plus=plus, concrete_dropout=concrete_dropout)
            context_dim += dim_head
        else:
            self.geometry_tokenizer = None
        if global_dim is not None:
            self.global_tokenizer = ContextProjector(global_dim, n_head, dim_head, dropout, slice_num, use_te, plus,
                                                     concrete_dropout=concrete_dropout)
            context_dim += dim_head
        else:
            self.global_tokenizer = None
        self._context_dim = context_dim

    def get_context_dim(self) -> int:
        return self._context_dim

    def build_context(self, local_embeddings, local_positions, geometry=None, global_embedding=None):
        """``(context [B, H, S, context_dim] | None, per-stream local features | None, detached geometry context | None)``."""
        if not torch.compiler.is_compiling():
            if len(local_embeddings) == 0:
                raise ValueError("Expected non-empty tuple of local embeddings")
            for i, emb in enumerate(local_embeddings):
                if emb.ndim != 3:
                    raise ValueError(f"Expected 3D local_embedding tensor (B, N, C) at index {i}, got {emb.ndim}D tensor with shape {tuple(emb.shape)}")
        parts, local_features, geometry_detached = [], None, None
        if local_positions is None and self.local_extractors is not None:
            raise ValueError("Local positions are required if local features are enabled.")
        if self.local_extractors is not None and geometry is not None:
            local_features = []
            for i in range(len(local_embeddings)):
                coords = local_positions[i]
                parts.extend(self.local_extractors[i].extract_context_features(coords, geometry))
                local_features.append(self.local_extractors[i].extract_local_features(coords, geometry))
        if self.geometry_tokenizer is not None and geometry is not None:
            gctx = self.geometry_tokenizer(geometry)
            geometry_detached = gctx.detach()
            parts.append(gctx)
        if self.global_tokenizer is not None and global_embedding is not None:
            parts.append(self.global_tokenizer(global_embedding))
        context = torch.cat(parts, dim=-1) if parts else None
        if context is not None and hasattr(context, "redistribute"):
            from ...parallel import Replicate

            context = context.redistribute(placements=[Replicate()])
        return context, local_features, geometry_detached

"""GeoTransolver: Transolver blocks whose slice tokens cross-attend to a geometry / global context.

Parity: ``physicsnemo/models/geotransolver/geotransolver.py`` (``GeoTransolver``: ``context_builder``,
``preprocess`` (one MLP per input stream), ``blocks`` of ``GALEBlock``, ``ln_mlp_out``; multi-stream
inputs sharing the blocks; structured 2-D / 3-D grids; optional ball-query local features appended to
the hidden state; ``return_embedding_states`` / ``return_point_features``).
"""
from __future__ import annotations

import math
from collections.abc import Sequence
from dataclasses import dataclass
from typing import Literal

import torch
import torch.nn as nn

from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.gale import GALEBlock
from ..transolver.transolver import _TransolverMlp
from .context_projector import GlobalContextBuilder


@dataclass
class GeoTransolverMetaData(ModelMetaData):
    name: str = "GeoTransolver"
    jit: bool = False
    cuda_graphs: bool = False
    amp: bool = True
    onnx_cpu: bool = False
    onnx_gpu: bool = True
    onnx_runtime: bool = True
    var_dim: int = 1
    func_torch: bool = False
    auto_grad: bool = False


def _normalize_dim(x) -> tuple[int, ...]:
    if isinstance(x, int):
        return (x,)
    if isinstance(x, Sequence) and not isinstance(x, (str, bytes)):
        return tuple(int(v) for v in x)
    raise TypeError(f"Invalid dim specifier {x!r}")


def _normalize_tensor(x) -> tuple[torch.Tensor, ...]:
    if isinstance(x, torch.Tensor):
        return (x,)
    if isinstance(x, Sequence):
        return tuple(x)
    raise TypeError("Invalid tensor structure")


def _structured_num_tokens(spatial_shape) -> int:
    return int(math.prod(spatial_shape))


def _flatten_for_structured(t: torch.Tensor, spatial_shape, name: str) -> torch.Tensor:
    n = _structured_num_tokens(spatial_shape)
    if t.ndim == 3:
        if not torch.compiler.is_compiling() and t.shape[1] != n:
            raise ValueError(f"{name} token count {t.shape[1]} != structured grid size {n}")
        return t
    if t.ndim == len(spatial_shape) + 2:
        if tuple(t.shape[1:-1]) != tuple(spatial_shape):
            raise ValueError(f"{name} spatial dims {tuple(t.shape[1:-1])} != structured_shape {tuple(spatial_shape)}")
        return t.reshape(t.shape[0], n, t.shape[-1])
    raise ValueError(f"{name}: expected (B,N,C) with N={n}, or spatial layout matching structured_shape "
                     f"{tuple(spatial_shape)}; got shape {tuple(t.shape)}")


class GeoTransolver(Module):
    def __init__(self, functional_dim, out_dim, geometry_dim: int | None = None, global_dim: int | None = None,
                 n_layers: int = 4, n_hidden: int = 256, dropout: float = 0.0, n_head: int = 8, act: str = "gelu",
                 mlp_ratio: int = 4, slice_num: int = 32, use_te: bool = False, time_input: bool = False, plus: bool = False,
                 include_local_features: bool = False, radii=None, neighbors_in_radius=None, n_hidden_local: int = 32,
                 structured_shape=None, attention_type: Literal["GALE", "GALE_FA"] = "GALE", concrete_dropout: bool = False,
                 state_mixing_mode: str = "weighted") -> None:
        super().__init__(meta=GeoTransolverMetaData())
        self.__name__ = "GeoTransolver"
        radii = [0.05, 0.25] if radii is None else radii
        neighbors_in_radius = [8, 32] if neighbors_in_radius is None else neighbors_in_radius
        if structured_shape is not None:
            if include_local_features:
                raise ValueError("include_local_features=True is not supported with structured_shape (ball-query path is mesh-only).")
            if len(structured_shape) not in (2, 3):
                raise ValueError(f"structured_shape must have length 2 or 3, got {structured_shape!r}")
            if not all(int(s) > 0 for s in structured_shape):
                raise ValueError(f"structured_shape must be positive ints, got {structured_shape!r}")
            structured_shape = tuple(int(s) for s in structured_shape)
        if n_head <= 0:
            raise ValueError(f"GeoTransolver requires n_head > 0, got {n_head}")
        if n_hidden % n_head != 0:
            raise ValueError(f"GeoTransolver requires n_hidden % n_head == 0, got n_hidden={n_hidden}, n_head={n_head}")
        self.include_local_features, self.use_te, self.structured_shape = include_local_features, False, structured_shape
        functional_dims, out_dims = _normalize_dim(functional_dim), _normalize_dim(out_dim)
        if len(functional_dims) != len(out_dims):
            raise ValueError(f"functional_dim and out_dim must be the same length, but instead got {len(functional_dims)} and {len(out_dims)}")
        self.radii = radii if include_local_features else []
        self.context_builder = GlobalContextBuilder(
            functional_dims=functional_dims, geometry_dim=geometry_dim, global_dim=global_dim, radii=radii,
            neighbors_in_radius=neighbors_in_radius, n_hidden_local=n_hidden_local, n_hidden=n_hidden, n_head=n_head,
            dropout=dropout, slice_num=slice_num, use_te=False, plus=plus, include_local_features=include_local_features,
            structured_shape=structured_shape, concrete_dropout=concrete_dropout)
        context_dim = self.context_builder.get_context_dim()
        self.preprocess = nn.ModuleList([_TransolverMlp(in_features=f, hidden_features=n_hidden * 2, out_features=n_hidden,
                                                        act_layer=act, use_te=False) for f in functional_dims])
        self.n_hidden = n_hidden
        width = n_hidden + n_hidden_local * len(self.radii) if include_local_features else n_hidden
        self.blocks = nn.ModuleList([
            GALEBlock(num_heads=n_head, hidden_dim=width, dropout=dropout, act=act, mlp_ratio=mlp_ratio, slice_num=slice_num,
                      last_layer=(i == n_layers - 1), use_te=False, plus=plus, context_dim=context_dim,
                      spatial_shape=structured_shape, attention_type=attention_type, concrete_dropout=concrete_dropout,
                      state_mixing_mode=state_mixing_mode) for i in range(n_layers)])
        self.ln_mlp_out = nn.ModuleList([nn.Sequential(nn.LayerNorm(width), nn.Linear(width, o)) for o in out_dims])
        self.time_input = time_input
        if time_input:
            self.time_fc = nn.Sequential(nn.Linear(n_hidden, n_hidden), nn.SiLU(), nn.Linear(n_hidden, n_hidden))

    def forward(self, local_embedding, local_positions=None, global_embedding=None, geometry=None, time=None, *,
                return_embedding_states: bool = False, return_point_features: bool = False):
        single = isinstance(local_embedding, torch.Tensor)
        if time is not None:
            raise NotImplementedError("Time input is not implemented yet. Error rather than silently ignoring it.")
        local_embedding = _normalize_tensor(local_embedding)
        if local_positions is not None:
            local_positions = _normalize_tensor(local_positions)
        unflatten = False
        if self.structured_shape is not None:
            unflatten = any(le.ndim in (4, 5) for le in local_embedding)
            local_embedding = tuple(_flatten_for_structured(le, self.structured_shape, f"local_embedding[{i}]")
                                    for i, le in enumerate(local_embedding))
            if geometry is not None:
                geometry = _flatten_for_structured(geometry, self.structured_shape, "geometry")
        if not torch.compiler.is_compiling():
            if len(local_embedding) != len(self.preprocess):
                raise ValueError(f"Expected {len(self.preprocess)} local_embedding stream(s) to match the model's configured "
                                 f"functional_dim/out_dim, got {len(local_embedding)}")
            if local_positions is not None and len(local_positions) != len(local_embedding):
                raise ValueError(f"Expected local_positions to provide the same number of streams as local_embedding "
                                 f"({len(local_embedding)}), got {len(local_positions)}")
            for i, t in enumerate(local_embedding):
                if t.ndim != 3:
                    raise ValueError(f"Expected 3D local_embedding tensor (B, N, C) at index {i}, got {t.ndim}D tensor with shape {tuple(t.shape)}")
            if geometry is not None and geometry.ndim != 3:
                raise ValueError(f"Expected 3D geometry tensor (B, N, C_geo), got {geometry.ndim}D tensor with shape {tuple(geometry.shape)}")
            if global_embedding is not None and global_embedding.ndim != 3:
                raise ValueError(f"Expected 3D global_embedding tensor (B, N_g, C_g), got {global_embedding.ndim}D tensor with shape {tuple(global_embedding.shape)}")
        states, local_bq, _ = self.context_builder.build_context(local_embedding, local_positions, geometry, global_embedding)
        x = [self.preprocess[i](le) for i, le in enumerate(local_embedding)]
        if self.include_local_features and local_bq is not None:
            x = [torch.cat([x[i], local_bq[i]], dim=-1) for i in range(len(x))]
        for block in self.blocks:
            x = block(tuple(x), states)
        point_features = list(x)
        x = [self.ln_mlp_out[i](x[i]) for i in range(len(x))]
        if self.structured_shape is not None and unflatten:
            x = [t.reshape(t.shape[0], *self.structured_shape, -1) for t in x]
        out = x[0] if single else tuple(x)
        pf = point_features[0] if single else tuple(point_features)
        if return_embedding_states and return_point_features:
            return out, states, pf
        if return_embedding_states:
            return out, states
        if return_point_features:
            return out, pf
        return out

"""Transolver: transformer PDE surrogate with physics (slice) attention.

Parity: ``physicsnemo/models/transolver/transolver.py`` — ``_TransolverMlp`` key remap
(``:76-134``), ``TransolverBlock`` (``:137-309``), ``Transolver`` (``:330-736``).  Constructor
arguments and state-dict keys are the reference's (``use_te=False`` layout: ``ln_1``,
``Attn.*``, ``ln_mlp1.0`` LayerNorm + ``ln_mlp1.1.layers.{0,2}``; last block ``ln_mlp2``).

``use_te`` is accepted and ignored: the Transformer-Engine role (fused LayerNorm / Linear
/ MLP) is played by this package's sm_100a kernels under the plain key names, so
checkpoints of the reference's ``use_te=False`` configuration load directly.

On CUDA with bf16 autocast a block runs as: LayerNorm kernel → fused physics attention
(4 tcgen05 GEMMs + 1 tcgen05 reduction, residual in the epilogue) → LayerNorm kernel →
MLP as 2 tcgen05 GEMMs (bias+GELU and bias+residual in the epilogues).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
import torch.nn as nn

from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.module.embedding_layers import PositionalEmbedding
from ...nn.module.layer_norm import LayerNorm
from ...nn.module.mlp_layers import Mlp
from ...nn.module.physics_attention import (
    PhysicsAttentionIrregularMesh,
    PhysicsAttentionStructuredMesh2D,
    PhysicsAttentionStructuredMesh3D,
)
from ... import ops


class _TransolverMlp(Mlp):
    """``Mlp`` that also loads the older ``linear_pre`` / ``linear_post`` key names."""

    _OLD_TO_NEW_KEYS = {
        "linear_pre.weight": "layers.0.weight",
        "linear_pre.bias": "layers.0.bias",
        "linear_post.weight": "layers.2.weight",
        "linear_post.bias": "layers.2.bias",
    }

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                              error_msgs):
        for old, new in self._OLD_TO_NEW_KEYS.items():
            if prefix + old in state_dict and prefix + new not in state_dict:
                state_dict[prefix + new] = state_dict.pop(prefix + old)
        return super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys,
                                             unexpected_keys, error_msgs)

    def forward(self, x, residual=None):
        if residual is not None and self._fusable and ops.fused_path_enabled(x):
            lin = [m for m in self.layers if isinstance(m, nn.Linear)]
            from ...nn.module.activations import activation_code

            acts_mods = [m for m in self.layers if not isinstance(m, (nn.Linear, nn.Dropout))]
            code = activation_code(acts_mods[0]) if acts_mods else 0
            if code is not None and len(lin) >= 1 and all(not isinstance(m, nn.Dropout) for m in self.layers):
                acts = [code] * (len(lin) - 1) + [0]
                return ops.mlp_chain(x, [l.weight for l in lin], [l.bias for l in lin], acts, residual=residual)
        y = super().forward(x)
        return y if residual is None else y + residual


class TransolverBlock(nn.Module):
    """Pre-norm block: ``x + Attn(LN(x))`` then ``x + MLP(LN(x))`` (+ output head on the last)."""

    def __init__(self, num_heads: int, hidden_dim: int, dropout: float, act: str = "gelu", mlp_ratio: int = 4,
                 last_layer: bool = False, out_dim: int = 1, slice_num: int = 32,
                 spatial_shape: tuple[int, ...] | None = None, use_te: bool = True, plus: bool = False):
        super().__init__()
        self.last_layer = last_layer
        self.ln_1 = LayerNorm(hidden_dim)
        common = dict(heads=num_heads, dim_head=hidden_dim // num_heads, dropout=dropout, slice_num=slice_num,
                      use_te=False, plus=plus)
        if spatial_shape is None:
            self.Attn = PhysicsAttentionIrregularMesh(hidden_dim, **common)
        elif len(spatial_shape) == 2:
            self.Attn = PhysicsAttentionStructuredMesh2D(hidden_dim, spatial_shape=spatial_shape, **common)
        elif len(spatial_shape) == 3:
            self.Attn = PhysicsAttentionStructuredMesh3D(hidden_dim, spatial_shape=spatial_shape, **common)
        else:
            raise ValueError(
                f"Unexpected length of spatial shape encountered in Transolver_block: {len(spatial_shape)}. Expected 2 or 3."
            )
        self.ln_mlp1 = nn.Sequential(
            LayerNorm(hidden_dim),
            _TransolverMlp(in_features=hidden_dim, hidden_features=hidden_dim * mlp_ratio, out_features=hidden_dim,
                           act_layer=act, use_te=False),
        )
        if self.last_layer:
            self.ln_mlp2 = nn.Sequential(LayerNorm(hidden_dim), nn.Linear(hidden_dim, out_dim))

    def forward(self, fx: torch.Tensor) -> torch.Tensor:
        ln1, ln2 = self.ln_1, self.ln_mlp1[0]
        xn, skip = ops.layer_norm(fx, ln1.weight, ln1.bias, ln1.eps, return_residual=True)
        fx = self.Attn(xn, residual=skip)
        xn, skip = ops.layer_norm(fx, ln2.weight, ln2.bias, ln2.eps, return_residual=True)
        fx = self.ln_mlp1[1](xn, residual=skip)
        if self.last_layer:
            h = self.ln_mlp2[0](fx)
            lin = self.ln_mlp2[1]
            return ops.linear(h, lin.weight, lin.bias)
        return fx


@dataclass
class MetaData(ModelMetaData):
    jit: bool = False
    cuda_graphs: bool = False
    amp: bool = True
    onnx_cpu: bool = False
    onnx_gpu: bool = True
    onnx_runtime: bool = True
    var_dim: int = 1
    func_torch: bool = False
    auto_grad: bool = False


class Transolver(Module):
    """Transolver model; see the module docstring for the execution paths.

    Parameters follow the reference: ``functional_dim, out_dim, embedding_dim=None, n_layers=4,
    n_hidden=256, dropout=0.0, n_head=8, act="gelu", mlp_ratio=4, slice_num=32, unified_pos=False,
    ref=8, structured_shape=None, use_te=True, time_input=False, plus=False``.

    Forward: ``fx`` (B, N, C_in) or (B, *structured_shape, C_in); ``embedding`` likewise
    (required unless ``unified_pos``); optional ``time`` (B,).  Output (B, N, out_dim).
    """

    def __init__(self, functional_dim: int, out_dim: int, embedding_dim: int | None = None, n_layers: int = 4,
                 n_hidden: int = 256, dropout: float = 0.0, n_head: int = 8, act: str = "gelu", mlp_ratio: int = 4,
                 slice_num: int = 32, unified_pos: bool = False, ref: int = 8,
                 structured_shape: None | tuple[int, ...] = None, use_te: bool = True, time_input: bool = False,
                 plus: bool = False) -> None:
        super().__init__(meta=MetaData())
        self.use_te = False
        if n_hidden % n_head != 0:
            raise ValueError(
                f"Transolver requires n_hidden % n_head == 0, but got n_hidden={n_hidden}, n_head={n_head} "
                f"(remainder={n_hidden % n_head})"
            )
        if structured_shape is not None:
            if len(structured_shape) not in (2, 3):
                raise ValueError(
                    f"Transolver only supports 2D or 3D structured data, got shape with {len(structured_shape)} dimensions"
                )
            if not all(s > 0 and s == int(s) for s in structured_shape):
                raise ValueError(f"Transolver requires positive integer shapes, got {structured_shape}")
            structured_shape = tuple(int(s) for s in structured_shape)
        elif unified_pos:
            raise ValueError("Transolver requires structured_shape when using unified_pos=True")
        self.structured_shape = structured_shape
        self.unified_pos = unified_pos
        if unified_pos:
            self.register_buffer("embedding", self.get_grid(ref))
            self.embedding_dim = ref * ref
            mlp_in = functional_dim + ref * ref
        else:
            if embedding_dim is None:
                raise ValueError("Transolver requires embedding_dim when unified_pos=False")
            self.embedding_dim = embedding_dim
            mlp_in = functional_dim + embedding_dim
        self.preprocess = _TransolverMlp(in_features=mlp_in, hidden_features=n_hidden * 2, out_features=n_hidden,
                                         act_layer=act, use_te=False)
        self.time_input = time_input
        self.n_hidden = n_hidden
        if time_input:
            self.time_embed = PositionalEmbedding(num_channels=n_hidden, max_positions=10000, endpoint=False,
                                                  learnable=False, embed_fn="cos_sin")
            self.time_fc = nn.Sequential(nn.Linear(n_hidden, n_hidden), nn.SiLU(), nn.Linear(n_hidden, n_hidden))
        self.blocks = nn.ModuleList([
            TransolverBlock(num_heads=n_head, hidden_dim=n_hidden, dropout=dropout, act=act, mlp_ratio=mlp_ratio,
                            out_dim=out_dim, slice_num=slice_num, spatial_shape=structured_shape,
                            last_layer=(i == n_layers - 1), use_te=False, plus=plus)
            for i in range(n_layers)
        ])
        self.initialize_weights()

    def initialize_weights(self) -> None:
        self.apply(self._init_weights)

    def _init_weights(self, m: nn.Module) -> None:
        if isinstance(m, nn.Linear):
            nn.init.trunc_normal_(m.weight, std=0.02)
            if m.bias is not None:
                nn.init.constant_(m.bias, 0)
        if isinstance(m, (nn.LayerNorm, nn.BatchNorm1d)):
            nn.init.constant_(m.bias, 0)
            nn.init.constant_(m.weight, 1.0)

    def get_grid(self, ref: int, batchsize: int = 1) -> torch.Tensor:
        """Distances of every grid point to a coarse ``ref × ref`` reference grid: (B, H*W, ref²)."""
        if self.structured_shape is None:
            raise ValueError("Cannot generate positional encoding grid: structured_shape is None.")
        size_x, size_y = self.structured_shape
        gx = torch.linspace(0, 1, size_x).reshape(1, size_x, 1, 1).repeat(batchsize, 1, size_y, 1)
        gy = torch.linspace(0, 1, size_y).reshape(1, 1, size_y, 1).repeat(batchsize, size_x, 1, 1)
        grid = torch.cat((gx, gy), dim=-1)
        rx = torch.linspace(0, 1, ref).reshape(1, ref, 1, 1).repeat(batchsize, 1, ref, 1)
        ry = torch.linspace(0, 1, ref).reshape(1, 1, ref, 1).repeat(batchsize, ref, 1, 1)
        grid_ref = torch.cat((rx, ry), dim=-1)
        pos = torch.sqrt(
            torch.sum((grid[:, :, :, None, None, :] - grid_ref[:, None, None, :, :, :]) ** 2, dim=-1)
        ).reshape(batchsize, -1, ref * ref).contiguous()
        return pos

    def forward(self, fx: torch.Tensor, embedding: torch.Tensor | None = None,
                time: torch.Tensor | None = None) -> torch.Tensor:
        if not torch.compiler.is_compiling():
            if fx.ndim < 2:
                raise ValueError(
                    f"Expected input tensor with at least 2 dimensions, got {fx.ndim}D tensor with shape {tuple(fx.shape)}"
                )
            if not self.unified_pos and embedding is None:
                raise ValueError("Embedding is required when unified_pos=False")
        unflatten = False
        n_tokens = 0
        if self.unified_pos:
            embedding = self.embedding.repeat(fx.shape[0], 1, 1)
        if self.structured_shape is not None:
            if fx.dim() != 3:
                unflatten = True
                fx = fx.reshape(fx.shape[0], -1, fx.shape[-1])
            if embedding is not None and embedding.dim() != 3:
                embedding = embedding.reshape(embedding.shape[0], -1, embedding.shape[-1])
        elif embedding is None:
            raise ValueError("Embedding is required for unstructured data")
        if embedding is not None:
            n_tokens = embedding.shape[1]
            fx = torch.cat((embedding, fx), -1)
        fx = self.preprocess(fx)
        if time is not None:
            emb = self.time_embed(time).unsqueeze(1).repeat(1, n_tokens, 1)
            fx = fx + self.time_fc(emb)
        for block in self.blocks:
            fx = block(fx)
        if self.structured_shape is not None and unflatten:
            fx = fx.reshape(fx.shape[0], *self.structured_shape, -1)
        return fx

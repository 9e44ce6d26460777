"""Transolver physics attention (slice tokens ↔ points).

Parity: ``physicsnemo/nn/module/physics_attention.py`` — ``_project_input`` (``:58-117``),
``_compute_slices_from_projections`` (``:120-206``), ``PhysicsAttentionBase`` (``:209-558``),
``PhysicsAttentionIrregularMesh`` (``:561-660``), ``…StructuredMesh2D/3D`` (``:663-907``).
Parameter names (``temperature``, ``in_project_slice``, ``qkv_project``, ``out_linear``,
``in_project_x``, ``in_project_fx``) and shapes match, so state dicts interchange.

Two execution paths:

* reference path (any device / dtype): the sequence of PyTorch ops of the reference;
* fused path (CUDA, bf16, irregular mesh, no dropout, standard variant): the whole block
  is four tcgen05 GEMMs plus one tcgen05 token reduction
  (``physicsnemo_b200.ops.physics_attention``), with the slice softmax, the output
  projection, the residual and all bias terms inside GEMM epilogues.
"""
from __future__ import annotations

from abc import ABC, abstractmethod

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import ops
from .gumbel_softmax import gumbel_softmax


def _split_heads(t: torch.Tensor, heads: int, dim_head: int, channels_first: bool) -> torch.Tensor:
    if channels_first:  # (B, H*D, *spatial) -> (B, N, H, D)
        B = t.shape[0]
        t = t.reshape(B, heads, dim_head, -1).permute(0, 3, 1, 2)
        return t
    B, N, _ = t.shape
    return t.reshape(B, N, heads, dim_head)


def _project_input(x, project_x, heads, dim_head, channels_first, project_fx=None):
    px = _split_heads(project_x(x), heads, dim_head, channels_first)
    if project_fx is None:
        return px
    return px, _split_heads(project_fx(x), heads, dim_head, channels_first)


def _compute_slices_from_projections(slice_projections, fx, temperature, plus, proj_temperature=None):
    """Slice weights (B,N,H,S) and slice tokens (B,H,S,D) from projections and features.

    Under domain parallelism the two sums over N are partial sums; a ``ShardTensor`` input
    resolves them with one all-reduce each (``physicsnemo_b200.parallel``).
    """
    if plus and proj_temperature is not None:
        temp = temperature + proj_temperature(fx)
        clamped = torch.clamp(temp, min=0.01).to(slice_projections.dtype)
        slice_weights = gumbel_softmax(slice_projections, clamped)
    else:
        clamped = torch.clamp(temperature, min=0.5, max=5).to(slice_projections.dtype)
        slice_weights = F.softmax(slice_projections / clamped, dim=-1)
    slice_weights = slice_weights.to(slice_projections.dtype)
    slice_norm = slice_weights.sum(1) + 1e-2  # (B, H, S)
    normed = slice_weights / slice_norm[:, None, :, :]
    slice_token = torch.matmul(normed.permute(0, 2, 3, 1), fx.permute(0, 2, 1, 3))
    return slice_weights, slice_token


class PhysicsAttentionBase(nn.Module, ABC):
    def __init__(self, dim, heads, dim_head, dropout, slice_num, use_te, plus):
        super().__init__()
        inner_dim = dim_head * heads
        self.dim, self.dim_head, self.heads, self.plus = dim, dim_head, heads, plus
        self.slice_num = slice_num
        self.scale = dim_head**-0.5
        self.use_te = False  # fused sm_100a kernels take the role of Transformer-Engine
        self.softmax = nn.Softmax(dim=-1)
        self.dropout = nn.Dropout(dropout)
        self.temperature = nn.Parameter(torch.ones([1, 1, heads, 1]) * 0.5)
        if plus:
            self.proj_temperature = nn.Sequential(
                nn.Linear(self.dim_head, slice_num), nn.GELU(), nn.Linear(slice_num, 1), nn.GELU()
            )
        self.in_project_slice = nn.Linear(dim_head, slice_num)
        nn.init.orthogonal_(self.in_project_slice.weight)
        self.qkv_project = nn.Linear(dim_head, 3 * dim_head, bias=False)
        self.out_linear = nn.Linear(inner_dim, dim)
        self.out_dropout = nn.Dropout(dropout)

    @abstractmethod
    def project_input_onto_slices(self, x):
        ...

    def _compute_slices_from_projections(self, slice_projections, fx):
        proj_temp = getattr(self, "proj_temperature", None) if self.plus else None
        return _compute_slices_from_projections(slice_projections, fx, self.temperature, self.plus, proj_temp)

    def _compute_slice_attention_sdpa(self, slice_tokens):
        qkv = self.qkv_project(slice_tokens)
        B, H, S, _ = qkv.shape
        qkv = qkv.reshape(B, H, S, 3, self.dim_head)
        if hasattr(qkv, "redistribute"):
            from ...parallel import Replicate

            qkv = qkv.redistribute(placements=[Replicate()])
        q, k, v = qkv.unbind(3)
        return F.scaled_dot_product_attention(q, k, v, is_causal=False)

    def _project_attention_outputs(self, out_slice_token, slice_weights):
        out_x = torch.einsum("bths,bhsd->bthd", slice_weights, out_slice_token)
        out_x = out_x.reshape(out_x.shape[0], out_x.shape[1], -1)
        return self.out_dropout(self.out_linear(out_x))

    def _fusable(self, x) -> bool:
        return False

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """``x``: (B, N, C).  ``residual`` (optional, same shape) is added to the result;
        on the fused path the addition happens in the last GEMM's epilogue."""
        if not torch.compiler.is_compiling():
            if x.ndim != 3:
                raise ValueError(f"Expected 3D input tensor (B, N, C), got {x.ndim}D tensor with shape {tuple(x.shape)}")
            if x.shape[-1] != self.dim:
                raise ValueError(f"Expected input feature dimension {self.dim}, got {x.shape[-1]}")
        if self._fusable(x):
            from ...ops.physics_attention import physics_attention_irregular

            return physics_attention_irregular(self, x, residual, exchange=getattr(self, "_exchange", None))
        projected = self.project_input_onto_slices(x)
        if self.plus:
            x_mid = projected
            fx_mid = x_mid
        else:
            x_mid, fx_mid = projected
        slice_projections = self.in_project_slice(x_mid)
        slice_weights, slice_tokens = self._compute_slices_from_projections(slice_projections, fx_mid)
        out_slice_token = self._compute_slice_attention_sdpa(slice_tokens)
        out = self._project_attention_outputs(out_slice_token, slice_weights)
        return out if residual is None else out + residual


def _fused_params_ok(mod) -> bool:
    from ...ops.physics_attention import fused_supported

    return fused_supported(mod)


class PhysicsAttentionIrregularMesh(PhysicsAttentionBase):
    """Physics attention for unstructured point sets (linear projections)."""

    def __init__(self, dim, heads=8, dim_head=64, dropout=0.0, slice_num=64, use_te=True, plus=False):
        super().__init__(dim, heads, dim_head, dropout, slice_num, use_te, plus)
        inner_dim = dim_head * heads
        self.in_project_x = nn.Linear(dim, inner_dim)
        if not plus:
            self.in_project_fx = nn.Linear(dim, inner_dim)

    def project_input_onto_slices(self, x):
        fx = None if self.plus else self.in_project_fx
        return _project_input(x, self.in_project_x, self.heads, self.dim_head, False, project_fx=fx)

    def _fusable(self, x) -> bool:
        inner = self.heads * self.dim_head
        return (
            not self.plus
            and self.slice_num == 64
            and inner % 64 == 0
            and self.dim % 8 == 0
            and (self.dropout.p == 0.0 or not self.training)
            and ops.fused_path_enabled(x)
            and _fused_params_ok(self)
        )


class PhysicsAttentionStructuredMesh2D(PhysicsAttentionBase):
    """Physics attention on a 2-D grid (3×3 conv projections)."""

    def __init__(self, dim, spatial_shape, heads=8, dim_head=64, dropout=0.0, slice_num=64, kernel=3, use_te=True,
                 plus=False):
        super().__init__(dim, heads, dim_head, dropout, slice_num, use_te, plus)
        inner_dim = dim_head * heads
        self.H, self.W = spatial_shape
        self.in_project_x = nn.Conv2d(dim, inner_dim, kernel, 1, kernel // 2)
        if not plus:
            self.in_project_fx = nn.Conv2d(dim, inner_dim, kernel, 1, kernel // 2)

    def project_input_onto_slices(self, x):
        B, _, C = x.shape
        x = x.view(B, self.H, self.W, C).permute(0, 3, 1, 2)
        fx = None if self.plus else self.in_project_fx
        return _project_input(x, self.in_project_x, self.heads, self.dim_head, True, project_fx=fx)


class PhysicsAttentionStructuredMesh3D(PhysicsAttentionBase):
    """Physics attention on a 3-D grid (3×3×3 conv projections)."""

    def __init__(self, dim, spatial_shape, heads=8, dim_head=64, dropout=0.0, slice_num=32, kernel=3, use_te=True,
                 plus=False):
        super().__init__(dim, heads, dim_head, dropout, slice_num, use_te, plus)
        inner_dim = dim_head * heads
        self.H, self.W, self.D = spatial_shape
        self.in_project_x = nn.Conv3d(dim, inner_dim, kernel, 1, kernel // 2)
        if not plus:
            self.in_project_fx = nn.Conv3d(dim, inner_dim, kernel, 1, kernel // 2)

    def project_input_onto_slices(self, x):
        B, _, C = x.shape
        x = x.view(B, self.H, self.W, self.D, C).permute(0, 4, 1, 2, 3)
        fx = None if self.plus else self.in_project_fx
        return _project_input(x, self.in_project_x, self.heads, self.dim_head, True, project_fx=fx)

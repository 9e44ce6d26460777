"""FIGConvUNet: factorized implicit global convolution U-Net for point clouds (drag and surface-field prediction).

Parity: ``physicsnemo/models/figconvnet/figconvunet.py`` (constructor arguments, ``forward(vertices, features=None) ->
(point_outputs [B, N, out_channels], scalar [B, 1] | None)``) and the building blocks in ``point_feature_conv.py``,
``point_feature_grid_ops.py``, ``point_feature_grid_conv.py``, ``grid_feature_group.py``, ``components/``: the 3-D domain is
represented by a *group* of factor grids, each high-resolution along two axes and low-resolution along the third, the third
axis being folded into the channels so that every grid is processed by 2-D convolutions; after every conv block the grids
exchange information by sampling each other trilinearly ("intra-communication", sum or product).

This implementation keeps the computation of the reference but stores a factor grid as one plain tensor
``[B, D_c · C, U, V]`` (compressed axis major) with its axis index, instead of the reference's vertex-carrying
``GridFeatures`` objects with switchable memory formats: node positions of a level are implied by its shape (nodes span the
bounding box), so nothing but features flows through the U-Net.  Parameter names therefore differ from the reference's
checkpoints.  Point→grid and grid→point graph convolutions search neighbours with the hash-grid ``radius_search`` /
``knn`` functionals (CUDA kernels on GPU) in voxel units.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from enum import Enum
from typing import List, Literal, Optional, Sequence, Tuple, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...core.meta import ModelMetaData
from ...core.module import Module
from ...nn.functional.neighbors import knn, radius_search

REDUCTION_TYPES = Literal["min", "max", "mean", "sum", "var", "std"]


class GridFeaturesMemoryFormat(Enum):
    """Which axis of a factor grid is folded into the channels (``b_x_y_z_c`` = none, a plain 3-D grid)."""

    b_x_y_z_c = -1
    b_xc_y_z = 0
    b_yc_x_z = 1
    b_zc_x_y = 2


# ---- small components ------------------------------------------------------------------------------------------------
class SinusoidalEncoding(nn.Module):
    """``[cos(2π 2^k x / range), sin(…)]`` for ``k < num_channels / 2``, per input coordinate."""

    def __init__(self, num_channels: int, data_range: float = 2.0):
        super().__init__()
        if num_channels % 2:
            raise ValueError(f"num_channels must be even for sin/cos, got {num_channels}")
        self.num_channels, self.data_range = num_channels, data_range

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        freqs = (2 * math.pi / self.data_range) * 2 ** torch.arange(self.num_channels // 2, device=x.device, dtype=x.dtype)
        ang = x.unsqueeze(-1) * freqs
        return torch.cat([ang.cos(), ang.sin()], dim=-1).flatten(start_dim=-2)


class MLPBlock(nn.Module):
    """Linear-LN-GELU-Linear-LN with a linear shortcut."""

    def __init__(self, in_channels: int, hidden_channels: int | None = None, out_channels: int | None = None):
        super().__init__()
        hidden_channels, out_channels = hidden_channels or in_channels, out_channels or in_channels
        self.in_channels = in_channels
        self.fc1, self.norm1 = nn.Linear(in_channels, hidden_channels), nn.LayerNorm(hidden_channels)
        self.fc2, self.norm2 = nn.Linear(hidden_channels, out_channels), nn.LayerNorm(out_channels)
        self.shortcut = nn.Linear(in_channels, out_channels)

    def forward(self, x):
        return F.gelu(self.norm2(self.fc2(F.gelu(self.norm1(self.fc1(x))))) + self.shortcut(x))


class _ResidualLinear(nn.Module):
    def __init__(self, cin, cout):
        super().__init__()
        self.blocks = nn.Sequential(nn.Linear(cin, cin), nn.LayerNorm(cin), nn.GELU(), nn.Linear(cin, cout), nn.LayerNorm(cout))
        self.shortcut = nn.Identity() if cin == cout else nn.Linear(cin, cout)

    def forward(self, x):
        return F.gelu(self.blocks(x) + self.shortcut(x))


class MLP(nn.Module):
    def __init__(self, in_channels: int, out_channels: int, hidden_channels: Sequence[int], use_residual: bool = False):
        super().__init__()
        ch = [in_channels, *hidden_channels, out_channels]
        self.layers = nn.ModuleList([
            _ResidualLinear(ch[i], ch[i + 1]) if use_residual and i < len(ch) - 2 else
            nn.Sequential(nn.Linear(ch[i], ch[i + 1], bias=False), nn.LayerNorm(ch[i + 1]), nn.GELU()) for i in range(len(ch) - 1)])

    def forward(self, x):
        for layer in self.layers:
            x = layer(x)
        return x


class LayerNorm2d(nn.LayerNorm):
    def forward(self, x):
        return F.layer_norm(x.permute(0, 2, 3, 1), self.normalized_shape, self.weight, self.bias, self.eps).permute(0, 3, 1, 2)


def segment_reduce(values: torch.Tensor, segment: torch.Tensor, n: int, reduction: str) -> torch.Tensor:
    """Reduce rows of ``values [E, C]`` into ``n`` segments given by ``segment [E]``; empty segments give zero."""
    C = values.shape[1]
    idx = segment.unsqueeze(1).expand(-1, C)
    if reduction in ("sum", "mean", "var", "std"):
        s = values.new_zeros(n, C).index_add_(0, segment, values)
        if reduction == "sum":
            return s
        cnt = values.new_zeros(n).index_add_(0, segment, values.new_ones(values.shape[0])).clamp_min(1).unsqueeze(1)
        mean = s / cnt
        if reduction == "mean":
            return mean
        var = (values.new_zeros(n, C).index_add_(0, segment, values * values) / cnt - mean * mean).clamp_min(0)
        return var if reduction == "var" else var.sqrt()
    if reduction in ("max", "min"):
        out = values.new_zeros(n, C).scatter_reduce_(0, idx, values, "amax" if reduction == "max" else "amin", include_self=False)
        return out
    raise ValueError(f"unknown reduction {reduction!r}")


def neighbour_pairs(points: torch.Tensor, queries: torch.Tensor, search: str, radius: float, k: int):
    """Flattened ``(query_index, point_index)`` pairs over a batch ``points [B, N, 3]``, ``queries [B, M, 3]``."""
    B, N, M = points.shape[0], points.shape[1], queries.shape[1]
    qs, ps = [], []
    with torch.no_grad():
        for b in range(B):
            if search == "knn":
                kk = min(k, N)
                idx = knn(points[b].float().contiguous(), queries[b].float().contiguous(), kk)[0].long()
                q = torch.arange(M, device=points.device).repeat_interleave(kk)
                p = idx.reshape(-1)
            elif search == "radius":
                pr = radius_search(points[b].float().contiguous(), queries[b].float().contiguous(), radius, max_points=None).long()
                q, p = pr[0], pr[1]
            else:
                raise ValueError(f"neighbor_search_type must be radius or knn, got {search}")
            qs.append(q + b * M)
            ps.append(p + b * N)
    return torch.cat(qs), torch.cat(ps)


class PointFeatureConv(nn.Module):
    """Graph convolution from source points to target points: edge MLP over [source feats, target feats, relative position
    (optionally sinusoidally encoded)], reduction(s) over the neighbours of every target, output MLP."""

    def __init__(self, in_channels: int, target_channels: int, out_channels: int, radius: float = math.sqrt(3), hidden_dim: int | None = None,
                 use_rel_pos: bool = True, use_rel_pos_encode: bool = False, pos_encode_dim: int = 32, pos_encode_range: float = 4.0,
                 reductions: Sequence[str] = ("mean",), neighbor_search_type: str = "radius", knn_k: int = 16):
        super().__init__()
        if not reductions:
            raise ValueError("reductions must be a non-empty list")
        self.radius, self.k, self.search = radius, knn_k, neighbor_search_type
        self.use_rel_pos, self.use_rel_pos_encode, self.reductions = use_rel_pos, use_rel_pos_encode, list(reductions)
        self.positional_encoding = SinusoidalEncoding(pos_encode_dim, pos_encode_range)
        hidden_dim = hidden_dim or 2 * out_channels
        edge_in = in_channels + target_channels + (3 * pos_encode_dim if use_rel_pos_encode else (3 if use_rel_pos else 0))
        self.edge_transform_mlp = MLPBlock(edge_in, hidden_dim, out_channels)
        self.out_transform_mlp = MLPBlock(out_channels * len(self.reductions), hidden_dim, out_channels)

    def forward(self, src_xyz, src_feat, dst_xyz, dst_feat, scaler: torch.Tensor | None = None):
        B, M = dst_xyz.shape[:2]
        sx, dx = (src_xyz * scaler, dst_xyz * scaler) if scaler is not None else (src_xyz, dst_xyz)
        q, p = neighbour_pairs(sx, dx, self.search, self.radius, self.k)
        edge = [src_feat.reshape(-1, src_feat.shape[-1])[p], dst_feat.reshape(-1, dst_feat.shape[-1])[q]]
        if self.use_rel_pos or self.use_rel_pos_encode:
            rel = src_xyz.reshape(-1, 3)[p] - dst_xyz.reshape(-1, 3)[q]
            edge.append(self.positional_encoding(rel) if self.use_rel_pos_encode else rel)
        e = self.edge_transform_mlp(torch.cat(edge, dim=1))
        out = torch.cat([segment_reduce(e, q, B * M, r) for r in self.reductions], dim=-1)
        return self.out_transform_mlp(out).reshape(B, M, -1)


# ---- factor grids ----------------------------------------------------------------------------------------------------
def _fold(x5: torch.Tensor, axis: int) -> torch.Tensor:
    """``[B, C, X, Y, Z]`` -> ``[B, D·C, U, V]`` with the compressed axis major in the channel dimension."""
    if axis < 0:
        return x5
    x = x5.movedim(2 + axis, 1)                                  # [B, D, C, U, V]
    return x.reshape(x.shape[0], -1, *x.shape[3:])


def _unfold(x4: torch.Tensor, axis: int, depth: int) -> torch.Tensor:
    if axis < 0:
        return x4
    B, DC, U, V = x4.shape
    return x4.reshape(B, depth, DC // depth, U, V).movedim(1, 2 + axis)


def _node_positions(shape3: Sequence[int], device, dtype) -> torch.Tensor:
    """Normalised ``[-1, 1]`` node coordinates of a grid of 3-D shape ``shape3`` in ``grid_sample`` (x=last axis) order."""
    axes = [torch.linspace(-1, 1, n, device=device, dtype=dtype) if n > 1 else torch.zeros(1, device=device, dtype=dtype) for n in shape3]
    gx, gy, gz = torch.meshgrid(*axes, indexing="ij")
    return torch.stack((gz, gy, gx), dim=-1)                      # grid_sample wants (W, H, D) = (z, y, x) for [B,C,X,Y,Z]


class GridConv2d(nn.Module):
    """2-D (transposed) convolution over a factor grid; the compressed axis rides along in the channels."""

    def __init__(self, in_channels, out_channels, kernel_size, depth, stride=1, up_stride=None):
        super().__init__()
        if up_stride is None:
            self.conv = nn.Conv2d(in_channels * depth, out_channels * depth, kernel_size, stride=stride, padding=(kernel_size - 1) // 2)
        else:
            self.conv = nn.ConvTranspose2d(in_channels * depth, out_channels * depth, kernel_size, stride=up_stride,
                                           padding=(kernel_size - 1) // 2 if kernel_size != up_stride else 0,
                                           output_padding=up_stride - 1 if kernel_size != up_stride else 0)

    def forward(self, x):
        return self.conv(x)


def pad_to_match(ref: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """Crop / zero-pad the trailing two axes of ``x`` to those of ``ref``."""
    x = x[..., :ref.shape[-2], :ref.shape[-1]]
    ph, pw = ref.shape[-2] - x.shape[-2], ref.shape[-1] - x.shape[-1]
    return F.pad(x, (0, pw, 0, ph)) if ph > 0 or pw > 0 else x


class GridConvBlock(nn.Module):
    """conv → LN → GELU → conv → LN, plus a (strided / transposed) shortcut."""

    def __init__(self, in_channels, out_channels, kernel_size, depth, stride=1, up_stride=None):
        super().__init__()
        self.conv1 = GridConv2d(in_channels, out_channels, kernel_size if up_stride is None else up_stride, depth, stride, up_stride)
        self.conv2 = GridConv2d(out_channels, out_channels, kernel_size, depth)
        self.norm1, self.norm2 = LayerNorm2d(out_channels * depth), LayerNorm2d(out_channels * depth)
        if up_stride is not None:
            self.shortcut = GridConv2d(in_channels, out_channels, up_stride, depth, up_stride=up_stride)
        elif stride > 1:
            self.shortcut = nn.Conv2d(in_channels * depth, out_channels * depth, stride, stride=stride)
        elif in_channels != out_channels:
            self.shortcut = nn.Conv2d(in_channels * depth, out_channels * depth, 1)
        else:
            self.shortcut = nn.Identity()

    def forward(self, x):
        out = self.norm2(self.conv2(F.gelu(self.norm1(self.conv1(x)))))
        return out + pad_to_match(out, self.shortcut(x))


class GroupConvAndCommunication(nn.Module):
    """One conv block per factor grid, then every grid adds (or multiplies in) the others sampled at its own nodes."""

    def __init__(self, in_channels, out_channels, kernel_size, depths, axes, stride=1, up_stride=None, communication_types=("sum",)):
        super().__init__()
        types = [communication_types] if isinstance(communication_types, str) else list(communication_types)
        if not 1 <= len(types) <= 2 or any(t not in ("sum", "mul") for t in types):
            raise NotImplementedError(f"communication_types must be one or two of 'sum' / 'mul', got {types}")
        self.types, self.depths, self.axes = types, list(depths), list(axes)
        self.convs = nn.ModuleList([GridConvBlock(in_channels, out_channels, kernel_size, d, stride, up_stride) for d in depths])
        if len(types) > 1:
            self.proj = nn.ModuleList([nn.Sequential(nn.Conv2d(out_channels * len(types) * d, out_channels * d, 1), LayerNorm2d(out_channels * d))
                                       for d in depths])
        else:
            self.proj = None

    def _communicate(self, grids5: List[torch.Tensor], kind: str) -> List[torch.Tensor]:
        out = []
        for i, g in enumerate(grids5):
            pos = _node_positions(g.shape[2:], g.device, g.dtype).unsqueeze(0).expand(g.shape[0], -1, -1, -1, -1)
            acc = g
            for j, other in enumerate(grids5):
                if i != j:
                    s = F.grid_sample(other, pos, align_corners=True)
                    acc = acc + s if kind == "sum" else acc * s
            out.append(acc)
        return out

    def forward(self, group: List[torch.Tensor]) -> List[torch.Tensor]:
        feats = [conv(g) for conv, g in zip(self.convs, group)]
        grids5 = [_unfold(f, a, d) for f, a, d in zip(feats, self.axes, self.depths)]
        mixed = [self._communicate(grids5, t) for t in self.types]
        if len(mixed) == 1:
            out5 = mixed[0]
        else:
            out5 = [torch.cat([m[i] for m in mixed], dim=1) for i in range(len(grids5))]
        out = [_fold(g, a) for g, a in zip(out5, self.axes)]
        if self.proj is not None:
            out = [p(o) for p, o in zip(self.proj, out)]
        return [F.gelu(o) for o in out]


class PointFeatureToGrid(nn.Module):
    """Scatter point features onto the nodes of one factor grid with a graph convolution (nodes carry a sinusoidal
    encoding of their position)."""

    def __init__(self, in_channels, out_channels, aabb_max, aabb_min, resolution, axis, use_rel_pos=True, use_rel_pos_encode=False,
                 pos_encode_dim=32, reductions=("mean",), neighbor_search_type="radius", knn_k=16, radius=math.sqrt(3)):
        super().__init__()
        for i in range(3):
            if aabb_max[i] <= aabb_min[i]:
                raise ValueError(f"aabb_max[{i}] ({aabb_max[i]}) must be greater than aabb_min[{i}] ({aabb_min[i]})")
        self.resolution, self.axis = [int(r) for r in resolution], axis
        lo, hi = torch.tensor(aabb_min, dtype=torch.float32), torch.tensor(aabb_max, dtype=torch.float32)
        axes = [torch.linspace(float(lo[i]), float(hi[i]), self.resolution[i]) for i in range(3)]
        nodes = torch.stack(torch.meshgrid(*axes, indexing="ij"), dim=-1).reshape(-1, 3)
        self.register_buffer("nodes", nodes, persistent=False)
        self.register_buffer("node_features", SinusoidalEncoding(pos_encode_dim, float(hi[0] - lo[0]))(nodes), persistent=False)
        self.register_buffer("scaler", torch.tensor(self.resolution, dtype=torch.float32) / (hi - lo), persistent=False)
        self.conv = PointFeatureConv(in_channels, 3 * pos_encode_dim, out_channels, radius=radius, use_rel_pos=use_rel_pos,
                                     use_rel_pos_encode=use_rel_pos_encode, pos_encode_dim=pos_encode_dim,
                                     pos_encode_range=float(hi[0] - lo[0]), reductions=reductions,
                                     neighbor_search_type=neighbor_search_type, knn_k=knn_k)

    def forward(self, xyz, feat):
        B = xyz.shape[0]
        nodes = self.nodes.to(xyz.dtype).unsqueeze(0).expand(B, -1, -1)
        nf = self.node_features.to(feat.dtype).unsqueeze(0).expand(B, -1, -1)
        out = self.conv(xyz, feat, nodes, nf, self.scaler.to(xyz.dtype))                       # [B, X·Y·Z, C]
        x5 = out.reshape(B, *self.resolution, -1).permute(0, 4, 1, 2, 3)
        return _fold(x5, self.axis)


class GridFeatureToPoint(nn.Module):
    """Read one factor grid at the points: graph convolution from the grid nodes, or trilinear interpolation + linear."""

    def __init__(self, grid_in_channels, point_in_channels, out_channels, aabb_max, aabb_min, use_rel_pos=True, use_rel_pos_embed=False,
                 pos_embed_dim=32, sample_method="graphconv", neighbor_search_type="radius", knn_k=16, reductions=("mean",)):
        super().__init__()
        self.sample_method = sample_method
        self.register_buffer("lo", torch.tensor(aabb_min, dtype=torch.float32), persistent=False)
        self.register_buffer("hi", torch.tensor(aabb_max, dtype=torch.float32), persistent=False)
        if sample_method == "graphconv":
            self.conv = PointFeatureConv(grid_in_channels, point_in_channels, out_channels, radius=math.sqrt(3), use_rel_pos=use_rel_pos,
                                         use_rel_pos_encode=use_rel_pos_embed, pos_encode_dim=pos_embed_dim,
                                         pos_encode_range=float(aabb_max[0] - aabb_min[0]), reductions=reductions,
                                         neighbor_search_type=neighbor_search_type, knn_k=knn_k)
        elif sample_method == "interp":
            self.transform = nn.Sequential(nn.Linear(grid_in_channels + point_in_channels, out_channels), nn.LayerNorm(out_channels))
        else:
            raise NotImplementedError(f"unknown sample method {sample_method!r}")

    def forward(self, grid5, xyz, feat):
        B, C = grid5.shape[:2]
        lo, hi = self.lo.to(xyz.dtype), self.hi.to(xyz.dtype)
        if self.sample_method == "interp":
            g = ((xyz - lo) / (hi - lo) * 2 - 1).flip(-1).reshape(B, 1, 1, -1, 3)
            sampled = F.grid_sample(grid5, g, align_corners=True).reshape(B, C, -1).transpose(1, 2)
            return self.transform(torch.cat((feat, sampled), dim=-1))
        res = grid5.shape[2:]
        axes = [torch.linspace(float(lo[i]), float(hi[i]), res[i], device=xyz.device, dtype=xyz.dtype) for i in range(3)]
        nodes = torch.stack(torch.meshgrid(*axes, indexing="ij"), dim=-1).reshape(1, -1, 3).expand(B, -1, -1)
        nf = grid5.permute(0, 2, 3, 4, 1).reshape(B, -1, C)
        scaler = torch.tensor(list(res), device=xyz.device, dtype=xyz.dtype) / (hi - lo)
        return self.conv(nodes, nf, xyz, feat, scaler)


class AttentionPool(nn.Module):
    def __init__(self, in_channels, out_channels, num_heads: int = 2, dropout: float = 0.0):
        super().__init__()
        self.num_heads, self.head_dim = num_heads, out_channels // num_heads
        self.qkv, self.out, self.dropout = nn.Linear(in_channels, out_channels * 3), nn.Linear(out_channels, out_channels), nn.Dropout(dropout)

    def forward(self, x):
        B, N, _ = x.shape
        q, k, v = self.qkv(x).reshape(B, N, 3, self.num_heads, self.head_dim).permute(2, 0, 3, 1, 4)
        q = q.max(dim=2, keepdim=True).values
        attn = self.dropout(F.softmax(q @ k.transpose(-2, -1) / self.head_dim ** 0.5, dim=-1))
        return self.out((attn @ v).reshape(B, -1))


class GridFeaturePool(nn.Module):
    def __init__(self, in_channels, out_channels, depth, pooling_type="max"):
        super().__init__()
        self.conv = nn.Conv2d(in_channels * depth, out_channels, 1)
        if pooling_type not in ("attention", "max", "mean"):
            raise NotImplementedError(f"Unknown pooling type: {pooling_type}")
        self.pooling_type = pooling_type
        self.pool = AttentionPool(out_channels, out_channels) if pooling_type == "attention" else None
        self.norm = nn.LayerNorm(out_channels)

    def forward(self, x):
        f = self.conv(x).flatten(2)
        if self.pooling_type == "attention":
            p = self.pool(f.transpose(1, 2))
        else:
            p = f.amax(dim=-1) if self.pooling_type == "max" else f.mean(dim=-1)
        return self.norm(p)


@dataclass
class MetaData(ModelMetaData):
    name: str = "FIGConvUNet"
    jit: bool = False
    cuda_graphs: bool = False
    amp_gpu: bool = True


_DEFAULT_PAIRS = ((GridFeaturesMemoryFormat.b_xc_y_z, (2, 128, 128)), (GridFeaturesMemoryFormat.b_yc_x_z, (128, 2, 128)),
                  (GridFeaturesMemoryFormat.b_zc_x_y, (128, 128, 2)))


class FIGConvUNet(Module):
    def __init__(self, in_channels: int, out_channels: int, kernel_size: int, hidden_channels: List[int], num_levels: int = 3,
                 num_down_blocks: Union[int, List[int]] = 1, num_up_blocks: Union[int, List[int]] = 1, mlp_channels: Optional[List[int]] = None,
                 aabb_max: Tuple[float, float, float] = (1.0, 1.0, 1.0), aabb_min: Tuple[float, float, float] = (0.0, 0.0, 0.0),
                 voxel_size: Optional[float] = None, resolution_memory_format_pairs=_DEFAULT_PAIRS, use_rel_pos: bool = True,
                 use_rel_pos_embed: bool = True, pos_encode_dim: int = 32, communication_types: List[str] = ("sum",),
                 to_point_sample_method: str = "graphconv", neighbor_search_type: str = "radius", knn_k: int = 16,
                 reductions: List[str] = ("mean",), use_scalar_output: bool = True, has_input_features: bool = False,
                 pooling_type: str = "max", pooling_layers: List[int] = None):
        super().__init__(meta=MetaData())
        mlp_channels = list(mlp_channels) if mlp_channels is not None else [512, 512]
        if len(hidden_channels) < num_levels + 1:
            raise ValueError("hidden_channels needs num_levels + 1 entries")
        self.in_channels, self.out_channels, self.hidden_channels, self.num_levels = in_channels, out_channels, list(hidden_channels), num_levels
        self.use_scalar_output, self.has_input_features = use_scalar_output, has_input_features
        axes, depths, self.point_feature_to_grids = [], [], nn.ModuleList()
        point_channels = in_channels if has_input_features else hidden_channels[0]
        for fmt, res in resolution_memory_format_pairs:
            fmt = GridFeaturesMemoryFormat[fmt] if isinstance(fmt, str) else fmt
            if fmt.value < 0:
                raise ValueError("factor grids need a compressed axis (b_xc_y_z, b_yc_x_z or b_zc_x_y)")
            axes.append(fmt.value)
            depths.append(int(res[fmt.value]))
            self.point_feature_to_grids.append(PointFeatureToGrid(
                point_channels, hidden_channels[0], aabb_max, aabb_min, res, fmt.value, use_rel_pos=use_rel_pos,
                use_rel_pos_encode=use_rel_pos_embed, pos_encode_dim=pos_encode_dim, reductions=reductions,
                neighbor_search_type=neighbor_search_type, knn_k=knn_k))
        self.axes, self.compressed_spatial_dims = axes, depths
        self.grid_feature_group_size = len(axes)
        nd = [num_down_blocks] * (num_levels + 1) if isinstance(num_down_blocks, int) else list(num_down_blocks)
        nu = [num_up_blocks] * (num_levels + 1) if isinstance(num_up_blocks, int) else list(num_up_blocks)
        mk = lambda ci, co, **kw: GroupConvAndCommunication(ci, co, kernel_size, depths, axes, communication_types=communication_types, **kw)  # noqa: E731
        self.down_blocks, self.up_blocks = nn.ModuleList(), nn.ModuleList()
        for lvl in range(num_levels):
            lo_c, hi_c = hidden_channels[lvl], hidden_channels[lvl + 1]
            self.down_blocks.append(nn.Sequential(mk(lo_c, hi_c, stride=2), *[mk(hi_c, hi_c, stride=1) for _ in range(1, nd[lvl])]))
            self.up_blocks.append(nn.Sequential(mk(hi_c, lo_c, up_stride=2), *[mk(lo_c, lo_c, up_stride=1) for _ in range(1, nu[lvl])]))
        if use_scalar_output:
            if pooling_layers is None:
                pooling_layers = [num_levels]
            elif not isinstance(pooling_layers, list):
                raise ValueError(f"pooling_layers must be a list, got {type(pooling_layers)}.")
            for layer in pooling_layers:
                if layer > num_levels:
                    raise ValueError(f"pooling_layer {layer} is greater than num_levels {num_levels}.")
            self.pooling_layers = pooling_layers
            self.grid_pools = nn.ModuleList([nn.ModuleList([GridFeaturePool(hidden_channels[layer], mlp_channels[0], d, pooling_type) for d in depths])
                                             for layer in pooling_layers])
            self.mlp = MLP(mlp_channels[0] * len(depths) * len(pooling_layers), mlp_channels[-1], mlp_channels, use_residual=True)
            self.mlp_projection = nn.Linear(mlp_channels[-1], 1)
        width = hidden_channels[0] * 2
        self.to_point = nn.ModuleList([GridFeatureToPoint(hidden_channels[0], point_channels, width // 2, aabb_max, aabb_min, use_rel_pos=use_rel_pos,
                                                          use_rel_pos_embed=use_rel_pos_embed, pos_embed_dim=pos_encode_dim,
                                                          sample_method=to_point_sample_method, neighbor_search_type=neighbor_search_type,
                                                          knn_k=knn_k, reductions=reductions) for _ in axes])
        self.projection = nn.Sequential(nn.Linear(width, width), nn.LayerNorm(width), nn.GELU(), nn.Linear(width, out_channels))
        if not has_input_features:
            self.vertex_to_point_features = nn.ModuleDict({"mlp": MLP(3 * pos_encode_dim, hidden_channels[0], [])})
            self._vertex_encoding = SinusoidalEncoding(pos_encode_dim, float(aabb_max[0] - aabb_min[0]))

    # ------------------------------------------------------------ checkpoints
    #: (pattern in the reference's parameter names, replacement here); applied in order to every incoming key
    _REFERENCE_KEY_RULES = (
        (r"^point_feature_to_grids\.(\d+)\.0\.", r"point_feature_to_grids.\1."),
        (r"\.norm(\d)\.feature_transform\.", r".norm\1."),
        (r"^(down_blocks\.\d+\.\d+\.convs\.\d+\.shortcut)\.conv\.", r"\1."),
        (r"^grid_pools\.(\d+)\.pools\.", r"grid_pools.\1."),
        (r"(mlp\.layers\.\d+)\.block\.", r"\1."),
        (r"^to_point\.conv_list\.(\d+)\.conv\.conv\.", r"to_point.\1.conv."),
        (r"^projection\.feature_transform\.", "projection."),
    )

    @classmethod
    def _from_reference_key(cls, key: str) -> str:
        import re

        for pattern, repl in cls._REFERENCE_KEY_RULES:
            key = re.sub(pattern, repl, key)
        return key

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        """Accept state dicts written by the reference implementation: its parameter names differ from the ones here only
        by wrapper levels (``.0.``, ``.pools.``, ``.block.``, ``.conv_list.N.conv.``, ``.feature_transform.``), which
        are renamed before loading.  Keys already in this package's naming pass through unchanged."""
        for key in [k for k in state_dict if k.startswith(prefix)]:
            new = prefix + self._from_reference_key(key[len(prefix):])
            if new != key and new not in state_dict:
                state_dict[new] = state_dict.pop(key)
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    def _grid_forward(self, xyz, feat):
        levels = [[to_grid(xyz, feat) for to_grid in self.point_feature_to_grids]]
        for block in self.down_blocks:
            levels.append(block(levels[-1]))
        scalar = None
        if self.use_scalar_output:
            pooled = [torch.cat([pool(g) for pool, g in zip(pools, levels[layer])], dim=-1) for pools, layer in zip(self.grid_pools, self.pooling_layers)]
            scalar = self.mlp_projection(self.mlp(torch.cat(pooled, dim=-1)))
        for lvl in reversed(range(self.num_levels)):
            up = self.up_blocks[lvl](levels[lvl + 1])
            levels[lvl] = [pad_to_match(skip, u) + skip for u, skip in zip(up, levels[lvl])]
        return [_unfold(g, a, d) for g, a, d in zip(levels[0], self.axes, self.compressed_spatial_dims)], scalar

    def forward(self, vertices: torch.Tensor, features: Optional[torch.Tensor] = None):
        if vertices.ndim != 3 or vertices.shape[2] != 3:
            raise ValueError(f"Expected vertices of shape (B, N, 3), got {tuple(vertices.shape)}")
        if features is not None:
            if features.ndim != 3 or features.shape[:2] != vertices.shape[:2]:
                raise ValueError(f"Expected features of shape (B, N, C) matching the vertices, got {tuple(features.shape)}")
            if features.shape[2] != self.in_channels:
                raise ValueError(f"Expected {self.in_channels} input feature channels, got {features.shape[2]} channels")
        if features is None:
            if self.has_input_features:
                raise ValueError("this model was built with has_input_features=True and needs features")
            features = self.vertex_to_point_features["mlp"](self._vertex_encoding(vertices))
        grids5, scalar = self._grid_forward(vertices, features)
        per_grid = [tp(g, vertices, features) for tp, g in zip(self.to_point, grids5)]
        add, mul = per_grid[0], per_grid[0]
        for cur in per_grid[1:]:
            add, mul = add + cur, mul * cur
        return self.projection(torch.cat((add, mul), dim=-1)), scalar

"""DPOT: auto-regressive operator transformer with AFNO-style Fourier mixing, 2-D and 3-D.

Parity: ``physicsnemo/models/dpot/dpot.py`` (``DPOT2DLayer``, ``ConvMlp``, ``Block``, ``PatchEmbed``,
``TimeAggregator``, ``DPOTNet``, ``resize_pos_embed``, ``checkpoint_filter_fn``) and ``dpot3d.py``
(``AFNO3DLayer``, ``ConvMlp3D``, ``Block3D``, ``PatchEmbed3D``, ``DPOTNet3D``); parameter names and
shapes are the reference's (``w1 [2, nb, bs, bs·f]`` … with index 0 = real part, 1 = imaginary part).

Both dimensionalities share one implementation.  The spectral mixer transforms only the retained
low-frequency corner: the block-diagonal two-layer complex MLP is evaluated as complex batched
products on that corner and the result is zero-padded to the full spectrum in one ``F.pad`` — the
full-size zero buffers and slice assignments of a literal formulation never exist.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Literal, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...core.meta import ModelMetaData
from ...core.module import Module

Tensor = torch.Tensor

_ACTIVATIONS = {"gelu": nn.GELU, "tanh": nn.Tanh, "sigmoid": nn.Sigmoid, "relu": nn.ReLU,
                "leaky_relu": lambda: nn.LeakyReLU(0.1), "softplus": nn.Softplus, "elu": nn.ELU, "silu": nn.SiLU}
_CONV = {2: nn.Conv2d, 3: nn.Conv3d}
_CONVT = {2: nn.ConvTranspose2d, 3: nn.ConvTranspose3d}


def get_activation(name: str) -> nn.Module:
    key = name.lower()
    if key not in _ACTIVATIONS:
        raise ValueError(f"Unsupported activation '{name}'. Available: {list(_ACTIVATIONS)}")
    return _ACTIVATIONS[key]()


def _tuple(v, nd: int):
    return (v,) * nd if isinstance(v, int) else tuple(v)


class _FourierMixer(nn.Module):
    """Block-diagonal complex MLP on the retained Fourier modes of a channels-first or channels-last grid."""

    nd = 2

    def __init__(self, width: int = 32, num_blocks: int = 8, sparsity_threshold: float = 0.01, modes: int = 32,
                 hidden_size_factor: int = 1, channel_first: bool = False, activation: str = "gelu",
                 temporal_modes: int | None = None):
        super().__init__()
        if width % num_blocks != 0:
            raise ValueError(f"width {width} must be divisible by num_blocks {num_blocks}")
        self.width, self.num_blocks, self.block_size = width, num_blocks, width // num_blocks
        self.sparsity_threshold, self.modes, self.temporal_modes = sparsity_threshold, modes, temporal_modes
        self.hidden_size_factor, self.channel_first = hidden_size_factor, channel_first
        self.act = get_activation(activation)
        bs, f = self.block_size, hidden_size_factor
        scale = 1.0 / (bs * bs * f)
        self.w1 = nn.Parameter(scale * torch.rand(2, num_blocks, bs, bs * f))
        self.b1 = nn.Parameter(scale * torch.rand(2, num_blocks, bs * f))
        self.w2 = nn.Parameter(scale * torch.rand(2, num_blocks, bs * f, bs))
        self.b2 = nn.Parameter(scale * torch.rand(2, num_blocks, bs))

    def _kept(self, spatial: Sequence[int], last_freq: int) -> list[int]:
        if self.nd == 2:
            k = min(self.modes, spatial[0], spatial[1] // 2 + 1)
            return [k, k]
        return [min(self.modes, spatial[0]), min(self.modes, spatial[1]), min(self.temporal_modes, last_freq)]

    def forward(self, x: Tensor) -> Tensor:
        nd = self.nd
        if not torch.compiler.is_compiling() and x.ndim != nd + 2:
            raise ValueError(f"Expected {nd + 2}D tensor, got shape {tuple(x.shape)}")
        if self.channel_first:
            x = x.permute(0, *range(2, nd + 2), 1)
        b, *spatial, c = x.shape
        dims = tuple(range(1, nd + 1))
        xf = torch.fft.rfftn(x.float(), dim=dims, norm="ortho")
        kept = self._kept(spatial, xf.shape[nd])
        corner = xf[(slice(None), *[slice(0, k) for k in kept])]
        corner = corner.reshape(*corner.shape[:-1], self.num_blocks, self.block_size)
        w1, w2 = torch.complex(self.w1[0], self.w1[1]), torch.complex(self.w2[0], self.w2[1])
        b1, b2 = torch.complex(self.b1[0], self.b1[1]), torch.complex(self.b2[0], self.b2[1])
        h = torch.einsum("...bi,bio->...bo", corner, w1) + b1
        h = torch.complex(self.act(h.real), self.act(h.imag))
        o = (torch.einsum("...bi,bio->...bo", h, w2) + b2).reshape(*corner.shape[:-2], c)
        pad = [0, 0]
        for k, full in zip(reversed(kept), reversed(xf.shape[1:nd + 1])):
            pad += [0, full - k]
        o = torch.view_as_complex(F.pad(torch.view_as_real(o), [0, 0] + pad))
        out = torch.fft.irfftn(o, s=tuple(spatial), dim=dims, norm="ortho").to(x.dtype) + x
        return out.permute(0, nd + 1, *range(1, nd + 1)) if self.channel_first else out


class DPOT2DLayer(_FourierMixer):
    nd = 2


class AFNO3DLayer(_FourierMixer):
    nd = 3

    def __init__(self, width: int = 32, num_blocks: int = 8, modes: int = 32, temporal_modes: int = 8,
                 hidden_size_factor: int = 1, activation: str = "gelu", channel_first: bool = True,
                 sparsity_threshold: float = 0.01):
        super().__init__(width, num_blocks, sparsity_threshold, modes, hidden_size_factor, channel_first, activation,
                         temporal_modes)


class _ConvMlp(nn.Module):
    nd = 2

    def __init__(self, width: int, mlp_ratio: float = 1.0, activation: str = "gelu"):
        super().__init__()
        hidden = int(width * mlp_ratio)
        self.act = get_activation(activation)
        self.fc1 = _CONV[self.nd](width, hidden, kernel_size=1)
        self.fc2 = _CONV[self.nd](hidden, width, kernel_size=1)

    def forward(self, x: Tensor) -> Tensor:
        return self.fc2(self.act(self.fc1(x)))


class ConvMlp(_ConvMlp):
    nd = 2


class ConvMlp3D(_ConvMlp):
    nd = 3


class _Block(nn.Module):
    nd = 2

    def __init__(self, width: int, num_blocks: int, mlp_ratio: float, modes: int, temporal_modes: int | None = None,
                 activation: str = "gelu", double_skip: bool = True, norm_groups: int = 8):
        super().__init__()
        self.norm1 = nn.GroupNorm(norm_groups, width)
        if self.nd == 2:
            self.filter = DPOT2DLayer(width=width, num_blocks=num_blocks, modes=modes, channel_first=True, activation=activation)
            self.mlp = ConvMlp(width=width, mlp_ratio=mlp_ratio, activation=activation)
        else:
            self.filter = AFNO3DLayer(width=width, num_blocks=num_blocks, modes=modes, temporal_modes=temporal_modes,
                                      channel_first=True, activation=activation)
            self.mlp = ConvMlp3D(width=width, mlp_ratio=mlp_ratio, activation=activation)
        self.norm2 = nn.GroupNorm(norm_groups, width)
        self.double_skip = double_skip

    def forward(self, x: Tensor) -> Tensor:
        residual = x
        x = self.filter(self.norm1(x))
        if self.double_skip:
            x = x + residual
            residual = x
        return self.mlp(self.norm2(x)) + residual


class Block(_Block):
    nd = 2

    def __init__(self, width, num_blocks, mlp_ratio, modes, activation="gelu", double_skip=True, norm_groups=8):
        super().__init__(width, num_blocks, mlp_ratio, modes, None, activation, double_skip, norm_groups)


class Block3D(_Block):
    nd = 3


class _PatchEmbed(nn.Module):
    nd = 2

    def __init__(self, inp_shape, patch_size, in_chans: int, embed_dim: int, out_dim: int, activation: str = "gelu"):
        super().__init__()
        self.inp_shape, self.patch_size = _tuple(inp_shape, self.nd), _tuple(patch_size, self.nd)
        self.out_size = tuple(s // p for s, p in zip(self.inp_shape, self.patch_size))
        self.act = get_activation(activation)
        conv = _CONV[self.nd]
        self.proj = nn.Sequential(conv(in_chans, embed_dim, kernel_size=self.patch_size, stride=self.patch_size), self.act,
                                  conv(embed_dim, out_dim, kernel_size=1))

    def forward(self, x: Tensor) -> Tensor:
        if tuple(x.shape[2:]) != self.inp_shape:
            raise ValueError(f"Input size {tuple(x.shape[2:])} doesn't match model {self.inp_shape}.")
        return self.proj(x)


class PatchEmbed(_PatchEmbed):
    nd = 2


class PatchEmbed3D(_PatchEmbed):
    nd = 3


class TimeAggregator(nn.Module):
    """Collapse the time axis of ``[..., T, C]`` with per-step channel mixing (optionally cosine-modulated)."""

    def __init__(self, in_channels: int, in_timesteps: int, embed_dim: int, mode: Literal["mlp", "exp_mlp"] = "exp_mlp"):
        super().__init__()
        if mode not in ("mlp", "exp_mlp"):
            raise ValueError(f"Unsupported TimeAggregator mode: {mode}")
        self.mode = mode
        self.w = nn.Parameter(torch.randn(in_timesteps, embed_dim, embed_dim) / (in_timesteps * embed_dim ** 0.5))
        if mode == "exp_mlp":
            self.gamma = nn.Parameter(2 ** torch.linspace(-10, 10, embed_dim).unsqueeze(0))

    def forward(self, x: Tensor) -> Tensor:
        if self.mode == "exp_mlp":
            t = torch.linspace(0, 1, x.shape[-2], device=x.device).unsqueeze(-1)
            x = x * torch.cos(t @ self.gamma).to(x.dtype)
        return torch.einsum("tij,...ti->...j", self.w.to(x.dtype), x)


@dataclass
class DPOTMeta(ModelMetaData):
    name: str = "DPOTNet"
    jit: bool = False
    amp: bool = True
    cuda_graphs: bool = False


@dataclass
class DPOT3DMeta(ModelMetaData):
    name: str = "DPOTNet3D"
    jit: bool = False
    amp: bool = True
    cuda_graphs: bool = False


class _DPOTBase(Module):
    nd = 2

    def __init__(self, meta, inp_shape, patch_size, mixing_type, in_channels, out_channels, in_timesteps, out_timesteps,
                 num_blocks, embed_dim, out_layer_dim, depth, modes, temporal_modes, mlp_ratio, normalize, activation,
                 time_agg, norm_groups):
        super().__init__(meta=meta)
        if mixing_type != "afno":
            raise ValueError("Currently only 'afno' mixing_type is supported.")
        nd = self.nd
        self.inp_shape, self.patch_size = _tuple(inp_shape, nd), _tuple(patch_size, nd)
        self.in_channels, self.out_channels = in_channels, out_channels
        self.in_timesteps, self.out_timesteps = in_timesteps, out_timesteps
        self.normalize, self.activation, self.embed_dim = normalize, activation, embed_dim
        extra = nd + 1                                    # coordinate channels: space + time
        embed_cls = PatchEmbed if nd == 2 else PatchEmbed3D
        self.patch_embed = embed_cls(inp_shape=inp_shape, patch_size=patch_size, in_chans=in_channels + extra,
                                     embed_dim=out_channels * max(self.patch_size) + extra, out_dim=embed_dim,
                                     activation=activation)
        self.pos_embed = nn.Parameter(torch.zeros(1, embed_dim, *self.patch_embed.out_size))
        if normalize:
            self.scale_mu = nn.Linear(2 * in_channels, embed_dim)
            self.scale_sigma = nn.Linear(2 * in_channels, embed_dim)
        self.time_agg_layer = TimeAggregator(in_channels=in_channels, in_timesteps=in_timesteps, embed_dim=embed_dim,
                                             mode=time_agg)
        if nd == 2:
            blocks = [Block(width=embed_dim, num_blocks=num_blocks, mlp_ratio=mlp_ratio, modes=modes, activation=activation,
                            double_skip=False, norm_groups=norm_groups) for _ in range(depth)]
        else:
            blocks = [Block3D(width=embed_dim, num_blocks=num_blocks, mlp_ratio=mlp_ratio, modes=modes,
                              temporal_modes=temporal_modes, activation=activation, double_skip=False,
                              norm_groups=norm_groups) for _ in range(depth)]
        self.blocks = nn.ModuleList(blocks)
        self.act = get_activation(activation)
        conv = _CONV[nd]
        self.reconstruct = nn.Sequential(
            _CONVT[nd](in_channels=embed_dim, out_channels=out_layer_dim, kernel_size=patch_size, stride=patch_size), self.act,
            conv(out_layer_dim, out_layer_dim, kernel_size=1), self.act,
            conv(out_layer_dim, out_channels * out_timesteps, kernel_size=1))
        nn.init.trunc_normal_(self.pos_embed, std=0.02)
        self.apply(self._init_weights)

    def _init_weights(self, m: nn.Module) -> None:
        if isinstance(m, (nn.Linear, _CONV[self.nd], _CONVT[self.nd])):
            nn.init.trunc_normal_(m.weight, std=0.02)
            if m.bias is not None:
                nn.init.constant_(m.bias, 0)
        elif isinstance(m, nn.LayerNorm):
            nn.init.constant_(m.bias, 0)
            nn.init.constant_(m.weight, 1.0)

    @staticmethod
    def _build_grid(x: Tensor) -> Tensor:
        """Normalised coordinates of every axis between batch and channel: ``[B, *axes, n_axes]``."""
        b, *axes, _ = x.shape
        coords = []
        for i, n in enumerate(axes):
            shape = [1] * (len(axes) + 2)
            shape[i + 1] = n
            coords.append(torch.linspace(0, 1, n, device=x.device, dtype=x.dtype).view(shape).expand(b, *axes, 1))
        return torch.cat(coords, dim=-1)

    def forward(self, x: Tensor) -> Tensor:
        nd = self.nd
        b, *spatial, t, c = x.shape
        if t != self.in_timesteps or c != self.in_channels:
            raise ValueError(f"Input has shape T={t}, C={c}; expected T={self.in_timesteps}, C={self.in_channels}.")
        red = tuple(range(1, nd + 2))
        if self.normalize:
            mu = x.mean(dim=red, keepdim=True)
            sigma = x.std(dim=red, keepdim=True) + 1e-6
            xn = (x - mu) / sigma
        else:
            mu = sigma = None
            xn = x
        feat = torch.cat([xn, self._build_grid(xn)], dim=-1)                                  # [B, *S, T, C + nd + 1]
        feat = feat.permute(0, nd + 1, nd + 2, *range(1, nd + 1)).reshape(b * t, -1, *spatial)  # [(B T), C', *S]
        feat = self.patch_embed(feat) + self.pos_embed
        sp = feat.shape[2:]
        feat = feat.reshape(b, t, self.embed_dim, *sp).permute(0, *range(3, nd + 3), 1, 2)   # [B, *S', T, E]
        feat = self.time_agg_layer(feat).permute(0, nd + 1, *range(1, nd + 1))                # [B, E, *S']
        if self.normalize:
            stats = torch.cat([mu, sigma], dim=-1)
            to_cf = lambda v: v.squeeze(-2).permute(0, nd + 1, *range(1, nd + 1))  # noqa: E731
            feat = to_cf(self.scale_sigma(stats)) * feat + to_cf(self.scale_mu(stats))
        for blk in self.blocks:
            feat = blk(feat)
        y = self.reconstruct(feat).permute(0, *range(2, nd + 2), 1)
        y = y.reshape(b, *spatial, self.out_timesteps, self.out_channels)
        return y * sigma + mu if self.normalize else y

    def extra_repr(self) -> str:
        return (f"in_channels={self.in_channels}, out_channels={self.out_channels}, in_timesteps={self.in_timesteps}, "
                f"out_timesteps={self.out_timesteps}, embed_dim={self.embed_dim}, depth={len(self.blocks)}")


class DPOTNet(_DPOTBase):
    """``forward(x [B, H, W, T_in, C_in]) -> [B, H, W, T_out, C_out]``."""

    nd = 2

    def __init__(self, inp_shape: int = 224, patch_size: int = 16, mixing_type: Literal["afno"] = "afno",
                 in_channels: int = 1, out_channels: int = 4, in_timesteps: int = 1, out_timesteps: int = 1,
                 num_blocks: int = 4, embed_dim: int = 768, out_layer_dim: int = 32, depth: int = 12, modes: int = 32,
                 mlp_ratio: float = 1.0, normalize: bool = False, activation: str = "gelu",
                 time_agg: Literal["mlp", "exp_mlp"] = "exp_mlp", norm_groups: int = 8):
        super().__init__(DPOTMeta(), inp_shape, patch_size, mixing_type, in_channels, out_channels, in_timesteps,
                         out_timesteps, num_blocks, embed_dim, out_layer_dim, depth, modes, None, mlp_ratio, normalize,
                         activation, time_agg, norm_groups)


class DPOTNet3D(_DPOTBase):
    """``forward(x [B, X, Y, Z, T_in, C_in]) -> [B, X, Y, Z, T_out, C_out]``."""

    nd = 3

    def __init__(self, inp_shape: int = 224, patch_size: int = 16, mixing_type: Literal["afno"] = "afno",
                 in_channels: int = 1, out_channels: int = 3, in_timesteps: int = 1, out_timesteps: int = 1,
                 num_blocks: int = 4, embed_dim: int = 768, out_layer_dim: int = 32, depth: int = 12, modes: int = 32,
                 temporal_modes: int = 8, mlp_ratio: float = 1.0, normalize: bool = False, activation: str = "gelu",
                 time_agg: Literal["mlp", "exp_mlp"] = "exp_mlp", norm_groups: int = 8):
        super().__init__(DPOT3DMeta(), inp_shape, patch_size, mixing_type, in_channels, out_channels, in_timesteps,
                         out_timesteps, num_blocks, embed_dim, out_layer_dim, depth, modes, temporal_modes, mlp_ratio,
                         normalize, activation, time_agg, norm_groups)


def resize_pos_embed(pos_embed: Tensor, new_pos_embed: Tensor) -> Tensor:
    if pos_embed.shape == new_pos_embed.shape:
        return pos_embed
    mode = "bilinear" if pos_embed.ndim == 4 else "trilinear"
    return F.interpolate(pos_embed, size=tuple(new_pos_embed.shape[2:]), mode=mode, align_corners=False)


def checkpoint_filter_fn(state_dict: dict, model: _DPOTBase) -> dict:
    """Adapt a checkpoint's positional embedding to the model's patch grid."""
    return {k: resize_pos_embed(v, model.pos_embed) if k == "pos_embed" and v.shape != model.pos_embed.shape else v
            for k, v in state_dict.items()}

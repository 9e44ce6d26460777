"""Layers of the Strata 3-D transformers: windowed / global / column attention, transformer blocks, patch embedding,
output head, and the pixel-stage block with per-pixel adaptive layer norm.

Counterpart of ``physicsnemo/experimental/models/strata/layers.py`` (``Natten3DSelfAttention`` :89,
``StrataTransformer3DBlock`` :291, ``PatchEmbed3D`` :399, ``FinalLayer3D`` :473, ``DepthwiseConv`` :614,
``StrataPixel3DBlock`` :691); parameter names are the same.

Device notes: 3-D neighbourhood attention runs on this package's own CUDA kernels (``nn.functional.na3d``); the patch
embedding is a GEMM on the unfolded patches that writes the token matrix ``[B, N, E]`` directly (no convolution output
to transpose); the 5x5 depthwise conditioning filter is applied in batch slices when the tensor exceeds 32-bit
indexing.
"""

from __future__ import annotations

from typing import Literal, Optional, Tuple, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from ....nn.functional.natten import na3d
from ....nn.module.mlp_layers import Mlp
from ....nn.module.rope import apply_rotary_pos_emb

__all__ = ["Natten3DSelfAttention", "StrataTransformer3DBlock", "StrataPixel3DBlock", "PatchEmbed3D", "FinalLayer3D", "RopeTables",
           "DepthwiseConv"]

RopeTables = Tuple[torch.Tensor, torch.Tensor]
_INT32_MAX = 2 ** 31 - 1


def _as_kernel_triple(attn_kernel: Union[int, Tuple[int, int, int]]) -> Tuple[int, int, int]:
    if isinstance(attn_kernel, int):
        return (attn_kernel,) * 3
    kernel = tuple(attn_kernel)
    if len(kernel) != 3:
        raise ValueError(f"attn_kernel tuple must have length 3 (kd, kh, kw); got {attn_kernel}")
    return kernel


class Natten3DSelfAttention(nn.Module):
    """Multi-head self attention over ``(d, h, w)`` tokens: global (``attn_kernel=-1``), neighbourhood
    (``attn_kernel=k`` or ``(kd, kh, kw)``), or along the vertical column of every ``(h, w)`` site
    (``do_depthwise_attention``); optional RMS norm of q / k, rotary embedding and sigmoid output gate."""

    def __init__(self, dim: int, num_heads: int = 8, qkv_bias: bool = False, qk_norm: bool = False, qk_norm_affine: bool = False,
                 attn_drop_rate: float = 0.0, proj_drop_rate: float = 0.0, attn_kernel: Union[int, Tuple[int, int, int]] = -1,
                 do_depthwise_attention: bool = False, na_dilation: int = 1, gated_attention: bool = False,
                 na3d_backend: Optional[str] = None):
        super().__init__()
        if dim % num_heads != 0:
            raise ValueError(f"dim ({dim}) must be divisible by num_heads ({num_heads})")
        _as_kernel_triple(attn_kernel)
        self.num_heads, self.head_dim = num_heads, dim // num_heads
        self.scale = self.head_dim ** -0.5
        self.attn_drop_rate, self.attn_kernel, self.na_dilation = attn_drop_rate, attn_kernel, na_dilation
        self.do_depthwise_attention, self.gated_attention, self.na3d_backend = do_depthwise_attention, gated_attention, na3d_backend
        self.qkv = nn.Linear(dim, dim * 3, bias=qkv_bias)
        norm = lambda: nn.RMSNorm(self.head_dim, elementwise_affine=qk_norm_affine, eps=1e-6) if qk_norm else nn.Identity()  # noqa: E731
        self.q_norm, self.k_norm = norm(), norm()
        self.proj = nn.Linear(dim, dim)
        self.proj_drop = nn.Dropout(proj_drop_rate) if proj_drop_rate > 0.0 else nn.Identity()
        self.gate_proj = nn.Linear(dim, dim) if gated_attention else nn.Identity()

    def forward(self, x: torch.Tensor, latent_dhw: Optional[Tuple[int, int, int]] = None,
                rope_tables: Optional[RopeTables] = None) -> torch.Tensor:
        B, N, C = x.shape
        H, hd = self.num_heads, self.head_dim
        q, k, v = self.qkv(x).view(B, N, 3, H, hd).unbind(2)                 # [B, N, H, hd] views
        q, k = self.q_norm(q), self.k_norm(k)
        if rope_tables is not None:
            cos, sin = (t.unsqueeze(-2) if t.dim() == 2 else t.transpose(1, 2) for t in rope_tables)   # -> [.., N, 1, hd]
            q, k = apply_rotary_pos_emb(q, cos, sin), apply_rotary_pos_emb(k, cos, sin)
        q, k = q.to(v.dtype), k.to(v.dtype)
        p = self.attn_drop_rate if self.training else 0.0
        local = self.do_depthwise_attention or self.attn_kernel != -1
        if local and not torch.compiler.is_compiling():
            if latent_dhw is None:
                raise ValueError("depth-axis attention requires latent_dhw" if self.do_depthwise_attention
                                 else "neighborhood attention requires latent_dhw")
            if N != latent_dhw[0] * latent_dhw[1] * latent_dhw[2]:
                raise ValueError(f"Expected N == D*H*W for latent_dhw={latent_dhw}, got N={N}")
        if self.do_depthwise_attention:
            d = latent_dhw[0]
            col = lambda t: t.reshape(B, d, N // d, H, hd).permute(0, 2, 3, 1, 4).reshape(B * (N // d), H, d, hd)  # noqa: E731
            o = F.scaled_dot_product_attention(col(q), col(k), col(v), dropout_p=p, scale=self.scale)
            out = o.reshape(B, N // d, H, d, hd).permute(0, 3, 1, 2, 4).reshape(B, N, C)
        elif self.attn_kernel == -1:
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), dropout_p=p, scale=self.scale)
            out = o.transpose(1, 2).reshape(B, N, C)
        else:
            grid = lambda t: t.reshape(B, *latent_dhw, H, hd)  # noqa: E731
            out = na3d(grid(q), grid(k), grid(v), _as_kernel_triple(self.attn_kernel), dilation=self.na_dilation,
                       is_causal=False).reshape(B, N, C)
        if self.gated_attention:
            out = out * torch.sigmoid(self.gate_proj(x))
        return self.proj_drop(self.proj(out))


class StrataTransformer3DBlock(nn.Module):
    """Pre-norm transformer block (parameter-free layer norms): ``x + attn(norm(x))``, ``x + mlp(norm(x))``."""

    def __init__(self, dim: int, num_heads: int, mlp_ratio: float = 4.0, qkv_bias: bool = True, qk_norm: bool = False,
                 qk_norm_affine: bool = False, mlp_drop_rate: float = 0.0, attn_drop_rate: float = 0.0,
                 attn_kernel: Union[int, Tuple[int, int, int]] = -1, do_depthwise_attention: bool = False, na_dilation: int = 1,
                 gated_attention: bool = False, na3d_backend: Optional[str] = None):
        super().__init__()
        self.do_depthwise_attention = do_depthwise_attention
        self.norm1 = nn.LayerNorm(dim, elementwise_affine=False, eps=1e-6)
        self.norm2 = nn.LayerNorm(dim, elementwise_affine=False, eps=1e-6)
        self.attn = Natten3DSelfAttention(dim, num_heads=num_heads, qkv_bias=qkv_bias, qk_norm=qk_norm, qk_norm_affine=qk_norm_affine,
                                          attn_drop_rate=attn_drop_rate, proj_drop_rate=mlp_drop_rate, attn_kernel=attn_kernel,
                                          do_depthwise_attention=do_depthwise_attention, na_dilation=na_dilation,
                                          gated_attention=gated_attention, na3d_backend=na3d_backend)
        self.mlp = Mlp(in_features=dim, hidden_features=int(dim * mlp_ratio), out_features=dim, act_layer=nn.GELU, drop=mlp_drop_rate)

    def forward(self, x, latent_dhw=None, rope_tables=None):
        x = x + self.attn(self.norm1(x), latent_dhw=latent_dhw, rope_tables=rope_tables)
        return x + self.mlp(self.norm2(x))


class PatchEmbed3D(nn.Module):
    """Non-overlapping ``(pd, ph, pw)`` patches to ``embed_dim`` features.  ``forward`` returns the convolution layout
    ``[B, E, d, h, w]``; ``tokens`` returns ``([B, d*h*w, E], (d, h, w))`` from one GEMM on the unfolded patches."""

    def __init__(self, depth: int, height: int, width: int, patch_size: Union[int, Tuple[int, int, int]] = 16, in_chans: int = 3,
                 embed_dim: int = 768):
        super().__init__()
        patch_size = (patch_size,) * 3 if isinstance(patch_size, int) else tuple(patch_size)
        for extent, p, what, kind in ((depth, patch_size[0], "Depth", "vertical"), (height, patch_size[1], "Height", "horizontal"),
                                      (width, patch_size[2], "Width", "horizontal")):
            if extent % p != 0:
                raise ValueError(f"{what} ({extent}) must be divisible by {kind} patch size ({p})")
        self.depth, self.height, self.width, self.patch_size = depth, height, width, patch_size
        self.num_patches = (depth // patch_size[0]) * (height // patch_size[1]) * (width // patch_size[2])
        self.proj = nn.Conv3d(in_chans, embed_dim, kernel_size=patch_size, stride=patch_size, bias=True)

    def tokens(self, x: torch.Tensor):
        B, C, D, Hh, W = x.shape
        pd, ph, pw = self.patch_size
        d, h, w = D // pd, Hh // ph, W // pw
        rows = x.reshape(B, C, d, pd, h, ph, w, pw).permute(0, 2, 4, 6, 1, 3, 5, 7).reshape(B, d * h * w, C * pd * ph * pw)
        wt = self.proj.weight.reshape(self.proj.out_channels, -1)
        return F.linear(rows, wt.to(rows.dtype), self.proj.bias.to(rows.dtype)), (d, h, w)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        t, (d, h, w) = self.tokens(x)
        return t.transpose(1, 2).reshape(x.shape[0], -1, d, h, w)


class FinalLayer3D(nn.Module):
    """Parameter-free layer norm (always fp32) followed by a linear head."""

    def __init__(self, hidden_size: int, out_features: int):
        super().__init__()
        self.norm = nn.LayerNorm(hidden_size, elementwise_affine=False, eps=1e-6)
        self.linear = nn.Linear(hidden_size, out_features)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        with torch.autocast(device_type=x.device.type, enabled=False):
            return self.linear(self.norm(x.float()).to(self.linear.weight.dtype))


class DepthwiseConv(nn.Conv2d):
    """Depthwise 2-D convolution; with ``chunk_size`` the batch is processed in slices of that many samples, which
    keeps every call below the 32-bit indexing limit of the convolution kernels."""

    def __init__(self, channels: int, *args, chunk_size: Optional[int] = None, **kwargs):
        if "groups" in kwargs:
            raise ValueError("DepthwiseConv does not accept a groups argument")
        super().__init__(channels, channels, *args, **kwargs, groups=channels)
        self.chunk_size = chunk_size

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.chunk_size is None or x.numel() <= _INT32_MAX and x.shape[0] <= self.chunk_size:
            return super().forward(x)
        per = max(1, min(self.chunk_size, _INT32_MAX // max(1, x[0].numel())))
        return torch.cat([super(DepthwiseConv, self).forward(part) for part in x.split(per, dim=0)], dim=0)


class StrataPixel3DBlock(nn.Module):
    """Transformer block at pixel resolution whose two layer norms are modulated (shift, scale, gate) per pixel by
    the backbone tokens: either every token emits the parameters of all pixels of its patch (``pixel_proj``), or the
    tokens are interpolated to the pixel grid, filtered by a 5x5 depthwise convolution, RMS-normalised and projected
    (``bilinear_dw``).  Both projections start at zero, so the block starts as the identity."""

    def __init__(self, dim: int, cond_dim: int, pixels_per_patch: int, num_heads: int, mlp_ratio: float = 4.0, qkv_bias: bool = True,
                 qk_norm: bool = False, qk_norm_affine: bool = False, mlp_drop_rate: float = 0.0, attn_drop_rate: float = 0.0,
                 attn_kernel: Union[int, Tuple[int, int, int]] = -1, na_dilation: int = 1, gated_attention: bool = False,
                 na3d_backend: Optional[str] = None, adaln_mode: Literal["pixel_proj", "bilinear_dw"] = "pixel_proj",
                 chunk_size_grouped_conv: int = 2, use_chunked_depthwise_conv: bool = True):
        super().__init__()
        if adaln_mode not in ("pixel_proj", "bilinear_dw"):
            raise ValueError(f"adaln_mode must be 'pixel_proj' or 'bilinear_dw'; got {adaln_mode!r}")
        self.adaln_mode, self.num_adaln_params = adaln_mode, 6
        self.attn = Natten3DSelfAttention(dim, num_heads=num_heads, qkv_bias=qkv_bias, qk_norm=qk_norm, qk_norm_affine=qk_norm_affine,
                                          attn_drop_rate=attn_drop_rate, proj_drop_rate=mlp_drop_rate, attn_kernel=attn_kernel,
                                          do_depthwise_attention=False, na_dilation=na_dilation, gated_attention=gated_attention,
                                          na3d_backend=na3d_backend)
        self.norm1 = nn.LayerNorm(dim, elementwise_affine=False, eps=1e-6)
        self.norm2 = nn.LayerNorm(dim, elementwise_affine=False, eps=1e-6)
        self.mlp = Mlp(in_features=dim, hidden_features=int(dim * mlp_ratio), out_features=dim, act_layer=nn.GELU, drop=mlp_drop_rate)
        if adaln_mode == "bilinear_dw":
            kw = dict(kernel_size=(5, 5), padding=(2, 2), bias=True, padding_mode="replicate")
            self.adaln_bilinear_dw_conv = (DepthwiseConv(cond_dim, chunk_size=chunk_size_grouped_conv, **kw) if use_chunked_depthwise_conv
                                           else nn.Conv2d(cond_dim, cond_dim, groups=cond_dim, **kw))
            with torch.no_grad():                                       # start as the identity filter
                self.adaln_bilinear_dw_conv.weight.zero_()
                self.adaln_bilinear_dw_conv.weight[:, 0, 2, 2] = 1.0
                self.adaln_bilinear_dw_conv.bias.zero_()
            self.adaln_bilinear_dw_norm = nn.RMSNorm(cond_dim, elementwise_affine=False)
            self.adaln_bilinear_dw_proj = nn.Linear(cond_dim, self.num_adaln_params * dim)
        else:
            self.pixels_per_patch = pixels_per_patch
            self.adaln_pixel_proj = nn.Sequential(nn.SiLU(), nn.Linear(cond_dim, pixels_per_patch * self.num_adaln_params * dim))
        self.reset_adaln_zero()

    def reset_adaln_zero(self) -> None:
        for lin in (getattr(self, "adaln_bilinear_dw_proj", None), getattr(self, "adaln_pixel_proj", [None])[-1]):
            if lin is not None:
                nn.init.zeros_(lin.weight)
                nn.init.zeros_(lin.bias)

    @staticmethod
    def _expand_cond_to_pixels(raw: torch.Tensor, pixel_dhw, backbone_dhw) -> torch.Tensor:
        """``[B, tokens, (pv ph pw m)] -> [B, pixels, m]``: every token scatters the parameters of its own patch."""
        (d, h, w), (sd, sh, sw) = pixel_dhw, backbone_dhw
        pv, ph, pw = d // sd, h // sh, w // sw
        t = raw.reshape(raw.shape[0], sd, sh, sw, pv, ph, pw, -1).permute(0, 1, 4, 2, 5, 3, 6, 7)
        return t.reshape(raw.shape[0], d * h * w, -1)

    @staticmethod
    def precompute_bilinear_cond(backbone_cond: torch.Tensor, pixel_dhw, backbone_dhw) -> torch.Tensor:
        """Backbone tokens interpolated to the pixel grid, ``[B, d, C, h, w]`` (shared by all pixel blocks)."""
        (d, h, w), (sd, sh, sw) = pixel_dhw, backbone_dhw
        B, _, C = backbone_cond.shape
        vol = backbone_cond.reshape(B, sd, sh, sw, C)
        if d == sd:
            planes = F.interpolate(vol.permute(0, 1, 4, 2, 3).reshape(B * sd, C, sh, sw), size=(h, w), mode="bilinear", align_corners=False)
            return planes.reshape(B, sd, C, h, w)
        return F.interpolate(vol.permute(0, 4, 1, 2, 3), size=(d, h, w), mode="trilinear", align_corners=False).transpose(1, 2)

    def _bilinear_dw_params(self, s: torch.Tensor):
        B, d, C, h, w = s.shape
        y = self.adaln_bilinear_dw_conv(s.reshape(B * d, C, h, w))
        y = self.adaln_bilinear_dw_norm(y.permute(0, 2, 3, 1)).reshape(B, d * h * w, C)
        return self.adaln_bilinear_dw_proj(F.gelu(y)).reshape(B, d * h * w, self.num_adaln_params, -1).unbind(dim=-2)

    def forward(self, x: torch.Tensor, backbone_cond: torch.Tensor, pixel_dhw, backbone_dhw, s_cond_bilinear: Optional[torch.Tensor] = None,
                rope_tables: Optional[RopeTables] = None) -> torch.Tensor:
        if self.adaln_mode == "bilinear_dw":
            if s_cond_bilinear is None:
                raise ValueError("s_cond_bilinear is required when adaln_mode='bilinear_dw'")
            shift1, scale1, gate1, shift2, scale2, gate2 = self._bilinear_dw_params(s_cond_bilinear)
        else:
            params = self._expand_cond_to_pixels(self.adaln_pixel_proj(backbone_cond), pixel_dhw, backbone_dhw)
            shift1, scale1, gate1, shift2, scale2, gate2 = params.chunk(self.num_adaln_params, dim=-1)
        x = x + gate1 * self.attn(torch.addcmul(shift1, self.norm1(x), 1 + scale1), latent_dhw=pixel_dhw, rope_tables=rope_tables)
        return x + gate2 * self.mlp(torch.addcmul(shift2, self.norm2(x), 1 + scale2))

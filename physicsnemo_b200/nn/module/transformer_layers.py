"""Earth-specific shifted-window transformer blocks (Pangu-Weather / FengWu / SwinRNN building blocks).

Parity: ``physicsnemo/nn/module/transformer_layers.py`` — ``Transformer3DBlock`` / ``Transformer2DBlock``
(pad → cyclic shift → longitude-major window partition → ``EarthAttention`` → reverse → crop → residual → MLP),
``FuserLayer``, ``EncoderLayer`` / ``DecoderLayer`` (FengWu per-variable encoders / decoders with one down / up
sampling stage and a skip), ``SwinTransformer`` (a plain Swin stage; implemented here because ``timm`` is not a
dependency).
"""
from collections.abc import Sequence

import torch
from torch import nn

from .attention_layers import EarthAttention2D, EarthAttention3D
from .drop import DropPath
from .mlp_layers import Mlp
from .resample_layers import DownSample2D, UpSample2D
from .utils import (PatchEmbed2D, PatchRecovery2D, crop2d, crop3d, get_pad2d, get_pad3d, get_shift_window_mask,
                    window_partition, window_reverse)


def _at(value, i):
    return value[i] if isinstance(value, Sequence) else value


class _EarthBlock(nn.Module):
    _ndim = 3
    _default_window = (2, 6, 12)
    _default_shift = (1, 3, 6)

    def __init__(self, dim, input_resolution, num_heads, window_size=None, shift_size=None, mlp_ratio=4.0, qkv_bias=True,
                 qk_scale=None, drop=0.0, attn_drop=0.0, drop_path=0.0, act_layer=nn.GELU, norm_layer=nn.LayerNorm):
        super().__init__()
        nd = self._ndim
        window_size = self._default_window if window_size is None else window_size
        shift_size = self._default_shift if shift_size is None else shift_size
        self.dim, self.input_resolution, self.num_heads = dim, input_resolution, num_heads
        self.window_size, self.shift_size, self.mlp_ratio = window_size, shift_size, mlp_ratio
        self.norm1 = norm_layer(dim)
        padding = get_pad3d(input_resolution, window_size) if nd == 3 else get_pad2d(input_resolution, window_size)
        self.pad = (nn.ZeroPad3d if nd == 3 else nn.ZeroPad2d)(padding)
        pad_res = list(input_resolution)
        for a in range(nd):  # padding lists the innermost axis first
            pad_res[nd - 1 - a] += padding[2 * a] + padding[2 * a + 1]
        attn_cls = EarthAttention3D if nd == 3 else EarthAttention2D
        self.attn = attn_cls(dim=dim, input_resolution=pad_res, window_size=window_size, num_heads=num_heads,
                             qkv_bias=qkv_bias, qk_scale=qk_scale, attn_drop=attn_drop, proj_drop=drop)
        self.drop_path = DropPath(drop_path) if drop_path > 0.0 else nn.Identity()
        self.norm2 = norm_layer(dim)
        self.mlp = Mlp(in_features=dim, hidden_features=int(dim * mlp_ratio), act_layer=act_layer, drop=drop)
        self.roll = all(bool(s) for s in shift_size)
        mask = get_shift_window_mask(pad_res, window_size, shift_size, ndim=nd) if self.roll else None
        self.register_buffer("attn_mask", mask)

    def forward(self, x: torch.Tensor):
        nd = self._ndim
        B, _, C = x.shape
        res = tuple(self.input_resolution)
        shortcut = x
        x = self.norm1(x).view(B, *res, C)
        x = self.pad(x.movedim(-1, 1)).movedim(1, -1)
        padded = x.shape[1:-1]
        dims = tuple(range(1, nd + 1))
        if self.roll:
            x = torch.roll(x, shifts=tuple(-s for s in self.shift_size), dims=dims)
        win = window_partition(x, self.window_size, ndim=nd)
        n_tok = 1
        for w in self.window_size:
            n_tok *= w
        out = self.attn(win.view(win.shape[0], win.shape[1], n_tok, C), mask=self.attn_mask)
        out = out.view(out.shape[0], out.shape[1], *self.window_size, C)
        names = ("Pl", "Lat", "Lon")[3 - nd:]
        x = window_reverse(out, self.window_size, ndim=nd, **dict(zip(names, padded)))
        if self.roll:
            x = torch.roll(x, shifts=tuple(self.shift_size), dims=dims)
        x = (crop3d if nd == 3 else crop2d)(x.movedim(-1, 1), res).movedim(1, -1).reshape(B, -1, C)
        x = shortcut + self.drop_path(x)
        return x + self.drop_path(self.mlp(self.norm2(x)))


class Transformer3DBlock(_EarthBlock):
    _ndim, _default_window, _default_shift = 3, (2, 6, 12), (1, 3, 6)


class Transformer2DBlock(_EarthBlock):
    _ndim, _default_window, _default_shift = 2, (6, 12), (3, 6)


def _stack(block, n, shift_zero, **kw):
    drop_path = kw.pop("drop_path")
    return nn.ModuleList([block(shift_size=shift_zero if i % 2 == 0 else None, drop_path=_at(drop_path, i), **kw)
                          for i in range(n)])


class FuserLayer(nn.Module):
    """``depth`` 3-D blocks alternating unshifted / shifted windows."""

    def __init__(self, dim, input_resolution, depth, num_heads, window_size, mlp_ratio=4.0, qkv_bias=True, qk_scale=None,
                 drop=0.0, attn_drop=0.0, drop_path=0.0, norm_layer=nn.LayerNorm):
        super().__init__()
        self.dim, self.input_resolution, self.depth = dim, input_resolution, depth
        self.blocks = _stack(Transformer3DBlock, depth, (0, 0, 0), dim=dim, input_resolution=input_resolution,
                             num_heads=num_heads, window_size=window_size, mlp_ratio=mlp_ratio, qkv_bias=qkv_bias,
                             qk_scale=qk_scale, drop=drop, attn_drop=attn_drop, drop_path=drop_path, norm_layer=norm_layer)

    def forward(self, x):
        for blk in self.blocks:
            x = blk(x)
        return x


def _split_cfg(drop_path, num_heads, depth):
    dp_mid = drop_path[depth:] if isinstance(drop_path, Sequence) else drop_path
    dp = drop_path[:depth] if isinstance(drop_path, Sequence) else drop_path
    h, h_mid = (num_heads[0], num_heads[1]) if isinstance(num_heads, Sequence) else (num_heads, num_heads)
    return dp, dp_mid, h, h_mid


class EncoderLayer(nn.Module):
    """Patch embed → 2-D blocks → down-sample → 2-D blocks at twice the width; returns ``(tokens, skip)``."""

    def __init__(self, img_size, patch_size, in_chans, dim, input_resolution, middle_resolution, depth, depth_middle,
                 num_heads, window_size, mlp_ratio=4.0, qkv_bias=True, qk_scale=None, drop=0.0, attn_drop=0.0,
                 drop_path=0.0, norm_layer=nn.LayerNorm):
        super().__init__()
        self.in_chans, self.dim, self.input_resolution = in_chans, dim, input_resolution
        self.depth, self.depth_middle = depth, depth_middle
        dp, dp_mid, h, h_mid = _split_cfg(drop_path, num_heads, depth)
        common = dict(window_size=window_size, mlp_ratio=mlp_ratio, qkv_bias=qkv_bias, qk_scale=qk_scale, drop=drop,
                      attn_drop=attn_drop, norm_layer=norm_layer)
        self.patchembed2d = PatchEmbed2D(img_size=img_size, patch_size=patch_size, in_chans=in_chans, embed_dim=dim)
        self.blocks = _stack(Transformer2DBlock, depth, (0, 0), dim=dim, input_resolution=input_resolution, num_heads=h,
                             drop_path=dp, **common)
        self.downsample = DownSample2D(in_dim=dim, input_resolution=input_resolution, output_resolution=middle_resolution)
        self.blocks_middle = _stack(Transformer2DBlock, depth_middle, (0, 0), dim=dim * 2,
                                    input_resolution=middle_resolution, num_heads=h_mid, drop_path=dp_mid, **common)

    def forward(self, x):
        x = self.patchembed2d(x)
        B, C, Lat, Lon = x.shape
        x = x.reshape(B, C, -1).transpose(1, 2)
        for blk in self.blocks:
            x = blk(x)
        skip = x.reshape(B, Lat, Lon, C)
        x = self.downsample(x)
        for blk in self.blocks_middle:
            x = blk(x)
        return x, skip


class DecoderLayer(nn.Module):
    """Mirror of ``EncoderLayer``: blocks → up-sample → blocks → concat skip → patch recovery."""

    def __init__(self, img_size, patch_size, out_chans, dim, output_resolution, middle_resolution, depth, depth_middle,
                 num_heads, window_size, mlp_ratio=4.0, qkv_bias=True, qk_scale=None, drop=0.0, attn_drop=0.0,
                 drop_path=0.0, norm_layer=nn.LayerNorm):
        super().__init__()
        self.out_chans, self.dim, self.output_resolution = out_chans, dim, output_resolution
        self.depth, self.depth_middle = depth, depth_middle
        dp, dp_mid, h, h_mid = _split_cfg(drop_path, num_heads, depth)
        common = dict(window_size=window_size, mlp_ratio=mlp_ratio, qkv_bias=qkv_bias, qk_scale=qk_scale, drop=drop,
                      attn_drop=attn_drop, norm_layer=norm_layer)
        self.blocks_middle = _stack(Transformer2DBlock, depth_middle, (0, 0), dim=dim * 2,
                                    input_resolution=middle_resolution, num_heads=h_mid, drop_path=dp_mid, **common)
        self.upsample = UpSample2D(in_dim=dim * 2, out_dim=dim, input_resolution=middle_resolution,
                                   output_resolution=output_resolution)
        self.blocks = _stack(Transformer2DBlock, depth, (0, 0), dim=dim, input_resolution=output_resolution, num_heads=h,
                             drop_path=dp, **common)
        self.patchrecovery2d = PatchRecovery2D(img_size, patch_size, 2 * dim, out_chans)

    def forward(self, x, skip):
        B, Lat, Lon, C = skip.shape
        for blk in self.blocks_middle:
            x = blk(x)
        x = self.upsample(x)
        for blk in self.blocks:
            x = blk(x)
        out = torch.cat([x, skip.reshape(B, -1, C)], dim=-1).transpose(1, 2).reshape(B, -1, Lat, Lon)
        return self.patchrecovery2d(out)


# ------------------------------------------------------------------ plain Swin stage
class _SwinWindowAttention(nn.Module):
    def __init__(self, dim, window_size, num_heads):
        super().__init__()
        self.dim, self.window_size, self.num_heads = dim, window_size, num_heads
        wh, ww = window_size
        self.relative_position_bias_table = nn.Parameter(torch.zeros((2 * wh - 1) * (2 * ww - 1), num_heads))
        coords = torch.stack(torch.meshgrid(torch.arange(wh), torch.arange(ww), indexing="ij")).flatten(1)
        rel = (coords[:, :, None] - coords[:, None, :]).permute(1, 2, 0).contiguous()
        rel[:, :, 0] += wh - 1
        rel[:, :, 1] += ww - 1
        rel[:, :, 0] *= 2 * ww - 1
        self.register_buffer("relative_position_index", rel.sum(-1), persistent=False)
        self.qkv = nn.Linear(dim, dim * 3)
        self.proj = nn.Linear(dim, dim)
        nn.init.trunc_normal_(self.relative_position_bias_table, std=0.02)

    def forward(self, x, mask=None):
        B_, N, C = x.shape
        H = self.num_heads
        q, k, v = self.qkv(x).reshape(B_, N, 3, H, C // H).permute(2, 0, 3, 1, 4)
        bias = self.relative_position_bias_table[self.relative_position_index.view(-1)].view(N, N, H).permute(2, 0, 1)[None]
        if mask is not None:
            nW = mask.shape[0]
            bias = (bias + mask[:, None]).repeat(B_ // nW, 1, 1, 1)
        out = torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=bias.to(q.dtype).expand(B_, -1, -1, -1))
        return self.proj(out.transpose(1, 2).reshape(B_, N, C))


class _SwinBlock(nn.Module):
    def __init__(self, dim, input_resolution, num_heads, window_size, shift):
        super().__init__()
        self.res, self.ws = tuple(input_resolution), tuple(window_size)
        self.shift = tuple(0 if r <= w else s for r, w, s in zip(self.res, self.ws, shift))
        self.norm1 = nn.LayerNorm(dim)
        self.attn = _SwinWindowAttention(dim, self.ws, num_heads)
        self.norm2 = nn.LayerNorm(dim)
        self.mlp = Mlp(in_features=dim, hidden_features=4 * dim, act_layer=nn.GELU)
        mask = None
        if any(self.shift):
            H, W = self.res
            lab = torch.zeros(1, H, W, 1)
            cnt = 0
            for hs in (slice(0, -self.ws[0]), slice(-self.ws[0], -self.shift[0] or None), slice(-self.shift[0] or H, None)):
                for wsl in (slice(0, -self.ws[1]), slice(-self.ws[1], -self.shift[1] or None), slice(-self.shift[1] or W, None)):
                    lab[:, hs, wsl, :] = cnt
                    cnt += 1
            win = self._part(lab).reshape(-1, self.ws[0] * self.ws[1])
            diff = win[:, None, :] - win[:, :, None]
            mask = torch.where(diff != 0, torch.full_like(diff, -100.0), torch.zeros_like(diff))
        self.register_buffer("attn_mask", mask, persistent=False)

    def _part(self, x):
        B, H, W, C = x.shape
        wh, ww = self.ws
        return x.view(B, H // wh, wh, W // ww, ww, C).permute(0, 1, 3, 2, 4, 5).reshape(-1, wh, ww, C)

    def forward(self, x):
        B, H, W, C = x.shape
        wh, ww = self.ws
        y = self.norm1(x)
        if any(self.shift):
            y = torch.roll(y, shifts=(-self.shift[0], -self.shift[1]), dims=(1, 2))
        win = self._part(y).reshape(-1, wh * ww, C)
        win = self.attn(win, self.attn_mask).view(B, H // wh, W // ww, wh, ww, C).permute(0, 1, 3, 2, 4, 5).reshape(B, H, W, C)
        if any(self.shift):
            win = torch.roll(win, shifts=self.shift, dims=(1, 2))
        x = x + win
        return x + self.mlp(self.norm2(x))


class SwinTransformer(nn.Module):
    """Zero-pad to a multiple of the window, run ``depth`` Swin blocks (alternating shift), crop back.
    Input / output ``[B, C, Lat, Lon]``."""

    def __init__(self, embed_dim, input_resolution, num_heads, window_size, depth):
        super().__init__()
        ws = (window_size, window_size) if isinstance(window_size, int) else tuple(window_size)
        self.padding = get_pad2d(input_resolution, ws)
        left, right, top, bottom = self.padding
        self.pad = nn.ZeroPad2d(self.padding)
        res = (input_resolution[0] + top + bottom, input_resolution[1] + left + right)
        self.layer = nn.Sequential(*[_SwinBlock(embed_dim, res, num_heads, ws, (0, 0) if i % 2 == 0 else (ws[0] // 2, ws[1] // 2))
                                     for i in range(depth)])

    def forward(self, x):
        left, right, top, bottom = self.padding
        x = self.pad(x)
        H, W = x.shape[2:]
        x = self.layer(x.permute(0, 2, 3, 1)).permute(0, 3, 1, 2)
        return x[:, :, top:H - bottom, left:W - right]

"""Padding of HEALPix faces with the data of their neighbouring faces.

Parity: ``physicsnemo/nn/module/hpx/padding.py`` (``HEALPixPadding``, ``HEALPixPaddingv2``,
``HEALPixFoldFaces``, ``HEALPixUnfoldFaces``).  The 12 faces (4 north, 4 equatorial, 4 south) are padded
with strips of their eight neighbours, rotated where the faces' local axes disagree; the two corners of
an equatorial face that have no neighbour are filled from the two adjacent faces, averaged on the diagonal.

The face-by-face procedure runs ONCE per (face size, padding) on an index image; what the layer executes
is a single gather ``out = ½ (x[idx₀] + x[idx₁])`` over a cached ``[2, 12, n+2p, n+2p]`` index table
(``idx₀ = idx₁`` everywhere except on those averaged diagonals), i.e. one launch instead of about a
hundred slice / rotate / concatenate launches per padded tensor.
"""
from __future__ import annotations

from functools import lru_cache

import torch


class HEALPixFoldFaces(torch.nn.Module):
    """``[B, F, C, H, W] → [B·F, C, H, W]``."""

    def __init__(self, enable_nhwc: bool = False) -> None:
        super().__init__()
        self.enable_nhwc = enable_nhwc

    def forward(self, tensor: torch.Tensor) -> torch.Tensor:
        if not torch.compiler.is_compiling() and tensor.ndim != 5:
            raise ValueError(f"HEALPixFoldFaces.forward requires 5D tensor, got {tensor.shape}")
        b, f, c, h, w = tensor.shape
        out = tensor.reshape(b * f, c, h, w)
        return out.to(memory_format=torch.channels_last) if self.enable_nhwc else out


class HEALPixUnfoldFaces(torch.nn.Module):
    """``[B·F, C, H, W] → [B, F, C, H, W]``."""

    def __init__(self, num_faces: int = 12, enable_nhwc: bool = False) -> None:
        super().__init__()
        self.num_faces, self.enable_nhwc = num_faces, enable_nhwc

    def forward(self, tensor: torch.Tensor) -> torch.Tensor:
        if not torch.compiler.is_compiling():
            if tensor.ndim != 4:
                raise ValueError(f"HEALPixUnfoldFaces.forward requires 4D tensor, got {tensor.shape}")
            if tensor.shape[0] % self.num_faces != 0:
                raise ValueError(f"HEALPixUnfoldFaces.forward invalid batch size: {tensor.shape[0]}")
        bf, c, h, w = tensor.shape
        return tensor.reshape(bf // self.num_faces, self.num_faces, c, h, w)


# ---- the face-adjacency procedure, written for any tensor whose last two axes are a face --------------------------
_D = (-2, -1)


def _north(p, c, t, tl, lft, bl, b, br, rgt, tr):
    mid = torch.cat((t.rot90(1, _D)[..., -p:, :], c, b[..., :p, :]), dim=-2)
    left = torch.cat((tl.rot90(2, _D)[..., -p:, -p:], lft.rot90(-1, _D)[..., -p:], bl[..., :p, -p:]), dim=-2)
    right = torch.cat((tr[..., -p:, :p], rgt[..., :p], br[..., :p, :p]), dim=-2)
    return torch.cat((left, mid, right), dim=-1)


def _equator(p, c, t, tl, lft, bl, b, br, rgt, tr):
    mid = torch.cat((t[..., -p:, :], c, b[..., :p, :]), dim=-2)
    left = torch.cat((tl[..., -p:, -p:], lft[..., -p:], bl[..., :p, -p:]), dim=-2)
    right = torch.cat((tr[..., -p:, :p], rgt[..., :p], br[..., :p, :p]), dim=-2)
    return torch.cat((left, mid, right), dim=-1)


def _south(p, c, t, tl, lft, bl, b, br, rgt, tr):
    mid = torch.cat((t[..., -p:, :], c, b.rot90(1, _D)[..., :p, :]), dim=-2)
    left = torch.cat((tl[..., -p:, -p:], lft[..., -p:], bl[..., :p, -p:]), dim=-2)
    right = torch.cat((tr[..., -p:, :p], rgt.rot90(-1, _D)[..., :p], br.rot90(2, _D)[..., :p, :p]), dim=-2)
    return torch.cat((left, mid, right), dim=-1)


def _corner_tl(p: int, top: torch.Tensor, lft: torch.Tensor) -> torch.Tensor:
    """Missing top-left corner of an equatorial face as index PAIRS ``[2, p, p]`` (averaged where they differ)."""
    a, b = torch.zeros(p, p, dtype=top.dtype), torch.zeros(p, p, dtype=top.dtype)
    a[-1, -1], b[-1, -1] = top[-1, 0], lft[0, -1]
    for i in range(1, p):
        a[-i - 1, -i:] = b[-i - 1, -i:] = top[-i - 1, :i]
        a[-i:, -i - 1] = b[-i:, -i - 1] = lft[:i, -i - 1]
        a[-i - 1, -i - 1], b[-i - 1, -i - 1] = top[-i - 1, 0], lft[0, -i - 1]
    return torch.stack((a, b))


def _corner_br(p: int, bot: torch.Tensor, rgt: torch.Tensor) -> torch.Tensor:
    a, b = torch.zeros(p, p, dtype=bot.dtype), torch.zeros(p, p, dtype=bot.dtype)
    a[0, 0], b[0, 0] = bot[0, -1], rgt[-1, 0]
    for i in range(1, p):
        a[:i, i] = b[:i, i] = rgt[-i:, i]
        a[i, :i] = b[i, :i] = bot[i, -i:]
        a[i, i], b[i, i] = bot[i, -1], rgt[-1, i]
    return torch.stack((a, b))


@lru_cache(maxsize=32)
def padding_index_table(n: int, p: int) -> torch.Tensor:
    """``[2, 12, n+2p, n+2p]`` indices into the flattened ``(face, row, col)`` axes of the unpadded faces."""
    if p > n:
        raise ValueError(f"padding {p} exceeds the face size {n}")
    ids = torch.arange(12 * n * n).reshape(12, n, n)
    f = [ids[k].expand(2, n, n) for k in range(12)]                     # pair images: both entries equal
    sq = lambda t: t if t.dim() == 3 else t.expand(2, *t.shape)  # noqa: E731

    def pad_corner(corner):          # corners come as [2, p, p]; make them full faces so the strips can slice them
        return corner

    out = []
    for k in range(4):               # north faces 0..3
        out.append(_north(p, f[k], f[(k + 1) % 4], f[(k + 2) % 4], f[(k + 3) % 4], f[(k + 3) % 4], f[4 + k], f[8 + k],
                          f[4 + (k + 1) % 4], f[(k + 1) % 4]))
    for k in range(4):               # equatorial faces 4..7
        t, lft, b, rgt = f[k], f[(k + 3) % 4], f[8 + (k + 3) % 4], f[8 + k]
        tl = torch.zeros(2, n, n, dtype=ids.dtype)
        tl[:, -p:, -p:] = _corner_tl(p, t[0], lft[0])
        br = torch.zeros(2, n, n, dtype=ids.dtype)
        br[:, :p, :p] = _corner_br(p, b[0], rgt[0])
        out.append(_equator(p, f[4 + k], t, tl, lft, f[4 + (k + 3) % 4], b, br, rgt, f[4 + (k + 1) % 4]))
    for k in range(4):               # south faces 8..11
        out.append(_south(p, f[8 + k], f[4 + (k + 1) % 4], f[k], f[4 + k], f[8 + (k + 3) % 4], f[8 + (k + 3) % 4],
                          f[8 + (k + 2) % 4], f[8 + (k + 1) % 4], f[8 + (k + 1) % 4]))
    return torch.stack(out, dim=1).contiguous()                          # [2, 12, n+2p, n+2p]


class HEALPixPadding(torch.nn.Module):
    """Pads ``[B·12, C, n, n]`` face tensors to ``[B·12, C, n+2p, n+2p]`` with neighbour data."""

    def __init__(self, padding: int, enable_nhwc: bool = False) -> None:
        super().__init__()
        if not isinstance(padding, int) or padding < 1:
            raise ValueError(f"invalid value for 'padding', expected int > 0 but got {padding}")
        self.p, self.d, self.enable_nhwc = padding, (-2, -1), enable_nhwc
        self.fold = HEALPixFoldFaces(enable_nhwc=enable_nhwc)
        self.unfold = HEALPixUnfoldFaces(num_faces=12, enable_nhwc=enable_nhwc)
        self._tables: dict = {}

    def _table(self, n: int, device) -> torch.Tensor:
        key = (n, str(device))
        if key not in self._tables:
            self._tables[key] = padding_index_table(n, self.p).to(device)
        return self._tables[key]

    def forward(self, data: torch.Tensor) -> torch.Tensor:
        if not torch.compiler.is_compiling() and data.ndim != 4:
            raise ValueError(f"HEALPixPadding.forward requires a 4D tensor, got {data.shape}")
        bf, c, n, _ = data.shape
        if bf % 12:
            raise ValueError(f"HEALPixPadding.forward invalid batch size: {bf}")
        idx = self._table(n, data.device)
        m = n + 2 * self.p
        flat = data.reshape(bf // 12, 12, c, n * n).transpose(1, 2).reshape(bf // 12, c, 12 * n * n)
        a = flat.index_select(-1, idx[0].reshape(-1))
        pair_differs = getattr(self, "_pair_differs", None)
        if pair_differs is None or pair_differs[0] != (n, str(data.device)):
            self._pair_differs = pair_differs = ((n, str(data.device)), bool((idx[0] != idx[1]).any()))
        if pair_differs[1]:
            a = 0.5 * a + 0.5 * flat.index_select(-1, idx[1].reshape(-1))
        out = a.reshape(bf // 12, c, 12, m, m).transpose(1, 2).reshape(bf, c, m, m)
        return out.contiguous(memory_format=torch.channels_last) if self.enable_nhwc else out


class HEALPixPaddingv2(HEALPixPadding):
    """Same result as ``HEALPixPadding`` (the reference's variant calls an external accelerated routine)."""

    def __init__(self, padding: int) -> None:
        super().__init__(padding)
        self.padding = padding

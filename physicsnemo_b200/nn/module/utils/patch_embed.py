"""Patch embedding / recovery convolutions with centred zero padding (parity:
``physicsnemo/nn/module/utils/patch_embed.py``)."""
import torch
from torch import nn


def _pads(sizes, patches):
    """Per-axis (lo, hi) padding that rounds each size up to a multiple of its patch."""
    out = []
    for n, p in zip(sizes, patches):
        total = (p - n % p) % p
        out.append((total // 2, total - total // 2))
    return out


class _PatchEmbed(nn.Module):
    def __init__(self, img_size, patch_size, in_chans, embed_dim, norm_layer=None):
        super().__init__()
        self.img_size = img_size
        nd = len(img_size)
        pads = _pads(img_size, patch_size)
        flat = [v for lo_hi in reversed(pads) for v in lo_hi]          # innermost axis first
        self.pad = (nn.ZeroPad2d if nd == 2 else nn.ZeroPad3d)(tuple(flat))
        self.proj = (nn.Conv2d if nd == 2 else nn.Conv3d)(in_chans, embed_dim, kernel_size=patch_size, stride=patch_size)
        self.norm = norm_layer(embed_dim) if norm_layer is not None else None

    def forward(self, x: torch.Tensor):
        x = self.proj(self.pad(x))
        if self.norm is not None:
            x = self.norm(x.movedim(1, -1)).movedim(-1, 1)
        return x


class PatchEmbed2D(_PatchEmbed):
    pass


class PatchEmbed3D(_PatchEmbed):
    pass


class _PatchRecovery(nn.Module):
    def __init__(self, img_size, patch_size, in_chans, out_chans):
        super().__init__()
        self.img_size = img_size
        conv = nn.ConvTranspose2d if len(img_size) == 2 else nn.ConvTranspose3d
        self.conv = conv(in_chans, out_chans, patch_size, patch_size)

    def forward(self, x):
        out = self.conv(x)
        sl = [slice(None), slice(None)]
        for have, want in zip(out.shape[2:], self.img_size):
            extra = have - want
            sl.append(slice(extra // 2, have - (extra - extra // 2)))
        return out[tuple(sl)]


class PatchRecovery2D(_PatchRecovery):
    pass


class PatchRecovery3D(_PatchRecovery):
    pass

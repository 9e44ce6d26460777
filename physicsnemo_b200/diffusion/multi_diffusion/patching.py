"""2-D patching for patch-based ("multi-diffusion") training and sampling.

Parity: ``physicsnemo/diffusion/multi_diffusion/patching.py`` — ``BasePatching2D`` (``:30``),
``RandomPatching2D`` (``:172``), ``GridPatching2D`` (``:398``), ``image_batching`` (``:645``),
``image_fuse`` (``:772``).  Patch order in the batch dimension is patch-major: ``(P, B)`` flattened
with, for the grid, the x index of the patch varying slowest.  Grid patches overlap by
``overlap_pix`` and carry ``boundary_pix`` of reflected context that is dropped when fusing;
overlaps are averaged.

Patches are extracted by one gather with pre-computed row / column index tables (instead
of ``unfold`` / ``fold``), which also serves integer inputs such as index grids directly.
"""
from __future__ import annotations

import math
import warnings
from abc import ABC, abstractmethod
from typing import Optional, Tuple, Union

import torch
from torch import Tensor


def _gather_patches(x: Tensor, py: Tensor, px: Tensor, hp: int, wp: int) -> Tensor:
    """Patches with top-left corners (py, px): (B, C, H, W) -> (P*B, C, hp, wp), patch-major."""
    B, C = x.shape[:2]
    P = py.numel()
    iy = (py[:, None] + torch.arange(hp, device=x.device))[:, :, None]  # (P, hp, 1)
    ix = (px[:, None] + torch.arange(wp, device=x.device))[:, None, :]  # (P, 1, wp)
    out = x[:, :, iy, ix]                                               # (B, C, P, hp, wp)
    return out.permute(2, 0, 1, 3, 4).reshape(P * B, C, hp, wp)


class BasePatching2D(torch.nn.Module, ABC):
    def __init__(self, img_shape: Tuple[int, int], patch_shape: Tuple[int, int]) -> None:
        super().__init__()
        if len(img_shape) != 2:
            raise ValueError(f"img_shape must be 2D, got {len(img_shape)}D")
        if len(patch_shape) != 2:
            raise ValueError(f"patch_shape must be 2D, got {len(patch_shape)}D")
        if any(p > i for p, i in zip(patch_shape, img_shape)):
            warnings.warn(f"Patch shape {patch_shape} is larger than image shape {img_shape}. "
                          f"Patches will be cropped to fit within the image.")
        self.img_shape = tuple(img_shape)
        self.patch_shape = tuple(min(p, i) for p, i in zip(patch_shape, img_shape))

    def forward(self, input: Tensor, **kwargs) -> Tensor:
        return self.apply(input, **kwargs)

    @abstractmethod
    def apply(self, input: Tensor, *args, **kwargs) -> Tensor: ...

    def fuse(self, input: Tensor, **kwargs) -> Tensor:
        raise NotImplementedError("'fuse' method must be implemented in subclasses.")

    def global_index(self, batch_size: int = 1, device: Union[torch.device, str] = "cpu") -> Tensor:
        """(P, 2, Hp, Wp) integer tensor: global (y, x) of every patch pixel."""
        return self._compute_global_index().to(device)

    def _compute_global_index(self) -> Tensor:
        ny = torch.arange(self.img_shape[0])
        nx = torch.arange(self.img_shape[1])
        grid = torch.stack(torch.meshgrid(ny, nx, indexing="ij"), dim=0).unsqueeze(0)
        dev = getattr(self, "patch_indices", grid).device
        return self.apply(grid.to(dev)).long()


class RandomPatching2D(BasePatching2D):
    """``patch_num`` patches at uniformly random positions (re-drawn by ``reset_patch_indices``)."""

    def __init__(self, img_shape: Tuple[int, int], patch_shape: Tuple[int, int], patch_num: int) -> None:
        super().__init__(img_shape, patch_shape)
        self._patch_num = patch_num
        self.reset_patch_indices()

    @property
    def patch_num(self) -> int:
        return self._patch_num

    def set_patch_num(self, value: int) -> None:
        self._patch_num = value
        self.reset_patch_indices()

    def reset_patch_indices(self, *, generator: Optional[torch.Generator] = None) -> None:
        has = isinstance(getattr(self, "patch_indices", None), Tensor)
        device = self.patch_indices.device if has else None
        max_y = self.img_shape[0] - self.patch_shape[0]
        max_x = self.img_shape[1] - self.patch_shape[1]
        py = torch.randint(0, max_y + 1, (self.patch_num,), dtype=torch.long, device=device, generator=generator)
        px = torch.randint(0, max_x + 1, (self.patch_num,), dtype=torch.long, device=device, generator=generator)
        new = torch.stack([py, px], dim=1)
        if has and new.shape == self.patch_indices.shape:
            self.patch_indices.copy_(new)
        else:
            self.register_buffer("patch_indices", new, persistent=False)

    def apply(self, input: Tensor, additional_input: Optional[Tensor] = None) -> Tensor:
        idx = self.patch_indices.to(input.device)
        out = _gather_patches(input, idx[:, 0], idx[:, 1], *self.patch_shape)
        if additional_input is not None:
            add = torch.nn.functional.interpolate(additional_input, size=self.patch_shape, mode="bilinear")
            out = torch.cat((out, add.repeat(self.patch_num, 1, 1, 1)), dim=1)
        return out

    def forward(self, input: Tensor, additional_input: Optional[Tensor] = None) -> Tensor:
        return self.apply(input, additional_input=additional_input)


def _grid_geometry(img_y, img_x, patch_y, patch_x, overlap_pix, boundary_pix):
    for name, p in (("x", patch_x), ("y", patch_y)):
        if p - overlap_pix - boundary_pix < 1:
            raise ValueError(f"patch_shape_{name} must verify patch_shape_{name} ({p}) >= 1 + overlap_pix "
                             f"({overlap_pix}) + boundary_pix ({boundary_pix})")
        if p <= overlap_pix + 2 * boundary_pix:
            raise ValueError(f"patch_shape_{name} ({p}) must verify patch_shape_{name} ({p}) > overlap_pix "
                             f"({overlap_pix}) + 2 * boundary_pix ({boundary_pix})")
    sx, sy = patch_x - overlap_pix - boundary_pix, patch_y - overlap_pix - boundary_pix
    nx, ny = math.ceil(img_x / sx), math.ceil(img_y / sy)
    pad_x = sx * (nx - 1) + patch_x + boundary_pix
    pad_y = sy * (ny - 1) + patch_y + boundary_pix
    return sx, sy, nx, ny, pad_x, pad_y


def _grid_origins(nx, ny, sx, sy, device):
    ix = torch.arange(nx, device=device).repeat_interleave(ny)  # x index varies slowest
    iy = torch.arange(ny, device=device).repeat(nx)
    return iy * sy, ix * sx


def image_batching(input: Tensor, patch_shape_y: int, patch_shape_x: int, overlap_pix: int, boundary_pix: int,
                   input_interp: Optional[Tensor] = None) -> Tensor:
    """Split (B, C, H, W) into a regular grid of overlapping patches: (P*B, C[+C_add], Hp, Wp)."""
    B, _, H, W = input.shape
    sx, sy, nx, ny, pad_x, pad_y = _grid_geometry(H, W, patch_shape_y, patch_shape_x, overlap_pix, boundary_pix)
    if input_interp is not None:
        if input_interp.shape[0] != B:
            raise ValueError(f"input_interp batch size ({input_interp.shape[0]}) must match input batch size ({B})")
        if input_interp.shape[2] != patch_shape_y or input_interp.shape[3] != patch_shape_x:
            raise ValueError(f"input_interp patch shape ({input_interp.shape[2]}, {input_interp.shape[3]}) must match "
                             f"specified patch shape ({patch_shape_y}, {patch_shape_x})")
    pads = (boundary_pix, pad_x - W - boundary_pix, boundary_pix, pad_y - H - boundary_pix)
    x = input
    as_float = not input.is_floating_point()
    if as_float:
        x = x.double()
    x = torch.nn.functional.pad(x, pads, mode="reflect")
    if as_float:
        x = x.round().to(input.dtype)
    py, px = _grid_origins(nx, ny, sx, sy, input.device)
    out = _gather_patches(x, py, px, patch_shape_y, patch_shape_x)
    if input_interp is not None:
        out = torch.cat((out, input_interp.repeat(nx * ny, 1, 1, 1)), dim=1)
    return out


def image_fuse(input: Tensor, img_shape_y: int, img_shape_x: int, batch_size: int, overlap_pix: int,
               boundary_pix: int, overlap_count: Optional[Tensor] = None) -> Tensor:
    """Inverse of ``image_batching``: average overlapping patch interiors back into (B, C, H, W)."""
    hp, wp = input.shape[2], input.shape[3]
    sx, sy, nx, ny, pad_x, pad_y = _grid_geometry(img_shape_y, img_shape_x, hp, wp, overlap_pix, boundary_pix)
    P, C = nx * ny, input.shape[1]
    py, px = _grid_origins(nx, ny, sx, sy, input.device)
    patches = input.reshape(P, batch_size, C, hp, wp)
    acc_dtype = input.dtype if input.is_floating_point() else torch.float64
    out = torch.zeros(batch_size, C, pad_y, pad_x, dtype=acc_dtype, device=input.device)
    iy = (py[:, None] + torch.arange(hp, device=input.device))[:, :, None]
    ix = (px[:, None] + torch.arange(wp, device=input.device))[:, None, :]
    flat = (iy * pad_x + ix).reshape(-1)                                   # (P*hp*wp,)
    src = patches.permute(1, 2, 0, 3, 4).reshape(batch_size, C, -1).to(acc_dtype)
    out.view(batch_size, C, -1).index_add_(2, flat, src)
    if overlap_count is None:
        overlap_count = GridPatching2D.get_overlap_count((hp, wp), (img_shape_y, img_shape_x), overlap_pix, boundary_pix)
    out = out / overlap_count.to(device=out.device, dtype=out.dtype)
    out = out[:, :, boundary_pix:boundary_pix + img_shape_y, boundary_pix:boundary_pix + img_shape_x]
    return out.to(input.dtype) if input.is_floating_point() else out.round().to(input.dtype)


class GridPatching2D(BasePatching2D):
    """Deterministic regular grid of overlapping patches with ``fuse`` as the inverse."""

    def __init__(self, img_shape: Tuple[int, int], patch_shape: Tuple[int, int], overlap_pix: int = 0,
                 boundary_pix: int = 0):
        super().__init__(img_shape, patch_shape)
        self.overlap_pix, self.boundary_pix = overlap_pix, boundary_pix
        _, _, nx, ny, _, _ = _grid_geometry(img_shape[0], img_shape[1], self.patch_shape[0], self.patch_shape[1],
                                            overlap_pix, boundary_pix)
        self.patch_num = nx * ny
        self.register_buffer("_overlap_count", self.get_overlap_count(self.patch_shape, self.img_shape, overlap_pix,
                                                                      boundary_pix), persistent=False)
        self.register_buffer("_global_index", self._compute_global_index(), persistent=False)

    def global_index(self, batch_size: int = 1, device="cpu") -> Tensor:
        return self._global_index.clone().to(device)

    def apply(self, input: Tensor, additional_input: Optional[Tensor] = None) -> Tensor:
        add = None
        if additional_input is not None:
            add = torch.nn.functional.interpolate(additional_input, size=self.patch_shape, mode="bilinear")
        return image_batching(input, self.patch_shape[0], self.patch_shape[1], self.overlap_pix, self.boundary_pix, add)

    def forward(self, input: Tensor, additional_input: Optional[Tensor] = None) -> Tensor:
        return self.apply(input, additional_input=additional_input)

    def fuse(self, input: Tensor, batch_size: int) -> Tensor:
        return image_fuse(input, self.img_shape[0], self.img_shape[1], batch_size, self.overlap_pix,
                          self.boundary_pix, self._overlap_count)

    @staticmethod
    def get_overlap_count(patch_shape, img_shape, overlap_pix: int, boundary_pix: int) -> Tensor:
        """(1, 1, Hpad, Wpad): number of patches covering each pixel of the padded image."""
        hp, wp = patch_shape
        sx, sy, nx, ny, pad_x, pad_y = _grid_geometry(img_shape[0], img_shape[1], hp, wp, overlap_pix, boundary_pix)
        cy = torch.zeros(pad_y)
        cx = torch.zeros(pad_x)
        for i in range(ny):
            cy[i * sy:i * sy + hp] += 1
        for i in range(nx):
            cx[i * sx:i * sx + wp] += 1
        return (cy[:, None] * cx[None, :]).reshape(1, 1, pad_y, pad_x)

"""Camera, colour and validation helpers shared by the renderers.

Parity: ``physicsnemo/nn/functional/rendering/utils.py`` (camera basis ``{eye, forward, right, up}``,
bounds tensor, RGBA normalisation of ``uint8`` / float colours, light direction default
``(-0.45, 0.75, -1)``, validators).  The device-side counterparts of the reference's Warp helper
functions live in ``csrc/render.cu``; the tensor versions here serve the PyTorch implementations.
"""
from __future__ import annotations

import ctypes
import math
from collections.abc import Sequence

import torch

from ....ops import _lib

FAR = 3.402823e38


def lib_render():
    lib = _lib.load(required=True)
    if not getattr(lib, "_render_declared", False):
        c = ctypes
        vp, i, f, ll = c.c_void_p, c.c_int, c.c_float, c.c_longlong
        lib.pnm_volume_render.argtypes = [vp, vp, vp, i, i, f, i, f, f, f, f, i, i, i, vp, vp, vp]
        lib.pnm_isosurface_render.argtypes = [vp] * 6 + [i, i, f, f, i, f, f, f, i, i, i, i, vp, vp, vp, vp]
        lib.pnm_mesh_raycast_render.argtypes = [vp, vp, vp, vp, i, vp, vp, vp, vp, i, i, f, f, f, f, i, vp, vp, vp, vp]
        lib.pnm_point_cloud_render.argtypes = [vp, vp, vp, vp, i, i, f, f, f, f, i, ll, f, ll, i, vp, vp, vp, vp]
        lib.pnm_wireframe_render.argtypes = [vp, vp, vp, i, i, f, f, f, f, i, ll, f, ll, vp, vp, vp, vp]
        lib.pnm_line_integral_convolution.argtypes = [vp, vp, f, i, f, i, i, i, vp, vp]
        lib.pnm_scalar_field_to_rgba.argtypes = [vp, ll, f, f, f, f, vp, vp]
        lib.pnm_vector_field_to_rgba.argtypes = [vp, vp, ll, f, f, f, f, vp, vp]
        for name in ("pnm_volume_render", "pnm_isosurface_render", "pnm_mesh_raycast_render", "pnm_point_cloud_render",
                     "pnm_wireframe_render", "pnm_line_integral_convolution", "pnm_scalar_field_to_rgba",
                     "pnm_vector_field_to_rgba"):
            getattr(lib, name).restype = c.c_int
        lib._render_declared = True
    return lib


def check(err: int, what: str) -> None:
    if err:
        raise RuntimeError(f"{what} failed (CUDA error {err})")
    from ....ops import gemm as _g

    _g.launch_count += 1


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def normalize(v: torch.Tensor, eps: float = 1.0e-12) -> torch.Tensor:
    return v / v.norm(dim=-1, keepdim=True).clamp_min(eps)


def as_vec3(value, *, name: str, device) -> torch.Tensor:
    if isinstance(value, torch.Tensor):
        value = value.to(device=device, dtype=torch.float32)
    else:
        value = torch.tensor(value, device=device, dtype=torch.float32)
    if value.shape != (3,):
        raise ValueError(f"{name} must have shape (3,), got {tuple(value.shape)}")
    return value


def camera_basis(eye, center, up, *, device) -> torch.Tensor:
    """``[4, 3]``: eye, forward, right, up — built on the host (12 floats) and shipped in one copy."""
    e = as_vec3(eye, name="eye", device="cpu")
    c = as_vec3(center, name="center", device="cpu")
    u = as_vec3(up, name="up", device="cpu")
    fwd = c - e
    if float(fwd.norm()) <= 1.0e-12:
        raise ValueError("eye and center must not be equal")
    fwd = normalize(fwd)
    right = torch.linalg.cross(normalize(u), fwd, dim=0)
    if float(right.norm()) <= 1.0e-12:
        raise ValueError("up must not be parallel to the camera direction")
    right = normalize(right)
    cam_up = normalize(torch.linalg.cross(fwd, right, dim=0))
    return torch.stack([e, fwd, right, cam_up]).contiguous().to(device)


def bounds_tensor(bounds_min, bounds_max, *, device) -> torch.Tensor:
    lo = as_vec3(bounds_min, name="bounds_min", device="cpu")
    hi = as_vec3(bounds_max, name="bounds_max", device="cpu")
    if bool((hi <= lo).any()):
        raise ValueError("bounds_max must be greater than bounds_min in all dimensions")
    return torch.stack([lo, hi]).contiguous().to(device)


def _to_unit_rgba(color: torch.Tensor) -> torch.Tensor:
    color = color.to(torch.float32) / 255.0 if color.dtype == torch.uint8 else color.to(torch.float32)
    if color.shape[-1] == 3:
        color = torch.cat([color, torch.ones_like(color[..., :1])], dim=-1)
    return color.contiguous().clamp(0.0, 1.0)


def color_tensor(color, *, device, shape_name: str, expected_rank: int) -> torch.Tensor:
    if color is None:
        return torch.zeros((1,) * (expected_rank - 1) + (4,), device=device)
    if color.ndim != expected_rank or color.shape[-1] not in (3, 4):
        raise ValueError(f"{shape_name} must have shape (..., 3) or (..., 4), got {tuple(color.shape)}")
    return _to_unit_rgba(color.to(device))


def uniform_color_tensor(surface_color, *, device) -> torch.Tensor:
    if surface_color is None:
        return torch.ones(1, 4, device=device)
    color = torch.as_tensor(surface_color)
    if color.shape not in ((3,), (4,)):
        raise ValueError(f"surface_color must have shape (3,) or (4,), got {tuple(color.shape)}")
    return _to_unit_rgba(color).reshape(1, 4).to(device)


def light_tensor(light_direction, *, device) -> torch.Tensor:
    if light_direction is None:
        light_direction = [-0.45, 0.75, -1.0]
    return normalize(as_vec3(light_direction, name="light_direction", device="cpu").reshape(1, 3)).contiguous().to(device)


def normalize_rgba_volume(v: torch.Tensor) -> torch.Tensor:
    if v.ndim != 4 or v.shape[-1] != 4:
        raise ValueError(f"rgba_volume must have shape (nx, ny, nz, 4), got {tuple(v.shape)}")
    if any(s < 2 for s in v.shape[:3]):
        raise ValueError("rgba_volume must have at least two samples per dimension")
    return _to_unit_rgba(v)


def validate_image_shape(h: int, w: int) -> None:
    if h <= 0 or w <= 0:
        raise ValueError("image_height and image_width must be strictly positive")


def validate_fov(fov: float) -> None:
    if fov <= 0.0 or fov >= 180.0:
        raise ValueError("fov_y_degrees must lie in the open interval (0, 180)")


def validate_ambient(a: float) -> None:
    if a < 0.0 or a > 1.0:
        raise ValueError("ambient must lie in the closed interval [0, 1]")


def validate_transfer_range(vmin: float, vmax: float) -> None:
    if not math.isfinite(vmin) or not math.isfinite(vmax) or vmax <= vmin:
        raise ValueError("vmax must be greater than vmin")


def validate_opacity(v: float, *, name: str) -> None:
    if not math.isfinite(v) or v < 0.0 or v > 1.0:
        raise ValueError(f"{name} must lie in the closed interval [0, 1]")


def validate_clip_range(near: float, far: float) -> None:
    if not math.isfinite(near) or not math.isfinite(far) or near <= 0.0 or far <= near:
        raise ValueError("near and far must satisfy 0 < near < far")


def validate_vector_field(v: torch.Tensor) -> None:
    if v.ndim != 4 or v.shape[-1] != 3:
        raise ValueError(f"vector_field must have shape (nx, ny, nz, 3), got {tuple(v.shape)}")
    if any(s < 2 for s in v.shape[:3]):
        raise ValueError("vector_field must have at least two samples per dimension")


def tan_half(fov_y_degrees: float) -> float:
    return float(math.tan(math.radians(float(fov_y_degrees)) * 0.5))


def finish_depth(depth: torch.Tensor) -> torch.Tensor:
    return torch.where(depth >= 3.0e38, torch.full_like(depth, torch.inf), depth)


# ---- tensor versions of the device helpers (PyTorch implementations / oracles) --------------------------------
def pixel_rays(camera: torch.Tensor, h: int, w: int, fov: float) -> torch.Tensor:
    """``[H*W, 3]`` unit directions, row-major pixels."""
    dev = camera.device
    t, aspect = tan_half(fov), float(w) / float(h)
    x = ((torch.arange(w, device=dev, dtype=torch.float32) + 0.5) / w * 2.0 - 1.0) * t * aspect
    y = (1.0 - (torch.arange(h, device=dev, dtype=torch.float32) + 0.5) / h * 2.0) * t
    d = camera[1] + x[None, :, None] * camera[2] + y[:, None, None] * camera[3]
    return normalize(d.reshape(-1, 3))


def ray_box(origin: torch.Tensor, d: torch.Tensor, bounds: torch.Tensor):
    """Slab test of rays from one origin: ``(hit [N], t_near [N], t_far [N])``."""
    lo, hi = bounds[0], bounds[1]
    par = d.abs() < 1.0e-12
    safe = torch.where(par, torch.ones_like(d), d)
    t0, t1 = (lo - origin) / safe, (hi - origin) / safe
    tmin = torch.where(par, torch.full_like(d, -FAR), torch.minimum(t0, t1))
    tmax = torch.where(par, torch.full_like(d, FAR), torch.maximum(t0, t1))
    outside = (par & ((origin < lo) | (origin > hi))).any(-1)
    tn = tmin.amax(-1).clamp_min(0.0)
    tf = tmax.amin(-1)
    return (~outside) & (tf >= tn), tn, tf


def trilinear(grid: torch.Tensor, p: torch.Tensor, bounds: torch.Tensor) -> torch.Tensor:
    """Sample ``grid [nx, ny, nz(, C)]`` at world points ``p [N, 3]`` (clamped to the boundary cells)."""
    n = torch.tensor(grid.shape[:3], device=p.device)
    s = (p - bounds[0]) / (bounds[1] - bounds[0]) * (n - 1).to(p.dtype)
    i0 = torch.minimum(torch.floor(s).long().clamp_min(0), n - 2)
    f = (s - i0.to(p.dtype)).clamp(0.0, 1.0)
    return _blend(grid, i0, i0 + 1, f)


def trilinear_index(grid: torch.Tensor, p: torch.Tensor) -> torch.Tensor:
    """Index-space sampling with clamped upper neighbours (streamline integrator convention)."""
    n = torch.tensor(grid.shape[:3], device=p.device)
    i0 = torch.minimum(torch.floor(p).long().clamp_min(0), n - 1)
    i1 = torch.minimum(i0 + 1, n - 1)
    f = (p - i0.to(p.dtype)).clamp(0.0, 1.0)
    return _blend(grid, i0, i1, f)


def _blend(grid, i0, i1, f):
    extra = grid.ndim - 3
    fx, fy, fz = (f[:, k].reshape(-1, *([1] * extra)) for k in range(3))

    def at(a, b, c):
        return grid[a[:, 0], b[:, 1], c[:, 2]]

    c00 = at(i0, i0, i0) * (1 - fx) + at(i1, i0, i0) * fx
    c10 = at(i0, i1, i0) * (1 - fx) + at(i1, i1, i0) * fx
    c01 = at(i0, i0, i1) * (1 - fx) + at(i1, i0, i1) * fx
    c11 = at(i0, i1, i1) * (1 - fx) + at(i1, i1, i1) * fx
    c0 = c00 * (1 - fy) + c10 * fy
    c1 = c01 * (1 - fy) + c11 * fy
    return c0 * (1 - fz) + c1 * fz


def shade(color: torch.Tensor, normal: torch.Tensor, light: torch.Tensor, ambient: float) -> torch.Tensor:
    k = ambient + (1.0 - ambient) * (normal * light).sum(-1, keepdim=True).clamp_min(0.0)
    return torch.cat([color[..., :3] * k, color[..., 3:]], dim=-1)


def jet_colormap(v: torch.Tensor) -> torch.Tensor:
    r = torch.minimum(4.0 * v - 1.5, -4.0 * v + 4.5).clamp(0.0, 1.0)
    g = torch.minimum(4.0 * v - 0.5, -4.0 * v + 3.5).clamp(0.0, 1.0)
    b = torch.minimum(4.0 * v + 0.5, -4.0 * v + 2.5).clamp(0.0, 1.0)
    return torch.stack([r, g, b], dim=-1)


def project_points(points: torch.Tensor, camera: torch.Tensor, h: int, w: int, fov: float):
    """Screen x, y (float pixels) and camera-space depth z of world points."""
    t, aspect = tan_half(fov), float(w) / float(h)
    rel = points - camera[0]
    z = rel @ camera[1]
    zs = torch.where(z.abs() > 1e-12, z, torch.ones_like(z))
    sx = ((rel @ camera[2]) / (zs * t * aspect) + 1.0) * 0.5 * w
    sy = (1.0 - ((rel @ camera[3]) / (zs * t) + 1.0) * 0.5) * h
    return sx, sy, z

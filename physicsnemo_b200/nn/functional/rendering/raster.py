"""Depth-tested splatting of point clouds and line segments.

Parity: ``physicsnemo/nn/functional/rendering/point_cloud_render`` and ``wireframe_render``: every
primitive writes a packed key ``int64(z · depth_scale) · N + id`` to the pixels it covers with an
atomic minimum, so the nearest primitive (ties: lowest id) wins each pixel; a second pass turns the
winner of every pixel into colour and depth.  Lines are clipped against the near / far planes in
camera space and walked with Bresenham's algorithm, depth interpolated along the walk.

``"cuda"``: two launches per image (``csrc/render.cu``; 64-bit ``atomicMin``).  ``"torch"``: the
point splat is a ``scatter_reduce(amin)``; the line walk is restated on the host.
"""
from __future__ import annotations

import numpy as np
import torch

from ....core.function_spec import FunctionSpec
from . import utils as U

_EMPTY = torch.iinfo(torch.int64).max


def _depth_scale(n: int, far: float) -> float:
    return min(1.0e6, float(_EMPTY // max(int(n), 1) - 1) / float(far))


def _point_prepare(points, image_height, image_width, fov_y_degrees, point_colors, point_color, point_size, near, far,
                   eye, center, up):
    if points.ndim != 2 or points.shape[-1] != 3:
        raise ValueError(f"points must have shape (num_points, 3), got {points.shape}")
    if points.shape[0] == 0:
        raise ValueError("points must contain at least one point")
    U.validate_image_shape(image_height, image_width)
    U.validate_fov(fov_y_degrees)
    if point_size <= 0:
        raise ValueError("point_size must be strictly positive")
    U.validate_clip_range(near, far)
    dev = points.device
    colors = torch.zeros(1, 4, device=dev)
    if point_colors is not None:
        if point_color is not None:
            raise ValueError("Pass either point_colors or point_color, not both")
        if point_colors.shape[0] != points.shape[0]:
            raise ValueError("point_colors must have one color per point")
        colors = U.color_tensor(point_colors, device=dev, shape_name="point_colors", expected_rank=2)
    return (points.to(torch.float32).contiguous(), colors, U.uniform_color_tensor(point_color, device=dev),
            U.camera_basis(eye, center, up, device=dev))


def _point_cuda(points, image_height, image_width, eye, center, up, fov_y_degrees, point_colors=None, point_color=None,
                point_size=1, near=0.01, far=1.0e8):
    pts, colors, uc, cam = _point_prepare(points, image_height, image_width, fov_y_degrees, point_colors, point_color,
                                          point_size, near, far, eye, center, up)
    dev, n = pts.device, pts.shape[0]
    rgba = torch.zeros(image_height, image_width, 4, device=dev)
    depth = torch.full((image_height, image_width), U.FAR, device=dev)
    winners = torch.full((image_height, image_width), _EMPTY, device=dev, dtype=torch.int64)
    U.check(U.lib_render().pnm_point_cloud_render(
        pts.data_ptr(), colors.data_ptr(), cam.data_ptr(), uc.data_ptr(), image_width, image_height,
        U.tan_half(fov_y_degrees), image_width / image_height, float(near), float(far), int(point_size), n,
        _depth_scale(n, far), _EMPTY, int(point_colors is not None), winners.data_ptr(), rgba.data_ptr(), depth.data_ptr(),
        U.stream()), "pnm_point_cloud_render")
    return rgba, U.finish_depth(depth)


def _point_torch(points, image_height, image_width, eye, center, up, fov_y_degrees, point_colors=None, point_color=None,
                 point_size=1, near=0.01, far=1.0e8):
    pts, colors, uc, cam = _point_prepare(points, image_height, image_width, fov_y_degrees, point_colors, point_color,
                                          point_size, near, far, eye, center, up)
    dev, n, H, W = pts.device, pts.shape[0], image_height, image_width
    sx, sy, z = U.project_points(pts, cam, H, W, fov_y_degrees)
    ok = (z > near) & (z < far) & (z > 1e-12)
    key = (z * _depth_scale(n, far)).long() * n + torch.arange(n, device=dev)
    cx, cy = sx.long(), sy.long()            # truncation toward zero, like the device cast
    winners = torch.full((H * W,), _EMPTY, device=dev, dtype=torch.int64)
    r = int(point_size) // 2
    for dy in range(-r, r + 1):
        for dx in range(-r, r + 1):
            x, y = cx + dx, cy + dy
            m = ok & (x >= 0) & (x < W) & (y >= 0) & (y < H)
            winners.scatter_reduce_(0, (y * W + x)[m], key[m], "amin")
    got = winners != _EMPTY
    pid = torch.where(got, winners % n, torch.zeros_like(winners))
    col = colors[pid] if point_colors is not None else uc.expand(H * W, 4)
    rgba = torch.where(got[:, None], col, torch.zeros(H * W, 4, device=dev))
    depth = torch.where(got, (pts[pid] - cam[0]) @ cam[1], torch.full((H * W,), U.FAR, device=dev))
    return rgba.reshape(H, W, 4), U.finish_depth(depth.reshape(H, W))


class PointCloudRender(FunctionSpec):
    """``(rgba [H, W, 4], depth [H, W])`` of points ``[N, 3]`` drawn as ``point_size``-pixel squares."""

    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(points, image_height, image_width, eye, center, up, fov_y_degrees, point_colors=None, point_color=None,
                     point_size=1, near=0.01, far=1.0e8):
        return _point_cuda(points, image_height, image_width, eye, center, up, fov_y_degrees, point_colors, point_color,
                           point_size, near, far)

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(points, image_height, image_width, eye, center, up, fov_y_degrees, point_colors=None, point_color=None,
                      point_size=1, near=0.01, far=1.0e8):
        return _point_torch(points, image_height, image_width, eye, center, up, fov_y_degrees, point_colors, point_color,
                            point_size, near, far)


def _wire_prepare(edges, image_height, image_width, fov_y_degrees, line_color, line_thickness, near, far, eye, center, up):
    if edges.ndim == 3:
        if tuple(edges.shape[1:]) != (2, 3):
            raise ValueError("edges must have shape (num_edges, 2, 3) or (num_edges, 6)")
        edges = edges.reshape(edges.shape[0], 6)
    elif edges.ndim != 2 or edges.shape[-1] != 6:
        raise ValueError("edges must have shape (num_edges, 2, 3) or (num_edges, 6)")
    if edges.shape[0] == 0:
        raise ValueError("edges must contain at least one edge")
    U.validate_image_shape(image_height, image_width)
    U.validate_fov(fov_y_degrees)
    if line_thickness <= 0:
        raise ValueError("line_thickness must be strictly positive")
    U.validate_clip_range(near, far)
    dev = edges.device
    return (edges.to(torch.float32).contiguous(), U.uniform_color_tensor(line_color, device=dev),
            U.camera_basis(eye, center, up, device=dev))


def _wire_cuda(edges, image_height, image_width, eye, center, up, fov_y_degrees, line_color=None, line_thickness=1,
               near=0.01, far=1.0e8):
    e, uc, cam = _wire_prepare(edges, image_height, image_width, fov_y_degrees, line_color, line_thickness, near, far, eye,
                               center, up)
    dev, n = e.device, e.shape[0]
    rgba = torch.zeros(image_height, image_width, 4, device=dev)
    depth = torch.full((image_height, image_width), U.FAR, device=dev)
    winners = torch.full((image_height, image_width), _EMPTY, device=dev, dtype=torch.int64)
    U.check(U.lib_render().pnm_wireframe_render(
        e.data_ptr(), cam.data_ptr(), uc.data_ptr(), image_width, image_height, U.tan_half(fov_y_degrees),
        image_width / image_height, float(near), float(far), int(line_thickness), n, _depth_scale(n, far), _EMPTY,
        winners.data_ptr(), rgba.data_ptr(), depth.data_ptr(), U.stream()), "pnm_wireframe_render")
    return rgba, U.finish_depth(depth)


def _wire_torch(edges, image_height, image_width, eye, center, up, fov_y_degrees, line_color=None, line_thickness=1,
                near=0.01, far=1.0e8):
    e, uc, cam = _wire_prepare(edges, image_height, image_width, fov_y_degrees, line_color, line_thickness, near, far, eye,
                               center, up)
    H, W, n = image_height, image_width, e.shape[0]
    f32 = np.float32
    cam_np = cam.cpu().numpy().astype(f32)
    E = e.cpu().numpy().astype(f32)
    t, aspect = f32(U.tan_half(fov_y_degrees)), f32(W / H)
    near, far, scale = f32(near), f32(far), f32(_depth_scale(n, far))
    winners = np.full(H * W, _EMPTY, dtype=np.int64)
    margin = f32(4.0 * (W + H))
    r = int(line_thickness) // 2
    for eid in range(n):
        p0, p1 = E[eid, :3].copy(), E[eid, 3:].copy()
        z0, z1 = f32(np.dot(p0 - cam_np[0], cam_np[1])), f32(np.dot(p1 - cam_np[0], cam_np[1]))
        if (z0 <= near and z1 <= near) or (z0 >= far and z1 >= far):
            continue
        if z0 < near:
            p0, z0 = p0 + (near - z0) / (z1 - z0) * (p1 - p0), near
        elif z1 < near:
            p1, z1 = p1 + (near - z1) / (z0 - z1) * (p0 - p1), near
        if z0 > far:
            p0, z0 = p0 + (far - z0) / (z1 - z0) * (p1 - p0), far
        elif z1 > far:
            p1, z1 = p1 + (far - z1) / (z0 - z1) * (p0 - p1), far

        def screen(p, z):
            rel = p - cam_np[0]
            return ((np.dot(rel, cam_np[2]) / (z * t * aspect) + 1) * 0.5 * W,
                    (1 - (np.dot(rel, cam_np[3]) / (z * t) + 1) * 0.5) * H)

        (fx0, fy0), (fx1, fy1) = screen(p0, z0), screen(p1, z1)
        x0, y0 = int(np.clip(fx0, -margin, margin)), int(np.clip(fy0, -margin, margin))
        x1, y1 = int(np.clip(fx1, -margin, margin)), int(np.clip(fy1, -margin, margin))
        dx, dy = abs(x1 - x0), abs(y1 - y0)
        sx, sy = (-1 if x0 > x1 else 1), (-1 if y0 > y1 else 1)
        steps, err = max(dx, dy), dx - dy
        for s in range(steps + 1):
            a = f32(s) / f32(steps) if steps > 0 else f32(0)
            z = z0 * (f32(1) - a) + z1 * a
            key = int(f32(z * scale)) * n + eid
            for oy in range(-r, r + 1):
                for ox in range(-r, r + 1):
                    x, y = x0 + ox, y0 + oy
                    if 0 <= x < W and 0 <= y < H and key < winners[y * W + x]:
                        winners[y * W + x] = key
            if x0 == x1 and y0 == y1:
                break
            e2 = 2 * err
            if e2 > -dy:
                err -= dy
                x0 += sx
            if e2 < dx:
                err += dx
                y0 += sy
    win = torch.from_numpy(winners).to(e.device)
    got = win != _EMPTY
    rgba = torch.where(got[:, None], uc.expand(H * W, 4), torch.zeros(H * W, 4, device=e.device))
    depth = torch.where(got, (win // n).float() / float(scale), torch.full((H * W,), U.FAR, device=e.device))
    return rgba.reshape(H, W, 4), U.finish_depth(depth.reshape(H, W))


class WireframeRender(FunctionSpec):
    """``(rgba, depth)`` of line segments ``[N, 2, 3]`` (or ``[N, 6]``) drawn ``line_thickness`` pixels wide."""

    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(edges, image_height, image_width, eye, center, up, fov_y_degrees, line_color=None, line_thickness=1,
                     near=0.01, far=1.0e8):
        return _wire_cuda(edges, image_height, image_width, eye, center, up, fov_y_degrees, line_color, line_thickness, near, far)

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(edges, image_height, image_width, eye, center, up, fov_y_degrees, line_color=None, line_thickness=1,
                      near=0.01, far=1.0e8):
        return _wire_torch(edges, image_height, image_width, eye, center, up, fov_y_degrees, line_color, line_thickness, near, far)


point_cloud_render = PointCloudRender.make_function("point_cloud_render")
wireframe_render = WireframeRender.make_function("wireframe_render")

"""Ray-marched renderers of volumetric data: emission / absorption volumes and isosurfaces.

Parity: ``physicsnemo/nn/functional/rendering/volume_render`` (front-to-back compositing of a
trilinearly sampled RGBA volume, early exit at ``opacity_threshold``, depth = first sample at which
the accumulated opacity reaches ``depth_threshold``, colour un-premultiplied at the end) and
``isosurface_render`` (march to the first bracket of ``threshold``, linear root refinement,
central-difference gradient normal facing the camera, Lambert shading with an ambient floor).

``"cuda"``: one thread per pixel (``csrc/render.cu``); the RGBA volume is read as one 16-byte
vector per vertex.  ``"torch"``: the same march vectorised over pixels; CPU path and oracle.
"""
from __future__ import annotations

import torch

from ....core.function_spec import FunctionSpec
from . import utils as U


def _volume_checks(image_height, image_width, fov_y_degrees, step_size, max_steps, opacity_threshold, depth_threshold):
    U.validate_image_shape(image_height, image_width)
    U.validate_fov(fov_y_degrees)
    if step_size <= 0.0:
        raise ValueError("step_size must be strictly positive")
    if max_steps <= 0:
        raise ValueError("max_steps must be strictly positive")
    U.validate_opacity(opacity_threshold, name="opacity_threshold")
    U.validate_opacity(depth_threshold, name="depth_threshold")


def _volume_cuda(rgba_volume, image_height, image_width, eye, center, up, fov_y_degrees, bounds_min, bounds_max,
                 step_size=0.01, max_steps=512, opacity_threshold=0.95, depth_threshold=0.1):
    _volume_checks(image_height, image_width, fov_y_degrees, step_size, max_steps, opacity_threshold, depth_threshold)
    dev = rgba_volume.device
    vol = U.normalize_rgba_volume(rgba_volume)
    cam = U.camera_basis(eye, center, up, device=dev)
    bounds = U.bounds_tensor(bounds_min, bounds_max, device=dev)
    rgba = torch.empty(image_height, image_width, 4, device=dev)
    depth = torch.empty(image_height, image_width, device=dev)
    U.check(U.lib_render().pnm_volume_render(
        vol.data_ptr(), cam.data_ptr(), bounds.data_ptr(), image_width, image_height, float(step_size), int(max_steps),
        U.tan_half(fov_y_degrees), image_width / image_height, float(opacity_threshold), float(depth_threshold),
        vol.shape[0], vol.shape[1], vol.shape[2], rgba.data_ptr(), depth.data_ptr(), U.stream()), "pnm_volume_render")
    return rgba, U.finish_depth(depth)


def _volume_torch(rgba_volume, image_height, image_width, eye, center, up, fov_y_degrees, bounds_min, bounds_max,
                  step_size=0.01, max_steps=512, opacity_threshold=0.95, depth_threshold=0.1):
    _volume_checks(image_height, image_width, fov_y_degrees, step_size, max_steps, opacity_threshold, depth_threshold)
    dev = rgba_volume.device
    vol = U.normalize_rgba_volume(rgba_volume)
    cam = U.camera_basis(eye, center, up, device=dev)
    bounds = U.bounds_tensor(bounds_min, bounds_max, device=dev)
    d = U.pixel_rays(cam, image_height, image_width, fov_y_degrees)
    hit, tn, tf = U.ray_box(cam[0], d, bounds)
    n = d.shape[0]
    acc = torch.zeros(n, 4, device=dev)
    first = torch.full((n,), U.FAR, device=dev)
    t = tn.clone()
    for _ in range(int(max_steps)):
        live = hit & (t <= tf) & (acc[:, 3] < opacity_threshold)
        if not bool(live.any()):
            break
        idx = live.nonzero().squeeze(1)
        smp = U.trilinear(vol, cam[0] + t[idx, None] * d[idx], bounds)
        a = smp[:, 3].clamp(0.0, 1.0)
        o = (1.0 - acc[idx, 3]) * a
        new = acc[idx] + torch.cat([smp[:, :3] * o[:, None], o[:, None]], 1)
        acc[idx] = torch.where((a > 0)[:, None], new, acc[idx])
        crossed = (a > 0) & (first[idx] >= 3.0e38) & (acc[idx, 3] >= depth_threshold)
        first[idx] = torch.where(crossed, t[idx], first[idx])
        t = torch.where(live, t + step_size, t)
    some = acc[:, 3] > 0
    rgb = acc[:, :3] / acc[:, 3:].clamp_min(1e-30)
    rgba = torch.where(some[:, None], torch.cat([rgb, acc[:, 3:]], 1), torch.zeros_like(acc))
    depth = torch.where(some, first, torch.full_like(first, U.FAR))
    return rgba.reshape(image_height, image_width, 4), U.finish_depth(depth.reshape(image_height, image_width))


class VolumeRender(FunctionSpec):
    """``(rgba [H, W, 4], depth [H, W])`` of an RGBA volume ``[nx, ny, nz, 4]`` (float in [0, 1] or ``uint8``)."""

    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(rgba_volume, image_height, image_width, eye, center, up, fov_y_degrees, bounds_min, bounds_max,
                     step_size=0.01, max_steps=512, opacity_threshold=0.95, depth_threshold=0.1):
        return _volume_cuda(rgba_volume, image_height, image_width, eye, center, up, fov_y_degrees, bounds_min, bounds_max,
                            step_size, max_steps, opacity_threshold, depth_threshold)

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(rgba_volume, image_height, image_width, eye, center, up, fov_y_degrees, bounds_min, bounds_max,
                      step_size=0.01, max_steps=512, opacity_threshold=0.95, depth_threshold=0.1):
        return _volume_torch(rgba_volume, image_height, image_width, eye, center, up, fov_y_degrees, bounds_min, bounds_max,
                             step_size, max_steps, opacity_threshold, depth_threshold)


def _iso_prepare(field, image_height, image_width, fov_y_degrees, bounds_min, bounds_max, step_size, max_steps,
                 color_field, surface_color, light_direction, ambient, eye, center, up):
    if field.ndim != 3:
        raise ValueError(f"field must have shape (nx, ny, nz), got {tuple(field.shape)}")
    if any(s < 2 for s in field.shape):
        raise ValueError("field must have at least two samples in each dimension")
    U.validate_image_shape(image_height, image_width)
    U.validate_fov(fov_y_degrees)
    U.validate_ambient(ambient)
    if step_size <= 0.0:
        raise ValueError("step_size must be strictly positive")
    if max_steps <= 0:
        raise ValueError("max_steps must be strictly positive")
    dev = field.device
    if color_field is not None and tuple(color_field.shape[:3]) != tuple(field.shape):
        raise ValueError(f"color_field spatial shape must match field, got {tuple(color_field.shape[:3])} "
                         f"and {tuple(field.shape)}")
    return (field.to(torch.float32).contiguous(), U.camera_basis(eye, center, up, device=dev),
            U.bounds_tensor(bounds_min, bounds_max, device=dev),
            U.color_tensor(color_field, device=dev, shape_name="color_field", expected_rank=4),
            U.uniform_color_tensor(surface_color, device=dev), U.light_tensor(light_direction, device=dev))


def _iso_cuda(field, image_height, image_width, eye, center, up, fov_y_degrees, bounds_min, bounds_max, threshold=0.0,
              step_size=0.01, max_steps=512, color_field=None, surface_color=None, light_direction=None, ambient=0.2):
    f, cam, bounds, cf, uc, light = _iso_prepare(field, image_height, image_width, fov_y_degrees, bounds_min, bounds_max,
                                                 step_size, max_steps, color_field, surface_color, light_direction, ambient,
                                                 eye, center, up)
    dev = f.device
    rgba = torch.empty(image_height, image_width, 4, device=dev)
    depth = torch.empty(image_height, image_width, device=dev)
    normal = torch.empty(image_height, image_width, 3, device=dev)
    U.check(U.lib_render().pnm_isosurface_render(
        f.data_ptr(), cf.data_ptr(), cam.data_ptr(), bounds.data_ptr(), uc.data_ptr(), light.data_ptr(), image_width,
        image_height, float(threshold), float(step_size), int(max_steps), U.tan_half(fov_y_degrees),
        image_width / image_height, float(ambient), int(color_field is not None), f.shape[0], f.shape[1], f.shape[2],
        rgba.data_ptr(), depth.data_ptr(), normal.data_ptr(), U.stream()), "pnm_isosurface_render")
    return rgba, U.finish_depth(depth), normal


def _iso_torch(field, image_height, image_width, eye, center, up, fov_y_degrees, bounds_min, bounds_max, threshold=0.0,
               step_size=0.01, max_steps=512, color_field=None, surface_color=None, light_direction=None, ambient=0.2):
    f, cam, bounds, cf, uc, light = _iso_prepare(field, image_height, image_width, fov_y_degrees, bounds_min, bounds_max,
                                                 step_size, max_steps, color_field, surface_color, light_direction, ambient,
                                                 eye, center, up)
    dev = f.device
    d = U.pixel_rays(cam, image_height, image_width, fov_y_degrees)
    hit, tn, tf = U.ray_box(cam[0], d, bounds)
    n = d.shape[0]
    found = torch.zeros(n, dtype=torch.bool, device=dev)
    hit_t = torch.full((n,), U.FAR, device=dev)
    pt = tn.clone()
    pv = U.trilinear(f, cam[0] + pt[:, None] * d, bounds)
    live = hit.clone()
    for _ in range(int(max_steps)):
        nt = pt + step_size
        live = live & ~found & (nt <= tf)
        if not bool(live.any()):
            break
        nv = U.trilinear(f, cam[0] + nt[:, None] * d, bounds)
        cross = live & ((pv - threshold) * (nv - threshold) <= 0.0)
        den = nv - pv
        den = torch.where(den.abs() < 1e-7, torch.where(den < 0, torch.full_like(den, -1e-7), torch.full_like(den, 1e-7)), den)
        alpha = ((threshold - pv) / den).clamp(0.0, 1.0)
        hit_t = torch.where(cross, pt + alpha * step_size, hit_t)
        found = found | cross
        pt = torch.where(live, nt, pt)
        pv = torch.where(live, nv, pv)
    p = cam[0] + torch.where(found, hit_t, torch.zeros_like(hit_t))[:, None] * d
    h = (bounds[1] - bounds[0]) / (torch.tensor(f.shape, device=dev, dtype=torch.float32) - 1)
    g = torch.stack([(U.trilinear(f, p + 0.5 * h[k] * e, bounds) - U.trilinear(f, p - 0.5 * h[k] * e, bounds)) / h[k]
                     for k, e in enumerate(torch.eye(3, device=dev))], -1)
    gl = g.norm(dim=-1, keepdim=True)
    nrm = torch.where(gl > 1e-12, g / gl.clamp_min(1e-30), torch.zeros_like(g))
    nrm = torch.where(((nrm * d).sum(-1) > 0)[:, None], -nrm, nrm)
    color = U.trilinear(cf, p, bounds) if color_field is not None else uc.expand(n, 4)
    rgba = torch.where(found[:, None], U.shade(color, nrm, light, ambient), torch.zeros(n, 4, device=dev))
    depth = torch.where(found, hit_t, torch.full_like(hit_t, U.FAR))
    nrm = torch.where(found[:, None], nrm, torch.zeros_like(nrm))
    return (rgba.reshape(image_height, image_width, 4), U.finish_depth(depth.reshape(image_height, image_width)),
            nrm.reshape(image_height, image_width, 3))


class IsosurfaceRender(FunctionSpec):
    """``(rgba, depth, normal)`` of the level set ``field == threshold`` of a scalar grid ``[nx, ny, nz]``."""

    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(field, image_height, image_width, eye, center, up, fov_y_degrees, bounds_min, bounds_max, threshold=0.0,
                     step_size=0.01, max_steps=512, color_field=None, surface_color=None, light_direction=None, ambient=0.2):
        return _iso_cuda(field, image_height, image_width, eye, center, up, fov_y_degrees, bounds_min, bounds_max, threshold,
                         step_size, max_steps, color_field, surface_color, light_direction, ambient)

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(field, image_height, image_width, eye, center, up, fov_y_degrees, bounds_min, bounds_max, threshold=0.0,
                      step_size=0.01, max_steps=512, color_field=None, surface_color=None, light_direction=None, ambient=0.2):
        return _iso_torch(field, image_height, image_width, eye, center, up, fov_y_degrees, bounds_min, bounds_max, threshold,
                          step_size, max_steps, color_field, surface_color, light_direction, ambient)


volume_render = VolumeRender.make_function("volume_render")
isosurface_render = IsosurfaceRender.make_function("isosurface_render")

"""Field → texture maps: line integral convolution and jet colour / opacity transfer functions.

Parity: ``physicsnemo/nn/functional/rendering/line_integral_convolution`` (midpoint streamline
integration from every voxel in both directions, linearly decaying weights, contrast stretch),
``scalar_field_to_rgba`` and ``vector_field_to_rgba`` (jet colour of the normalised value /
magnitude; opacity = value above a threshold, or LIC texture × magnitude).  Outputs of the two
colour maps are ``uint8`` RGBA volumes ready for ``volume_render``.
"""
from __future__ import annotations

import torch

from ....core.function_spec import FunctionSpec
from . import utils as U


def _lic_checks(vector_field, seed, step_size, num_steps, contrast):
    U.validate_vector_field(vector_field)
    if tuple(seed.shape) != tuple(vector_field.shape[:3]):
        raise ValueError("seed must have shape matching vector_field spatial dimensions, got "
                         f"{tuple(seed.shape)} and {tuple(vector_field.shape[:3])}")
    if step_size <= 0.0:
        raise ValueError("step_size must be strictly positive")
    if num_steps <= 0:
        raise ValueError("num_steps must be strictly positive")
    if contrast <= 0.0:
        raise ValueError("contrast must be strictly positive")


def _lic_cuda(vector_field, seed, step_size=0.5, num_steps=20, contrast=1.4):
    _lic_checks(vector_field, seed, step_size, num_steps, contrast)
    v = vector_field.to(torch.float32).contiguous()
    s = seed.to(device=v.device, dtype=torch.float32).contiguous()
    out = torch.empty_like(s)
    U.check(U.lib_render().pnm_line_integral_convolution(v.data_ptr(), s.data_ptr(), float(step_size), int(num_steps),
                                                         float(contrast), s.shape[0], s.shape[1], s.shape[2], out.data_ptr(),
                                                         U.stream()), "pnm_line_integral_convolution")
    return out


def _lic_torch(vector_field, seed, step_size=0.5, num_steps=20, contrast=1.4):
    _lic_checks(vector_field, seed, step_size, num_steps, contrast)
    v = vector_field.to(torch.float32)
    s = seed.to(device=v.device, dtype=torch.float32)
    dev = v.device
    nx, ny, nz = s.shape
    pos = torch.stack(torch.meshgrid(torch.arange(nx, device=dev), torch.arange(ny, device=dev), torch.arange(nz, device=dev),
                                     indexing="ij"), -1).reshape(-1, 3).float()
    hi = torch.tensor([nx - 1, ny - 1, nz - 1], device=dev, dtype=torch.float32)
    total = s.reshape(-1).clone()
    wsum = torch.ones_like(total)
    for sgn in (1.0, -1.0):
        cur = pos.clone()
        live = torch.ones(pos.shape[0], dtype=torch.bool, device=dev)
        for step in range(int(num_steps)):
            vec = U.trilinear_index(v, cur)
            ln = vec.norm(dim=-1)
            live = live & (ln > 1e-6)
            vec = sgn * vec / ln.clamp_min(1e-30)[:, None]
            mv = U.trilinear_index(v, cur + 0.5 * step_size * vec)
            ml = mv.norm(dim=-1)
            live = live & (ml > 1e-6)
            nxt = cur + step_size * sgn * mv / ml.clamp_min(1e-30)[:, None]
            live = live & ((nxt >= 0) & (nxt <= hi)).all(-1)
            if not bool(live.any()):
                break
            cur = torch.where(live[:, None], nxt, cur)
            w = 1.0 - (step + 1) / (num_steps + 1)
            total = total + torch.where(live, U.trilinear_index(s, cur) * w, torch.zeros_like(total))
            wsum = wsum + torch.where(live, torch.full_like(wsum, w), torch.zeros_like(wsum))
    val = (total / wsum.clamp_min(1e-6)).clamp(0.0, 1.0)
    return (((val - 0.5) * contrast + 0.5).clamp(0.0, 1.0)).reshape(nx, ny, nz)


class LineIntegralConvolution(FunctionSpec):
    """LIC texture ``[nx, ny, nz]`` in [0, 1] of a vector field ``[nx, ny, nz, 3]`` and a noise ``seed``."""

    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(vector_field, seed, step_size=0.5, num_steps=20, contrast=1.4):
        return _lic_cuda(vector_field, seed, step_size, num_steps, contrast)

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(vector_field, seed, step_size=0.5, num_steps=20, contrast=1.4):
        return _lic_torch(vector_field, seed, step_size, num_steps, contrast)


def _to_uint8(color, alpha):
    return (torch.cat([color, alpha.unsqueeze(-1)], -1) * 255.0).clamp(0.0, 255.0).to(torch.uint8)


def _scalar_checks(field, vmin, vmax, max_opacity, opacity_threshold):
    if field.ndim != 3:
        raise ValueError(f"field must have shape (nx, ny, nz), got {tuple(field.shape)}")
    U.validate_transfer_range(vmin, vmax)
    U.validate_opacity(max_opacity, name="max_opacity")
    U.validate_opacity(opacity_threshold, name="opacity_threshold")


class ScalarFieldToRGBA(FunctionSpec):
    """Jet colours and value-proportional opacity; ``uint8 [nx, ny, nz, 4]``."""

    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(field, vmin, vmax, max_opacity=0.8, opacity_threshold=0.1):
        _scalar_checks(field, vmin, vmax, max_opacity, opacity_threshold)
        f = field.to(torch.float32).contiguous()
        out = torch.empty(*f.shape, 4, dtype=torch.uint8, device=f.device)
        U.check(U.lib_render().pnm_scalar_field_to_rgba(f.data_ptr(), f.numel(), float(vmin), float(vmax), float(max_opacity),
                                                        float(opacity_threshold), out.data_ptr(), U.stream()),
                "pnm_scalar_field_to_rgba")
        return out

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(field, vmin, vmax, max_opacity=0.8, opacity_threshold=0.1):
        _scalar_checks(field, vmin, vmax, max_opacity, opacity_threshold)
        v = ((field.to(torch.float32) - vmin) / (vmax - vmin)).clamp(0.0, 1.0)
        alpha = (torch.where(v < opacity_threshold, torch.zeros_like(v), v) * max_opacity).clamp(0.0, 1.0)
        return _to_uint8(U.jet_colormap(v), alpha)


def _vector_checks(vector_field, lic_field, vmin, vmax, max_opacity, lic_threshold):
    if vector_field.ndim != 4 or vector_field.shape[-1] != 3:
        raise ValueError(f"vector_field must have shape (nx, ny, nz, 3), got {tuple(vector_field.shape)}")
    if tuple(lic_field.shape) != tuple(vector_field.shape[:3]):
        raise ValueError("lic_field must have shape matching vector_field spatial dimensions")
    U.validate_transfer_range(vmin, vmax)
    U.validate_opacity(max_opacity, name="max_opacity")
    U.validate_opacity(lic_threshold, name="lic_threshold")


class VectorFieldToRGBA(FunctionSpec):
    """Jet colours of the magnitude, opacity = LIC texture × magnitude; ``uint8 [nx, ny, nz, 4]``."""

    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(vector_field, lic_field, vmin, vmax, max_opacity=0.8, lic_threshold=0.5):
        _vector_checks(vector_field, lic_field, vmin, vmax, max_opacity, lic_threshold)
        v = vector_field.to(torch.float32).contiguous()
        lic = lic_field.to(device=v.device, dtype=torch.float32).contiguous()
        out = torch.empty(*lic.shape, 4, dtype=torch.uint8, device=v.device)
        U.check(U.lib_render().pnm_vector_field_to_rgba(v.data_ptr(), lic.data_ptr(), lic.numel(), float(vmin), float(vmax),
                                                        float(max_opacity), float(lic_threshold), out.data_ptr(), U.stream()),
                "pnm_vector_field_to_rgba")
        return out

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(vector_field, lic_field, vmin, vmax, max_opacity=0.8, lic_threshold=0.5):
        _vector_checks(vector_field, lic_field, vmin, vmax, max_opacity, lic_threshold)
        mag = ((vector_field.to(torch.float32).norm(dim=-1) - vmin) / (vmax - vmin)).clamp(0.0, 1.0)
        lic = lic_field.to(device=vector_field.device, dtype=torch.float32).clamp(0.0, 1.0)
        lic = torch.where(lic < lic_threshold, torch.zeros_like(lic), lic)
        return _to_uint8(U.jet_colormap(mag), (lic * mag * max_opacity).clamp(0.0, 1.0))


line_integral_convolution = LineIntegralConvolution.make_function("line_integral_convolution")
scalar_field_to_rgba = ScalarFieldToRGBA.make_function("scalar_field_to_rgba")
vector_field_to_rgba = VectorFieldToRGBA.make_function("vector_field_to_rgba")

"""Greedy farthest point sampling.

Parity: ``physicsnemo/nn/functional/geometry/farthest_point_sampling`` — ``(N, D)`` or ``(B, N, D)``
clouds, ``num_samples`` indices per cloud (int64), start at index 0 or at a random point.
``"cuda"``: one 1024-thread CTA per cloud runs the whole selection loop on the device (running
minimum distances in global memory, block-wide arg-max per step, ties to the smaller index;
``csrc/neighbors.cu``) — no per-step launch or host synchronisation.
"""
from __future__ import annotations

import torch

from ....core.function_spec import FunctionSpec
from ....ops import gemm as _g
from ..neighbors.radius_search import _lib_nb


def validate_inputs(points, num_samples):
    if points.ndim == 2:
        points, unb = points.unsqueeze(0), True
    elif points.ndim == 3:
        unb = False
    else:
        raise ValueError(f"points must have shape (N, D) or (B, N, D), got {tuple(points.shape)}")
    if not isinstance(num_samples, int) or num_samples < 1 or num_samples > points.shape[1]:
        raise ValueError(f"num_samples must satisfy 1 <= num_samples <= N ({points.shape[1]}), got {num_samples}")
    return points, unb


@torch.no_grad()
def _fps_torch(points, num_samples, random_start=False):
    points, unb = validate_inputs(points, num_samples)
    pts = points.float()
    B, N, _ = pts.shape
    cur = torch.randint(0, N, (B,), device=pts.device) if random_start else torch.zeros(B, dtype=torch.long, device=pts.device)
    sel = torch.empty(B, num_samples, dtype=torch.long, device=pts.device)
    best = torch.full((B, N), float("inf"), device=pts.device)
    rows = torch.arange(B, device=pts.device)
    for i in range(num_samples):
        sel[:, i] = cur
        if i + 1 == num_samples:
            break
        best = torch.minimum(best, ((pts - pts[rows, cur][:, None]) ** 2).sum(-1))
        cur = best.argmax(dim=1)
    return sel[0] if unb else sel


@torch.no_grad()
def _fps_cuda(points, num_samples, random_start=False):
    points, unb = validate_inputs(points, num_samples)
    if points.shape[-1] != 3:
        out = _fps_torch(points, num_samples, random_start)
        return out
    lib = _lib_nb()
    pts = points.float().contiguous()
    B, N, _ = pts.shape
    sel = torch.empty(B, num_samples, dtype=torch.int64, device=pts.device)
    sel[:, 0] = torch.randint(0, N, (B,), device=pts.device) if random_start else 0
    scratch = torch.empty(B, N, dtype=torch.float32, device=pts.device)
    err = lib.pnm_fps(pts.data_ptr(), scratch.data_ptr(), sel.data_ptr(), B, N, num_samples,
                      torch.cuda.current_stream().cuda_stream)
    if err:
        raise RuntimeError(f"pnm_fps failed ({err})")
    _g.launch_count += 1
    return sel[0] if unb else sel


class FarthestPointSampling(FunctionSpec):
    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(points, num_samples, random_start=False):
        return _fps_cuda(points, num_samples, random_start)

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(points, num_samples, random_start=False):
        return _fps_torch(points, num_samples, random_start)


farthest_point_sampling = FarthestPointSampling.make_function("farthest_point_sampling")

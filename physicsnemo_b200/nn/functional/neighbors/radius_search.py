"""Fixed-radius neighbour search.

Parity: ``physicsnemo/nn/functional/neighbors/radius_search`` — ``radius_search(points, queries,
radius, max_points=None, return_dists=False, return_points=False)`` on ``(N, 3)`` / ``(B, N, 3)``
clouds.  ``max_points=None`` returns the ragged list ``[query; point]`` (``[batch; query; point]``
when batched); with ``max_points`` every query gets a fixed-width row holding its nearest hits
(index 0 / zero distance / zero point where there is none).

``"cuda"``: points are bucketed into a uniform cell list (cell edge = radius, enlarged when the
grid would exceed 2^22 cells; sort and prefix sums by library calls), then count → fill or a
per-query sorted top-K kernel (``csrc/neighbors.cu``).  Distances and gathered points are
recomputed from the indices with PyTorch ops, so gradients reach ``points`` and ``queries``.
"""
from __future__ import annotations

import ctypes

import torch

from ....core.function_spec import FunctionSpec
from ....ops import _lib
from ....ops import gemm as _g

_MAX_CELLS = 1 << 22


def validate_inputs(points, queries):
    if points.ndim == 2 and queries.ndim == 2:
        return points.unsqueeze(0), queries.unsqueeze(0), True
    if points.ndim == 3 and queries.ndim == 3:
        if points.shape[0] != queries.shape[0]:
            raise ValueError(f"Batch dimensions must match: points has {points.shape[0]}, queries has {queries.shape[0]}")
        return points, queries, False
    raise ValueError(f"points and queries must be 2D (N, 3) or 3D (B, N, 3), got {points.ndim}D and {queries.ndim}D")


def format_returns(indices, points, distances, return_dists, return_points):
    if return_points:
        return (indices, points, distances) if return_dists else (indices, points)
    return (indices, distances) if return_dists else indices


# ------------------------------------------------------------------------ torch
def _ragged_torch(p, q, radius):
    d = torch.cdist(q, p, compute_mode="donot_use_mm_for_euclid_dist")
    return torch.nonzero(d <= radius, as_tuple=False).t().contiguous()          # [2, total]: query, point


def _capped_torch(p, q, radius, max_points):
    d = torch.cdist(q, p, compute_mode="donot_use_mm_for_euclid_dist")          # [Q, N]
    k = min(max_points, d.shape[1])
    vals, idx = torch.topk(d, k=k, dim=1, largest=False)
    if k < max_points:
        vals = torch.nn.functional.pad(vals, (0, max_points - k), value=float("inf"))
        idx = torch.nn.functional.pad(idx, (0, max_points - k), value=0)
    ok = vals <= radius
    return torch.where(ok, idx, 0), ok


def _finish(points, queries, pairs_or_idx, ok, radius, max_points, return_dists, return_points, unb):
    """Gather points / distances from indices with differentiable ops and shape the outputs."""
    B = points.shape[0]
    if max_points is None:
        sel = pairs_or_idx                                                    # [3, total]
        b, qi, pi = sel[0], sel[1], sel[2]
        pts_out = points[b, pi] if return_points else points.new_empty((0, points.shape[-1]))
        dists = (points[b, pi] - queries[b, qi]).norm(dim=-1) if return_dists else points.new_empty((0,))
        return format_returns(sel[1:] if unb else sel, pts_out, dists, return_dists, return_points)
    idx = pairs_or_idx                                                        # [B, Q, K]
    gathered = torch.gather(points[:, None].expand(-1, idx.shape[1], -1, -1), 2,
                            idx[..., None].expand(-1, -1, -1, points.shape[-1])) if (return_points or return_dists) else None
    if return_points:
        pts_out = gathered * ok[..., None]
    else:
        pts_out = points.new_empty((0, max_points, 3))
    if return_dists:
        delta = gathered - queries[:, :, None]
        dists = torch.where(ok, (delta * delta).sum(-1).clamp_min(0).sqrt(), torch.zeros((), dtype=points.dtype, device=points.device))
    else:
        dists = points.new_empty((0,))
    if unb:
        idx = idx[0]
        pts_out = pts_out[0] if return_points else pts_out
        dists = dists[0] if return_dists else dists
    return format_returns(idx, pts_out, dists, return_dists, return_points)


def _radius_search_torch(points, queries, radius, max_points=None, return_dists=False, return_points=False):
    points, queries, unb = validate_inputs(points, queries)
    B = points.shape[0]
    with torch.no_grad():
        if max_points is None:
            rows = []
            for b in range(B):
                pr = _ragged_torch(points[b], queries[b], radius)
                rows.append(torch.cat([torch.full((1, pr.shape[1]), b, dtype=pr.dtype, device=pr.device), pr]))
            sel, ok = torch.cat(rows, dim=1), None
        else:
            pairs = [_capped_torch(points[b], queries[b], radius, max_points) for b in range(B)]
            sel, ok = torch.stack([a for a, _ in pairs]), torch.stack([m for _, m in pairs])
    return _finish(points, queries, sel, ok, radius, max_points, return_dists, return_points, unb)


# ------------------------------------------------------------------------- cuda
def _lib_nb():
    lib = _lib.load(required=True)
    if not getattr(lib, "_nb_declared", False):
        c = ctypes
        vp, fp, ip = c.c_void_p, c.POINTER(c.c_float), c.POINTER(c.c_int)
        lib.pnm_radius_count.argtypes = [vp, vp, vp, vp, vp, fp, c.c_float, ip, c.c_int, c.c_float, vp]
        lib.pnm_radius_fill.argtypes = [vp, vp, vp, vp, vp, vp, vp, c.c_longlong, fp, c.c_float, ip, c.c_int, c.c_float, vp]
        lib.pnm_radius_topk.argtypes = [vp, vp, vp, vp, vp, vp, vp, fp, c.c_float, ip, c.c_int, c.c_int, c.c_float, vp]
        lib.pnm_knn.argtypes = [vp, vp, vp, vp, c.c_int, c.c_int, c.c_int, c.c_int, vp]
        lib.pnm_fps.argtypes = [vp, vp, vp, c.c_int, c.c_int, c.c_int, vp]
        for f in (lib.pnm_radius_count, lib.pnm_radius_fill, lib.pnm_radius_topk, lib.pnm_knn, lib.pnm_fps, lib.pnm_knn_max_k):
            f.restype = c.c_int
        lib._nb_declared = True
    return lib


class CellList:
    """Points of one cloud sorted by cell of a uniform grid."""

    def __init__(self, p: torch.Tensor, radius: float):
        lo, hi = p.amin(0), p.amax(0)
        ext = (hi - lo).clamp_min(1e-12)
        cell = float(radius)
        ext_h = ext.tolist()
        while True:
            n = [int(e / cell) + 1 for e in ext_h]
            if n[0] * n[1] * n[2] <= _MAX_CELLS:
                break
            cell *= 1.26
        self.cell, self.n, self.lo = cell, n, lo.tolist()
        c = ((p - lo) / cell).floor().long()
        for a in range(3):
            c[:, a].clamp_(0, n[a] - 1)
        cid = (c[:, 0] * n[1] + c[:, 1]) * n[2] + c[:, 2]
        cid_sorted, order = torch.sort(cid)
        self.order = order.int()
        self.pts = p[order].contiguous()
        bounds = torch.searchsorted(cid_sorted, torch.arange(n[0] * n[1] * n[2] + 1, device=p.device))
        self.start, self.end = bounds[:-1].int().contiguous(), bounds[1:].int().contiguous()
        self.c_lo = (ctypes.c_float * 3)(*self.lo)
        self.c_n = (ctypes.c_int * 3)(*n)


def _radius_search_cuda(points, queries, radius, max_points=None, return_dists=False, return_points=False):
    points, queries, unb = validate_inputs(points, queries)
    if points.shape[-1] != 3 or queries.shape[-1] != 3:
        raise ValueError("radius_search expects 3-D coordinates")
    lib = _lib_nb()
    st = torch.cuda.current_stream().cuda_stream
    B, Q = queries.shape[0], queries.shape[1]
    rows, idxs, oks = [], [], []
    with torch.no_grad():
        for b in range(B):
            p = points[b].detach().float().contiguous()
            q = queries[b].detach().float().contiguous()
            cl = CellList(p, radius)
            if max_points is None:
                counts = torch.empty(Q, dtype=torch.int32, device=p.device)
                err = lib.pnm_radius_count(cl.pts.data_ptr(), cl.start.data_ptr(), cl.end.data_ptr(), q.data_ptr(),
                                           counts.data_ptr(), cl.c_lo, cl.cell, cl.c_n, Q, radius, st)
                offsets = torch.zeros(Q + 1, dtype=torch.int64, device=p.device)
                offsets[1:] = torch.cumsum(counts, 0)
                total = int(offsets[-1])
                pairs = torch.empty(2, total, dtype=torch.int64, device=p.device)
                err |= lib.pnm_radius_fill(cl.pts.data_ptr(), cl.order.data_ptr(), cl.start.data_ptr(), cl.end.data_ptr(),
                                           q.data_ptr(), offsets.data_ptr(), pairs.data_ptr(), total, cl.c_lo, cl.cell,
                                           cl.c_n, Q, radius, st)
                if err:
                    raise RuntimeError(f"radius search kernels failed ({err})")
                _g.launch_count += 2
                rows.append(torch.cat([torch.full((1, total), b, dtype=torch.int64, device=p.device), pairs]))
            else:
                idx = torch.empty(Q, max_points, dtype=torch.int64, device=p.device)
                d2 = torch.empty(Q, max_points, dtype=torch.float32, device=p.device)
                err = lib.pnm_radius_topk(cl.pts.data_ptr(), cl.order.data_ptr(), cl.start.data_ptr(), cl.end.data_ptr(),
                                          q.data_ptr(), idx.data_ptr(), d2.data_ptr(), cl.c_lo, cl.cell, cl.c_n, Q,
                                          max_points, radius, st)
                if err:
                    raise RuntimeError(f"radius search kernel failed ({err})")
                _g.launch_count += 1
                ok = idx >= 0
                idxs.append(idx.clamp_min(0))
                oks.append(ok)
    if max_points is None:
        return _finish(points, queries, torch.cat(rows, dim=1), None, radius, None, return_dists, return_points, unb)
    return _finish(points, queries, torch.stack(idxs), torch.stack(oks), radius, max_points, return_dists, return_points, unb)


class RadiusSearch(FunctionSpec):
    @FunctionSpec.register(name="cuda", rank=0)
    def cuda_forward(points, queries, radius, max_points=None, return_dists=False, return_points=False):
        return _radius_search_cuda(points, queries, radius, max_points, return_dists, return_points)

    @FunctionSpec.register(name="torch", rank=1, baseline=True)
    def torch_forward(points, queries, radius, max_points=None, return_dists=False, return_points=False):
        return _radius_search_torch(points, queries, radius, max_points, return_dists, return_points)


radius_search = RadiusSearch.make_function("radius_search")

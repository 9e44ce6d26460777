"""Neighbour searches on point clouds whose points and / or queries are sharded over ranks.

Parity: ``physicsnemo/domain_parallel/shard_utils/knn.py:36-165`` (ring kNN) and ``point_cloud_ops.py:48-717`` (ring ball
query).  The point blocks travel around the ring of the mesh dimension; every rank searches the visiting block for ITS
queries with the ordinary single-device function (the CUDA kernels on a GPU) and merges the block's candidates into a
running list of the best ``k`` (or ``max_points``) by distance, carrying the candidates' GLOBAL indices and coordinates.
After ``n`` steps every rank holds exact results for its queries; nothing of size points × queries ever exists, and
no rank ever holds more than two point blocks.  Distances are recomputed from the carried coordinates, so they are
differentiable with respect to the queries (remote points are treated as constants, as in the reference).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch.distributed.tensor import Replicate, Shard

from .. import collectives as C
from ._common import MissingShardPatch, ShardTensor, is_st, local, resolved, wrap


def _row_shard(t):
    """Mesh dimension over which dim 0 (the point index) of ``t`` is sharded, or None when ``t`` is whole on every rank."""
    if not is_st(t):
        return None
    for md, p in enumerate(t._spec.placements):
        if isinstance(p, Shard):
            if p.dim != t.dim() - 2:
                raise MissingShardPatch("point clouds may only be sharded along their point dimension")
            return md
    return None


def _ring_blocks(block: torch.Tensor, sizes, group, rank: int):
    """Yield ``(owner, points of the owner)`` for all ranks of ``group``, own block first, others as they arrive."""
    n = len(sizes)
    cur = block.detach()
    yield rank, cur
    for step in range(1, n):
        owner = (rank - step) % n
        shape = list(block.shape)
        shape[0] = sizes[owner]
        cur = C.RingShift.apply(cur, tuple(shape), group, 1)
        yield owner, cur


def _merge_topk(best, cand, k: int):
    """Keep the ``k`` closest of two candidate sets ``(dist [Q, *], index [Q, *], xyz [Q, *, D])``."""
    if best is None:
        d, i, x = cand
    else:
        d, i, x = (torch.cat([a, b], dim=1) for a, b in zip(best, cand))
    if d.shape[1] > k:
        d, sel = torch.topk(d, k, dim=1, largest=False, sorted=True)
        i = torch.gather(i, 1, sel)
        x = torch.gather(x, 1, sel[..., None].expand(-1, -1, x.shape[-1]))
    return d, i, x


def _knn_rule(func, types, args, kwargs):
    names = ["points", "queries", "k"]
    a = dict(zip(names, args))
    a.update({key: v for key, v in kwargs.items() if key in names})
    points, queries, k = a["points"], a["queries"], int(a.get("k", 3))
    impl = {key: v for key, v in kwargs.items() if key not in names}
    ref = points if is_st(points) else queries
    mesh = ref._spec.mesh
    points = resolved(points) if is_st(points) else points
    queries = resolved(queries) if is_st(queries) else queries
    mp, mq = _row_shard(points), _row_shard(queries)
    q_loc = local(queries) if is_st(queries) else queries
    if mp is None:
        # every rank has all points: a local search, global indices as they are
        idx, dist_ = func(local(points) if is_st(points) else points, q_loc, k, **impl)
    else:
        group, r = mesh.get_group(mp), mesh.get_local_rank(mp)
        sizes = [int(s) for s in points._spec.sharding_sizes[mp]]
        starts = [sum(sizes[:i]) for i in range(len(sizes))]
        if k > sum(sizes):
            raise ValueError(f"k = {k} exceeds the {sum(sizes)} points of the cloud")
        best = None
        q_det = q_loc.detach()
        for owner, block in _ring_blocks(local(points), sizes, group, r):
            kk = min(k, block.shape[0])
            if kk == 0:
                continue
            bi, bd = func(block, q_det, kk, **impl)
            best = _merge_topk(best, (bd, bi + starts[owner], block[bi]), k)
        _, idx, xyz = best
        dist_ = (xyz - q_loc[:, None]).norm(dim=-1)              # differentiable in the queries
        if mq is None:
            # replicated queries: all ranks now hold the same exact answer (every block visited every rank)
            pass
    if mq is None and not is_st(queries):
        return idx, dist_
    placements = queries._spec.placements if is_st(queries) else [Replicate()] * mesh.ndim
    sizes_q = queries._spec.sharding_sizes if is_st(queries) else {}
    return wrap(idx, mesh, placements, sizes_q), wrap(dist_, mesh, placements, sizes_q)


def _radius_rule(func, types, args, kwargs):
    names = ["points", "queries", "radius", "max_points", "return_dists", "return_points"]
    a = dict(zip(names, args))
    a.update({key: v for key, v in kwargs.items() if key in names})
    impl = {key: v for key, v in kwargs.items() if key not in names}
    points, queries, radius = a["points"], a["queries"], float(a["radius"])
    max_points = a.get("max_points")
    want_d, want_p = bool(a.get("return_dists", False)), bool(a.get("return_points", False))
    ref = points if is_st(points) else queries
    mesh = ref._spec.mesh
    points = resolved(points) if is_st(points) else points
    queries = resolved(queries) if is_st(queries) else queries
    mp, mq = _row_shard(points), _row_shard(queries)
    q_loc = local(queries) if is_st(queries) else queries
    p_loc = local(points) if is_st(points) else points
    if q_loc.dim() != 2:
        raise MissingShardPatch("sharded radius_search takes unbatched [N, 3] clouds")
    placements = queries._spec.placements if is_st(queries) else [Replicate()] * mesh.ndim
    sizes_q = queries._spec.sharding_sizes if is_st(queries) else {}

    def pack(idx, pts, dists):
        out = [wrap(idx, mesh, placements, sizes_q) if idx.dim() == 2 and max_points is not None else idx]
        if want_p:
            out.append(wrap(pts, mesh, placements, sizes_q) if max_points is not None else pts)
        if want_d:
            out.append(wrap(dists, mesh, placements, sizes_q) if max_points is not None else dists)
        return out[0] if len(out) == 1 else tuple(out)

    if mp is None:
        res = func(p_loc, q_loc, radius, max_points, True, True, **impl)
        return pack(*res)
    if max_points is None:
        raise MissingShardPatch("the ragged (max_points=None) radius search needs the points whole on every rank")
    group, r = mesh.get_group(mp), mesh.get_local_rank(mp)
    sizes = [int(s) for s in points._spec.sharding_sizes[mp]]
    starts = [sum(sizes[:i]) for i in range(len(sizes))]
    best = None
    q_det = q_loc.detach()
    inf = torch.tensor(float("inf"), device=q_loc.device, dtype=q_loc.dtype)
    for owner, block in _ring_blocks(p_loc, sizes, group, r):
        if block.shape[0] == 0:
            continue
        bi, bp, bd = func(block, q_det, radius, max_points, True, True, **impl)
        # a slot without a neighbour holds index 0 and a zero vector: it is told apart by not being the point it names
        true_d = (bp - q_det[:, None]).norm(dim=-1)
        hit = (bp == block[bi]).all(dim=-1) & (true_d <= radius * (1 + 1e-6))
        bd = torch.where(hit, true_d, inf)
        best = _merge_topk(best, (bd, torch.where(hit, bi + starts[owner], torch.zeros_like(bi)), bp), max_points)
    d, idx, xyz = best
    ok = torch.isfinite(d)
    idx = torch.where(ok, idx, torch.zeros_like(idx))
    pts = xyz * ok[..., None]
    dists = torch.where(ok, (pts - q_loc[:, None]).norm(dim=-1), torch.zeros_like(d))
    return pack(idx, pts, dists)


ShardTensor.register_named_function_handler("knn", _knn_rule)
ShardTensor.register_named_function_handler("radius_search", _radius_rule)


def _sdf_rule(func, types, args, kwargs):
    """Signed distance of sharded query points to a mesh (reference: ``shard_utils/mesh_ops.py:27-120``): a distance
    query needs the whole surface, so a sharded mesh is gathered once; the queries stay where they are and the
    outputs (distance, closest point, closest face) are sharded like them."""
    names = ["mesh_vertices", "mesh_indices", "input_points"]
    a = dict(zip(names, args[:3]))
    a.update({key: kwargs[key] for key in names if key in kwargs})
    rest_args = args[3:]
    rest_kwargs = {key: v for key, v in kwargs.items() if key not in names}
    pts = a["input_points"]
    whole = [resolved(t).full_tensor() if is_st(t) else t for t in (a["mesh_vertices"], a["mesh_indices"])]
    if not is_st(pts):
        return func(whole[0], whole[1], pts, *rest_args, **rest_kwargs)
    pts = resolved(pts)
    out = func(whole[0], whole[1], local(pts), *rest_args, **rest_kwargs)
    mesh, spec = pts._spec.mesh, pts._spec
    outs = out if isinstance(out, tuple) else (out,)
    wrapped = tuple(wrap(o, mesh, spec.placements, spec.sharding_sizes) if torch.is_tensor(o) and o.dim() >= 1
                    and o.shape[0] == local(pts).shape[0] else o for o in outs)
    return wrapped if isinstance(out, tuple) else wrapped[0]


ShardTensor.register_named_function_handler("signed_distance_field", _sdf_rule)

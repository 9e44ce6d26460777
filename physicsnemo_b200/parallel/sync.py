"""One-time synchronisation of a module's parameters and buffers over a mesh.

Parity: ``physicsnemo/domain_parallel/sync.py:38-242`` — coalesced broadcast of plain parameters
and buffers from the first rank of a 1-D mesh, optional verification (metadata must match on
every rank; value check-sums compared through MIN / MAX all-reduces); modules holding meta
tensors or already-sharded parameters are refused.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

_BUCKET_BYTES = 250 * 1024 * 1024


@torch.no_grad()
def sync_module_over_mesh(module: torch.nn.Module, mesh, src_rank: int = 0, verify: bool = False) -> torch.nn.Module:
    """Make every rank of the (1-D) ``mesh`` hold the parameters / buffers of its rank ``src_rank``."""
    if mesh.ndim != 1:
        raise ValueError("sync_module_over_mesh expects a 1-D mesh (slice a sub-mesh by name)")
    group = mesh.get_group()
    if dist.get_world_size(group) == 1:
        return module
    tensors = []
    for name, t in list(module.named_parameters()) + list(module.named_buffers()):
        if t.is_meta:
            raise ValueError(f"'{name}' is a meta tensor; materialise the module before synchronising")
        if type(t).__name__ in ("DTensor", "ShardTensor") or type(getattr(t, "data", t)).__name__ in ("DTensor", "ShardTensor"):
            raise ValueError(f"'{name}' is already distributed; sync_module_over_mesh handles plain tensors only")
        tensors.append((name, t))
    if verify:
        meta = [(n, tuple(t.shape), str(t.dtype)) for n, t in tensors]
        gathered = [None] * dist.get_world_size(group)
        dist.all_gather_object(gathered, meta, group=group)
        if any(g != gathered[0] for g in gathered):
            raise RuntimeError("module structure differs between ranks of the mesh")
    src_global = dist.get_global_rank(group, src_rank)
    bucket, nbytes = [], 0

    def flush():
        nonlocal bucket, nbytes
        if not bucket:
            return
        by_dtype = {}
        for t in bucket:
            by_dtype.setdefault(t.dtype, []).append(t)
        for dt, ts in by_dtype.items():
            flat = torch.cat([t.detach().reshape(-1) for t in ts])
            dist.broadcast(flat, src=src_global, group=group)
            off = 0
            for t in ts:
                t.detach().copy_(flat[off:off + t.numel()].reshape(t.shape))
                off += t.numel()
        bucket, nbytes = [], 0

    for _, t in tensors:
        bucket.append(t)
        nbytes += t.numel() * t.element_size()
        if nbytes >= _BUCKET_BYTES:
            flush()
    flush()
    if verify:
        sums = torch.stack([t.detach().double().sum() for _, t in tensors if t.is_floating_point()]) if tensors else None
        if sums is not None and sums.numel():
            lo, hi = sums.clone(), sums.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=group)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=group)
            if not torch.equal(lo, hi):
                raise RuntimeError("parameter check-sums differ between ranks after synchronisation")
    return module

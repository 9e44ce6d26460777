"""Attention as two tcgen05 GEMMs around a row softmax, forward and backward, with sequence-sharded keys / values staged
over peer memory.

For head widths that the TMEM flash kernel does not cover — above all the single 512-wide head over 16 384 tokens of the
SongUNet bottleneck — the products ``Q Kᵀ`` and ``P V`` are compute bound (arithmetic intensity ≈ D), so computing
them with the library's own GEMM kernel around a materialised bf16 score matrix costs one extra pass over that matrix
and nothing else: ``S = Q Kᵀ`` (``gemm_tn``), ``P = softmax(scale · S)`` in place (``pnm_softmax_rows_fwd``), ``O = P V``
(``gemm_tn`` against ``Vᵀ``).  The backward is four GEMMs and the softmax Jacobian kernel:
``dV = Pᵀ dO`` and ``dK = dSᵀ Q`` (``gemm_nt``), ``dP = dO Vᵀ`` and ``dQ = dS K`` (``gemm_tn``),
``dS = scale · P ∘ (dP − rowsum(dP ∘ P))``.  No library attention or GEMM is called.

Sequence sharding (``sharded_attention``; reference: ``RingSDPA`` in
``physicsnemo/domain_parallel/shard_utils/attention_patches.py:136-503``, which rotates K / V blocks with send / recv and
merges block results in log space).  Every rank publishes its K / V block in symmetric memory; a side stream pulls the
peers' blocks (each crosses NVLink once) while the tensor cores already work on the rank's own block, and the score
matrix is filled owner by owner, so the softmax runs once over complete rows and nothing is merged.  In the backward
every rank computes its queries' contributions to ``dK`` / ``dV`` of ALL keys and the owner of a block sums the
contributions with direct peer loads (pull model, fixed order, no atomics).
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from . import _lib
from . import gemm as G


def _lib_sm():
    lib = _lib.load(required=True)
    if not getattr(lib, "_softmax_rows_declared", False):
        c = ctypes
        vp, i, ll, f = c.c_void_p, c.c_int, c.c_longlong, c.c_float
        lib.pnm_softmax_rows_fwd.argtypes = [vp, ll, ll, i, f, vp, vp]
        lib.pnm_softmax_rows_bwd.argtypes = [vp, ll, vp, ll, ll, i, f, vp]
        lib.pnm_softmax_rows_fwd.restype = lib.pnm_softmax_rows_bwd.restype = i
        lib._softmax_rows_declared = True
    return lib


def _st():
    return torch.cuda.current_stream().cuda_stream


def softmax_rows_(s: torch.Tensor, scale: float, lse: Optional[torch.Tensor] = None) -> torch.Tensor:
    """In place: ``s[r, :] = softmax(scale * s[r, :])`` for a bf16 matrix with contiguous rows."""
    rows, L = s.shape
    rc = _lib_sm().pnm_softmax_rows_fwd(s.data_ptr(), s.stride(0), rows, L, float(scale), None if lse is None else lse.data_ptr(), _st())
    G._check(rc, "pnm_softmax_rows_fwd")
    G.launch_count += 1
    return s


def softmax_rows_bwd_(p: torch.Tensor, dp: torch.Tensor, scale: float) -> torch.Tensor:
    """In place over ``dp``: ``scale * p * (dp - rowsum(dp * p))``."""
    rows, L = p.shape
    rc = _lib_sm().pnm_softmax_rows_bwd(p.data_ptr(), p.stride(0), dp.data_ptr(), dp.stride(0), rows, L, float(scale), _st())
    G._check(rc, "pnm_softmax_rows_bwd")
    G.launch_count += 1
    return dp


def supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    if not (q.is_cuda and q.dim() >= 3 and k.shape == v.shape and q.shape[:-2] == k.shape[:-2] and q.shape[-1] == k.shape[-1]):
        return False
    D, Sq, Skv = q.shape[-1], q.shape[-2], k.shape[-2]
    return D % 8 == 0 and Skv % 8 == 0 and Sq > 0 and Skv > 0 and _lib.available()


def _bh(t: torch.Tensor) -> torch.Tensor:
    """``[..., S, D]`` → contiguous bf16 ``[BH, S, D]``."""
    t = t.reshape(-1, t.shape[-2], t.shape[-1])
    if t.dtype != torch.bfloat16:
        t = t.to(torch.bfloat16)
    return t.contiguous()


class _GemmAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale: float):
        q3, k3, v3 = _bh(q), _bh(k), _bh(v)
        BH, Sq, D = q3.shape
        Skv = k3.shape[1]
        P = torch.empty(BH, Sq, Skv, dtype=torch.bfloat16, device=q.device)
        out = torch.empty(BH, Sq, D, dtype=torch.bfloat16, device=q.device)
        for b in range(BH):
            G.gemm_tn(q3[b], k3[b], out=P[b])
            softmax_rows_(P[b], scale)
            G.gemm_tn(P[b], v3[b].t().contiguous(), out=out[b])
        ctx.save_for_backward(q3, k3, v3, P)
        ctx.scale, ctx.shapes, ctx.dtypes = scale, (q.shape, k.shape), (q.dtype, k.dtype, v.dtype)
        return out.reshape(q.shape).to(q.dtype)

    @staticmethod
    def backward(ctx, do):
        q3, k3, v3, P = ctx.saved_tensors
        BH, Sq, D = q3.shape
        Skv = k3.shape[1]
        do3 = _bh(do)
        dq = torch.empty_like(q3)
        dk = torch.zeros(BH, Skv, D, dtype=torch.float32, device=do.device)
        dv = torch.zeros_like(dk)
        dP = torch.empty(Sq, Skv, dtype=torch.bfloat16, device=do.device)
        for b in range(BH):
            G.gemm_nt(P[b], do3[b], out=dv[b])
            G.gemm_tn(do3[b], v3[b], out=dP)
            softmax_rows_bwd_(P[b], dP, ctx.scale)
            G.gemm_tn(dP, k3[b].t().contiguous(), out=dq[b])
            G.gemm_nt(dP, q3[b], out=dk[b])
        qs, ks = ctx.shapes
        dt = ctx.dtypes
        return dq.reshape(qs).to(dt[0]), dk.reshape(ks).to(dt[1]), dv.reshape(ks).to(dt[2]), None


def gemm_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
    """``softmax(scale · q kᵀ) v`` for ``[..., S, D]`` tensors on the library's GEMM and softmax kernels (bf16 compute)."""
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    return _GemmAttention.apply(q, k, v, scale)


# ------------------------------------------------------------------------------------------------- sequence sharded
class KVExchange:
    """Symmetric buffers of one group for ``sharded_attention``: the published K / V blocks (bf16) and the partial
    ``dK`` / ``dV`` of all keys (fp32), plus the side stream that pulls the peers' blocks."""

    def __init__(self, group, kv_elems: int, grad_floats: int):
        from ..parallel.peer import PeerRegions

        self.kv = PeerRegions(group, region_floats=kv_elems // 2 + 64, n_regions=2)
        self.grad = PeerRegions(group, region_floats=grad_floats + 64, n_regions=2)
        self.world, self.rank = self.kv.rt.world, self.kv.rt.rank
        self.stream = torch.cuda.Stream()
        self.kv_elems, self.grad_floats = kv_elems, grad_floats


_exchanges = {}


def _exchange_for(group, kv_elems: int, grad_floats: int) -> KVExchange:
    key = (group.group_name, kv_elems, grad_floats)
    ex = _exchanges.get(key)
    if ex is None:
        ex = KVExchange(group, kv_elems, grad_floats)
        _exchanges[key] = ex
    return ex


def _gather_kv(ex: KVExchange, k3: torch.Tensor, v3: torch.Tensor):
    """Publish this rank's ``[BH, S_loc, D]`` blocks and pull everybody's into ``[world, BH, S_loc, D]`` (K and V).

    Returns ``(K_all, V_all, events)``: ``events[o]`` fires when owner ``o``'s block has landed (own block: at once)."""
    rt = ex.kv.rt
    n = k3.numel()
    view, ptrs = ex.kv.region(n, k3.device)                     # n bf16 for K followed by n bf16 for V = n floats
    flat = view.view(torch.bfloat16)
    flat[:n].view_as(k3).copy_(k3)
    flat[n:2 * n].view_as(v3).copy_(v3)
    peer = ex.kv.publish()
    epoch = peer[3]
    K_all = torch.empty(ex.world, *k3.shape, dtype=torch.bfloat16, device=k3.device)
    V_all = torch.empty_like(K_all)
    K_all[ex.rank].copy_(k3)
    V_all[ex.rank].copy_(v3)
    events = [None] * ex.world
    cur = torch.cuda.current_stream()
    ex.stream.wait_stream(cur)
    loop = len(ptrs) != ex.world                                 # loopback: no peer traffic, the blocks stay this rank's own
    with torch.cuda.stream(ex.stream):
        for i in range(1, ex.world):
            o = (ex.rank + i) % ex.world
            if loop:
                K_all[o].copy_(k3)
                V_all[o].copy_(v3)
            else:
                rt.pull(ptrs[o], K_all[o], n * 2, epoch, flag_from=o, max_ctas=32)
                rt.pull(ptrs[o] + n * 2, V_all[o], n * 2, epoch, flag_from=o, max_ctas=32)
            ev = torch.cuda.Event()
            ev.record(ex.stream)
            events[o] = ev
    return K_all, V_all, events


class _ShardedAttention(torch.autograd.Function):
    """q, k, v: this rank's ``[..., S_loc, D]`` slices of sequences sharded evenly over ``group`` (no mask, no dropout)."""

    @staticmethod
    def forward(ctx, q, k, v, scale: float, group):
        q3, k3, v3 = _bh(q), _bh(k), _bh(v)
        BH, Sq, D = q3.shape
        Sl = k3.shape[1]
        ex = _exchange_for(group, 2 * k3.numel(), 2 * BH * Sl * D * torch.distributed.get_world_size(group))
        W = ex.world
        K_all, V_all, events = _gather_kv(ex, k3, v3)
        P = torch.empty(BH, Sq, W * Sl, dtype=torch.bfloat16, device=q.device)
        out = torch.empty(BH, Sq, D, dtype=torch.bfloat16, device=q.device)
        cur = torch.cuda.current_stream()
        for i in range(W):                                        # own block first: the pulls of the others are in flight
            o = (ex.rank + i) % W
            if events[o] is not None:
                cur.wait_event(events[o])
            for b in range(BH):
                G.gemm_tn(q3[b], K_all[o, b], out=P[b, :, o * Sl:(o + 1) * Sl])
        VT = V_all.permute(1, 3, 0, 2).reshape(BH, D, W * Sl).contiguous()   # [BH, D, all keys]
        for b in range(BH):
            softmax_rows_(P[b], scale)
            G.gemm_tn(P[b], VT[b], out=out[b])
        ctx.save_for_backward(q3, K_all, V_all, P)
        ctx.scale, ctx.group, ctx.ex = scale, group, ex
        ctx.shapes, ctx.dtypes = (q.shape, k.shape), (q.dtype, k.dtype, v.dtype)
        return out.reshape(q.shape).to(q.dtype)

    @staticmethod
    def backward(ctx, do):
        q3, K_all, V_all, P = ctx.saved_tensors
        ex = ctx.ex
        W = ex.world
        BH, Sq, D = q3.shape
        Sl = K_all.shape[2]
        do3 = _bh(do)
        dq = torch.empty_like(q3)
        # partial dK / dV of ALL keys, laid out [owner][dK | dV][BH, Sl, D] so that an owner's share is one contiguous block
        block = 2 * BH * Sl * D
        view, ptrs = ex.grad.region(W * block, do.device)
        view.zero_()
        part = view[: W * block].view(W, 2, BH, Sl, D)
        dP = torch.empty(Sq, W * Sl, dtype=torch.bfloat16, device=do.device)
        Vf = V_all.permute(1, 0, 2, 3).reshape(BH, W * Sl, D)      # views when BH == 1, copies otherwise
        KT = K_all.permute(1, 3, 0, 2).reshape(BH, D, W * Sl).contiguous()
        for b in range(BH):
            G.gemm_tn(do3[b], Vf[b].contiguous(), out=dP)
            for o in range(W):
                G.gemm_nt(P[b, :, o * Sl:(o + 1) * Sl], do3[b], out=part[o, 1, b])
            softmax_rows_bwd_(P[b], dP, ctx.scale)
            G.gemm_tn(dP, KT[b], out=dq[b])
            for o in range(W):
                G.gemm_nt(dP[:, o * Sl:(o + 1) * Sl], q3[b], out=part[o, 0, b])
        peer = ex.grad.publish()
        mine = torch.empty(2, BH, Sl, D, dtype=torch.float32, device=do.device)
        _sum_blocks(ex, mine, ptrs, block, peer)
        qs, ks = ctx.shapes
        dt = ctx.dtypes
        return dq.reshape(qs).to(dt[0]), mine[0].reshape(ks).to(dt[1]), mine[1].reshape(ks).to(dt[2]), None, None


def _sum_blocks(ex: KVExchange, dst: torch.Tensor, ptrs, block: int, peer) -> None:
    """``dst = Σ_r region_r[rank * block : (rank + 1) * block]`` after every rank's flag of the call (direct peer loads)."""
    lib = _lib.load(required=True)
    if not getattr(lib, "_sumblocks_declared", False):
        c = ctypes
        lib.pnm_peer_sum_blocks.argtypes = [c.c_void_p, c.c_void_p, c.c_longlong, c.c_int, c.c_void_p, c.c_int, c.c_int, c.c_uint,
                                            c.c_longlong, c.c_double, c.c_void_p, c.c_void_p, c.c_int]
        lib.pnm_peer_sum_blocks.restype = c.c_int
        lib._sumblocks_declared = True
    loop = len(ptrs) != ex.world
    srcs = [p + (0 if loop else ex.rank) * block * 4 for p in ptrs]
    srcs = srcs + [srcs[0]] * (8 - len(srcs))
    bases, rank, world, epoch, cap, budget, ebase = peer
    rc = lib.pnm_peer_sum_blocks(dst.data_ptr(), (ctypes.c_void_p * 8)(*srcs), block, 1, bases, rank, world, epoch, cap, budget,
                                 ebase, _st(), 0)
    G._check(rc, "pnm_peer_sum_blocks")
    G.launch_count += 1


def sharded_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group, scale: Optional[float] = None) -> torch.Tensor:
    """Attention of this rank's queries over the keys / values of ALL ranks of ``group`` (equal shards, no mask)."""
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    return _ShardedAttention.apply(q, k, v, scale, group)

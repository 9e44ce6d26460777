"""Scaled dot-product attention on sequence-sharded inputs.

Parity: ``physicsnemo/domain_parallel/shard_utils/attention_patches.py`` — cases (``:965-1140``):
K/V replicated → local attention; Q, K, V sharded along the sequence dim (dim -2) → ring
attention (K/V blocks travel around the ring, block results merged with running max /
log-sum-exp, ``:136-503``); Q replicated with K/V sharded → local attention per shard, merged by
an all-reduce of the (max, sum, output) triple (``ReplicatedQSDPA`` ``:836-962``).  No causal
masks, no dropout, no grouped-query attention on the sharded paths, one mesh dimension.

The ring is written with differentiable ring shifts, so the backward pass (K/V gradients
travelling back to their owners) follows from autograd.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch.distributed.tensor import Replicate, Shard

from .. import collectives as C
from ._common import MissingShardPatch, NO_TF, ShardTensor, is_st, local, register, resolved, wrap


def _flash_block_ok(q, k, v) -> bool:
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        return False
    if not q.is_cuda:
        return False
    from ...ops import attention as _fa

    return _fa.supported(q, k, v)


def _peer_attention_ok(q, k, v, k_sizes, q_sizes, group) -> bool:
    """Sequence-sharded attention on the library's GEMM / softmax kernels with K / V staged over peer memory: CUDA,
    16-bit tensors, every rank holding the same number of keys (and of queries), peer memory available."""
    if not (q.is_cuda and q.dtype in (torch.bfloat16, torch.float16)):
        return False
    if len({tuple(s) if isinstance(s, (tuple, list, torch.Size)) else s for s in k_sizes}) != 1:
        return False
    if len({tuple(s) if isinstance(s, (tuple, list, torch.Size)) else s for s in q_sizes}) != 1:
        return False
    from ...ops import gemm_attention as _ga
    from ..peer import peer_available

    return _ga.supported(q, k, v) and peer_available(q)


def _block(q, k, v, scale, mask=None):
    """Un-normalised attention of one K/V block: (max, sumexp, weighted values), fp32."""
    acc = torch.float32 if q.dtype in (torch.bfloat16, torch.float16) else q.dtype
    if mask is None and _flash_block_ok(q, k, v):
        # flash kernel: normalised output + log-sum-exp, i.e. the triple (lse, 1, out); no S matrix in memory.
        # Only without autograd: the merge differentiates through the log-sum-exp, which the kernel does not.
        from ...ops import attention as _fa

        out, lse = _fa.flash_forward(q, k, v, False, scale)
        return lse.unsqueeze(-1), torch.ones_like(lse).unsqueeze(-1), out.to(acc)
    s = torch.matmul(q, k.transpose(-2, -1)).to(acc) * scale
    if mask is not None:
        s = s + mask
    m = s.amax(dim=-1, keepdim=True)
    p = torch.exp(s - m)
    return m, p.sum(dim=-1, keepdim=True), torch.matmul(p.to(v.dtype), v).to(acc)


def _merge(acc, new):
    if acc is None:
        return new
    m0, l0, o0 = acc
    m1, l1, o1 = new
    m = torch.maximum(m0, m1)
    a0, a1 = torch.exp(m0 - m), torch.exp(m1 - m)
    return m, l0 * a0 + l1 * a1, o0 * a0 + o1 * a1


@register(F.scaled_dot_product_attention)
def _sdpa(func, types, args, kwargs):
    names = ["query", "key", "value", "attn_mask", "dropout_p", "is_causal", "scale", "enable_gqa"]
    a = dict(zip(names, args))
    a.update(kwargs)
    q, k, v = a["query"], a["key"], a["value"]
    ref = next(t for t in (q, k, v) if is_st(t))
    mesh = ref._spec.mesh
    q, k, v = (resolved(t) if is_st(t) else t for t in (q, k, v))

    def seq_shard(t):
        if not is_st(t):
            return None
        for md, p in enumerate(t._spec.placements):
            if isinstance(p, Shard) and p.dim == t.dim() - 2:
                return md
        return None

    mq, mk, mv = seq_shard(q), seq_shard(k), seq_shard(v)
    if mk is None and mv is None:
        # keys / values are whole on every rank: plain attention on the local queries
        from ..local_rule import apply_local_rule

        return apply_local_rule(func, args, kwargs)
    if a.get("is_causal", False) or a.get("dropout_p", 0.0) or a.get("enable_gqa", False):
        raise MissingShardPatch("sharded attention supports neither causal masks, dropout nor GQA")
    if mk != mv:
        raise MissingShardPatch("key and value must be sharded alike")
    mask = a.get("attn_mask")
    if mask is not None:
        raise MissingShardPatch("attention masks on sequence-sharded keys are not supported")
    md = mk
    group = mesh.get_group(md)
    n = mesh.size(md)
    lq, lk, lv = local(q), local(k), local(v)
    scale = a.get("scale") or 1.0 / math.sqrt(lq.shape[-1])
    k_sizes = k._spec.sharding_sizes[md]
    r = mesh.get_local_rank(md)
    with NO_TF():
        if mq is None:
            # replicated queries: every rank attends to its K/V shard, then the triples are merged
            m, l, o = _block(lq, lk, lv, scale)
            gm = _GlobalMax.apply(m, group)
            w = torch.exp(m - gm)
            packed = torch.cat([l * w, o * w], dim=-1)
            packed = C.AllReduceSum.apply(packed, group)
            out = (packed[..., 1:] / packed[..., :1]).to(lq.dtype)
            spec = q._spec if is_st(q) else None
            placements = spec.placements if spec else [Replicate()] * mesh.ndim
            return wrap(out, mesh, placements, spec.sharding_sizes if spec else {})
        if mq != md:
            raise MissingShardPatch("queries and keys are sharded over different mesh dimensions")
        if _peer_attention_ok(lq, lk, lv, k_sizes, q._spec.sharding_sizes[md], group):
            # equal shards on CUDA: K / V blocks pulled over peer memory under the first block's GEMMs, softmax once
            from ...ops import gemm_attention as _ga

            out = _ga.sharded_attention(lq, lk, lv, group, scale)
            return wrap(out, mesh, q._spec.placements, q._spec.sharding_sizes)
        acc = None
        kb, vb = lk, lv
        for step in range(n):
            acc = _merge(acc, _block(lq, kb, vb, scale))
            if step < n - 1:
                src = (r - step - 1) % n  # owner of the block that arrives next
                ks, vs = list(lk.shape), list(lv.shape)
                ks[-2] = vs[-2] = k_sizes[src]
                kb = C.RingShift.apply(kb, tuple(ks), group, 1)
                vb = C.RingShift.apply(vb, tuple(vs), group, 1)
        m, l, o = acc
        out = (o / l).to(lq.dtype)
    return wrap(out, mesh, q._spec.placements, q._spec.sharding_sizes)


class _GlobalMax(torch.autograd.Function):
    """Element-wise max over the group; treated as a constant in the backward (it cancels)."""

    @staticmethod
    def forward(ctx, m, group):
        import torch.distributed as dist

        out = m.contiguous().clone()
        dist.all_reduce(out, op=dist.ReduceOp.MAX, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        return torch.zeros_like(g), None

"""GroupNorm with an optional fused SiLU on the library's kernels (``csrc/groupnorm.cu``).

Covers bf16 / fp32 tensors ``(B, C, *spatial)`` in channels-first or channels-last memory format;
statistics are fp32 and the backward recomputes the activation derivative, so only ``x``, the
per-group mean and rstd are kept for backward (no pre-activation tensor).  ``supported(x)`` tells
whether the kernels cover a tensor; callers fall back to ``F.group_norm`` otherwise (CPU, other
dtypes, spatial sizes that are not a multiple of the 16-byte vector in channels-first layout).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from . import gemm as _g

_DT = {torch.bfloat16: 0, torch.float32: 1}


def _lib_gn():
    lib = _lib.load(required=True)
    if not getattr(lib, "_gn_declared", False):
        c = ctypes
        vp, i, ll, f = c.c_void_p, c.c_int, c.c_longlong, c.c_float
        lib.pnm_groupnorm_scratch_floats.argtypes = [i, i, i, i]
        lib.pnm_groupnorm_scratch_floats.restype = ll
        lib.pnm_groupnorm_fwd.argtypes = [vp] * 7 + [i, i, ll, i, i, i, i, i, f, vp]
        lib.pnm_groupnorm_bwd.argtypes = [vp] * 10 + [i, i, ll, i, i, i, i, i, vp]
        lib.pnm_groupnorm_fwd.restype = lib.pnm_groupnorm_bwd.restype = i
        u, d = c.c_uint, c.c_double
        peer = [vp, i, i, u, ll, d, vp, vp, vp]   # bases, rank, world, epoch, capacity, budget_s, epoch_base, counter, stream
        lib.pnm_groupnorm_fwd_sharded.argtypes = [vp] * 7 + [i, i, ll, ll, i, i, i, i, f] + peer
        lib.pnm_groupnorm_bwd_sharded.argtypes = [vp] * 10 + [i, i, ll, ll, i, i, i, i] + peer
        lib.pnm_groupnorm_fwd_sharded.restype = lib.pnm_groupnorm_bwd_sharded.restype = i
        lib._gn_declared = True
    return lib


def _layout(x: torch.Tensor):
    """0 channels-first, 1 channels-last, None if neither (the caller makes the tensor contiguous)."""
    if x.is_contiguous():
        return 0
    if x.dim() == 4 and x.is_contiguous(memory_format=torch.channels_last):
        return 1
    if x.dim() == 5 and x.is_contiguous(memory_format=torch.channels_last_3d):
        return 1
    return None


def supported(x: torch.Tensor, num_groups: int) -> bool:
    if not x.is_cuda or x.dtype not in _DT or x.dim() < 3 or x.numel() == 0:
        return False
    B, C = x.shape[:2]
    hw = x.numel() // (B * C)
    v = 8 if x.dtype == torch.bfloat16 else 4
    lay = _layout(x)
    if lay == 1:
        return C % v == 0 and C // v <= 256 and C <= 6144 and B <= 65535 and C % num_groups == 0
    return hw % v == 0 and B * C <= 65535 and C % num_groups == 0


def _slices(B: int, C: int, hw: int, layout: int, v: int) -> int:
    target = 4 * 148
    if layout == 0:
        base, most = B * C, max(1, (hw // v) // 256)
        return int(max(1, min(128, most, -(-target // base))))
    # channels-last: the grid is (S, B), so a batch of one needs hundreds of slices to fill 148 SMs with 4 CTAs each; the
    # slices' partials are folded by the last CTA of the statistics kernels, not by their consumers
    ppi = max(1, 256 // (C // v))
    most = max(1, hw // (8 * ppi))
    return int(max(1, min(2048, most, -(-target // B))))


class _GroupNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, num_groups: int, eps: float, silu: bool):
        lay = _layout(x)
        if lay is None:
            x = x.contiguous()
            lay = 0
        B, C = x.shape[:2]
        hw = x.numel() // (B * C)
        v = 8 if x.dtype == torch.bfloat16 else 4
        S = _slices(B, C, hw, lay, v)
        lib = _lib_gn()
        dev = x.device
        gamma = weight.detach().float().contiguous()
        beta = bias.detach().float().contiguous()
        y = torch.empty_like(x)                       # preserves the memory format
        mean = torch.empty(B * num_groups, dtype=torch.float32, device=dev)
        rstd = torch.empty_like(mean)
        scratch = torch.empty(lib.pnm_groupnorm_scratch_floats(B, C, num_groups, S), dtype=torch.float32, device=dev)
        err = lib.pnm_groupnorm_fwd(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y.data_ptr(), mean.data_ptr(),
                                    rstd.data_ptr(), scratch.data_ptr(), B, C, hw, num_groups, S, lay, _DT[x.dtype],
                                    int(silu), float(eps), torch.cuda.current_stream().cuda_stream)
        if err:
            raise RuntimeError(f"pnm_groupnorm_fwd failed ({err})")
        _g.launch_count += 2
        ctx.save_for_backward(x, gamma, beta, mean, rstd)
        ctx.cfg = (num_groups, S, lay, bool(silu), weight.dtype, bias.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, gamma, beta, mean, rstd = ctx.saved_tensors
        G, S, lay, silu, wdt, bdt = ctx.cfg
        B, C = x.shape[:2]
        hw = x.numel() // (B * C)
        # dy must share x's memory format
        if lay == 0:
            dy = dy.contiguous()
        else:
            dy = dy.contiguous(memory_format=torch.channels_last if x.dim() == 4 else torch.channels_last_3d)
        if dy.dtype != x.dtype:
            dy = dy.to(x.dtype)
        lib = _lib_gn()
        dev = x.device
        dx = torch.empty_like(x)
        dgb = torch.zeros(2, C, dtype=torch.float32, device=dev)
        scratch = torch.empty(lib.pnm_groupnorm_scratch_floats(B, C, G, S), dtype=torch.float32, device=dev)
        err = lib.pnm_groupnorm_bwd(x.data_ptr(), dy.data_ptr(), gamma.data_ptr(), beta.data_ptr(), mean.data_ptr(),
                                    rstd.data_ptr(), dx.data_ptr(), dgb[0].data_ptr(), dgb[1].data_ptr(), scratch.data_ptr(),
                                    B, C, hw, G, S, lay, _DT[x.dtype], int(silu), torch.cuda.current_stream().cuda_stream)
        if err:
            raise RuntimeError(f"pnm_groupnorm_bwd failed ({err})")
        _g.launch_count += 3
        return dx, dgb[0].to(wdt), dgb[1].to(bdt), None, None, None


def group_norm(x: torch.Tensor, num_groups: int, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5,
               silu: bool = False) -> torch.Tensor:
    """``silu(group_norm(x))`` (or plain ``group_norm``) on the CUDA kernels; ``supported(x, G)`` must hold."""
    return _GroupNormFn.apply(x, weight, bias, int(num_groups), float(eps), bool(silu))


class _GroupNormShardedFn(torch.autograd.Function):
    """GroupNorm(+SiLU) of one rank's rows of a row-sharded channels-last image; moments over all ranks' rows.

    The (B, G) sums cross the ranks inside the normalising kernels (``csrc/groupnorm.cu``, "_sh" kernels): one peer
    publication + flag per pass, read by direct peer loads — the reference does one packed all-reduce forward and
    two backward (``physicsnemo/domain_parallel/shard_utils/normalization_patches.py:47-349``).
    """

    @staticmethod
    def forward(ctx, x, weight, bias, num_groups: int, eps: float, silu: bool, rt, hw_global: int):
        if _layout(x) != 1:
            x = x.contiguous(memory_format=torch.channels_last)
        B, C = x.shape[:2]
        hw = x.numel() // (B * C)
        v = 8 if x.dtype == torch.bfloat16 else 4
        S = _slices(B, C, hw, 1, v)
        lib = _lib_gn()
        dev = x.device
        gamma = weight.detach().float().contiguous()
        beta = bias.detach().float().contiguous()
        y = torch.empty_like(x)
        mean = torch.empty(B * num_groups, dtype=torch.float32, device=dev)
        rstd = torch.empty_like(mean)
        scratch = torch.empty(lib.pnm_groupnorm_scratch_floats(B, C, num_groups, S), dtype=torch.float32, device=dev)
        counter = _counter(rt)
        err = lib.pnm_groupnorm_fwd_sharded(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y.data_ptr(), mean.data_ptr(),
                                            rstd.data_ptr(), scratch.data_ptr(), B, C, hw, int(hw_global), num_groups, S,
                                            _DT[x.dtype], int(silu), float(eps), *rt.peer_args(rt.next_epoch()),
                                            counter.data_ptr(), torch.cuda.current_stream().cuda_stream)
        if err:
            raise RuntimeError(f"pnm_groupnorm_fwd_sharded failed ({err})")
        _g.launch_count += 3
        ctx.save_for_backward(x, gamma, beta, mean, rstd)
        ctx.cfg = (num_groups, S, bool(silu), weight.dtype, bias.dtype, rt, int(hw_global))
        return y

    @staticmethod
    def backward(ctx, dy):
        x, gamma, beta, mean, rstd = ctx.saved_tensors
        G, S, silu, wdt, bdt, rt, hw_global = ctx.cfg
        B, C = x.shape[:2]
        hw = x.numel() // (B * C)
        dy = dy.contiguous(memory_format=torch.channels_last)
        if dy.dtype != x.dtype:
            dy = dy.to(x.dtype)
        lib = _lib_gn()
        dev = x.device
        dx = torch.empty_like(x)
        dgb = torch.zeros(2, C, dtype=torch.float32, device=dev)
        scratch = torch.empty(lib.pnm_groupnorm_scratch_floats(B, C, G, S), dtype=torch.float32, device=dev)
        err = lib.pnm_groupnorm_bwd_sharded(x.data_ptr(), dy.data_ptr(), gamma.data_ptr(), beta.data_ptr(), mean.data_ptr(),
                                            rstd.data_ptr(), dx.data_ptr(), dgb[0].data_ptr(), dgb[1].data_ptr(),
                                            scratch.data_ptr(), B, C, hw, hw_global, G, S, _DT[x.dtype], int(silu),
                                            *rt.peer_args(rt.next_epoch()), _counter(rt).data_ptr(),
                                            torch.cuda.current_stream().cuda_stream)
        if err:
            raise RuntimeError(f"pnm_groupnorm_bwd_sharded failed ({err})")
        _g.launch_count += 4
        return dx, dgb[0].to(wdt), dgb[1].to(bdt), None, None, None, None, None


def _counter(rt) -> torch.Tensor:
    c = getattr(rt, "_gn_counter", None)
    if c is None:
        c = torch.zeros(4, dtype=torch.int32, device=rt.device)
        rt._gn_counter = c
    return c


def sharded_supported(x_local: torch.Tensor, num_groups: int, rt) -> bool:
    if not x_local.is_cuda or x_local.dtype not in _DT or x_local.dim() != 4 or x_local.numel() == 0:
        return False
    B, C = x_local.shape[:2]
    v = 8 if x_local.dtype == torch.bfloat16 else 4
    return (C % v == 0 and C // v <= 256 and C <= 6144 and B <= 65535 and C % num_groups == 0
            and 2 * B * num_groups <= rt.capacity)


def group_norm_sharded(x_local: torch.Tensor, num_groups: int, weight: torch.Tensor, bias: torch.Tensor, eps: float,
                       silu: bool, rt, hw_global: int) -> torch.Tensor:
    """GroupNorm (+ SiLU) of this rank's rows ``x_local [B, C, H_local, W]`` with statistics over the whole image
    (``hw_global`` pixels per image); ``rt`` is the ``PeerRuntime`` of the sharding group."""
    return _GroupNormShardedFn.apply(x_local, weight, bias, int(num_groups), float(eps), bool(silu), rt, int(hw_global))

"""tcgen05 GEMM primitives and the autograd functions built on them.

``gemm_tn``  : ``C = epilogue(A @ B.T)``  — forward / data-gradient GEMMs (``csrc/gemm_tn.cuh``)
``gemm_nt``  : ``out += A.T @ B``         — weight gradients and token reductions (``csrc/gemm_nt.cuh``)
``mlp_chain``: ``Linear → act → … → Linear (+ residual)`` as one autograd node whose
backward fuses ``act'(z)`` into the data-gradient GEMM epilogue and obtains the bias
gradient from the same pass as the weight gradient.

These replace cuBLAS ``F.linear`` + separate activation kernels of the reference
(``physicsnemo/nn/module/mlp_layers.py:171-173``, ``mesh_graph_mlp.py:120-206``).
Every function has a plain PyTorch path (CPU, fp32, or when the library is not loaded)
that doubles as the numerical oracle in the tests.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from . import _lib

ACT_NONE, ACT_GELU, ACT_SILU, ACT_RELU, ACT_SOFTMAX64 = 0, 1, 2, 3, 4
AUX_NONE, AUX_ADD, AUX_DGELU, AUX_DSOFTMAX, AUX_DSILU, AUX_DRELU = 0, 1, 2, 3, 4, 5
_DACT = {ACT_GELU: AUX_DGELU, ACT_SILU: AUX_DSILU, ACT_RELU: AUX_DRELU}

launch_count = 0  # number of library kernels launched by this process (bench bookkeeping)


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _check(code: int, what: str):
    if code != 0:
        raise RuntimeError(f"{what} failed with code {code}")


def _rowmajor2d(t: torch.Tensor) -> torch.Tensor:
    """2-D view whose last dim is contiguous and whose row stride is a multiple of 8."""
    assert t.dim() == 2
    if t.stride(1) != 1 or t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
        t = t.contiguous()
    return t


def gemm_tn(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    bias: Optional[torch.Tensor] = None,
    scale: Optional[torch.Tensor] = None,
    act: int = ACT_NONE,
    aux: Optional[torch.Tensor] = None,
    aux_mode: int = AUX_NONE,
    a2: Optional[torch.Tensor] = None,
    a3: Optional[torch.Tensor] = None,
    z_out: bool = False,
    out: Optional[torch.Tensor] = None,
    group_out: Optional[torch.Tensor] = None,
    scale_post: bool = False,
    bn: int = 0,
    max_ctas: int = 0,
):
    """``epilogue([a | a2] @ b.T)`` on tcgen05; bf16 operands, fp32 accumulation, bf16 result.

    a: [M, K1], a2 / a3: further column blocks of A (optional, K-concatenated), b: [N, K]; bias / scale: fp32 [N];
    aux: bf16 [M, N] consumed according to ``aux_mode``; ``z_out`` also returns the
    pre-activation.  Returns ``out`` or ``(out, z)``.
    """
    global launch_count
    lib = _lib.load(required=True)
    a = _rowmajor2d(a)
    b = _rowmajor2d(b)
    M, K1 = a.shape
    N, K = b.shape
    K2 = K
    if a2 is not None:
        a2 = _rowmajor2d(a2)
        K2 = K1 + a2.shape[1]
        if a3 is not None:
            a3 = _rowmajor2d(a3)
            assert a3.shape[0] == M and K2 + a3.shape[1] == K
        else:
            assert a2.shape[0] == M and K2 == K
    else:
        assert K1 == K, f"A has K={K1} but B has K={K}"
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    z = torch.empty((M, N), dtype=torch.bfloat16, device=a.device) if z_out else None
    if aux is not None:
        aux = _rowmajor2d(aux)
        assert aux.shape == (M, N) and aux.dtype == torch.bfloat16
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N and bias.is_contiguous()
    if scale is not None:
        assert scale.dtype == torch.float32 and scale.numel() == N and scale.is_contiguous()
    code = lib.pnm_gemm_tn(
        _ptr(a), a.stride(0), _ptr(a2), 0 if a2 is None else a2.stride(0), _ptr(a3), 0 if a3 is None else a3.stride(0),
        _ptr(b), b.stride(0),
        _ptr(out), out.stride(0), _ptr(z), 0 if z is None else z.stride(0),
        _ptr(aux), 0 if aux is None else aux.stride(0),
        M, N, K, K1, K2, _ptr(bias), _ptr(scale), _ptr(group_out), act, aux_mode, int(scale_post), bn, max_ctas,
        _stream(),
    )
    _check(code, "pnm_gemm_tn")
    launch_count += 1
    return (out, z) if z_out else out


def gemm_nt(a: torch.Tensor, b: torch.Tensor, *, colsum: bool = False, out: Optional[torch.Tensor] = None,
            colsum_out: Optional[torch.Tensor] = None, max_ctas: int = 0):
    """``a.T @ b`` in fp32 (a: [M, Na], b: [M, Nb], bf16), optionally the column sums of ``a``.

    ``out`` / ``colsum_out`` accumulate when given (they must hold valid fp32 data).
    """
    global launch_count
    lib = _lib.load(required=True)
    a = _rowmajor2d(a)
    b = _rowmajor2d(b)
    M, Na = a.shape
    Nb = b.shape[1]
    assert b.shape[0] == M
    if out is None:
        out = torch.zeros((Na, Nb), dtype=torch.float32, device=a.device)
    cs = None
    if colsum or colsum_out is not None:
        cs = colsum_out if colsum_out is not None else torch.zeros((Na,), dtype=torch.float32, device=a.device)
    code = lib.pnm_gemm_nt(_ptr(a), a.stride(0), _ptr(b), b.stride(0), _ptr(out), out.stride(0), _ptr(cs),
                           M, Na, Nb, max_ctas, _stream())
    _check(code, "pnm_gemm_nt")
    launch_count += 1
    return (out, cs) if cs is not None else out


# ------------------------------------------------------------------ oracles
def gemm_tn_stacked(a: torch.Tensor, b: torch.Tensor, *, bias: Optional[torch.Tensor] = None, act: int = ACT_NONE,
                    aux: Optional[torch.Tensor] = None, aux_mode: int = AUX_NONE, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[p] = epilogue(a[p] @ b[p].T)`` for ``a: [P, Mp, K]``, ``b: [P, N, K]`` (contiguous bf16, ``Mp % 128 == 0``),
    ``bias: [P, N]`` fp32, ``aux: [P, Mp, N]`` — all problems in ONE launch of the tcgen05 kernel."""
    global launch_count
    lib = _lib.load(required=True)
    P, Mp, K = a.shape
    N = b.shape[1]
    assert a.is_contiguous() and b.is_contiguous() and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert b.shape == (P, N, K) and Mp % 128 == 0
    if out is None:
        out = torch.empty((P, Mp, N), dtype=torch.bfloat16, device=a.device)
    assert out.is_contiguous() and out.shape == (P, Mp, N)
    if aux is not None:
        assert aux.is_contiguous() and aux.shape == (P, Mp, N) and aux.dtype == torch.bfloat16
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.is_contiguous() and bias.shape == (P, N)
    code = lib.pnm_gemm_tn_stacked(_ptr(a), K, _ptr(b), K, _ptr(out), N, _ptr(aux), N if aux is not None else 0, Mp, N, K, P,
                                   _ptr(bias), act, aux_mode, 0, _stream())
    _check(code, "pnm_gemm_tn_stacked")
    launch_count += 1
    return out


def gemm_nt_stacked(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, colsum: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[p] += a[p].T @ b[p]`` (and ``colsum[p] += a[p].sum(0)``) for ``a: [P, Mp, Na]``, ``b: [P, Mp, Nb]`` contiguous
    bf16 with ``Mp % 64 == 0``; ``out: [P, Na, Nb]`` / ``colsum: [P, Na]`` fp32, accumulated into.  One launch."""
    global launch_count
    lib = _lib.load(required=True)
    P, Mp, Na = a.shape
    Nb = b.shape[2]
    assert a.is_contiguous() and b.is_contiguous() and b.shape[:2] == (P, Mp) and Mp % 64 == 0
    assert out.is_contiguous() and out.shape == (P, Na, Nb) and out.dtype == torch.float32
    if colsum is not None:
        assert colsum.is_contiguous() and colsum.shape == (P, Na) and colsum.dtype == torch.float32
    code = lib.pnm_gemm_nt_stacked(_ptr(a), Na, _ptr(b), Nb, _ptr(out), _ptr(colsum), Mp, Na, Nb, P, 0, _stream())
    _check(code, "pnm_gemm_nt_stacked")
    launch_count += 1
    return out


def act_torch(x: torch.Tensor, act: int) -> torch.Tensor:
    if act == ACT_GELU:
        return F.gelu(x)
    if act == ACT_SILU:
        return F.silu(x)
    if act == ACT_RELU:
        return F.relu(x)
    if act == ACT_SOFTMAX64:
        shp = x.shape
        return torch.softmax(x.reshape(*shp[:-1], shp[-1] // 64, 64), dim=-1).reshape(shp)
    return x


def gemm_tn_reference(a, b, *, bias=None, scale=None, act=ACT_NONE, aux=None, aux_mode=AUX_NONE, a2=None,
                      a3=None, scale_post=False):
    """fp32 PyTorch statement of what ``gemm_tn`` computes (used by the tests)."""
    af = torch.cat([t.float() for t in (a, a2, a3) if t is not None], dim=1)
    x = af @ b.float().t()
    if bias is not None:
        x = x + bias
    if scale is not None and not scale_post:
        x = x * scale
    z = x
    y = act_torch(x, act)
    if aux_mode == AUX_ADD:
        y = y + aux.float()
    elif aux_mode in (AUX_DGELU, AUX_DSILU, AUX_DRELU):
        t = aux.float().detach().requires_grad_(True)
        with torch.enable_grad():
            f = act_torch(t, {AUX_DGELU: ACT_GELU, AUX_DSILU: ACT_SILU, AUX_DRELU: ACT_RELU}[aux_mode])
            (g,) = torch.autograd.grad(f.sum(), t)
        y = y * g
    elif aux_mode == AUX_DSOFTMAX:
        p = aux.float()
        shp = y.shape
        y4, p4 = y.reshape(shp[0], -1, 64), p.reshape(shp[0], -1, 64)
        y = (p4 * (y4 - (y4 * p4).sum(-1, keepdim=True))).reshape(shp)
    if scale is not None and scale_post:
        y = y * scale
    return y, z


# ----------------------------------------------------------------- dispatch
def fused_path_enabled(x: torch.Tensor) -> bool:
    """True when ``x`` should take the sm_100a kernels (CUDA + bf16 compute)."""
    if not isinstance(x, torch.Tensor) or not x.is_cuda:
        return False
    if type(x) is not torch.Tensor and type(x).__name__ != "Parameter":
        return False  # tensor subclasses (ShardTensor) dispatch through their own handlers
    if torch.is_autocast_enabled("cuda"):
        dt = torch.get_autocast_dtype("cuda")
    else:
        dt = x.dtype
    if dt != torch.bfloat16:
        return False
    _lib.load(required=True)  # a CUDA box without the library is an error, not a fallback
    return True


_wcache: dict = {}


def _bf16_weight(w: torch.Tensor, transpose: bool = False) -> torch.Tensor:
    """bf16 (optionally transposed) copy of a parameter, cached until the parameter changes."""
    if w.dtype == torch.bfloat16 and not transpose:
        return w.detach()
    key = (id(w), transpose)
    ver = (w._version, w.data_ptr(), tuple(w.shape))
    hit = _wcache.get(key)
    if hit is not None and hit[0] == ver:
        return hit[1]
    src = w.detach()
    val = (src.t() if transpose else src).to(torch.bfloat16).contiguous()
    if len(_wcache) > 4096:
        _wcache.clear()
    _wcache[key] = (ver, val)
    return val


def _pad_cols(t: torch.Tensor, mult: int = 8) -> torch.Tensor:
    k = t.shape[-1]
    pad = (-k) % mult
    return F.pad(t, (0, pad)) if pad else t


class _MlpChainFn(torch.autograd.Function):
    """``h_i = act_i(h_{i-1} W_i^T + b_i)``, last layer optionally ``+ residual``.

    The input of the first layer may be given as up to three column blocks (K-concatenated
    inside the GEMM, no materialised concatenation)."""

    @staticmethod
    def forward(ctx, residual, acts, n_layers, need_z, n_src, *rest):
        srcs = list(rest[:n_src])
        weights = rest[n_src:n_src + n_layers]
        biases = rest[n_src + n_layers:]
        acts = list(acts)
        hs, zs = [], []
        h = None
        for i in range(n_layers):
            w = _bf16_weight(weights[i])
            k_in = sum(t.shape[1] for t in srcs) if i == 0 else h.shape[1]
            if w.shape[1] != k_in:  # K padded to a multiple of 8
                w = _pad_cols(w)
            n_true = w.shape[0]
            if n_true % 8:
                w = F.pad(w, (0, 0, 0, (-n_true) % 8))
            b = biases[i]
            if b is not None:
                b = b.detach().float().contiguous()
                if b.numel() != w.shape[0]:
                    b = F.pad(b, (0, w.shape[0] - b.numel()))
            last = i == n_layers - 1
            use_res = last and residual is not None and acts[i] == ACT_NONE
            a_kw = {}
            if i == 0:
                a = srcs[0]
                if n_src > 1:
                    a_kw["a2"] = srcs[1]
                if n_src > 2:
                    a_kw["a3"] = srcs[2]
            else:
                a = h
            if acts[i] != ACT_NONE and need_z:
                h, z = gemm_tn(a, w, bias=b, act=acts[i], z_out=True, **a_kw)
                zs.append(z)
            else:
                h = gemm_tn(a, w, bias=b, act=acts[i], aux=residual if use_res else None,
                            aux_mode=AUX_ADD if use_res else AUX_NONE, **a_kw)
                zs.append(None)
            if last and residual is not None and not use_res:
                h = h + residual
            if n_true != h.shape[1]:
                h = h[:, :n_true]
            hs.append(h)
        ctx.acts, ctx.n_layers, ctx.n_src = acts, n_layers, n_src
        ctx.has_res = residual is not None
        ctx.src_widths = [t.shape[1] for t in srcs]
        ctx.save_for_backward(*srcs, *hs[:-1], *[z for z in zs if z is not None], *weights)
        ctx.z_mask = [z is not None for z in zs]
        ctx.bias_mask = [b is not None for b in biases]
        return hs[-1]

    @staticmethod
    def backward(ctx, dy):
        n, ns = ctx.n_layers, ctx.n_src
        saved = ctx.saved_tensors
        srcs = list(saved[:ns])
        hs = [None] + list(saved[ns:ns + n - 1])  # hs[i] = input of layer i (i >= 1)
        nz = sum(ctx.z_mask)
        zlist = list(saved[ns + n - 1:ns + n - 1 + nz])
        weights = saved[ns + n - 1 + nz:]
        zs, zi = [], 0
        for m in ctx.z_mask:
            zs.append(zlist[zi] if m else None)
            zi += int(m)
        acts = ctx.acts
        dres = dy if ctx.has_res else None
        g = dy.contiguous()
        if acts[n - 1] != ACT_NONE:
            # activation on the output layer: no upstream GEMM to fuse into
            z = zs[n - 1][:, :g.shape[1]].float().requires_grad_(True)
            with torch.enable_grad():
                f = act_torch(z, acts[n - 1])
            g = torch.autograd.grad(f, z, g.float())[0].to(torch.bfloat16)
        base = 5 + ns  # index of the first weight among the forward inputs
        dws, dbs = [None] * n, [None] * n
        dsrc = [None] * ns
        for i in range(n - 1, -1, -1):
            w = weights[i]
            n_true, k_true = w.shape
            gi = g
            if gi.shape[1] % 8:
                gi = _pad_cols(gi)
            need_b = ctx.bias_mask[i] and ctx.needs_input_grad[base + n + i]
            if ctx.needs_input_grad[base + i] or need_b:
                if i == 0 and ns > 1:
                    # weight gradient per column block of the K-concatenated input
                    parts, db = [], None
                    for j, t in enumerate(srcs):
                        res = gemm_nt(gi, t, colsum=need_b and j == 0)
                        if need_b and j == 0:
                            res, db = res
                        parts.append(res[:n_true])
                    dw = torch.cat(parts, dim=1)[:, :k_true]
                else:
                    hin = srcs[0] if i == 0 else hs[i]
                    res = gemm_nt(gi, hin, colsum=need_b)
                    dw, db = (res if need_b else (res, None))
                    dw = dw[:n_true, :k_true]
                dws[i] = dw if dw.dtype == w.dtype else dw.to(w.dtype)
                if db is not None:
                    dbs[i] = db[:n_true]
            need_dx = i > 0 or any(ctx.needs_input_grad[5 + j] for j in range(ns))
            if need_dx:
                wt = _bf16_weight(w, transpose=True)  # [K, N]
                if wt.shape[1] % 8:
                    wt = _pad_cols(wt)
                if wt.shape[0] % 8:
                    wt = F.pad(wt, (0, 0, 0, (-wt.shape[0]) % 8))
                if i > 0 and zs[i - 1] is not None:
                    zprev = zs[i - 1]
                    g = gemm_tn(gi, wt, aux=zprev if zprev.shape[1] == wt.shape[0] else _pad_cols(zprev),
                                aux_mode=_DACT[acts[i - 1]])
                else:
                    g = gemm_tn(gi, wt)
                if i == 0:
                    off = 0
                    for j, wdt in enumerate(ctx.src_widths):
                        if ctx.needs_input_grad[5 + j]:
                            dsrc[j] = g[:, off:off + wdt]
                        off += wdt
                elif g.shape[1] != hs[i].shape[1]:
                    g = g[:, :hs[i].shape[1]]
        return (dres, None, None, None, None, *dsrc, *dws, *dbs)


def mlp_chain(x, weights: Sequence[torch.Tensor], biases: Sequence[Optional[torch.Tensor]],
              acts: Sequence[int], residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Apply ``len(weights)`` linear layers with activations ``acts`` (codes) between them.

    ``x``: [..., K] or a list / tuple of up to three tensors [..., K_j] that are treated as
    the column blocks of one input (every block but the last a multiple of 64 wide);
    returns [..., N_last] (+ ``residual`` when given).  CUDA bf16 inputs run on the tcgen05
    kernels, anything else through PyTorch.
    """
    xs = list(x) if isinstance(x, (list, tuple)) else [x]
    if not fused_path_enabled(xs[0]):
        h = xs[0] if len(xs) == 1 else torch.cat(xs, dim=-1)
        for w, b, a in zip(weights, biases, acts):
            h = act_torch(F.linear(h, w, b), a)
        return h if residual is None else h + residual
    shp = xs[0].shape
    multi_ok = len(xs) <= 3 and all(t.shape[-1] % 64 == 0 for t in xs[:-1])
    if len(xs) > 1 and not multi_ok:
        xs = [torch.cat(xs, dim=-1)]
    x2s = []
    for t in xs:
        t2 = t.reshape(-1, t.shape[-1])
        if t2.dtype != torch.bfloat16:
            t2 = t2.to(torch.bfloat16)
        x2s.append(t2)
    if x2s[-1].shape[1] % 8:
        x2s[-1] = _pad_cols(x2s[-1])
    r2 = None
    if residual is not None:
        r2 = residual.reshape(-1, residual.shape[-1])
        if r2.dtype != torch.bfloat16:
            r2 = r2.to(torch.bfloat16)
    n = len(weights)
    need_z = torch.is_grad_enabled() and (
        any(t.requires_grad for t in xs) or any(w.requires_grad for w in weights)
        or (residual is not None and residual.requires_grad)
    )
    y = _MlpChainFn.apply(r2, tuple(acts), n, need_z, len(x2s), *x2s, *weights, *biases)
    return y.reshape(*shp[:-1], y.shape[-1])


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, act: int = ACT_NONE,
           residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``act(x @ weight.T + bias) (+ residual)`` — single-layer ``mlp_chain``."""
    return mlp_chain(x, [weight], [bias], [act], residual)

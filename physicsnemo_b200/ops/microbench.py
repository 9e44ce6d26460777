"""Kernel micro-benchmarks: CUDA-event timing and roofline fractions of the library kernels.

``python -m physicsnemo_b200.ops.microbench <kernel> [--m ROWS] [--iters N]`` with ``<kernel>``
one of ``gemm_tn``, ``gemm_tn_gelu_z``, ``gemm_tn_softmax``, ``gemm_tn_aux``, ``gemm_nt``,
``layernorm``, ``all``; ``conv`` (implicit-GEMM 3×3 convolutions at U-Net shapes next to the framework's
cuDNN call on the same channels-last bf16 tensors) and ``groupnorm`` (GroupNorm+SiLU forward / backward in both
memory formats next to ``F.group_norm`` + ``F.silu``).  Inputs are larger than the 126 MB L2 at the default size; the small
sizes (``--m 262144``) are meant for profiler captures.  Denominators come from
``MEASURED_PEAKS.json`` at the repository root when present (measured copy bandwidth and
cuBLAS bf16 throughput), else from the fallback 6.65 TB/s / 1.59 PFLOP/s.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import gemm as G
from .norm import layer_norm


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def _time(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.add_(1.0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def _r(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def cases(M):
    bias256, bias512, bias1024 = (torch.randn(n, device="cuda") for n in (256, 512, 1024))
    a256, a1024 = _r(M, 256), _r(M, 1024, scale=0.3)
    w256, w512, w1024, wk1024 = _r(256, 256, scale=0.05), _r(512, 256, scale=0.05), _r(1024, 256, scale=0.05), _r(256, 1024, scale=0.03)
    aux = _r(M, 256)
    p512 = _r(M, 512, scale=0.1)
    out = {}
    out["gemm_tn"] = (lambda: G.gemm_tn(a256, w256, bias=bias256), 2.0 * M * 256 * 256, M * 256 * 2 * 2)
    out["gemm_tn_k1024"] = (lambda: G.gemm_tn(a1024, wk1024, bias=bias256), 2.0 * M * 256 * 1024, M * (1024 + 256) * 2)
    out["gemm_tn_gelu_z"] = (lambda: G.gemm_tn(a256, w1024, bias=bias1024, act=G.ACT_GELU, z_out=True),
                             2.0 * M * 1024 * 256, M * (256 + 2 * 1024) * 2)
    out["gemm_tn_softmax"] = (lambda: G.gemm_tn(a256, w512, bias=bias512, act=G.ACT_SOFTMAX64),
                              2.0 * M * 512 * 256, M * (256 + 512) * 2)
    out["gemm_tn_aux"] = (lambda: G.gemm_tn(a256, w256, bias=bias256, aux=aux, aux_mode=G.AUX_ADD),
                          2.0 * M * 256 * 256, M * 256 * 2 * 3)
    out["gemm_nt"] = (lambda: G.gemm_nt(p512, a256, colsum=True), 2.0 * M * 512 * 256, M * (512 + 256) * 2)
    g, b = torch.ones(256, device="cuda"), torch.zeros(256, device="cuda")
    out["layernorm"] = (lambda: layer_norm(a256, g, b), 0.0, M * 256 * 2 * 2)
    gp, bp = g.clone().requires_grad_(True), b.clone().requires_grad_(True)
    xr = a256.detach().requires_grad_(True)
    y_keep = layer_norm(xr, gp, bp)
    dy = _r(M, 256)

    def ln_bwd():                                   # backward only: dy, x read, dx written (+ small dgamma / dbeta)
        torch.autograd.grad(y_keep, (xr, gp, bp), dy, retain_graph=True)

    out["layernorm_bwd"] = (ln_bwd, 0.0, M * 256 * 2 * 3)
    return out


def conv_cases():
    import torch.nn.functional as F

    from . import conv as C

    out = {}
    for name, (n, c, h, w, co) in {"c128_512": (8, 128, 512, 512, 128), "c256_256": (8, 256, 256, 256, 256),
                                   "c512_128": (8, 512, 128, 128, 512), "c128_1024x256": (2, 128, 1024, 256, 128)}.items():
        x = _r(n, c, h, w).contiguous(memory_format=torch.channels_last)
        wt = _r(co, c, 3, 3, scale=(9 * c) ** -0.5)
        b = torch.randn(co, device="cuda")
        flops = 2.0 * n * h * w * 9 * c * co
        nbytes = (n * h * w * (c + co) + 9 * c * co) * 2
        out[f"conv3x3_{name}"] = (lambda x=x, wt=wt, b=b: C.conv2d_same(x, wt, b), flops, nbytes)
        out[f"cudnn3x3_{name}"] = (lambda x=x, wt=wt, b=b: F.conv2d(x, wt, b.to(torch.bfloat16), padding=1), flops, nbytes)
    return out


def groupnorm_cases():
    import torch.nn.functional as F

    from . import group_norm as GN

    out = {}
    n, c, h, w, g = 8, 128, 512, 512, 32
    wgt, bias = torch.rand(c, device="cuda") + 0.5, torch.randn(c, device="cuda")
    for fmt, tag in ((torch.contiguous_format, "cf"), (torch.channels_last, "cl")):
        x = _r(n, c, h, w).contiguous(memory_format=fmt)
        dy = _r(n, c, h, w).contiguous(memory_format=fmt)
        nbytes = x.numel() * 2 * 3                          # stats pass + normalise pass reads, one write
        out[f"groupnorm_silu_fwd_{tag}"] = (lambda x=x: GN.group_norm(x, g, wgt, bias, 1e-5, silu=True), 0.0, nbytes)
        out[f"torch_groupnorm_silu_fwd_{tag}"] = (lambda x=x: F.silu(F.group_norm(x, g, wgt.to(x.dtype), bias.to(x.dtype), 1e-5)), 0.0, nbytes)

        def fwd_bwd(x=x, dy=dy):
            xr = x.detach().requires_grad_(True)
            GN.group_norm(xr, g, wgt, bias, 1e-5, silu=True).backward(dy)

        out[f"groupnorm_silu_fwd_bwd_{tag}"] = (fwd_bwd, 0.0, x.numel() * 2 * 8)
    return out


def attention_cases(small: bool = False):
    """Forward attention: SongUNet bottleneck (one head, 16 384 tokens, D=128 stands in for the split 512-wide head),
    a DiT-like shape (16 heads, D=64) and a causal case; each against ``F.scaled_dot_product_attention``."""
    import torch.nn.functional as F

    from . import attention as A

    shapes = {"b8_h4_s16384_d128": (8, 4, 16384, 128, False), "b8_h16_s4096_d64": (8, 16, 4096, 64, False),
              "b4_h16_s8192_d128_causal": (4, 16, 8192, 128, True)}
    if small:
        shapes = {"b2_h8_s4096_d128": (2, 8, 4096, 128, False), "b2_h8_s4096_d64": (2, 8, 4096, 64, False)}
    out = {}
    for name, (b, h, s, d, causal) in shapes.items():
        q, k, v = (_r(b, h, s, d) for _ in range(3))
        flops = 4.0 * b * h * s * s * d * (0.5 if causal else 1.0)
        nbytes = 4 * b * h * s * d * 2
        out[f"flash_{name}"] = (lambda q=q, k=k, v=v, c=causal: A.flash_forward(q, k, v, c, p_in_tmem=False), flops, nbytes)
        out[f"flash_ptmem_{name}"] = (lambda q=q, k=k, v=v, c=causal: A.flash_forward(q, k, v, c, p_in_tmem=True), flops, nbytes)
        out[f"torch_sdpa_{name}"] = (lambda q=q, k=k, v=v, c=causal: F.scaled_dot_product_attention(q, k, v, is_causal=c), flops, nbytes)
    return out


def sh_norm_cases(small=False):
    """Equivariant norms on spherical-harmonic grids [B, 7, 3, 2, 128] (lmax 6, mmax 2): own kernel against the same
    operator written with tensor operations.  Bytes: valid rows read, all rows written (forward); x and dy read, dx
    written (backward)."""
    from ..experimental.nn.symmetry import EquivariantLayerNorm, EquivariantLayerNormTied, EquivariantRMSNorm
    from . import sh_norm as S

    B, L, M, C = (8192 if small else 65536), 7, 3, 128
    out = {}
    for name, cls in (("rms", EquivariantRMSNorm), ("ln", EquivariantLayerNorm), ("tied", EquivariantLayerNormTied)):
        for dt in (torch.float32, torch.bfloat16):
            mod = cls(L - 1, M - 1, C).cuda()
            x = torch.randn(B, L, M, 2, C, device="cuda").to(dt).requires_grad_(True)
            valid = int(mod.grid_mask_3d.sum())
            esz = x.element_size()
            tag = f"sh_{name}_{'f32' if dt == torch.float32 else 'bf16'}"
            out[tag + "_fwd"] = (lambda mod=mod, x=x: mod(x.detach()), 0.0, B * C * esz * (valid + L * M * 2))
            y = mod(x)
            dy = torch.randn_like(y)
            out[tag + "_bwd"] = (lambda y=y, x=x, dy=dy, mod=mod: torch.autograd.grad(y, [x] + list(mod.parameters()), dy,
                                                                                      retain_graph=True),
                                 0.0, B * C * esz * (2 * valid + L * M * 2))
            if name == "rms":
                args = (mod.affine_weight, mod.affine_bias, mod._wstat, mod.grid_mask_3d, mod._group, mod.eps, True)
                out[tag + "_fwd_torch_ops"] = (lambda x=x, args=args: S.reference(x.detach(), *args), 0.0,
                                               B * C * esz * (valid + L * M * 2))
    return out

def pixel_attention_cases(small=False):
    """Variable-length token-space attention of 49 152 pixels (HEALPix nside 64) over ~20 observation tokens each, 32 heads,
    token width 64: own kernel against the same operator on dense-padded tensors.  Bytes: tokens once per block of 16 heads,
    qk read, ctx written (forward); plus dctx read, dqk and fp32 dtok written (backward)."""
    from . import pixel_attention as PA

    P, H, Dt = (8192 if small else 49152), 32, 64
    torch.manual_seed(0)
    counts = torch.randint(0, 41, (P,), device="cuda")
    cu = torch.zeros(P + 1, dtype=torch.int32, device="cuda")
    cu[1:] = counts.cumsum(0)
    N = int(cu[-1])
    out = {}
    for dt, tag in ((torch.bfloat16, "bf16"), (torch.float32, "f32")):
        qk = (torch.randn(P, H, Dt, device="cuda") * 0.3).to(dt).requires_grad_(True)
        tok = torch.randn(N, Dt, device="cuda").to(dt).requires_grad_(True)
        esz = qk.element_size()
        flops = 4.0 * N * H * Dt
        fwd_bytes = N * Dt * esz * (H // 16) + 2 * P * H * Dt * esz
        out[f"pixattn_{tag}_fwd"] = (lambda qk=qk, tok=tok: PA.token_attention(qk.detach(), tok.detach(), cu), flops, fwd_bytes)
        y = PA.token_attention(qk, tok, cu)
        dy = torch.randn_like(y)
        out[f"pixattn_{tag}_bwd"] = (lambda y=y, qk=qk, tok=tok, dy=dy: torch.autograd.grad(y, [qk, tok], dy, retain_graph=True), 2.5 * flops,
                                     fwd_bytes + P * H * Dt * (esz + 4) + N * Dt * 4)
        out[f"pixattn_{tag}_fwd_dense_padded_torch"] = (lambda qk=qk, tok=tok: PA.token_attention_reference(qk.detach(), tok.detach(), cu),
                                                        flops, fwd_bytes)
    return out

def afno_filter_cases(small: bool = False):
    """Stages of the AFNO spectral filter on the FourCastNet grid (2 x 90 x 180 tokens, 768 channels in 8 blocks; the small
    variant is 1 x 90 x 180 with 4 blocks): pruned row transforms, column transforms, the stacked-batch block MLP."""
    import ctypes

    from . import afno_spectral as A
    from . import gemm as G

    B, H, W, nb = (1, 90, 180, 4) if small else (2, 90, 180, 8)
    C = 96 * nb
    geo = A.FilterGeometry(B, H, W, C, nb, H // 2 + 1)
    lib = A._lib_af()
    st = torch.cuda.current_stream().cuda_stream
    tok = _r(B * H * W, C)
    out = torch.empty_like(tok)
    Y = torch.empty(B * H, geo.KX, C, 2, device="cuda")
    Z = torch.zeros(nb, geo.Mp, 192, device="cuda", dtype=torch.bfloat16)
    O = torch.empty_like(Z)
    w = _r(nb, 192, 192, scale=0.05)
    bias = torch.randn(nb, 192, device="cuda")
    dw = torch.zeros(nb, 192, 192, device="cuda")
    ptr = lambda t: (ctypes.c_void_p * 8)(*([t.data_ptr()] * 8))            # noqa: E731
    rows_flops = 2.0 * B * H * C * geo.KX * W * 2 / 2                          # folded real-input transform
    cols_flops = 8.0 * B * geo.KX * C * H * (geo.H1 + geo.H2)
    spec_bytes = B * H * geo.KX * C * 8
    return {
        "afno_rows_r2c": (lambda: lib.pnm_afno_rows_r2c(ptr(tok), Y.data_ptr(), geo.arr, geo.Tp, 0, 0, None, 0, 1, 0, 0, 1.0, None, st),
                          rows_flops, tok.numel() * 2 + spec_bytes),
        "afno_rows_c2r": (lambda: lib.pnm_afno_rows_c2r(Y.data_ptr(), ptr(out), geo.arr, geo.Tp, 1, 0, None, 0, 1, 0, 0, None, None, st),
                          rows_flops, tok.numel() * 2 + spec_bytes),
        "afno_cols_dft": (lambda: lib.pnm_afno_cols_dft(Y.data_ptr(), Z.data_ptr(), None, geo.arr, geo.Mp, 0.0, st),
                          cols_flops, spec_bytes + Z.numel() * 2),
        "afno_cols_idft": (lambda: lib.pnm_afno_cols_idft(Z.data_ptr(), Y.data_ptr(), geo.arr, geo.Mp, 0.01, st),
                           cols_flops, spec_bytes + Z.numel() * 2),
        "afno_block_mlp_layer": (lambda: G.gemm_tn_stacked(Z, w, bias=bias, act=G.ACT_RELU, out=O),
                                 2.0 * nb * geo.Mp * 192 * 192, 2 * Z.numel() * 2),
        "afno_block_mlp_wgrad": (lambda: G.gemm_nt_stacked(O, Z, dw), 2.0 * nb * geo.Mp * 192 * 192, 2 * Z.numel() * 2),
    }


def mlp_gemm_cases(M: int = 32400):
    """The six GEMMs of one AFNO channel MLP (768 -> 3072 -> 768 over ``M`` tokens, forward and backward) and the
    patch head: compute-bound shapes, which run as 256 x 256 tiles on CTA pairs (``tcgen05.mma.cta_group::2``) unless
    ``PNM_GEMM_PAIR=0`` keeps them on the single-CTA kernel.  Each has a ``cublas_*`` twin (``torch`` matmul, without
    the fused epilogue) as the library figure for the same product."""
    x, h, z, dy, g1 = _r(M, 768), _r(M, 3072), _r(M, 3072), _r(M, 768), _r(M, 3072)
    res = _r(M, 768)
    w1, w2 = _r(3072, 768, scale=0.03), _r(768, 3072, scale=0.02)
    w1t, w2t = w1.t().contiguous(), w2.t().contiguous()
    b1, b2 = torch.randn(3072, device="cuda"), torch.randn(768, device="cuda")
    wh, dh = _r(4672, 768, scale=0.03), _r(M, 4672)
    wht = wh.t().contiguous()
    fl = 2.0 * M * 768 * 3072
    flh = 2.0 * M * 768 * 4672
    out = {}
    out["fc1_gelu_z"] = (lambda: G.gemm_tn(x, w1, bias=b1, act=G.ACT_GELU, z_out=True), fl, M * (768 + 2 * 3072) * 2)
    out["cublas_fc1"] = (lambda: x @ w1.t(), fl, M * (768 + 3072) * 2)
    out["fc2_residual"] = (lambda: G.gemm_tn(h, w2, bias=b2, aux=res, aux_mode=G.AUX_ADD), fl, M * (3072 + 2 * 768) * 2)
    out["cublas_fc2"] = (lambda: h @ w2.t(), fl, M * (3072 + 768) * 2)
    out["dgrad2_dgelu"] = (lambda: G.gemm_tn(dy, w2t, aux=z, aux_mode=G.AUX_DGELU), fl, M * (768 + 2 * 3072) * 2)
    out["dgrad1"] = (lambda: G.gemm_tn(g1, w1t), fl, M * (3072 + 768) * 2)
    out["wgrad2_colsum"] = (lambda: G.gemm_nt(dy, h, colsum=True), fl, M * (3072 + 768) * 2)
    out["cublas_wgrad2"] = (lambda: dy.t() @ h, fl, M * (3072 + 768) * 2)
    out["head"] = (lambda: G.gemm_tn(x, wh), flh, M * (768 + 4672) * 2)
    out["cublas_head"] = (lambda: x @ wh.t(), flh, M * (768 + 4672) * 2)
    out["head_dgrad"] = (lambda: G.gemm_tn(dh, wht), flh, M * (768 + 4672) * 2)
    return out


def gemm_attention_cases(small: bool = False):
    """The 512-wide single head of the SongUNet bottleneck over 16 384 tokens (4 096 in the small variant): forward and
    forward + backward of attention as GEMMs around the row softmax."""
    from . import gemm_attention as GA

    S = 4096 if small else 16384
    q, k, v = (_r(1, 1, S, 512).requires_grad_(True) for _ in range(3))
    do = _r(1, 1, S, 512)
    P = _r(S, S)

    def fwd():
        with torch.no_grad():
            GA.gemm_attention(q, k, v)

    def fwd_bwd():
        GA.gemm_attention(q, k, v).backward(do)
        q.grad = k.grad = v.grad = None

    fl = 4.0 * S * S * 512
    return {"gemm_attention_fwd": (fwd, fl, 2 * S * S * 2 * 2), "gemm_attention_fwd_bwd": (fwd_bwd, 3.5 * fl, 8 * S * S * 2),
            "softmax_rows": (lambda: GA.softmax_rows_(P, 0.044), 5.0 * S * S, 2 * S * S * 2)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel")
    ap.add_argument("--m", type=int, default=1_000_000)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    hbm, tflops, src = _peaks()
    flush = torch.empty(256 * 1024 * 1024 // 4, device="cuda")
    if args.kernel == "conv":
        table = conv_cases()
        names = list(table)
    elif args.kernel == "groupnorm":
        table = groupnorm_cases()
        names = list(table)
    elif args.kernel in ("pixel_attention", "pixel_attention_small"):
        table = pixel_attention_cases(small=args.kernel == "pixel_attention_small")
        names = list(table)
    elif args.kernel in ("sh_norm", "sh_norm_small"):
        table = sh_norm_cases(small=args.kernel == "sh_norm_small")
        names = list(table)
    elif args.kernel in ("afno_filter", "afno_filter_small"):
        table = afno_filter_cases(small=args.kernel == "afno_filter_small")
        names = list(table)
    elif args.kernel in ("gemm_attention", "gemm_attention_small"):
        table = gemm_attention_cases(small=args.kernel == "gemm_attention_small")
        names = list(table)
    elif args.kernel in ("mlp_gemm", "mlp_gemm_small"):
        args.m = 8192 if args.kernel == "mlp_gemm_small" else 32400
        table = mlp_gemm_cases(args.m)
        names = list(table)
    elif args.kernel in ("attention", "attention_small"):
        table = attention_cases(small=args.kernel == "attention_small")
        names = list(table)
    else:
        table = cases(args.m)
        names = list(table) if args.kernel == "all" else [args.kernel]
    for name in names:
        fn, flops, nbytes = table[name]
        ms = _time(fn, args.iters, flush)
        t_roof = max(flops / (tflops * 1e12), nbytes / (hbm * 1e9)) * 1e3
        print(json.dumps({"kernel": name, "M": args.m, "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1),
                          "gbs": round(nbytes / ms / 1e6, 1), "roofline_ms": round(t_roof, 4),
                          "frac_of_roofline": round(t_roof / ms, 3), "peaks": src}))
    from . import device_error

    assert device_error() == 0


if __name__ == "__main__":
    main()

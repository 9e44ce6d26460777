"""Numerics of the tcgen05 GEMM family against fp32 PyTorch statements of the same ops."""
import pytest
import torch

from physicsnemo_b200 import ops
from physicsnemo_b200.ops import gemm as G

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def _close(out, ref, tol=2e-2):
    """Element-wise: |out - ref| <= tol/2 * |ref| + tol/2 * rms(ref) (bf16 rounding is 0.4 % of the element; the floor
    covers entries that are small because their terms cancel, whose error scales with the typical size instead)."""
    out, ref = out.float(), ref.float()
    rms = ref.pow(2).mean().sqrt().item() + 1e-6
    excess = (out - ref).abs() - (0.5 * tol * ref.abs() + 0.5 * tol * rms)
    worst = excess.max().item()
    assert worst <= 0, f"worst excess over the element-wise bound {worst} (rms of the reference {rms})"


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (300, 256, 256), (1000, 64, 128), (257, 264, 72), (20000, 512, 256)])
@pytest.mark.parametrize("bn", [0, 128])
def test_gemm_tn_plain(M, N, K, bn):
    a, b = _rand(M, K), _rand(N, K, scale=0.1)
    bias = torch.randn(N, device="cuda")
    out = ops.gemm_tn(a, b, bias=bias, bn=bn)
    ref, _ = ops.gemm_tn_reference(a, b, bias=bias)
    _close(out, ref)
    assert ops.device_error() == 0


@pytest.mark.parametrize("act", [G.ACT_GELU, G.ACT_SILU, G.ACT_RELU, G.ACT_SOFTMAX64])
def test_gemm_tn_activation_and_z(act):
    M, N, K = 777, 256, 128
    a, b = _rand(M, K), _rand(N, K, scale=0.2)
    bias = torch.randn(N, device="cuda")
    scale = torch.rand(N, device="cuda") + 0.5
    out, z = ops.gemm_tn(a, b, bias=bias, scale=scale, act=act, z_out=True)
    ref, zref = ops.gemm_tn_reference(a, b, bias=bias, scale=scale, act=act)
    _close(z, zref)
    _close(out, ref)
    out2 = ops.gemm_tn(a, b, bias=bias, scale=scale, act=act)
    _close(out2, ref)


@pytest.mark.parametrize("aux_mode", [G.AUX_ADD, G.AUX_DGELU, G.AUX_DSILU, G.AUX_DRELU, G.AUX_DSOFTMAX])
def test_gemm_tn_aux(aux_mode):
    M, N, K = 1500, 384, 192
    a, b = _rand(M, K), _rand(N, K, scale=0.2)
    if aux_mode == G.AUX_DSOFTMAX:
        aux = torch.softmax(torch.randn(M, N // 64, 64, device="cuda"), -1).reshape(M, N).to(torch.bfloat16)
    else:
        aux = _rand(M, N)
    scale = torch.rand(N, device="cuda") + 0.5
    grp = torch.zeros(N // 64, device="cuda") if aux_mode == G.AUX_DSOFTMAX else None
    out = ops.gemm_tn(a, b, aux=aux, aux_mode=aux_mode, scale=scale, scale_post=True, group_out=grp)
    ref, _ = ops.gemm_tn_reference(a, b, aux=aux, aux_mode=aux_mode, scale=scale, scale_post=True)
    _close(out, ref, tol=3e-2)
    if grp is not None:
        y = (a.float() @ b.float().t()).reshape(M, -1, 64)
        p = aux.float().reshape(M, -1, 64)
        ds = p * (y - (y * p).sum(-1, keepdim=True))
        gref = (ds * torch.log(p.clamp_min(1e-30)) * (p > 0)).sum((0, 2))
        _close(grp, gref, tol=5e-2)
    assert ops.device_error() == 0


def test_gemm_tn_k_concat():
    M, N, K1, K2 = 900, 256, 128, 192
    a, a2, b = _rand(M, K1), _rand(M, K2), _rand(N, K1 + K2, scale=0.1)
    out = ops.gemm_tn(a, b, a2=a2)
    ref, _ = ops.gemm_tn_reference(a, b, a2=a2)
    _close(out, ref)


@pytest.mark.parametrize("M,Na,Nb", [(64, 128, 128), (5000, 256, 256), (4097, 512, 256), (1000, 64, 32), (30000, 1024, 256),
                                     # >= 8192 rows and >= 256 output rows: the CTA-pair kernel (ragged edges in all three sizes)
                                     (32400, 768, 3072), (9001, 264, 136), (8192, 256, 128)])
def test_gemm_nt(M, Na, Nb):
    a, b = _rand(M, Na, scale=0.3), _rand(M, Nb, scale=0.3)
    out, cs = ops.gemm_nt(a, b, colsum=True)
    ref = a.float().t() @ b.float()
    _close(out, ref, tol=1e-2)
    _close(cs, a.float().sum(0), tol=1e-2)
    assert ops.device_error() == 0


@pytest.mark.parametrize("P,Mp,N,K", [(8, 8320, 192, 192), (3, 256, 64, 64), (2, 384, 264, 136)])
def test_gemm_stacked_batches(P, Mp, N, K):
    """`P` equal problems in one launch: forward with bias + ReLU, data gradient with the ReLU mask, weight gradient
    with column sums — each against the per-problem fp32 statement."""
    a, w = _rand(P, Mp, K), _rand(P, N, K, scale=0.1)
    bias = torch.randn(P, N, device="cuda")
    out = G.gemm_tn_stacked(a, w, bias=bias, act=G.ACT_RELU)
    ref = torch.relu(torch.einsum("pmk,pnk->pmn", a.float(), w.float()) + bias[:, None])
    _close(out, ref)
    gy = _rand(P, Mp, N)
    wt = w.transpose(1, 2).contiguous()
    # the mask has the product's shape: dx = (gy @ w) where aux > 0
    dref = torch.einsum("pmn,pnk->pmk", gy.float(), w.float())
    aux = _rand(P, Mp, K)
    dx = G.gemm_tn_stacked(gy, wt, aux=aux, aux_mode=G.AUX_DRELU)
    _close(dx, dref * (aux.float() > 0))
    dw = torch.zeros(P, N, K, device="cuda")
    db = torch.zeros(P, N, device="cuda")
    G.gemm_nt_stacked(gy, a, dw, db)
    _close(dw, torch.einsum("pmn,pmk->pnk", gy.float(), a.float()), tol=1e-2)
    _close(db, gy.float().sum(1), tol=1e-2)
    assert ops.device_error() == 0


@pytest.mark.parametrize("C", [128, 256, 768])
def test_layernorm(C):
    M = 3001
    x = _rand(M, C).requires_grad_(True)
    w = (torch.rand(C, device="cuda") + 0.5).requires_grad_(True)
    b = torch.randn(C, device="cuda").requires_grad_(True)
    y = ops.layer_norm(x, w, b)
    dy = _rand(M, C)
    y.backward(dy)
    xr = x.detach().float().requires_grad_(True)
    wr, br = w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    yr = torch.nn.functional.layer_norm(xr, (C,), wr, br)
    yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad, tol=3e-2)
    _close(w.grad, wr.grad, tol=2e-2)
    _close(b.grad, br.grad, tol=2e-2)


def test_mlp_chain_matches_torch():
    M = 2050
    x = _rand(M, 6).requires_grad_(True)
    res = _rand(M, 256).requires_grad_(True)
    ws = [torch.randn(512, 6, device="cuda") * 0.3, torch.randn(256, 512, device="cuda") * 0.05]
    bs = [torch.randn(512, device="cuda") * 0.1, torch.randn(256, device="cuda") * 0.1]
    for t in ws + bs:
        t.requires_grad_(True)
    y = ops.mlp_chain(x, ws, bs, [G.ACT_GELU, G.ACT_NONE], residual=res)
    dy = _rand(M, 256)
    y.backward(dy)
    got = [x.grad, res.grad] + [t.grad for t in ws + bs]
    xr = x.detach().float().requires_grad_(True)
    rr = res.detach().float().requires_grad_(True)
    wr = [t.detach().clone().requires_grad_(True) for t in ws]
    br = [t.detach().clone().requires_grad_(True) for t in bs]
    h = torch.nn.functional.gelu(xr @ wr[0].t() + br[0]) @ wr[1].t() + br[1] + rr
    h.backward(dy.float())
    _close(y, h, tol=3e-2)
    for g, r in zip(got, [xr.grad, rr.grad] + [t.grad for t in wr + br]):
        _close(g, r, tol=4e-2)
    assert ops.device_error() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(1000, 128, 128), (257, 72, 72), (90000, 128, 320), (512, 128, 64)])
def test_gemm_tn_split_m_tiles(M, N, K):
    """256-row x 128-column tiles (two row sub-tiles sharing one B tile), forced with bn = -256 and, for the large M,
    chosen by the launcher itself."""
    a, b = _rand(M, K), _rand(N, K, scale=0.1)
    bias = torch.randn(N, device="cuda")
    ref, _ = ops.gemm_tn_reference(a, b, bias=bias, act=G.ACT_SILU)
    _close(ops.gemm_tn(a, b, bias=bias, act=G.ACT_SILU, bn=-256), ref)
    _close(ops.gemm_tn(a, b, bias=bias, act=G.ACT_SILU), ref)
    assert ops.device_error() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(2, 64, 128, 24, 40, 3), (1, 128, 64, 17, 33, 3), (3, 64, 72, 8, 16, 1), (1, 192, 256, 40, 24, 5),
                                   (1, 128, 128, 296, 272, 3), (1, 64, 96, 320, 256, 1),
                                   # >= 8192 pixels and K >= 512: the CTA-pair tiles (256 x 128 and 256 x 256), with ragged image
                                   # edges, a ragged channel edge, an odd number of pixel tiles and a 1 x 1 window
                                   (1, 128, 256, 90, 100, 3), (1, 64, 192, 100, 90, 3), (1, 128, 128, 72, 144, 3),
                                   (1, 512, 128, 96, 96, 1), (1, 256, 256, 64, 136, 3)])
def test_conv2d_same_implicit_gemm(shape):
    from physicsnemo_b200.ops import conv as C

    n, cin, cout, h, w, k = shape
    torch.manual_seed(0)
    x = torch.randn(n, cin, h, w, device="cuda").to(memory_format=torch.channels_last).requires_grad_(True)
    wt = (torch.randn(cout, cin, k, k, device="cuda") / (cin * k * k) ** 0.5).requires_grad_(True)
    b = torch.randn(cout, device="cuda").requires_grad_(True)
    assert C.supported(x, wt)
    y = C.conv2d_same(x, wt, b)
    assert y.shape == (n, cout, h, w) and y.is_contiguous(memory_format=torch.channels_last)
    xr, wr, br = (t.detach().clone().requires_grad_(True) for t in (x, wt, b))
    ref = torch.nn.functional.conv2d(xr, wr, br, padding=k // 2)
    assert (y.float() - ref).abs().max() < 4e-2
    dy = torch.randn_like(ref)
    y.backward(dy.to(y.dtype))
    ref.backward(dy)
    assert (x.grad - xr.grad).abs().max() < 6e-2 * max(1.0, float(xr.grad.abs().max()))
    assert (wt.grad - wr.grad).abs().max() < 3e-2 * float(wr.grad.abs().max())
    assert (b.grad - br.grad).abs().max() < 2e-2 * float(br.grad.abs().max())
    fused = C.conv2d_same(x.detach(), wt.detach(), b.detach(), act="silu")
    assert (fused.float() - torch.nn.functional.silu(ref.detach())).abs().max() < 4e-2


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(2048, 256, 512), (4000, 768, 1024), (32400, 1096, 768), (2304, 520, 584)])
@pytest.mark.parametrize("mode", ["plain", "gelu_z", "add", "dgelu", "drelu"])
def test_gemm_tn_cta_pair_tiles(M, N, K, mode):
    """Compute-bound shapes (K >= 512, N >= 256, M >= 2048) run as 256 x 256 tiles on CTA pairs (cta_group::2): ragged M,
    N and K edges, every epilogue the pair kernel carries, against the fp32 statement and against the single-CTA kernel."""
    a, b = _rand(M, K), _rand(N, K, scale=0.05)
    bias = torch.randn(N, device="cuda")
    aux = _rand(M, N)
    kw = {"plain": dict(bias=bias), "gelu_z": dict(bias=bias, act=G.ACT_GELU, z_out=True),
          "add": dict(bias=bias, aux=aux, aux_mode=G.AUX_ADD), "dgelu": dict(aux=aux, aux_mode=G.AUX_DGELU),
          "drelu": dict(aux=aux, aux_mode=G.AUX_DRELU)}[mode]
    out = ops.gemm_tn(a, b, **kw)
    ref_kw = {k: v for k, v in kw.items() if k != "z_out"}
    ref, zref = ops.gemm_tn_reference(a, b, **ref_kw)
    single = ops.gemm_tn(a, b, bn=128 if mode == "plain" else 0, max_ctas=148, **kw)      # max_ctas keeps it off the pair kernel
    if mode == "gelu_z":
        (out, z), (single, zs) = out, single
        _close(z, zref)
        _close(z, zs, tol=1e-2)
    _close(out, ref)
    assert (out.float() - single.float()).abs().max().item() <= 2e-2 * ref.abs().max().item()
    assert ops.device_error() == 0

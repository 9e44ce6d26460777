"""Numerics of the normalisation kernels against PyTorch fp32 references (GPU)."""
import pytest
import torch


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("channels_last", [False, True])
@pytest.mark.parametrize("silu", [False, True])
def test_group_norm_kernels(dtype, channels_last, silu):
    from physicsnemo_b200.ops import group_norm as G

    torch.manual_seed(0)
    for (B, C, H, W, groups) in [(2, 128, 24, 40, 32), (3, 64, 16, 16, 16), (1, 256, 8, 8, 32)]:
        x = (torch.randn(B, C, H, W, device="cuda") * 2 + 0.5).to(dtype)
        if channels_last:
            x = x.contiguous(memory_format=torch.channels_last)
        w = torch.randn(C, device="cuda") * 0.5 + 1
        b = torch.randn(C, device="cuda") * 0.2
        assert G.supported(x, groups)
        xr = x.detach().float().requires_grad_(True)
        wr, br = w.clone().requires_grad_(True), b.clone().requires_grad_(True)
        ref = torch.nn.functional.group_norm(xr, groups, wr, br, 1e-5)
        ref = torch.nn.functional.silu(ref) if silu else ref
        dy = torch.randn_like(ref)
        ref.backward(dy)
        xk = x.detach().clone().requires_grad_(True)
        wk, bk = w.clone().requires_grad_(True), b.clone().requires_grad_(True)
        out = G.group_norm(xk, groups, wk, bk, 1e-5, silu=silu)
        assert out.stride() == x.stride()
        out.backward(dy.to(dtype))
        tol = 3e-2 if dtype == torch.bfloat16 else 2e-4
        assert (out.float() - ref).abs().max() < tol * 2
        assert (xk.grad.float() - xr.grad).abs().max() < tol * 3
        scale = wr.grad.abs().max()
        assert (wk.grad - wr.grad).abs().max() < tol * scale and (bk.grad - br.grad).abs().max() < tol * br.grad.abs().max()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fused_silu_derivative_chain(dtype):
    from physicsnemo_b200.nn.module.fused_silu import FusedSiLU, _kernel, silu_derivative_reference

    x = torch.randn(3, 1001, device="cuda").to(dtype)            # odd length exercises the scalar tail
    g = torch.randn_like(x)
    tol = 4e-2 if dtype == torch.bfloat16 else 1e-5
    for order in range(5):
        want = silu_derivative_reference(x.double(), order) * g.double()
        got = _kernel(x, g, order)
        assert (got.double() - want).abs().max() < tol, order
    xr = x.float().requires_grad_(True)
    y = FusedSiLU.apply(xr)
    (g1,) = torch.autograd.grad(y.sum(), xr, create_graph=True)
    (g2,) = torch.autograd.grad(g1.sum(), xr, create_graph=True)
    (g3,) = torch.autograd.grad(g2.sum(), xr)
    ref = silu_derivative_reference(x.double(), 3)
    assert (g3.double() - ref).abs().max() < 1e-4


@pytest.mark.gpu
@pytest.mark.parametrize("case", [((37,), 7, 1), ((21, 18), (5, 3), 1), ((16, 20), 3, (2, 3)), ((6, 7, 9), 3, 1)])
def test_neighbourhood_attention_kernels(case):
    from physicsnemo_b200.nn.functional.natten import na1d, na2d, na3d

    shape, kernel, dilation = case
    fn = {1: na1d, 2: na2d, 3: na3d}[len(shape)]
    torch.manual_seed(0)
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 3e-2)):
        q, k, v = (torch.randn(2, *shape, 3, 24, device="cuda").to(dtype).requires_grad_(True) for _ in range(3))
        out = fn(q, k, v, kernel, dilation=dilation, implementation="cuda")
        dy = torch.randn_like(out)
        gq, gk, gv = torch.autograd.grad(out, (q, k, v), dy)
        qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
        ref = fn(qr, kr, vr, kernel, dilation=dilation, implementation="torch")
        rq, rk, rv = torch.autograd.grad(ref, (qr, kr, vr), dy.float())
        assert (out.float() - ref).abs().max() < tol
        for a, b in ((gq, rq), (gk, rk), (gv, rv)):
            assert (a.float() - b).abs().max() < tol * 4 * max(1.0, float(b.abs().max()))

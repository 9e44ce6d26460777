"""Numerics of the normalisation kernels against PyTorch fp32 references (GPU)."""
import math

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


# ---- flash attention (tcgen05) ---------------------------------------------------------------------------------------
def _sdpa_fp32(q, k, v, causal, scale):
    s = (q.float() @ k.float().transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(q.shape[-2], k.shape[-2], dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    return torch.softmax(s, dim=-1) @ v.float(), torch.logsumexp(s, dim=-1)


@pytest.mark.gpu
@pytest.mark.parametrize("p_tmem", [False, True])
@pytest.mark.parametrize("layout", ["natural", "transposed"])
@pytest.mark.parametrize("shape", [(2, 3, 256, 256, 64, False), (1, 2, 384, 384, 128, False), (2, 2, 200, 333, 64, False),
                                   (1, 2, 130, 77, 128, False), (1, 3, 512, 512, 128, True), (2, 1, 300, 300, 64, True),
                                   (1, 1, 1024, 2048, 128, False)])
def test_flash_attention_forward(shape, layout, p_tmem):
    from physicsnemo_b200.ops import attention as A
    from physicsnemo_b200.ops import device_error

    b, h, sq, skv, d, causal = shape
    torch.manual_seed(0)
    q = torch.randn(b, h, sq, d, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(b, h, skv, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(b, h, skv, d, device="cuda", dtype=torch.bfloat16)
    scale = 0.7 / d ** 0.5
    out, lse = A.flash_forward(q, k, v, causal, scale, v_layout=layout, p_in_tmem=p_tmem)
    torch.cuda.synchronize()
    assert device_error() == 0
    ref, ref_lse = _sdpa_fp32(q, k, v, causal, scale)
    assert torch.isfinite(out.float()).all()
    err = (out.float() - ref).abs().max().item()
    assert err < 2e-2, f"max abs err {err}"
    assert (lse - ref_lse).abs().max().item() < 2e-3


@pytest.mark.gpu
def test_flash_attention_autograd_and_fallback():
    from physicsnemo_b200.ops import attention as A

    torch.manual_seed(0)
    q, k, v = (torch.randn(2, 4, 256, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
    out = A.sdpa(q, k, v, is_causal=True)
    out.float().square().sum().backward()
    qr, kr, vr = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    ref = torch.nn.functional.scaled_dot_product_attention(qr, kr, vr, is_causal=True)
    ref.float().square().sum().backward()
    assert (out - ref).abs().max().item() < 2e-2
    for a, b in ((q, qr), (k, kr), (v, vr)):
        assert (a.grad.float() - b.grad.float()).abs().max().item() < 5e-2 * b.grad.float().abs().max().item() + 1e-3
    x = torch.randn(2, 4, 64, 32, device="cuda")                                  # fp32, D=32: PyTorch operator
    assert torch.allclose(A.sdpa(x, x, x), torch.nn.functional.scaled_dot_product_attention(x, x, x))


@pytest.mark.gpu
@pytest.mark.parametrize("p_tmem", [False, True])
@pytest.mark.parametrize("d", [64, 128])
def test_flash_attention_growing_scores_rescale_the_accumulator(d, p_tmem):
    """Later key tiles carry much larger scores, so the running reference must move (by more than 2^8 and, for the last
    tile, by more than 2^64) and the TMEM accumulator is corrected in place."""
    from physicsnemo_b200.ops import attention as A
    from physicsnemo_b200.ops import device_error

    torch.manual_seed(1)
    q = torch.randn(1, 2, 256, d, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(1, 2, 640, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(1, 2, 640, d, device="cuda", dtype=torch.bfloat16)
    ramp = torch.tensor([0.2, 1.0, 3.0, 3.0, 30.0], device="cuda").repeat_interleave(128)     # per key tile
    k = (k.float() * ramp[None, None, :, None]).to(torch.bfloat16)
    scale = 1.0 / d ** 0.5
    out, lse = A.flash_forward(q, k, v, False, scale, p_in_tmem=p_tmem)
    torch.cuda.synchronize()
    assert device_error() == 0
    ref, ref_lse = _sdpa_fp32(q, k, v, False, scale)
    assert torch.isfinite(out.float()).all()
    assert (out.float() - ref).abs().max().item() < 3e-2
    assert ((lse - ref_lse).abs() / ref_lse.abs().clamp_min(1.0)).max().item() < 2e-3


@pytest.mark.gpu
def test_ring_attention_blocks_merge_with_flash_kernel():
    """Two K/V blocks processed by the flash kernel and merged by their log-sum-exp equal attention over the whole sequence."""
    from physicsnemo_b200.parallel.patches.attention import _block, _merge

    torch.manual_seed(0)
    q = torch.randn(2, 4, 256, 64, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(2, 4, 512, 64, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(2, 4, 512, 64, device="cuda", dtype=torch.bfloat16)
    scale = 1 / 8.0
    with torch.no_grad():
        acc = None
        for lo, hi in ((0, 200), (200, 512)):                    # uneven shards, as a ring over ranks would deliver them
            acc = _merge(acc, _block(q, k[:, :, lo:hi].contiguous(), v[:, :, lo:hi].contiguous(), scale))
        m, l, o = acc
        got = o / l
    ref, _ = _sdpa_fp32(q, k, v, False, scale)
    assert (got - ref).abs().max().item() < 2e-2


# ---- EDM conditioning --------------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_edm_conditioning_kernel(dtype):
    from physicsnemo_b200.ops import conditioning as C

    torch.manual_seed(0)
    B, Cn, E = 8, 128, 512
    noise = (torch.randn(B, device="cuda") * 1.2 - 1.2).exp()
    freqs = (1 / 10000) ** (torch.arange(Cn // 2, device="cuda") / (Cn // 2 - 1))
    w0 = (torch.randn(E, Cn, device="cuda") / Cn ** 0.5).to(dtype).requires_grad_(True)
    b0 = (0.1 * torch.randn(E, device="cuda")).to(dtype).requires_grad_(True)
    w1 = (torch.randn(E, E, device="cuda") / E ** 0.5).to(dtype).requires_grad_(True)
    b1 = (0.1 * torch.randn(E, device="cuda")).to(dtype).requires_grad_(True)
    extra = (0.3 * torch.randn(B, Cn, device="cuda")).requires_grad_(True)
    assert C.supported(noise, freqs, w0, w1)
    out = C.edm_conditioning(noise, freqs, w0, b0, w1, b1, extra)
    ref = C.reference(noise, freqs, w0, b0, w1, b1, extra)
    assert out.dtype == torch.float32 and (out - ref).abs().max().item() < (2e-5 if dtype == torch.float32 else 2e-3)
    g = torch.randn_like(out)
    got = torch.autograd.grad(out, (w0, b0, w1, b1, extra), g)
    want = torch.autograd.grad(ref, (w0, b0, w1, b1, extra), g)
    for a, b in zip(got, want):
        assert torch.allclose(a.float(), b.float(), atol=1e-4, rtol=1e-3)


@pytest.mark.gpu
def test_song_unet_uses_fused_conditioning():
    from physicsnemo_b200.models.diffusion_unets import SongUNet
    from physicsnemo_b200.ops import conditioning as C

    torch.manual_seed(0)
    net = SongUNet(img_resolution=16, in_channels=2, out_channels=2, label_dim=3, augment_dim=2, model_channels=32, channel_mult=[1, 2],
                   num_blocks=1, attn_resolutions=[8]).cuda().eval()
    x, sigma = torch.randn(4, 2, 16, 16, device="cuda"), torch.rand(4, device="cuda") + 0.1
    labels, aug = torch.randn(4, 3, device="cuda"), torch.randn(4, 2, device="cuda")
    assert net._fused_conditioning_ok(sigma)
    with torch.no_grad():
        fused = net.conditioning_embedding(x, sigma, labels, aug)
        emb = net.map_noise(sigma)
        emb = torch.cat([emb[:, emb.shape[1] // 2:], emb[:, :emb.shape[1] // 2]], dim=1)
        emb = emb + net.map_label(labels * 3 ** 0.5) + net.map_augment(aug)
        plain = torch.nn.functional.silu(net.map_layer1(torch.nn.functional.silu(net.map_layer0(emb))))
    assert torch.allclose(fused, plain, atol=1e-4)


# ---- spectral mode contraction -------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("nd", [1, 2, 3])
def test_spectral_conv_fused_corner_contraction(nd):
    from physicsnemo_b200.nn.module import spectral_layers as SL

    torch.manual_seed(0)
    cls = {1: SL.SpectralConv1d, 2: SL.SpectralConv2d, 3: SL.SpectralConv3d}[nd]
    modes = {1: (5,), 2: (4, 3), 3: (3, 2, 3)}[nd]
    shape = {1: (24,), 2: (16, 12), 3: (8, 6, 10)}[nd]
    layer = cls(6, 5, *modes)
    x = torch.randn(3, 6, *shape)
    ref_layer, xr = layer, x.clone().requires_grad_(True)                    # CPU: einsum path
    y_ref = ref_layer(xr)
    g = torch.randn_like(y_ref)
    y_ref.backward(g)
    ref_grads = [p.grad.clone() for p in ref_layer.parameters()]
    for p in ref_layer.parameters():
        p.grad = None
    gpu = layer.cuda()
    xg = x.cuda().requires_grad_(True)
    y = gpu(xg)                                                              # CUDA: fused corner kernel
    y.backward(g.cuda())
    assert torch.allclose(y.cpu(), y_ref, atol=2e-5, rtol=1e-4)
    assert torch.allclose(xg.grad.cpu(), xr.grad, atol=2e-5, rtol=1e-4)
    for p, r in zip(gpu.parameters(), ref_grads):
        assert torch.allclose(p.grad.cpu(), r, atol=2e-4, rtol=1e-3)


# ------------------------------------------------------------------------------------- spherical-harmonic norms
@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["rms", "rms_plain", "ln", "tied"])
@pytest.mark.parametrize("lmc", [(6, 2, 128), (5, 5, 64), (2, 2, 32), (3, 3, 20), (1, 1, 7)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sh_norm_kernel_matches_tensor_ops(kind, lmc, dtype):
    """Forward and backward of the grouped spherical-harmonic norm kernel against the same operator in fp32 tensor ops."""
    from physicsnemo_b200.experimental.nn.symmetry import EquivariantLayerNorm, EquivariantLayerNormTied, EquivariantRMSNorm
    from physicsnemo_b200.ops import device_error
    from physicsnemo_b200.ops import gemm as G
    from physicsnemo_b200.ops import sh_norm as S

    lmax, mmax, C = lmc
    torch.manual_seed(0)
    mod = {"rms": lambda: EquivariantRMSNorm(lmax, mmax, C), "rms_plain": lambda: EquivariantRMSNorm(lmax, mmax, C, subtract_mean=False,
                                                                                                    std_balance_degrees=False),
           "ln": lambda: EquivariantLayerNorm(lmax, mmax, C), "tied": lambda: EquivariantLayerNormTied(lmax, mmax, C)}[kind]().cuda()
    with torch.no_grad():
        for p in mod.parameters():
            p.add_(0.3 * torch.randn_like(p))
    B = 777
    x = (torch.randn(B, lmax + 1, mmax + 1, 2, C, device="cuda") * 2 + 0.5).to(dtype)
    assert S.supported(x)
    xa, xb = x.clone().requires_grad_(True), x.float().clone().requires_grad_(True)
    before = G.launch_count
    y = mod(xa)
    assert G.launch_count == before + 1 and y.dtype == dtype
    if kind == "tied":
        aff, bias = torch.cat([mod.norm_l0.weight[None], mod.affine_weight], 0), mod.norm_l0.bias
    else:
        aff, bias = mod.affine_weight, mod.affine_bias
    ref = S.reference(xb, aff, bias, mod._wstat, mod.grid_mask_3d, mod._group, mod.eps, mod._centre)
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert (y.float() - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())
    dy = torch.randn_like(ref)
    params = list(mod.parameters())
    got = torch.autograd.grad(y, [xa] + params, dy.to(dtype))
    want = torch.autograd.grad(ref, [xb] + params, dy.to(dtype).float())
    for g, w in zip(got, want):
        scale = max(1.0, w.abs().max().item())
        assert (g.float() - w).abs().max().item() <= (2e-4 if dtype == torch.float32 else 4e-2) * scale, (kind, g.shape)
    assert device_error() == 0


# ---------------------------------------------------------------------------------- pixel / observation attention
@pytest.mark.gpu
@pytest.mark.parametrize("cfg", [(300, 16, 64, 40), (257, 40, 32, 100), (64, 32, 128, 9), (50, 16, 96, 0)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_attention_kernel(cfg, dtype):
    """Forward and backward of the variable-length token-space attention kernel against dense-padded fp32 tensor ops."""
    from physicsnemo_b200.ops import device_error
    from physicsnemo_b200.ops import pixel_attention as PA

    P, H, Dt, nmax = cfg
    torch.manual_seed(0)
    counts = torch.randint(0, nmax + 1, (P,), device="cuda")
    counts[::7] = 0
    if nmax:
        counts[1] = nmax
    cu = torch.zeros(P + 1, dtype=torch.int32, device="cuda")
    cu[1:] = counts.cumsum(0)
    N = max(int(cu[-1]), 1)
    qk = (torch.randn(P, H, Dt, device="cuda") * 0.4).to(dtype)
    tok = torch.randn(N, Dt, device="cuda").to(dtype)
    assert PA.token_attention_supported(qk, tok)
    qa, ta = qk.clone().requires_grad_(True), tok.clone().requires_grad_(True)
    qb, tb = qk.float().clone().requires_grad_(True), tok.float().clone().requires_grad_(True)
    out = PA.token_attention(qa, ta, cu)
    ref, _ = PA.token_attention_reference(qb, tb, cu)
    tol = 2e-4 if dtype == torch.float32 else 3e-2
    assert (out.float() - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())
    empty = counts == 0
    assert float(out.detach()[empty].float().abs().max()) == 0.0
    g = torch.randn_like(ref)
    got = torch.autograd.grad(out, [qa, ta], g.to(dtype))
    if nmax == 0:
        assert all(float(a.float().abs().max()) == 0.0 for a in got)
    else:
        want = torch.autograd.grad(ref, [qb, tb], g.to(dtype).float())
        for a, b in zip(got, want):
            assert (a.float() - b).abs().max().item() <= (5e-4 if dtype == torch.float32 else 6e-2) * max(1.0, b.abs().max().item())
    assert device_error() == 0


@pytest.mark.gpu
def test_pixel_cross_attention_module_on_gpu_matches_cpu():
    from physicsnemo_b200.experimental.models.healda import PixelCrossAttention, prepare_obs_context

    torch.manual_seed(0)
    b, t, x, hid, Dt = 2, 2, 50, 64, 32
    P = b * t * x
    nobs = 3000
    flat = torch.randint(0, P, (nobs,))
    flat[flat % 11 == 0] = 1
    z = torch.zeros(nobs, dtype=torch.long)
    cpu = prepare_obs_context(torch.randn(nobs), torch.randn(nobs, 2), z, z, z, flat, P)
    gpu = prepare_obs_context(torch.randn(nobs).cuda(), torch.randn(nobs, 2).cuda(), z.cuda(), z.cuda(), z.cuda(), flat.cuda(), P)
    assert torch.equal(cpu.cu_seqlens_k, gpu.cu_seqlens_k.cpu()) and cpu.max_seqlen_k == gpu.max_seqlen_k
    # the packed order inside a pixel may differ: build the tokens from the pixel index so that both orders agree
    attn = PixelCrossAttention(hid, Dt, n_q_heads=32, n_kv_heads=2, d_head=16, use_proj_bias=True)
    h = torch.randn(b, t, x, hid)
    tok = torch.randn(nobs, Dt)
    order_cpu = torch.argsort(flat, stable=True)
    from physicsnemo_b200.ops.pixel_attention import counting_sort_and_pack
    order_gpu, counts = counting_sort_and_pack(flat.cuda(), P)
    assert torch.equal(flat.cuda()[order_gpu.long()], flat[order_cpu].cuda()) and torch.equal(counts.cpu(), torch.bincount(flat, minlength=P))
    y_cpu = attn(h, tok[order_cpu], cpu.cu_seqlens_k, cpu.max_seqlen_k)
    attn = attn.cuda()
    y_gpu = attn(h.cuda(), tok.cuda()[order_gpu.long()], gpu.cu_seqlens_k, gpu.max_seqlen_k)
    assert (y_gpu.cpu() - y_cpu).abs().max().item() < 2e-4


# ------------------------------------------------------------------ experimental models on their own GPU kernels
@pytest.mark.gpu
def test_strata_runs_on_neighbourhood_attention_kernels():
    """Strata with 3-D windows: the CUDA neighbourhood-attention kernels against the tensor-operation path of the same model."""
    from physicsnemo_b200.experimental.models import Strata
    from physicsnemo_b200.ops import device_error
    from physicsnemo_b200.ops import gemm as G

    torch.manual_seed(0)
    backbone = dict(in_channels=3, out_channels=2, input_shape=(4, 16, 16), patch_size=(2, 2, 2), embed_dim=64, num_heads=4, num_layers=2,
                    attn_kernel=(1, 3, 3))
    net = Strata(backbone_config=backbone, embed_dim_pixel=32, num_layers_pixel=2, num_heads_pixel=2, attn_kernel_pixel=3)
    with torch.no_grad():
        for p in net.parameters():
            p.add_(0.05 * torch.randn_like(p))
    x = torch.randn(2, 3, 4, 16, 16)
    ref = net(x)
    net, xg = net.cuda(), x.cuda().requires_grad_(True)
    before = G.launch_count
    y = net(xg)
    assert G.launch_count > before                                   # the window attention ran on the library kernels
    assert (y.cpu() - ref).abs().max().item() < 2e-3 * max(1.0, ref.abs().max().item())
    y.square().sum().backward()
    assert xg.grad is not None and bool(torch.isfinite(xg.grad).all()) and all(p.grad is not None for p in net.parameters())
    assert device_error() == 0


@pytest.mark.gpu
def test_video_healda_on_gpu_matches_cpu():
    from physicsnemo_b200.experimental.models import VideoHealDA
    from physicsnemo_b200.experimental.models.healda import prepare_obs_context
    from physicsnemo_b200.ops import gemm as G

    torch.manual_seed(0)
    net = VideoHealDA(in_channels=2, out_channels=3, hidden_size=64, num_layers=2, num_heads=4, level_in=3, level_model=2, time_length=2,
                      condition_embed_dim=32, noise_channels=32, obs_token_dim=32, obs_meta_dim=5, obs_film_hidden_dim=32,
                      pixel_attn_n_q_heads=32, pixel_attn_n_kv_heads=2, pixel_attn_head_dim=16, drop_path=0.0).eval()
    with torch.no_grad():
        for p in net.parameters():
            p.add_(0.05 * torch.randn_like(p))
    B, T, npix_c, npix = 2, 2, 12 * 16, 12 * 64
    P, n = B * T * npix_c, 5000
    ids, flat = torch.randint(0, 5, (n,)), torch.randint(0, P, (n,))
    obs, meta = torch.randn(n), torch.randn(n, 5)
    x, t = torch.randn(B, 2, T, npix), torch.rand(B)
    sod, doy = torch.rand(B, T) * 86400, torch.rand(B, T) * 365
    with torch.no_grad():
        ref = net(x, t, sod, doy, prepare_obs_context(obs, meta, ids, ids, ids, flat, P))
    net = net.cuda()
    ctx = prepare_obs_context(obs.cuda(), meta.cuda(), ids.cuda(), ids.cuda(), ids.cuda(), flat.cuda(), P)
    before = G.launch_count
    xg = x.cuda().requires_grad_(True)
    y = net(xg, t.cuda(), sod.cuda(), doy.cuda(), ctx)
    assert G.launch_count >= before + 2                              # one pixel-attention launch per block
    assert (y.detach().cpu() - ref).abs().max().item() < 2e-3 * max(1.0, ref.abs().max().item())
    y.square().sum().backward()
    assert bool(torch.isfinite(xg.grad).all()) and all(p.grad is not None for p in net.parameters())


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(2, 64, 128, 24, 40), (1, 16, 64, 16, 32), (2, 128, 4, 20, 48), (1, 192, 64, 9, 17)])
def test_conv3x3_forward_dgrad_wgrad_kernels(shape):
    """Implicit-GEMM convolution incl. the split-reduction weight-gradient kernel (and channel padding) vs fp32 conv2d."""
    from physicsnemo_b200 import ops
    from physicsnemo_b200.ops import conv as C

    n, cin, cout, h, w = shape
    torch.manual_seed(0)
    x = torch.randn(n, cin, h, w, device="cuda")
    wt = torch.randn(cout, cin, 3, 3, device="cuda") / (9 * cin) ** 0.5
    b = torch.randn(cout, device="cuda")
    dy = torch.randn(n, cout, h, w, device="cuda")
    xr, wr, br = x.clone().requires_grad_(True), wt.clone().requires_grad_(True), b.clone().requires_grad_(True)
    ref = torch.nn.functional.conv2d(xr, wr, br, padding=1)
    ref.backward(dy)
    xk, wk, bk = x.clone().requires_grad_(True), wt.clone().requires_grad_(True), b.clone().requires_grad_(True)
    assert C.supported(xk, wk)
    before = ops.kernel_launches()
    out = C.conv2d_same(xk, wk, bk)
    out.backward(dy.to(out.dtype))
    assert ops.kernel_launches() - before >= 3          # forward, input gradient, weight gradient: all library kernels

    def rel(a, r):
        return float((a.float() - r).abs().max()) / float(r.abs().max())

    assert rel(out, ref) < 2e-2
    assert rel(xk.grad, xr.grad) < 2e-2
    assert rel(wk.grad, wr.grad) < 2e-2
    assert rel(bk.grad, br.grad) < 2e-2
    assert ops.device_error() == 0


@pytest.mark.gpu
def test_conv1x1_kernels_and_box_resampling():
    from physicsnemo_b200.nn.module.conv_layers import Conv2d

    torch.manual_seed(0)
    for kw in (dict(kernel=1), dict(kernel=3, down=True), dict(kernel=3, up=True), dict(kernel=0, down=True)):
        m = Conv2d(64, 64 if kw["kernel"] == 0 else 128, amp_mode=True, **kw).cuda()
        x = torch.randn(2, 64, 16, 24, device="cuda")
        xr = x.clone().requires_grad_(True)
        w = m.weight
        # oracle: the definition with depth-wise (transposed) convolutions in fp32
        f = m.resample_filter
        y = xr
        if m.up:
            y = torch.nn.functional.conv_transpose2d(y, f.mul(4).tile([64, 1, 1, 1]), groups=64, stride=2)
        if m.down:
            y = torch.nn.functional.conv2d(y, f.tile([64, 1, 1, 1]), groups=64, stride=2)
        if w is not None:
            y = torch.nn.functional.conv2d(y, w, m.bias, padding=w.shape[-1] // 2)
        xk = x.clone().requires_grad_(True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out = m(xk)
        assert out.shape == y.shape
        assert float((out.float() - y).abs().max()) < 3e-2 * max(1.0, float(y.abs().max()))
        dy = torch.randn_like(y)
        y.backward(dy)
        out.backward(dy.to(out.dtype))
        assert float((xk.grad - xr.grad).abs().max()) < 3e-2 * float(xr.grad.abs().max())


@pytest.mark.gpu
def test_bounded_wait_gives_up_and_context_survives():
    """A wait on a flag that nothing sets returns status 0 after its budget, sets error word 6 and leaves the device usable."""
    import ctypes

    from physicsnemo_b200.ops import _lib

    lib = _lib.load(required=True)
    lib.pnm_peer_wait_probe.argtypes = [ctypes.c_void_p, ctypes.c_uint, ctypes.c_double, ctypes.c_void_p, ctypes.c_void_p]
    lib.pnm_peer_wait_probe.restype = ctypes.c_int
    assert lib.pnm_reset_error() == 0
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.full((1,), 7, dtype=torch.int32, device="cuda")
    rc = lib.pnm_peer_wait_probe(flag.data_ptr(), 1, 0.005, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0                      # gave up
    assert lib.pnm_get_error() == 6                     # ERR_WAIT_PEER
    assert lib.pnm_reset_error() == 0 and lib.pnm_get_error() == 0
    flag.fill_(1)                                       # a satisfied wait returns status 1 and raises nothing
    rc = lib.pnm_peer_wait_probe(flag.data_ptr(), 1, 0.005, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0 and int(status.item()) == 1 and lib.pnm_get_error() == 0
    a = torch.randn(64, 64, device="cuda")
    assert torch.isfinite(a @ a).all()                  # the context is intact


def _afno_filter_bf16_oracle(x, layer):
    from physicsnemo_b200.ops.afno_spectral import _expand_weight

    B, H, W, C = x.shape
    nb, Cb = layer.num_blocks, layer.block_size
    KX = min(H // 2 + 1, W // 2)
    r = lambda t: t.to(torch.bfloat16).float()                                   # noqa: E731
    X = torch.fft.rfft2(x, dim=(1, 2), norm="ortho")[:, :, :KX].reshape(B, H, KX, nb, Cb)
    z = r(torch.cat([X.real, X.imag], dim=-1))
    w1, w2 = _expand_weight(layer.w1).float(), _expand_weight(layer.w2).float()  # [nb, 2Cb out, 2Cb in], bf16-rounded
    b1 = torch.cat([layer.b1[0], layer.b1[1]], dim=1)
    b2 = torch.cat([layer.b2[0], layer.b2[1]], dim=1)
    o1 = r(torch.relu(torch.einsum("bhkni,noi->bhkno", z, w1) + b1))
    o2 = r(torch.einsum("bhkni,noi->bhkno", o1, w2) + b2)
    s = torch.nn.functional.softshrink(o2, layer.sparsity_threshold)
    spec = torch.complex(s[..., :Cb], s[..., Cb:]).reshape(B, H, KX, C)
    spec = torch.nn.functional.pad(spec, (0, 0, 0, W // 2 + 1 - KX))
    return torch.fft.irfft2(spec, s=(H, W), dim=(1, 2), norm="ortho")


@pytest.mark.gpu
@pytest.mark.parametrize("mlp", ["fp32", "bf16"])
@pytest.mark.parametrize("shape", [(2, 90, 180, 768, 8), (1, 12, 20, 64, 2), (2, 15, 36, 96, 1)])
def test_afno_spectral_filter_kernels(shape, mlp):
    """Own Fourier kernels (pruned row DFTs, two-level column DFT, soft-shrink) with the complex block MLP either in
    fp32 inside the column kernel or as tcgen05 GEMMs on the bf16 spectrum, vs torch.fft + einsum in fp32."""
    from physicsnemo_b200.nn.module.afno_layers import AFNO2DLayer
    from physicsnemo_b200.ops import afno_spectral as A

    B, H, W, C, nb = shape
    torch.manual_seed(0)
    layer = AFNO2DLayer(C, num_blocks=nb, sparsity_threshold=0.01).cuda()
    with torch.no_grad():
        for p in layer.parameters():
            p.mul_(5.0)                                    # well away from the shrink threshold
    x = torch.randn(B, H, W, C, device="cuda").to(torch.bfloat16)
    xr = x.float().requires_grad_(True)
    if mlp == "fp32":
        ref = layer(xr) - xr                               # the filter without its residual
    else:
        # ReLU and soft-shrink have discontinuous derivatives: an oracle that rounds differently flips masks and with them
        # whole gradient entries.  The oracle of the bf16 path therefore rounds to bf16 where the kernels do (spectrum,
        # weights, both MLP outputs) and is exact everywhere else.
        ref = _afno_filter_bf16_oracle(xr, layer)
    dy = torch.randn_like(ref)
    ref.backward(dy)
    gref = [p.grad.clone() for p in layer.parameters()]
    layer.zero_grad()
    kept = int((H // 2 + 1) * layer.hard_thresholding_fraction)
    geo = A.FilterGeometry(B, H, W, C, nb, kept)
    assert geo.supported()
    tok = x.reshape(-1, C).clone().requires_grad_(True)
    out = A.afno_filter(tok, layer.w1, layer.b1, layer.w2, layer.b2, geo, layer.sparsity_threshold, mlp=mlp)
    out.backward(dy.reshape(-1, C).to(out.dtype))

    def rel(a, r):
        return float((a.float() - r.float()).abs().max()) / max(float(r.float().abs().max()), 1e-12)

    def rel2(a, r):
        return float((a.float() - r.float()).norm() / r.float().norm().clamp_min(1e-12))

    tol = 2e-2 if mlp == "fp32" else 6e-2        # worst element, relative to the largest reference magnitude
    tol2 = 1e-2 if mlp == "fp32" else 1.5e-2     # relative L2 error
    pairs = [(out.reshape(B, H, W, C), ref), (tok.grad.reshape(B, H, W, C), xr.grad)]
    pairs += [(p.grad, g) for p, g in zip(layer.parameters(), gref)]
    for got, want in pairs:
        assert rel(got, want) < tol
        assert rel2(got, want) < tol2


@pytest.mark.gpu
@pytest.mark.parametrize("dims", [(2, 90, 46, 96, 2), (1, 12, 5, 32, 1)])
def test_afno_column_transforms(dims):
    """Column DFT into the bf16 [real | imag] layout (with the soft-shrink mask of the backward) and its inverse
    (with the soft-shrink of the forward) vs torch.fft on the same inputs."""
    import ctypes

    from physicsnemo_b200.ops import afno_spectral as A

    B, H, KX, Cb, nblk = dims
    lib = A._lib_af()
    geo = A.FilterGeometry(B, H, 2 * KX, Cb * nblk, nblk, KX)
    st = torch.cuda.current_stream().cuda_stream
    torch.manual_seed(0)
    Y = torch.randn(B * H, KX, nblk * Cb, 2, device="cuda")
    Mb = B * KX * H
    mask = torch.randn(nblk, Mb, 2 * Cb, device="cuda").to(torch.bfloat16)
    E = torch.empty_like(mask)
    lam = 0.7
    assert lib.pnm_afno_cols_dft(Y.data_ptr(), E.data_ptr(), mask.data_ptr(), geo.arr, Mb, lam, st) == 0
    Yc = torch.view_as_complex(Y).reshape(B, H, KX, nblk, Cb)
    F = torch.fft.fft(Yc, dim=1, norm="ortho")
    ref = torch.cat([F.real, F.imag], dim=-1).permute(3, 0, 2, 1, 4).reshape(nblk, Mb, 2 * Cb)   # rows (b, kx, ky)
    ref = ref * (mask.float().abs() > lam)
    scale = float(ref.abs().max())
    assert float((E.float() - ref).abs().max()) < 6e-3 * scale
    Y2 = torch.empty_like(Y)
    assert lib.pnm_afno_cols_idft(mask.data_ptr(), Y2.data_ptr(), geo.arr, Mb, lam, st) == 0
    m = torch.nn.functional.softshrink(mask.float(), lam).reshape(nblk, B, KX, H, 2 * Cb)
    Mc = torch.complex(m[..., :Cb], m[..., Cb:]).permute(1, 3, 2, 0, 4)          # [B, ky, KX, nblk, Cb]
    ref2 = torch.fft.ifft(Mc, dim=1, norm="ortho")
    got = torch.view_as_complex(Y2).reshape(B, H, KX, nblk, Cb)
    assert float((got - ref2).abs().max()) < 1e-4 * float(ref2.abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(1, 1, 2048, 512), (2, 2, 520, 256), (1, 1, 16384 + 64, 64)])
def test_gemm_attention_vs_fp32(shape):
    """Attention as tcgen05 GEMMs around the row softmax kernel (wide heads), forward and gradients, vs fp32 math."""
    from physicsnemo_b200.ops import gemm_attention as GA

    B, Hh, S, D = shape
    torch.manual_seed(0)
    q, k, v = (torch.randn(B, Hh, S, D, device="cuda").to(torch.bfloat16).requires_grad_(True) for _ in range(3))
    assert GA.supported(q, k, v)
    out = GA.gemm_attention(q, k, v)
    do = torch.randn_like(out)
    out.backward(do)
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    s = (qf @ kf.transpose(-1, -2)) / math.sqrt(D)
    ref = torch.softmax(s, dim=-1) @ vf
    ref.backward(do.float())

    def rel(a, r):
        return float((a.float() - r).norm() / r.norm())

    assert rel(out, ref) < 1.5e-2
    for a, r in ((q.grad, qf.grad), (k.grad, kf.grad), (v.grad, vf.grad)):
        assert rel(a, r) < 2.5e-2


@pytest.mark.gpu
def test_softmax_rows_kernels():
    from physicsnemo_b200.ops import gemm_attention as GA

    torch.manual_seed(1)
    for rows, L in ((37, 264), (5, 16384), (3, 16384 + 4096)):
        s = (torch.randn(rows, L, device="cuda") * 4).to(torch.bfloat16)
        ref = torch.softmax(s.float() * 0.3, dim=-1)
        p = GA.softmax_rows_(s.clone(), 0.3)
        assert float((p.float() - ref).abs().max()) < 4e-3 * float(ref.max()) + 1e-6
        dp = torch.randn(rows, L, device="cuda").to(torch.bfloat16)
        pr = p.float()
        dref = 0.3 * pr * (dp.float() - (dp.float() * pr).sum(-1, keepdim=True))
        ds = GA.softmax_rows_bwd_(p, dp.clone(), 0.3)
        assert float((ds.float() - dref).abs().max()) < 1e-2 * float(dref.abs().max()) + 1e-7


@pytest.mark.gpu
def test_box_resample_kernels():
    """2 x 2 mean / replication on channels-last bf16 images, with their backward passes, vs avg_pool2d / interpolate."""
    from physicsnemo_b200.ops import resample as R

    torch.manual_seed(0)
    for (n, c, h, w) in [(2, 64, 24, 40), (1, 8, 6, 2), (3, 136, 10, 14)]:
        x = torch.randn(n, c, h, w, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        assert R.supported(x)
        for fn, ref in ((R.down2x, lambda t: torch.nn.functional.avg_pool2d(t, 2)),
                        (R.up2x, lambda t: torch.nn.functional.interpolate(t, scale_factor=2, mode="nearest"))):
            a = x.clone().requires_grad_(True)
            b = x.float().clone().requires_grad_(True)
            ya, yb = fn(a), ref(b)
            assert ya.shape == yb.shape and ya.is_contiguous(memory_format=torch.channels_last)
            assert float((ya.float() - yb).abs().max()) <= 8e-3 * float(yb.abs().max())
            g = torch.randn_like(yb)
            ya.backward(g.to(torch.bfloat16))
            yb.backward(g.to(torch.bfloat16).float())
            assert float((a.grad.float() - b.grad).abs().max()) <= 1e-2 * float(b.grad.abs().max())


@pytest.mark.gpu
def test_add_scale_kernel():
    from physicsnemo_b200.ops.resample import add_scale

    torch.manual_seed(0)
    for fmt in (torch.contiguous_format, torch.channels_last):
        a = torch.randn(2, 16, 12, 10, device="cuda").to(torch.bfloat16).contiguous(memory_format=fmt).requires_grad_(True)
        b = torch.randn(2, 16, 12, 10, device="cuda").to(torch.bfloat16).contiguous(memory_format=fmt).requires_grad_(True)
        y = add_scale(a, b, 0.70710678)
        ref = (a.detach().float() + b.detach().float()) * 0.70710678
        assert y.stride() == a.stride() and float((y.float() - ref).abs().max()) < 2e-2
        g = torch.randn_like(y)
        y.backward(g)
        assert torch.allclose(a.grad.float(), g.float() * 0.70710678, atol=2e-2) and torch.equal(a.grad, b.grad)


@pytest.mark.gpu
@pytest.mark.parametrize("dims", [(2, 6, 45, 8, 8, 73), (1, 3, 5, 4, 16, 3), (2, 4, 7, 2, 3, 5), (1, 2, 40, 8, 8, 20)])
def test_unpatchify_kernel_matches_permute(dims):
    """Token -> image rearrangement and its gradient against the plain reshape / permute, bit for bit (a pure copy)."""
    from physicsnemo_b200.ops import patch_loss as pl

    B, h, w, p0, p1, C = dims
    g = torch.Generator(device="cuda").manual_seed(3)
    tokens = torch.randn(B, h, w, p0 * p1 * C, device="cuda", generator=g).to(torch.bfloat16).requires_grad_(True)
    image = pl.unpatchify(tokens, h, w, p0, p1, C)
    ref = pl._unpatchify_reference(tokens.detach(), h, w, p0, p1, C)
    assert image.shape == (B, C, h * p0, w * p1)
    assert torch.equal(image, ref)
    dimage = torch.randn(image.shape, device="cuda", generator=g).to(torch.bfloat16)
    image.backward(dimage)
    assert torch.equal(tokens.grad, pl._patchify_reference(dimage, h, w, p0, p1, C))


@pytest.mark.gpu
@pytest.mark.parametrize("pd,td,n", [(torch.bfloat16, torch.float32, 1 << 20), (torch.bfloat16, torch.bfloat16, 4099),
                                     (torch.float32, torch.float32, 77777), (torch.float32, torch.bfloat16, 8)])
def test_squared_error_kernel(pd, td, n):
    """Fused sum of squared differences and its gradient against the fp32 expression of the same loss."""
    from physicsnemo_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(5)
    pred = torch.randn(n, device="cuda", generator=g).to(pd).requires_grad_(True)
    tgt = torch.randn(n, device="cuda", generator=g).to(td)
    loss = ops.squared_error(pred, tgt, scale=0.37 / n)
    (3.0 * loss).backward()
    p32 = pred.detach().float().requires_grad_(True)
    ref = ((p32 - tgt.float()) ** 2).sum() * (0.37 / n)
    (3.0 * ref).backward()
    assert loss.dtype == torch.float32 and loss.ndim == 0
    assert abs(loss.item() - ref.item()) <= 1e-5 * abs(ref.item())
    tol = 1e-2 if pd == torch.bfloat16 else 1e-6
    assert torch.allclose(pred.grad.float(), p32.grad, rtol=tol, atol=tol * p32.grad.abs().max().item())


def test_patch_loss_host_paths():
    """On the host both ops are the plain tensor expressions."""
    from physicsnemo_b200 import ops

    tokens = torch.randn(2, 3, 4, 2 * 2 * 5)
    image = ops.unpatchify(tokens, 3, 4, 2, 2, 5)
    assert image.shape == (2, 5, 6, 8)
    assert image[1, 3, 2 * 2 + 1, 3 * 2 + 0] == tokens[1, 2, 3, (1 * 2 + 0) * 5 + 3]
    a, b = torch.randn(10, requires_grad=True), torch.randn(10)
    loss = ops.squared_error(a, b)
    assert torch.allclose(loss, torch.nn.functional.mse_loss(a, b))
    loss.backward()
    assert torch.allclose(a.grad, 2 * (a.detach() - b) / 10)
    with pytest.raises(ValueError):
        ops.squared_error(a, torch.randn(5))


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(2, 90, 180, 768, 8), (1, 12, 20, 64, 2)])
def test_afno_filter_fused_residuals(shape):
    """``afno_filter(add_input, residual)`` (sums in the store of the inverse row transform) against the same filter
    followed by the two additions in fp32: output and all gradients."""
    from physicsnemo_b200.nn.module.afno_layers import AFNO2DLayer
    from physicsnemo_b200.ops import afno_spectral as A

    B, H, W, C, nb = shape
    torch.manual_seed(1)
    layer = AFNO2DLayer(C, num_blocks=nb, sparsity_threshold=0.01).cuda()
    with torch.no_grad():
        for p in layer.parameters():
            p.mul_(5.0)
    geo = A.FilterGeometry(B, H, W, C, nb, H // 2 + 1)
    args = (layer.w1, layer.b1, layer.w2, layer.b2, geo, layer.sparsity_threshold)
    x = torch.randn(B * H * W, C, device="cuda").to(torch.bfloat16)
    r = torch.randn(B * H * W, C, device="cuda").to(torch.bfloat16)
    dy = torch.randn(B * H * W, C, device="cuda").to(torch.bfloat16)

    x0, r0 = x.clone().requires_grad_(True), r.clone().requires_grad_(True)
    ref = A.afno_filter(x0, *args).float() + x0.float() + r0.float()
    ref.backward(dy.float())
    gref = [p.grad.clone() for p in layer.parameters()]
    layer.zero_grad()

    x1, r1 = x.clone().requires_grad_(True), r.clone().requires_grad_(True)
    out = A.afno_filter(x1, *args, add_input=True, residual=r1)
    out.backward(dy)
    assert out.dtype == torch.bfloat16
    scale = ref.abs().max().item()
    assert (out.float() - ref).abs().max().item() <= 2 ** -7 * scale           # one bf16 rounding of the sum
    gscale = x0.grad.abs().max().item()
    assert (x1.grad.float() - x0.grad.float()).abs().max().item() <= 2 ** -6 * gscale
    assert torch.equal(r1.grad, dy)
    for p, g in zip(layer.parameters(), gref):
        assert torch.allclose(p.grad, g, rtol=1e-5, atol=1e-6 * g.abs().max().item())


@pytest.mark.gpu
def test_afno_block_fused_residuals_match_plain_block():
    """The AFNO block without separate elementwise kernels against the same block written with tensor additions."""
    from physicsnemo_b200.models.afno.afno import Block

    torch.manual_seed(2)
    for double_skip in (True, False):
        blk = Block(64, num_blocks=2, double_skip=double_skip).cuda()
        with torch.no_grad():
            for p in blk.filter.parameters():
                p.mul_(5.0)
        x = torch.randn(1, 12, 20, 64, device="cuda").to(torch.bfloat16)
        dy = torch.randn_like(x)
        res = []
        for fused in (True, False):
            blk.zero_grad()
            xi = x.clone().requires_grad_(True)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                if fused:
                    assert blk._fused_residuals(xi)
                    y = blk(xi)
                else:
                    mixed = blk.filter(blk.norm1(xi))
                    skip = xi
                    if double_skip:
                        mixed = skip = mixed + xi
                    y = blk.mlp(blk.norm2(mixed), residual=skip)
            y.backward(dy)
            res.append((y.detach().float(), xi.grad.float(), [p.grad.clone() for p in blk.parameters()]))
        (y1, g1, p1), (y0, g0, p0) = res
        assert (y1 - y0).abs().max().item() <= 3e-2 * y0.abs().max().item()
        assert (g1 - g0).norm().item() <= 3e-2 * g0.norm().item()
        for a, b in zip(p1, p0):
            assert (a - b).norm().item() <= 5e-2 * b.norm().item() + 1e-6

"""experimental: LoRA adapters and the variational GP head."""
import numpy as np
import pytest
import torch
import torch.nn as nn


class _Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.embed = nn.Linear(4, 16)
        self.blocks = nn.ModuleList([nn.Sequential(nn.Linear(16, 16), nn.GELU(), nn.Linear(16, 16)) for _ in range(2)])
        self.norm = nn.LayerNorm(16)
        self.head = nn.Linear(16, 3)

    def forward(self, x):
        x = self.embed(x)
        for b in self.blocks:
            x = x + b(x)
        return self.head(self.norm(x))


def test_lora_apply_train_save_load_merge(tmp_path):
    from physicsnemo_b200.experimental.peft import (LoRAConfig, apply_lora, is_lora_layer, load_adapter, merge_lora, save_adapter,
                                                    set_adapter_enabled, split_params_for_optimizer)

    torch.manual_seed(0)
    base = _Net()
    ref_state = {k: v.clone() for k, v in base.state_dict().items()}
    x = torch.randn(5, 4)
    y0 = base(x)
    res = apply_lora(base, LoRAConfig(rank=4, alpha=8, target_pattern=r"blocks\.\d+\.[02]$", extras_trainable=["norm"]))
    assert res.n_wrapped == 4 and res.n_trainable == 4 * (16 * 4 + 4 * 16) + 32
    assert torch.allclose(base(x), y0)                                            # lora_B starts at zero
    groups = split_params_for_optimizer(base)
    assert len(groups["lora"]) == 8 and len(groups["extras"]) == 2 and all(not p.requires_grad for p in groups["frozen"])
    opt = torch.optim.Adam(groups["lora"] + groups["extras"], lr=1e-2)
    for _ in range(5):
        opt.zero_grad()
        (base(x) - 1.0).square().mean().backward()
        opt.step()
    y1 = base(x)
    assert not torch.allclose(y1, y0)
    assert torch.equal(base.embed.weight, ref_state["embed.weight"])              # the base stays frozen
    set_adapter_enabled(base, False)
    assert torch.allclose(_hidden(base, x), _hidden_of_state(ref_state, x), atol=1e-6)   # adapters off: the frozen trunk is unchanged
    set_adapter_enabled(base, True)
    save_adapter(base, tmp_path / "adapter.zip")
    fresh = _Net()
    fresh.load_state_dict(ref_state)
    load_adapter(fresh, tmp_path / "adapter.zip")
    assert torch.allclose(fresh(x), y1, atol=1e-6)
    merged = merge_lora(fresh)
    assert not any(is_lora_layer(m) for m in merged.modules()) and torch.allclose(merged(x), y1, atol=1e-5)
    other = nn.Sequential(nn.Linear(4, 3))
    with pytest.raises(ValueError):
        load_adapter(other, tmp_path / "adapter.zip")                             # different architecture
    with pytest.raises(ValueError):
        LoRAConfig(rank=4)
    with pytest.raises(ValueError):
        apply_lora(base, LoRAConfig(target_modules=["embed"]))                    # not re-entrant


def _hidden_of_state(state, x):
    net = _Net()
    net.load_state_dict(state)
    return _hidden(net, x)


def _hidden(net, x):
    h = net.embed(x)
    for b in net.blocks:
        h = h + b(h)
    return h


def test_variational_gp_head_fits_a_function():
    from physicsnemo_b200.experimental.uq import VariationalGPHead

    torch.manual_seed(0)
    x = torch.linspace(-2, 2, 120).unsqueeze(1)
    y = torch.sin(2 * x[:, 0]) + 0.05 * torch.randn(120)
    head = VariationalGPHead(input_dim=1, n_train=120, n_inducing=16, inducing_points=torch.linspace(-2, 2, 16).unsqueeze(1), lengthscale_range=(0.05, 5.0))
    first = float(head.loss(x, y))
    opt = torch.optim.Adam(head.parameters(), lr=0.05)
    for _ in range(250):
        opt.zero_grad()
        loss = head.loss(x, y)
        loss.backward()
        opt.step()
    assert float(loss) < first - 0.5
    pred = head.predict(x)
    assert pred.mean.dtype == torch.float32 and float((pred.mean - torch.sin(2 * x[:, 0])).abs().mean()) < 0.1
    inside = ((y > pred.lower) & (y < pred.upper)).float().mean()
    assert float(inside) > 0.85
    far = head.predict(torch.tensor([[6.0]]))
    assert float(far.variance) > 2 * float(pred.variance.mean())                   # uncertainty grows away from the data
    dist = head(x[:5])
    assert dist.covariance_matrix.shape == (5, 5) and torch.allclose(dist.covariance_matrix, dist.covariance_matrix.t(), atol=1e-6)
    assert float(head.gp_layer.kl_divergence()) >= 0


def test_ood_guard_bounds_and_knn():
    from physicsnemo_b200.experimental.guardrails import OODGuard

    torch.manual_seed(0)
    guard = OODGuard(buffer_size=64, global_dim=2, geometry_embed_dim=8, knn_k=4, sensitivity=1.5)
    base = torch.randn(8)
    for _ in range(5):                                                # 80 samples through a 64-slot ring buffer
        guard.collect(torch.rand(16, 2) * 2 + 1, base + 0.1 * torch.randn(16, 8))
    assert bool(guard.geo_full) and float(guard.global_min.min()) >= 1.0 and float(guard.global_max.max()) <= 3.0
    flags = guard.check(torch.tensor([[2.0, 2.0], [5.0, 2.0]]), torch.stack([base + 0.1 * torch.randn(8), -base]))
    assert flags["global"].tolist() == [False, True] and flags["geometry"].tolist() == [False, True]
    assert torch.isfinite(guard.knn_threshold)
    state = guard.state_dict()
    clone = OODGuard(buffer_size=64, global_dim=2, geometry_embed_dim=8, knn_k=4)
    clone.load_state_dict(state)
    assert torch.equal(clone.geo_embeddings, guard.geo_embeddings)
    with pytest.raises(ValueError):
        guard.check(geometry_latent=torch.randn(2, 3, 8))


def test_torch_gmm_recovers_two_clusters():
    from physicsnemo_b200.experimental.guardrails import TorchGMM

    torch.manual_seed(0)
    a = torch.randn(300, 2) * 0.3 + torch.tensor([2.0, 0.0])
    b = torch.randn(200, 2) * 0.5 + torch.tensor([-2.0, 1.0])
    gmm = TorchGMM(2, max_iter=200, tol=1e-5).fit(torch.cat([a, b]))
    order = gmm.means_[:, 0].argsort()
    assert torch.allclose(gmm.means_[order], torch.tensor([[-2.0, 1.0], [2.0, 0.0]], dtype=gmm.means_.dtype), atol=0.15)
    assert torch.allclose(gmm.weights_[order], torch.tensor([0.4, 0.6], dtype=gmm.weights_.dtype), atol=0.03)
    inside, outside = gmm.score_samples(torch.tensor([[2.0, 0.0]])), gmm.score_samples(torch.tensor([[0.0, -6.0]]))
    assert float(inside) > float(outside) + 10
    other = TorchGMM(2)
    other.set_state(gmm.get_state())
    assert torch.allclose(other.score_samples(a[:5]), gmm.score_samples(a[:5]).cpu())


def test_rope_tables_and_projection():
    import math

    from physicsnemo_b200.experimental.nn import (apply_rope, build_axial_rope_cos_sin_2d_continuous, spherical_centroid,
                                                  stereographic_projection)

    torch.manual_seed(0)
    q, k = torch.randn(2, 5, 8), torch.randn(2, 5, 8)
    xa, ya = torch.rand(5) * 3, torch.rand(5) * 3
    cos, sin = build_axial_rope_cos_sin_2d_continuous(xa, ya, 8)
    shift = torch.tensor(0.7)
    cos2, sin2 = build_axial_rope_cos_sin_2d_continuous(xa + shift, ya - shift, 8)
    s1 = apply_rope(q, cos, sin) @ apply_rope(k, cos, sin).transpose(-1, -2)
    s2 = apply_rope(q, cos2, sin2) @ apply_rope(k, cos2, sin2).transpose(-1, -2)
    assert torch.allclose(s1, s2, atol=1e-4)                         # scores depend on relative positions only
    assert torch.allclose(apply_rope(q, cos, sin).norm(dim=-1), q.norm(dim=-1), atol=1e-5)
    lat = torch.tensor([[0.1, 0.2], [0.15, 0.25]])
    lon = torch.tensor([[1.0, 1.1], [1.05, 1.2]])
    lat0, lon0 = spherical_centroid(lat, lon)
    x, y = stereographic_projection(lat0, lon0, lat0, lon0)
    assert abs(float(x)) < 1e-6 and abs(float(y)) < 1e-6           # the centre maps to the origin
    x, y = stereographic_projection(lat, lon, lat0, lon0)
    assert float(torch.hypot(x, y).max()) < 0.2
    with pytest.raises(ValueError):
        build_axial_rope_cos_sin_2d_continuous(xa, ya, 6)
    assert math.isclose(float(cos[0, 0]), math.cos(float(xa[0])), rel_tol=1e-5)


def test_cached_dataset_and_prefetch(tmp_path):
    from physicsnemo_b200.experimental.utils import CachedPreprocessingDataset, prefetch_map

    calls = []

    class DS(CachedPreprocessingDataset):
        @staticmethod
        def preprocess(sample_path):
            calls.append(sample_path.name)
            return {"n": torch.tensor(int(sample_path.stem))}

    for i in range(3):
        (tmp_path / f"{i}.txt").write_text("x")
    ds = DS([tmp_path / f"{i}.txt" for i in range(3)], cache_dir=tmp_path / "cache")
    assert [int(ds[i]["n"]) for i in range(3)] == [0, 1, 2] and [int(ds[i]["n"]) for i in range(3)] == [0, 1, 2]
    assert calls == ["0.txt", "1.txt", "2.txt"]                      # the second pass came from the cache
    assert list(prefetch_map(range(5), lambda v: v * v)) == [0, 1, 4, 9, 16] and len(prefetch_map(range(5), abs)) == 5
    with pytest.raises(FileNotFoundError):
        DS([tmp_path / "missing.txt"])


def test_tedm_preconditioner_and_loss():
    from physicsnemo_b200.experimental.models import tEDMPrecondSuperRes, tEDMResidualLoss

    torch.manual_seed(0)
    net = tEDMPrecondSuperRes(img_resolution=16, img_in_channels=2, img_out_channels=3, model_type="SongUNet", nu=5, model_channels=32,
                              channel_mult=[1, 2], num_blocks=1, attn_resolutions=[8])
    x, lr, sigma = torch.randn(2, 3, 16, 16), torch.randn(2, 2, 16, 16), torch.tensor([0.5, 2.0])
    out = net(x, lr, sigma.clone())
    assert out.shape == x.shape and torch.allclose(sigma, torch.tensor([0.5, 2.0]))          # the caller's sigma is not modified
    loss = tEDMResidualLoss(regression_net=lambda *a, **k: torch.zeros(2, 3, 16, 16), nu=5)
    n, s, w = loss.get_noise_params(torch.zeros(4000, 1, 1, 1))
    assert n.shape == (4000, 1, 1, 1) and float(w.min()) > 0
    ratio = (n / s).flatten()
    assert float(ratio.abs().max()) > 4.5                                                      # heavy tails: beyond what 4000 Gaussians reach
    with pytest.raises(ValueError):
        tEDMResidualLoss(regression_net=None, nu=2)


# ------------------------------------------------------------------------------------------------ 3-D diffusion U-Net
def test_conv3d_box_resampling_matches_filtered_convolution():
    """The pooled / replicated fast path of the default box filter equals the depthwise (transposed) convolution."""
    from physicsnemo_b200.experimental.nn import Conv3D
    import torch.nn.functional as F

    torch.manual_seed(0)
    x = torch.randn(2, 3, 4, 6, 8)
    f = torch.ones(1, 1, 2, 2, 2) / 8
    down = Conv3D(3, 3, kernel=0, down=True)
    assert torch.allclose(down(x), F.conv3d(x, f.tile(3, 1, 1, 1, 1), groups=3, stride=2), atol=1e-6)
    up = Conv3D(3, 3, kernel=0, up=True)
    assert torch.allclose(up(x), F.conv_transpose3d(x, (4 * f).tile(3, 1, 1, 1, 1), groups=3, stride=2), atol=1e-6)
    # resampling fused with a 3x3x3 convolution keeps the expected shapes
    assert Conv3D(3, 5, kernel=3, down=True)(x).shape == (2, 5, 2, 3, 4)
    assert Conv3D(3, 5, kernel=3, up=True, resample_filter=[1, 3, 3, 1])(x).shape == (2, 5, 8, 12, 16)


def test_groupnorm3d_eval_uses_unbiased_variance():
    from physicsnemo_b200.experimental.nn import GroupNorm3D

    torch.manual_seed(0)
    gn = GroupNorm3D(8, num_groups=2).eval()
    with torch.no_grad():
        gn.weight.uniform_(0.5, 1.5); gn.bias.normal_()
    x = torch.randn(2, 8, 2, 3, 4)
    g = x.view(2, 2, -1)
    ref = ((g - g.mean(-1, keepdim=True)) * (g.var(-1, keepdim=True) + gn.eps).rsqrt()).view_as(x)
    ref = ref * gn.weight.view(1, -1, 1, 1, 1) + gn.bias.view(1, -1, 1, 1, 1)
    assert torch.allclose(gn(x), ref, atol=1e-5)


@pytest.mark.parametrize("enc,dec,emb", [("standard", "standard", "positional"), ("skip", "skip", "fourier"),
                                         ("residual", "standard", "zero")])
def test_diffusion_unet_3d(enc, dec, emb):
    from physicsnemo_b200.experimental.models import DiffusionUNet3D

    torch.manual_seed(0)
    vec = 0 if emb == "zero" else 3
    net = DiffusionUNet3D(x_channels=2, vol_cond_channels=1, vec_cond_dim=vec, num_levels=2, model_channels=8, channel_mult=[1, 2],
                          num_blocks=1, attention_levels=[1], encoder_type=enc, decoder_type=dec, embedding_type=emb, dropout=0.0,
                          checkpoint_level=1)
    x, t = torch.randn(2, 2, 4, 8, 8, requires_grad=True), torch.rand(2)
    cond = {"volume": torch.randn(2, 1, 4, 8, 8)}
    if vec:
        cond["vector"] = torch.randn(2, vec)
    y = net(x, t, cond)
    assert y.shape == x.shape
    y.square().sum().backward()
    assert x.grad is not None and all(p.grad is not None for p in net.parameters())
    with pytest.raises(ValueError):
        net(torch.randn(2, 2, 4, 8, 7), t, None)            # 7 is neither a power of two nor a multiple of 2
    with pytest.raises(ValueError):
        net(x, t, {"volume": cond["volume"], "other": t})


# ------------------------------------------------------------------------------------------------------- xDeepONet
def test_xdeeponet_padding_helpers():
    from physicsnemo_b200.experimental.models.xdeeponet._padding import (compute_right_pad_to_multiple, pad_right_nd,
                                                                          pad_spatial_right)
    import torch.nn.functional as F

    assert compute_right_pad_to_multiple((5, 8, 16), multiple=8) == (3, 0, 0)
    assert compute_right_pad_to_multiple((5, 8, 13), multiple=8, min_right_pad=4) == (11, 8, 11)
    x = torch.randn(2, 3, 5, 4, 2)
    y = pad_spatial_right(x, spatial_ndim=2, right_pad=(2, 3))
    ref = F.pad(x.reshape(2, 3, 5, 8).permute(0, 3, 1, 2), (0, 3, 0, 2), mode="replicate").permute(0, 2, 3, 1).reshape(2, 5, 8, 4, 2)
    assert torch.equal(y, ref)
    z = pad_right_nd(x, dims=[1, -1], right_pad=[1, 2], mode="constant", constant_value=7.0)
    assert z.shape == (2, 4, 5, 4, 4) and torch.equal(z[:, :3, :, :, :2], x) and bool((z[:, 3] == 7).all()) and bool((z[..., 2:] == 7).all())
    with pytest.raises(ValueError):
        pad_spatial_right(x, spatial_ndim=2, right_pad=(1,))


def _mlp(i, w):
    from physicsnemo_b200.models.mlp import FullyConnected
    return FullyConnected(i, w, w, 2, "tanh")


@pytest.mark.parametrize("decoder", ["mlp", "conv", "temporal_projection"])
def test_xdeeponet_trunked_variants(decoder):
    from physicsnemo_b200.experimental.models import DeepONet, SpatialBranch

    torch.manual_seed(0)
    W = 8
    net = DeepONet(SpatialBranch(2, width=W, num_fourier_layers=1, num_conv_layers=1, modes1=3, modes2=3, coord_features=True),
                   trunk=_mlp(1, W), branch2=_mlp(4, W), width=W, out_channels=2, decoder_type=decoder, decoder_width=16,
                   output_window=3 if decoder == "temporal_projection" else None)
    u, t, v = torch.randn(2, 8, 12, 3), torch.rand(5), torch.randn(2, 4)
    y = net(u, t, v)
    assert y.shape == (2, 8, 12, 3 if decoder == "temporal_projection" else 5, 2)
    assert torch.allclose(y, net(u, t, x_branch2=v))
    y.square().sum().backward()
    assert all(p.grad is not None for p in net.parameters())
    if decoder != "temporal_projection":
        # the operator is separable in time: evaluating one query time alone gives the same slice
        with torch.no_grad():
            net.eval()
            assert torch.allclose(net(u, t, v)[..., 2:3, :], net(u, t[2:3], v), atol=1e-6)
    with pytest.raises(TypeError):
        net(u)
    with pytest.raises(TypeError):
        net(u, t, v, x_branch2=v)


def test_xdeeponet_packed_and_trunkless_modes():
    from physicsnemo_b200.experimental.models import DeepONet, FNO4DWrapper, SpatialBranch

    torch.manual_seed(0)
    W = 8
    packed = DeepONet(SpatialBranch(2, width=W, num_fourier_layers=1, modes1=3, modes2=3), trunk=_mlp(3, W), width=W,
                      auto_pad=True, padding=5, trunk_input="grid")
    assert packed.padding == 8
    x = torch.randn(2, 10, 12, 4, 6)
    assert packed(x).shape == (2, 10, 12, 4, 1)
    assert packed(x, target_times=torch.rand(7)).shape == (2, 10, 12, 7, 1)

    xfno = DeepONet(SpatialBranch(3, width=W, num_fourier_layers=1, modes1=2, modes2=2, modes3=2), dimension=3, width=W,
                    auto_pad=True, time_modes=2, decoder_type="conv", decoder_layers=1)
    vol = torch.randn(1, 4, 4, 5, 3)
    assert xfno(vol).shape == (1, 4, 4, 5, 1)
    assert xfno(vol, target_times=torch.rand(2)).shape == (1, 4, 4, 2, 1)
    with pytest.raises(ValueError):
        DeepONet(_mlp(3, W), trunk=_mlp(1, W), width=W, decoder_type="conv")
    with pytest.raises(ValueError):
        DeepONet(SpatialBranch(2, width=W, num_conv_layers=1), width=W, time_modes=2)

    f4 = FNO4DWrapper(3, 1, latent_channels=4, num_fno_layers=1, num_fno_modes=2, padding=1)
    x6 = torch.randn(1, 4, 4, 4, 3, 3)
    assert f4(x6).shape == (1, 4, 4, 4, 3) and f4(x6, torch.rand(2)).shape == (1, 4, 4, 4, 2)


# --------------------------------------------------------------------------------------------- symmetry: norms
def _sh_input(B, lmax, mmax, C):
    return torch.randn(B, lmax + 1, mmax + 1, 2, C, dtype=torch.float64)


def test_equivariant_rms_norm_formula():
    """Direct restatement: masked input, centred scalar row, one balanced RMS, per-degree weight, bias on the scalar row."""
    from physicsnemo_b200.experimental.nn.symmetry import (EquivariantRMSNorm, make_degree_balance_weight, make_grid_mask,
                                                          make_m0_imag_mask)

    torch.manual_seed(0)
    lmax, mmax, C = 3, 2, 6
    mod = EquivariantRMSNorm(lmax, mmax, C).double()
    with torch.no_grad():
        mod.affine_weight.uniform_(0.5, 1.5); mod.affine_bias.normal_()
    x = _sh_input(4, lmax, mmax, C)
    mask = make_grid_mask(lmax, mmax).double()[None, :, :, None, None] * make_m0_imag_mask(mmax).double()
    xm = x * mask
    xm[:, 0, 0, 0] -= xm[:, 0, 0, 0].mean(-1, keepdim=True)
    w = make_degree_balance_weight(lmax, mmax).double()
    ms = torch.einsum("blmrc,lm->b", xm ** 2, w) / (2 * C)
    want = xm * (ms + mod.eps).rsqrt()[:, None, None, None, None] * mod.affine_weight[None, :, None, None, :]
    want[:, 0, 0, 0] += mod.affine_bias
    want = want * mask
    assert torch.allclose(mod(x), want, atol=1e-12)
    assert float(w.sum()) == pytest.approx(1.0)           # every degree carries 1 / (lmax + 1)


def test_equivariant_norms_are_rotation_equivariant_about_z():
    """A rotation about z multiplies order m by exp(i m phi): the norms commute with it and ignore invalid entries."""
    from physicsnemo_b200.experimental.nn.symmetry import (EquivariantLayerNorm, EquivariantLayerNormTied, EquivariantRMSNorm,
                                                          FusedEquivariantRMSNorm)

    torch.manual_seed(0)
    lmax, mmax, C = 4, 3, 5
    x = _sh_input(3, lmax, mmax, C)
    phi = 0.7
    m = torch.arange(mmax + 1, dtype=torch.float64)
    cos, sin = torch.cos(m * phi)[None, None, :, None], torch.sin(m * phi)[None, None, :, None]

    def rotate(t):
        re, im = t[..., 0, :], t[..., 1, :]
        return torch.stack([cos * re - sin * im, sin * re + cos * im], dim=-2)

    for cls in (EquivariantRMSNorm, EquivariantLayerNorm, EquivariantLayerNormTied, FusedEquivariantRMSNorm):
        mod = cls(lmax, mmax, C).double()
        with torch.no_grad():
            for p in mod.parameters():
                p.add_(0.2 * torch.randn_like(p))
        y = mod(x)
        valid = mod.grid_mask_3d[None, :, :, :, None].double()
        assert torch.allclose(mod(rotate(x * valid)), rotate(y), atol=1e-10), cls.__name__
        junk = x + (1 - valid) * 100.0
        assert torch.allclose(mod(junk), y, atol=1e-12) and bool((y * (1 - valid) == 0).all())
    with pytest.raises(ValueError):
        EquivariantLayerNormTied(0, 0, 4)
    with pytest.raises(ValueError):
        EquivariantRMSNorm(2, 3, 4)
    with pytest.raises(ValueError):
        EquivariantRMSNorm(2, 1, 4)(torch.randn(2, 3, 2, 2, 5))


def test_equivariant_layer_norm_tied_scalar_row_is_layer_norm():
    from physicsnemo_b200.experimental.nn.symmetry import EquivariantLayerNormTied

    torch.manual_seed(0)
    mod = EquivariantLayerNormTied(3, 2, 8).double()
    with torch.no_grad():
        mod.norm_l0.weight.uniform_(0.5, 1.5); mod.norm_l0.bias.normal_()
    x = _sh_input(5, 3, 2, 8).requires_grad_(True)
    y = mod(x)
    assert torch.allclose(y[:, 0, 0, 0], mod.norm_l0(x[:, 0, 0, 0]), atol=1e-12)
    y.square().sum().backward()
    assert mod.norm_l0.weight.grad is not None and mod.affine_weight.grad is not None and x.grad is not None
    # scaling the l > 0 part leaves its normalised output unchanged (up to eps)
    x2 = x.detach().clone(); x2[:, 1:] *= 7.0
    assert torch.allclose(mod(x2)[:, 1:], y[:, 1:].detach(), atol=1e-4)


# ------------------------------------------------------------------------ symmetry: linear maps, gates, rotations
def _random_rotation_angles(B):
    return tuple(torch.rand(B, dtype=torch.float64) * 6.0 - 3.0 for _ in range(3))


def test_wigner_matrices_form_a_representation():
    """D is orthogonal, D(identity) = 1, D(R1) D(R2) = D(R1 R2) for rotations about one axis, and l = 1 rotates vectors."""
    from physicsnemo_b200.experimental.nn.symmetry import compute_wigner_d_matrices

    torch.manual_seed(0)
    a, b, g = _random_rotation_angles(5)
    D = compute_wigner_d_matrices(a, b, g, 4)
    eye = torch.eye(25, dtype=torch.float64)
    assert D.shape == (5, 25, 25) and torch.allclose(D @ D.transpose(1, 2), eye.expand(5, -1, -1), atol=1e-10)
    zero = torch.zeros(5, dtype=torch.float64)
    assert torch.allclose(compute_wigner_d_matrices(zero, zero, zero, 4), eye.expand(5, -1, -1), atol=1e-12)
    D1 = compute_wigner_d_matrices(a, zero, zero, 3)
    D2 = compute_wigner_d_matrices(b, zero, zero, 3)
    assert torch.allclose(D1 @ D2, compute_wigner_d_matrices(a + b, zero, zero, 3), atol=1e-10)
    # block structure: nothing couples different degrees
    off = D.clone()
    for l in range(5):
        off[:, l * l:(l + 1) ** 2, l * l:(l + 1) ** 2] = 0
    assert float(off.abs().max()) == 0.0
    # the l = 1 block is a proper rotation (determinant +1)
    assert torch.allclose(torch.linalg.det(D[:, 1:4, 1:4]), torch.ones(5, dtype=torch.float64), atol=1e-10)


def test_edge_rotation_aligns_and_inverts():
    from physicsnemo_b200.experimental.nn.symmetry import EdgeRotation, edge_vectors_to_euler_angles

    torch.manual_seed(0)
    rot = EdgeRotation(3, 2).double()
    ev = torch.randn(4, 5, 3, dtype=torch.float64)
    mask = torch.rand(4, 5) > 0.3
    with pytest.raises(RuntimeError):
        rot(torch.randn(4, 5, 16, 2, dtype=torch.float64))
    W = rot.get_wigner_matrices(ev, mask)
    assert W.shape == (4, 5, rot._reduced_dim, 16) and rot._reduced_dim == 1 + 3 + 5 + 5
    x = torch.randn(4, 5, 16, 6, dtype=torch.float64)
    y = rot(x)
    assert torch.allclose(y, W @ x, atol=1e-12)                            # block application = dense matrix
    assert torch.allclose(rot(y, inverse=True), W.transpose(-1, -2) @ y, atol=1e-12)
    # rows of an orthogonal matrix: W W^T = 1 on the reduced space; masked edges carry the selection matrix
    assert torch.allclose(W @ W.transpose(-1, -2), torch.eye(rot._reduced_dim, dtype=torch.float64).expand(4, 5, -1, -1), atol=1e-6)   # J is stored in fp32
    sel = W[~mask]
    assert bool(((sel == 0) | (sel == 1)).all()) and bool((sel.sum(-1) == 1).all())
    # with mmax = lmax the round trip is exact
    full = EdgeRotation(3).double()
    full.get_wigner_matrices(ev)
    assert torch.allclose(full(full(x), inverse=True), x, atol=1e-6)
    # the pole direction has finite gradients
    pole = torch.tensor([[[0.0, 1.0, 0.0]]], dtype=torch.float64, requires_grad=True)
    a, b, _ = edge_vectors_to_euler_angles(pole)
    (a.sum() + b.sum()).backward()
    assert bool(torch.isfinite(pole.grad).all())
    rot.clear_cache()
    assert rot._cached_wigner is None


def test_so3_layers_commute_with_rotations():
    """Per-degree linear maps and the gated block commute with any rotation of the grid.  (The grid norms weight the
    stored orders m >= 0 once each, so they commute with rotations about the polar axis only; see the test above.)"""
    from physicsnemo_b200.experimental.nn.symmetry import SO3ConvolutionBlock, SO3LinearGrid, rotate_grid_coefficients

    torch.manual_seed(0)
    lmax, C = 3, 4
    x = torch.randn(2, lmax + 1, lmax + 1, 2, C, dtype=torch.float64)
    x = rotate_grid_coefficients(x, (0.0, 0.0, 0.0))                     # project on the valid coefficients
    rot = _random_rotation_angles(2)
    for layer in (SO3LinearGrid(C, 5, lmax, lmax), SO3ConvolutionBlock(C, 6, lmax, lmax)):
        layer = layer.double()
        a = layer(rotate_grid_coefficients(x, rot))
        b = rotate_grid_coefficients(layer(x), rot)
        assert torch.allclose(a, b, atol=1e-9), type(layer).__name__


def test_so2_convolution_is_complex_linear_per_order():
    from physicsnemo_b200.experimental.nn.symmetry import GateActivation, SO2Convolution, rotate_grid_coefficients

    torch.manual_seed(0)
    lmax, mmax, C, O = 3, 2, 4, 5
    conv = SO2Convolution(C, O, lmax, mmax, edge_channels=3, produce_gates=True).double()
    x = torch.randn(6, lmax + 1, mmax + 1, 2, C, dtype=torch.float64)
    e = torch.randn(6, 3, dtype=torch.float64)
    y = conv(x, e)
    assert y.shape == (6, lmax + 1, mmax + 1, 2, O + lmax * O)
    # gate channels live on the scalar row only
    assert float(y[:, 1:, :, :, O:].abs().max()) == 0.0 and float(y[:, 0, 1:, :, O:].abs().max()) == 0.0
    # complex arithmetic of order m = 1 at degree l = 2
    xm = x * conv.rad_func(e).view(6, lmax + 1, mmax + 1, 2, C)
    z = torch.complex(xm[:, 2, 1, 0], xm[:, 2, 1, 1]) @ torch.complex(conv.W_r[1], conv.W_i[1])
    assert torch.allclose(y[:, 2, 1, 0, :O], z.real[:, :O], atol=1e-12) and torch.allclose(y[:, 2, 1, 1, :O], z.imag[:, :O], atol=1e-12)
    # equivariance about the edge axis (rotation by gamma only multiplies order m by a phase)
    plain = SO2Convolution(C, O, lmax, mmax).double()
    xs = rotate_grid_coefficients(torch.randn(6, lmax + 1, lmax + 1, 2, C, dtype=torch.float64), (0.0, 0.0, 0.0))[:, :, :mmax + 1]
    m = torch.arange(mmax + 1, dtype=torch.float64)
    c, s = torch.cos(0.9 * m)[None, None, :, None], torch.sin(0.9 * m)[None, None, :, None]
    spin = lambda t: torch.stack([c * t[..., 0, :] - s * t[..., 1, :], s * t[..., 0, :] + c * t[..., 1, :]], dim=-2)  # noqa: E731
    assert torch.allclose(plain(spin(xs)), spin(plain(xs)), atol=1e-10)
    gate = GateActivation(lmax, mmax, O).double()
    assert gate(y).shape == (6, lmax + 1, mmax + 1, 2, O)
    with pytest.raises(ValueError):
        conv(x)


# ------------------------------------------------------------------------------------------------------ Strata
def _latlon(B, H, W):
    lat = torch.linspace(30, 40, H)[None, :, None].expand(B, H, W)
    lon = torch.linspace(10, 25, W)[None, None, :].expand(B, H, W)
    return torch.stack([lat, lon], 1)


def test_strata_patch_embed_equals_strided_convolution():
    from physicsnemo_b200.experimental.models.strata.layers import PatchEmbed3D

    torch.manual_seed(0)
    pe = PatchEmbed3D(4, 8, 6, patch_size=(2, 4, 3), in_chans=3, embed_dim=10)
    x = torch.randn(2, 3, 4, 8, 6)
    ref = torch.nn.functional.conv3d(x, pe.proj.weight, pe.proj.bias, stride=(2, 4, 3))
    assert torch.allclose(pe(x), ref, atol=1e-5)
    tok, dhw = pe.tokens(x)
    assert dhw == (2, 2, 2) and torch.allclose(tok, ref.flatten(2).transpose(1, 2), atol=1e-5)
    with pytest.raises(ValueError):
        PatchEmbed3D(4, 8, 6, patch_size=(3, 4, 3))


@pytest.mark.parametrize("kw", [dict(attn_kernel=-1), dict(attn_kernel=(1, 3, 3), do_interleaved_dilation=True, na_dilation=1),
                                dict(attn_kernel=3, do_alt_depthwise_attn=True, gated_attention=True, qk_norm=True, rope_mode="axial"),
                                dict(attn_kernel=-1, rope_mode="stereographic", activation_checkpointing=0.5)])
def test_strata_transformer_3d(kw):
    from physicsnemo_b200.experimental.models import StrataTransformer3D

    torch.manual_seed(0)
    net = StrataTransformer3D(in_channels=3, out_channels=2, input_shape=(4, 8, 8), patch_size=(1, 2, 2), embed_dim=32, num_heads=4,
                              num_layers=3, **kw)
    x = torch.randn(2, 3, 4, 8, 8)
    pos = _latlon(2, 8, 8) if kw.get("rope_mode") == "stereographic" else None
    assert float(net(x, pos).abs().max()) == 0.0               # the head starts at zero
    with torch.no_grad():
        net.final_layer.linear.weight.normal_(std=0.1)
    y = net(x, pos)
    assert y.shape == (2, 2, 4, 8, 8)
    y.square().sum().backward()
    assert all(p.grad is not None for p in net.parameters())
    tok, dhw = net.forward_tokens(x, pos)
    assert tok.shape == (2, 4 * 4 * 4, 32) and dhw == (4, 4, 4)
    with pytest.raises(ValueError):
        net(torch.randn(2, 3, 4, 8, 6), pos)
    if kw.get("rope_mode") == "stereographic":
        with pytest.raises(ValueError):
            net(x)


def test_strata_neighbourhood_attention_is_local():
    """With a 3x3x3 window and one layer, a perturbation only reaches tokens within one patch step."""
    from physicsnemo_b200.experimental.models import StrataTransformer3D

    torch.manual_seed(0)
    net = StrataTransformer3D(in_channels=2, input_shape=(8, 8, 8), patch_size=1, embed_dim=16, num_heads=2, num_layers=1,
                              attn_kernel=3, include_head=False).eval()
    x = torch.randn(1, 2, 8, 8, 8)
    x2 = x.clone()
    x2[0, :, 3, 4, 4] += 1.0
    with torch.no_grad():
        diff = (net(x2) - net(x)).abs().sum(-1).reshape(8, 8, 8)
    touched = diff > 1e-7
    assert bool(touched[3, 4, 4]) and not bool(touched[0].any()) and not bool(touched[:, 0].any()) and not bool(touched[:, :, 7].any())
    assert int(touched.sum()) <= 27


@pytest.mark.parametrize("mode", ["pixel_proj", "bilinear_dw"])
def test_strata_two_stage(mode):
    from physicsnemo_b200.experimental.models import Strata
    from physicsnemo_b200.experimental.models.strata.layers import StrataPixel3DBlock, StrataTransformer3DBlock

    torch.manual_seed(0)
    backbone = dict(in_channels=3, out_channels=2, input_shape=(4, 8, 8), patch_size=(2, 2, 2), embed_dim=32, num_heads=4, num_layers=1,
                    attn_kernel=-1)
    net = Strata(backbone_config=backbone, embed_dim_pixel=16, num_layers_pixel=2, num_heads_pixel=2, attn_kernel_pixel=(1, 3, 3),
                 adaln_mode=mode, first_block_only_adaln=True, rope_mode_pixel="stereographic", activation_checkpointing_pixel=True)
    assert isinstance(net.pixel_blocks[0], StrataPixel3DBlock) and isinstance(net.pixel_blocks[1], StrataTransformer3DBlock)
    assert net.backbone.final_layer is None
    with torch.no_grad():
        for p in net.parameters():
            p.add_(0.05 * torch.randn_like(p))
    x, pos = torch.randn(2, 3, 4, 8, 8), _latlon(2, 8, 8)
    y = net(x, pos)
    assert y.shape == (2, 2, 4, 8, 8)
    y.square().sum().backward()
    assert all(p.grad is not None for p in net.parameters())
    with pytest.raises(ValueError):
        net(x)                                                  # stereographic rotary needs lat / lon


def test_strata_chunked_depthwise_conv_matches_plain():
    from physicsnemo_b200.experimental.models.strata.layers import DepthwiseConv

    torch.manual_seed(0)
    conv = DepthwiseConv(6, kernel_size=(5, 5), padding=(2, 2), bias=True, padding_mode="replicate", chunk_size=2)
    x = torch.randn(5, 6, 7, 9)
    ref = torch.nn.functional.conv2d(torch.nn.functional.pad(x, (2, 2, 2, 2), mode="replicate"), conv.weight, conv.bias, groups=6)
    assert torch.allclose(conv(x), ref, atol=1e-6)
    with pytest.raises(ValueError):
        DepthwiseConv(6, kernel_size=3, groups=2)


# ------------------------------------------------------------------------------------------- HealDA attention
def _naive_pixel_attention(Q, tokens, W_k, W_v, cu, n_kv, scale, B_v=None):
    P, Hq, dh = Q.shape
    out = torch.zeros_like(Q)
    for p in range(P):
        s, e = int(cu[p]), int(cu[p + 1])
        if s == e:
            continue
        K = (tokens[s:e] @ W_k.t()).view(-1, n_kv, dh)
        V = tokens[s:e] @ W_v.t()
        V = (V + B_v if B_v is not None else V).view(-1, n_kv, dh)
        for h in range(Hq):
            kv = h // (Hq // n_kv)
            out[p, h] = torch.softmax(K[:, kv] @ Q[p, h] * scale, 0) @ V[:, kv]
    return out


def test_pixel_attention_matches_per_pixel_softmax():
    from physicsnemo_b200.ops.pixel_attention import pixel_attention

    torch.manual_seed(0)
    P, n_kv, g, dh, Dt = 9, 2, 3, 8, 12
    counts = torch.tensor([3, 0, 5, 1, 0, 2, 4, 0, 7])
    cu = torch.zeros(P + 1, dtype=torch.int32)
    cu[1:] = counts.cumsum(0)
    Q = torch.randn(P, n_kv * g, dh, dtype=torch.float64, requires_grad=True)
    tok = torch.randn(int(cu[-1]), Dt, dtype=torch.float64, requires_grad=True)
    Wk, Wv = (torch.randn(n_kv * dh, Dt, dtype=torch.float64, requires_grad=True) for _ in range(2))
    Bv = torch.randn(n_kv * dh, dtype=torch.float64, requires_grad=True)
    out = pixel_attention(Q, tok, Wk, Wv, cu, 7, n_kv_heads=n_kv, scale=0.3, B_v=Bv, B_k=torch.randn(n_kv * dh, dtype=torch.float64))
    ref = _naive_pixel_attention(Q, tok, Wk, Wv, cu, n_kv, 0.3, Bv)
    assert torch.allclose(out, ref, atol=1e-10)
    assert float(out[1].abs().max()) == 0.0 and float(out[4].abs().max()) == 0.0          # pixels without observations
    w = torch.randn_like(out)
    got = torch.autograd.grad((out * w).sum(), [Q, tok, Wk, Wv, Bv])
    want = torch.autograd.grad((ref * w).sum(), [Q, tok, Wk, Wv, Bv])
    for a, b in zip(got, want):
        assert torch.allclose(a, b, atol=1e-9)
    # no observation at all
    none = pixel_attention(Q, tok[:0], Wk, Wv, torch.zeros(P + 1, dtype=torch.int32), 0, n_kv_heads=n_kv, scale=0.3, B_v=Bv)
    assert none.shape == Q.shape and float(none.abs().max()) == 0.0


def test_obs_context_packs_by_pixel():
    from physicsnemo_b200.experimental.models.healda import build_pixel_group_map, prepare_obs_context

    torch.manual_seed(0)
    nobs, P = 50, 12
    flat = torch.randint(0, P, (nobs,))
    flat[flat == 5] = 6                                             # one empty pixel
    obs, meta = torch.randn(nobs), torch.randn(nobs, 4)
    typ, ch, plat = (torch.randint(0, 5, (nobs,)) for _ in range(3))
    ctx = prepare_obs_context(obs, meta, typ, ch, plat, flat, P)
    counts = torch.bincount(flat, minlength=P)
    assert torch.equal(ctx.cu_seqlens_k[1:].long(), counts.cumsum(0)) and ctx.max_seqlen_k == int(counts.max())
    for p in range(P):
        s, e = int(ctx.cu_seqlens_k[p]), int(ctx.cu_seqlens_k[p + 1])
        assert sorted(ctx.obs[s:e].tolist()) == sorted(obs[flat == p].tolist())
    gm = build_pixel_group_map(ctx.cu_seqlens_k)
    assert sorted(gm.program_pixels.tolist()) == torch.nonzero(counts > 0).flatten().tolist()
    assert int(gm.program_ptr[-1]) == gm.program_pixels.numel()
    empty = prepare_obs_context(obs[:0], meta[:0], typ[:0], ch[:0], plat[:0], flat[:0], P)
    assert empty.max_seqlen_k == 0 and int(empty.cu_seqlens_k[-1]) == 0 and empty.group_map.program_pixels.numel() == 0
    assert ctx.to(torch.float64).float_metadata.dtype == torch.float64 and ctx.to(torch.float64).channel.dtype == ch.dtype
    with pytest.raises(ValueError):
        prepare_obs_context(obs, meta[:3], typ, ch, plat, flat, P)


def test_healda_attention_layers():
    from physicsnemo_b200.experimental.models.healda import PixelCrossAttention, TemporalAttention, prepare_obs_context

    torch.manual_seed(0)
    b, t, x, hid, Dt = 2, 2, 3, 16, 8
    P = b * t * x
    flat = torch.randint(0, P, (40,))
    z = torch.zeros(40, dtype=torch.long)
    ctx = prepare_obs_context(torch.randn(40), torch.randn(40, 2), z, z, z, flat, P)
    attn = PixelCrossAttention(hid, Dt, n_q_heads=16, n_kv_heads=1, d_head=4, use_proj_bias=True)
    h = torch.randn(b, t, x, hid, requires_grad=True)
    tok = torch.randn(40, Dt, requires_grad=True)
    y = attn(h, tok, ctx.cu_seqlens_k, ctx.max_seqlen_k, group_map=ctx.group_map)
    assert y.shape == h.shape
    y.square().sum().backward()
    assert h.grad is not None and tok.grad is not None and all(p.grad is not None for p in attn.parameters())
    with pytest.raises(ValueError):
        attn(h, tok, ctx.cu_seqlens_k[:-1], ctx.max_seqlen_k)
    with pytest.raises(ValueError):
        PixelCrossAttention(hid, Dt, n_q_heads=15, n_kv_heads=3, d_head=4)

    # causal softmax attention over time: the output at step q ignores later steps
    ta = TemporalAttention(hidden_size=hid, num_heads=4, use_rope=False, is_causal=True, linear_attention=False)
    x1 = torch.randn(1, 4, 3, hid)
    x2 = x1.clone()
    x2[:, 3] += 1.0
    with torch.no_grad():
        d = (ta(x1) - ta(x2)).abs().amax(dim=(0, 2, 3))
    assert float(d[:3].max()) < 1e-6 and float(d[3]) > 1e-4
    with pytest.raises(ValueError):
        TemporalAttention(hidden_size=hid, num_heads=4)(x1)        # rope tables missing
    with pytest.raises(ValueError):
        TemporalAttention(hidden_size=hid, num_heads=4, causal_window=2)


def test_healda_film_tokenizer_reassociated_first_layer():
    """Projected-table gathers give the same tokens and gradients as the concatenate-then-multiply form."""
    from physicsnemo_b200.experimental.models.healda import ObsTokenizerFiLM

    torch.manual_seed(0)
    tok = ObsTokenizerFiLM(3, 8, platform_embed_dim=2, channel_embed_dim=5).double()
    n = 64
    obs, meta = torch.randn(n, dtype=torch.float64), torch.randn(n, 3, dtype=torch.float64)
    ids = [torch.randint(0, 1024, (n,)) for _ in range(3)]
    a = tok(obs, meta, *ids)
    ga = torch.autograd.grad(a.square().sum(), list(tok.parameters()))
    tok.use_fused_mlp = False
    b = tok(obs, meta, *ids)
    gb = torch.autograd.grad(b.square().sum(), list(tok.parameters()))
    assert a.shape == (n, 8) and torch.allclose(a, b, atol=1e-12)
    assert all(torch.allclose(u, v, atol=1e-10) for u, v in zip(ga, gb))
    with pytest.raises(ValueError):
        tok(obs, meta, ids[0], ids[1])                              # platform ids missing
    with pytest.raises(ValueError):
        tok(obs, meta[:, :2], *ids)


def test_healda_scatter_aggregator():
    from physicsnemo_b200.experimental.models.healda import ScatterAggregator, scatter_mean

    torch.manual_seed(0)
    x = torch.randn(30, 4)
    bi, px, bk = torch.randint(0, 2, (30,)), torch.randint(0, 5, (30,)), torch.randint(0, 3, (30,))
    mean, present = scatter_mean(x, torch.stack([bi, px, bk], -1), (2, 5, 3))
    for b in range(2):
        for p in range(5):
            for k in range(3):
                sel = (bi == b) & (px == p) & (bk == k)
                assert bool(present[b, p, k]) == bool(sel.any())
                if sel.any():
                    assert torch.allclose(mean[b, p, k], x[sel].mean(0), atol=1e-6)
                else:
                    assert bool(torch.isnan(mean[b, p, k]).all())
    agg = ScatterAggregator(4, 6, 3)
    y = agg(x.requires_grad_(True), bi, px, bk, 2, 5)
    assert y.shape == (2, 5, 6)
    y.sum().backward()
    assert x.grad is not None


def test_healda_adaln_helpers():
    from physicsnemo_b200.experimental.models.healda import AdaLNModulation, gated_residual, modulate

    torch.manual_seed(0)
    x, c = torch.randn(2, 3, 5, 8), torch.randn(2, 6)
    mod = AdaLNModulation(8, 6, n_blocks=2)
    parts = mod(c)
    assert len(parts) == 6 and all(p.shape == (2, 8) and float(p.abs().max()) == 0.0 for p in parts)
    assert torch.equal(modulate(x, parts[0], parts[1]), x) and torch.equal(gated_residual(x, x, parts[2]), x)
    shift, scale, gate = torch.randn(2, 8), torch.randn(2, 8), torch.randn(2, 8)
    assert torch.allclose(modulate(x, shift, scale), x * (1 + scale[:, None, None]) + shift[:, None, None], atol=1e-6)
    assert torch.allclose(gated_residual(x, 2 * x, gate), x + gate[:, None, None] * 2 * x, atol=1e-6)
    assert float(AdaLNModulation(8, 6, zero_init=False)(c)[0].abs().max()) > 0


def test_healda_multi_sensor_embedder():
    from physicsnemo_b200.experimental.models.healda import MultiSensorObsEmbedder

    torch.manual_seed(0)
    emb = MultiSensorObsEmbedder(nchannel_per_sensor=[2, 3], nplatform_per_sensor=[1, 2], sensor_names=["amsu", "iasi"], embed_dim=8,
                                 meta_dim=3, fusion_dim=12, gradient_checkpointing=True)
    B, T, npix = 2, 2, 6
    counts = torch.randint(1, 6, (2, B, T))
    offsets = counts.flatten().cumsum(0).view(2, B, T)
    n = int(offsets[-1, -1, -1])
    obs, meta = torch.randn(n, requires_grad=True), torch.randn(n, 3)
    pix, lc, lp, ty = torch.randint(0, npix, (n,)), torch.randint(0, 2, (n,)), torch.zeros(n, dtype=torch.long), torch.randint(0, 9, (n,))
    out = emb(obs, meta, pix, lc, lp, ty, offsets, npix)
    assert out.shape == (B, 12, T, npix)
    out.square().sum().backward()
    assert obs.grad is not None and all(p.grad is not None for p in emb.parameters())
    # an observation only influences its own (batch, time, pixel) site
    obs2 = obs.detach().clone()
    obs2[0] += 1.0
    with torch.no_grad():
        d = (emb(obs2, meta, pix, lc, lp, ty, offsets, npix) - emb(obs.detach(), meta, pix, lc, lp, ty, offsets, npix)).abs().sum(1)
    hit = torch.nonzero(d > 1e-7)
    assert hit.shape[0] == 1 and hit[0].tolist() == [0, 0, int(pix[0])]
    with pytest.raises(ValueError):
        emb(obs, meta, pix, lc, lp, ty, offsets[:1], npix)
    with pytest.raises(ValueError):
        MultiSensorObsEmbedder([1, 2], [1])


def test_guarded_geotransolver_collects_in_training_and_checks_in_eval():
    import warnings

    from physicsnemo_b200.experimental.guardrails import GuardedGeoTransolver, OODGuardConfig, attach_ood_guard
    from physicsnemo_b200.models.geotransolver import GeoTransolver

    torch.manual_seed(0)
    model = GeoTransolver(functional_dim=3, out_dim=2, geometry_dim=3, global_dim=4, n_layers=1, n_hidden=32, n_head=4, slice_num=8)
    guard = attach_ood_guard(model, OODGuardConfig(buffer_size=64, knn_k=3, sensitivity=1.5))
    assert isinstance(guard, GuardedGeoTransolver) and guard.ood_guard.global_min.shape == (4,)
    x, geo = torch.randn(2, 50, 3), torch.randn(2, 50, 3)
    glob = torch.rand(2, 1, 4)
    guard.train()
    for _ in range(4):
        y = guard(x, global_embedding=torch.rand(2, 1, 4), geometry=torch.randn(2, 50, 3))
    assert y.shape == (2, 50, 2) and bool(torch.isfinite(guard.ood_guard.global_min).all())
    guard.eval()
    out = guard(x, global_embedding=glob * 0.5 + 0.25, geometry=geo)          # inside the training range
    assert not bool(guard.ood_guard.last_flags["global"].any())
    guard(x, global_embedding=glob + 50.0, geometry=geo)                      # far outside: flagged (and logged)
    assert bool(guard.ood_guard.last_flags["global"].all()) and guard.ood_guard.last_flags["geometry"] is not None
    assert torch.equal(out, model(x, global_embedding=glob * 0.5 + 0.25, geometry=geo))
    with pytest.raises(ValueError):
        guard(x, global_embedding=torch.rand(2, 1, 5), geometry=geo)
    guard.close()
    assert guard._geo_hook_handle is None


# ------------------------------------------------------------------------------------------- geometry guardrail
def _ellipsoid(scale, shift=(0.0, 0.0, 0.0)):
    from physicsnemo_b200.mesh import Mesh
    from physicsnemo_b200.mesh.primitives import icosphere

    m = icosphere(subdivisions=2)
    pts = m.points * torch.tensor(scale, dtype=m.points.dtype) + torch.tensor(shift, dtype=m.points.dtype)
    return Mesh(points=pts, cells=m.cells)


@pytest.mark.parametrize("method", ["gmm", "pce"])
def test_geometry_guardrail_flags_unusual_shapes(tmp_path, method):
    from physicsnemo_b200.datapipes.mesh_dataset import save_mesh_npz
    from physicsnemo_b200.experimental.guardrails.geometry import FeatureSchema, GeometryGuardrail, extract_features

    torch.manual_seed(0)
    train = [_ellipsoid((1.0 + 0.1 * float(a), 0.6 + 0.05 * float(b), 0.4 + 0.05 * float(c)), (0.02 * float(d), 0.0, 0.0))
             for a, b, c, d in torch.randn(60, 4)]
    f = extract_features(train[0])
    assert f.shape == (FeatureSchema.dim,) == (22,) and abs(f[18] - float(train[0].cell_areas.sum())) < 1e-5
    assert f[12] > f[13] > f[14] > 0 and f[9] >= f[10] >= f[11] > 0           # extents and principal variances of an ellipsoid
    guard = GeometryGuardrail(method=method, warn_pct=95.0, reject_pct=99.5, pce_components=3)
    guard.fit(train)
    inside = guard.query([_ellipsoid((1.02, 0.61, 0.41))])[0]
    far = guard.query([_ellipsoid((4.0, 0.2, 3.0), (5.0, 0.0, 0.0))])[0]
    assert inside["status"] == "OK" and far["status"] == "REJECT" and far["percentile"] == 100.0
    path = tmp_path / "guard.npz"
    guard.save(path)
    again = GeometryGuardrail.load(path)
    probe = [_ellipsoid((1.3, 0.7, 0.5)), _ellipsoid((1.0, 0.6, 0.4))]
    assert [r["percentile"] for r in again.query(probe)] == pytest.approx([r["percentile"] for r in guard.query(probe)])
    d = tmp_path / "meshes"
    d.mkdir()
    for i, m in enumerate(probe):
        save_mesh_npz(m, d / f"m{i}.npz")
    named = again.query_from_dir(d)
    assert [r["name"] for r in named] == ["m0", "m1"] and {"percentile", "status"} <= set(named[0])
    with pytest.raises(ValueError):
        guard.query([])
    with pytest.raises(RuntimeError):
        GeometryGuardrail(method=method).save(tmp_path / "x.npz")
    with pytest.raises(ValueError):
        GeometryGuardrail(method="kde")


def test_field_variational_gp_head_learns_a_field_and_flags_far_inputs():
    """Two-channel field of a 1-D feature: the ELBO falls, the mean fits, and the epistemic variance grows away from data."""
    from physicsnemo_b200.experimental.uq import FieldVariationalGPHead, FieldVariationalGPPrediction

    torch.manual_seed(0)
    x = torch.rand(2, 150, 1) * 4 - 2
    y = torch.cat([torch.sin(2 * x), 0.5 * x ** 2], dim=-1) + 0.05 * torch.randn(2, 150, 2)
    head = FieldVariationalGPHead(1, n_train=300, num_tasks=2, n_inducing=20, lengthscale_range=(0.05, 5.0))
    head.set_inducing_points(x)
    opt = torch.optim.Adam(head.parameters(), lr=0.05)
    first = None
    for _ in range(150):
        opt.zero_grad()
        mean, nelbo = head.forward_and_loss(x, y)
        first = float(nelbo) if first is None else first
        nelbo.backward()
        opt.step()
    assert mean.shape == (2, 150, 2) and float(nelbo) < first - 0.5
    pred = head.predict(x)
    assert isinstance(pred, FieldVariationalGPPrediction) and pred.mean.shape == (2, 150, 2)
    assert float((pred.mean - y).abs().mean()) < 0.15
    assert bool((pred.upper > pred.lower).all()) and bool((pred.variance >= pred.epistemic_variance).all())
    far = head.predict(torch.full((1, 5, 1), 6.0))
    assert float(far.epistemic_variance.mean()) > 5 * float(pred.epistemic_variance.mean())
    # heteroscedastic noise MLP and radial feature normalisation: shapes and a finite objective
    het = FieldVariationalGPHead(3, n_train=100, num_tasks=2, n_inducing=8, mlp_hidden=[6], feature_norm="l2_radial",
                                 noise_mlp_hidden=[4], use_double=False)
    assert het.gp_input_dim == 7 and het.heteroscedastic
    m, l = het.forward_and_loss(torch.randn(4, 9, 3), torch.randn(4, 9, 2))
    assert m.shape == (4, 9, 2) and torch.isfinite(l)
    l.backward()
    assert het.noise_head[-1].weight.grad is not None


def test_geometry_features_from_a_directory_of_stl_files(tmp_path):
    from physicsnemo_b200.experimental.guardrails.geometry import FeatureSchema, extract_features
    from physicsnemo_b200.experimental.guardrails.geometry.mesh_io import load_features_from_dir
    from physicsnemo_b200.mesh import io, primitives

    shapes = {"a_sphere": primitives.icosphere(2), "b_torus": primitives.torus(24, 12), "c_cube": primitives.cube_surface(3)}
    for name, mesh in shapes.items():
        io.write_stl(mesh, tmp_path / f"{name}.stl")
    (tmp_path / "d_broken.stl").write_bytes(b"solid x\nfacet normal 0 0 0\nouter loop\nvertex 0 0\n")
    (tmp_path / "notes.txt").write_text("not a mesh")
    feats, names = load_features_from_dir(tmp_path, n_workers=1)
    assert names == ["a_sphere.stl", "b_torus.stl", "c_cube.stl"] and all(f.shape == (FeatureSchema.dim,) for f in feats)
    direct = extract_features(io.read_stl(tmp_path / "b_torus.stl"), return_tensor=False)
    assert np.allclose(feats[1], direct)
    pooled, names2 = load_features_from_dir(tmp_path, n_workers=2)
    assert names2 == names and all(np.allclose(a, b) for a, b in zip(feats, pooled))
    empty = tmp_path / "none"
    empty.mkdir()
    with pytest.raises(RuntimeError, match="No valid STL"):
        load_features_from_dir(empty)

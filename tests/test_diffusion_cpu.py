"""Diffusion tool-kit on CPU: scheduler identities, preconditioner algebra, a DSM training step of
a small SongUNet, and sampling with every solver."""
import pytest
import torch

from physicsnemo_b200.diffusion.metrics import EDMLoss, MSEDSMLoss, WeightedMSEDSMLoss
from physicsnemo_b200.diffusion.multi_diffusion import GridPatching2D, RandomPatching2D
from physicsnemo_b200.diffusion.noise_schedulers import (EDMNoiseScheduler, IDDPMNoiseScheduler, VENoiseScheduler,
                                                          VPNoiseScheduler)
from physicsnemo_b200.diffusion.preconditioners import EDMPrecond, EDMPreconditioner, VPPreconditioner
from physicsnemo_b200.diffusion.samplers import sample, stochastic_sampler
from physicsnemo_b200.diffusion.utils import ConcatConditionWrapper
from physicsnemo_b200.models.diffusion_unets import SongUNet


@pytest.mark.parametrize("sched", [EDMNoiseScheduler(), VPNoiseScheduler(), VENoiseScheduler(), IDDPMNoiseScheduler()])
def test_scheduler_identities(sched):
    t = sched.sample_time(6, dtype=torch.float64)
    assert torch.allclose(sched.sigma_inv(sched.sigma(t)), t, rtol=1e-4, atol=1e-6)
    x0 = torch.randn(6, 2, 4, 4, dtype=torch.float64)
    xt = sched.add_noise(x0, t)
    score = sched.x0_to_score(x0, xt, t)
    assert torch.allclose(sched.score_to_x0(score, xt, t), x0, atol=1e-8)
    eps = sched.x0_to_epsilon(x0, xt, t)
    assert torch.allclose(sched.epsilon_to_x0(eps, xt, t), x0, atol=1e-8)
    assert torch.allclose(sched.epsilon_to_score(eps, t), score, atol=1e-6)
    steps = sched.timesteps(8)
    assert steps.shape == (9,) and steps[-1] == 0 and bool((steps[:-1] > steps[1:]).all())


def test_edm_preconditioner_and_dsm_step():
    torch.manual_seed(0)
    net = SongUNet(img_resolution=16, in_channels=2 + 3, out_channels=2, model_channels=8, channel_mult=[1, 2],
                   num_blocks=1, attn_resolutions=[8], dropout=0.0)
    model = EDMPreconditioner(ConcatConditionWrapper(net), sigma_data=[0.5, 0.7])
    assert any(k.startswith("model.model.enc") for k in model.state_dict()) and "sigma_data" in model.state_dict()
    sched = EDMNoiseScheduler(sigma_data=torch.tensor([0.5, 0.7]))
    loss_fn = MSEDSMLoss(model, sched)
    x0, cond = torch.randn(3, 2, 16, 16), torch.randn(3, 3, 16, 16)
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    first = None
    for _ in range(5):
        loss = loss_fn(x0, t=torch.full((3,), 0.8), condition=cond)
        first = first or loss.item()
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert loss.item() < first
    w = WeightedMSEDSMLoss(model, sched, reduction="none")(x0, torch.ones_like(x0), condition=cond)
    assert w.shape == x0.shape
    # sigma -> 0: D(x) -> x ; large sigma: c_skip -> 0
    c_in, c_noise, c_out, c_skip = EDMPreconditioner(net, 0.5).compute_coefficients(torch.tensor([[[[1e-6]]]]))
    assert torch.allclose(c_skip, torch.ones_like(c_skip), atol=1e-6) and c_out.abs().max() < 1e-5


@pytest.mark.parametrize("solver", ["euler", "heun", "edm_stochastic_euler", "edm_stochastic_heun"])
def test_sampling_recovers_gaussian_mean(solver):
    torch.manual_seed(0)
    sched = EDMNoiseScheduler(sigma_max=10.0)
    mu, s0 = 2.0, 0.1
    # exact x0-predictor for data ~ N(mu, s0^2): posterior mean
    x0_pred = lambda x, t: (x * s0 ** 2 + mu * t.reshape(-1, 1) ** 2) / (s0 ** 2 + t.reshape(-1, 1) ** 2)  # noqa: E731
    den = sched.get_denoiser(x0_predictor=x0_pred)
    tN = torch.full((4096,), 10.0)
    xN = sched.init_latents((1,), tN)
    x = sample(den, xN, sched, num_steps=30, solver=solver,
               solver_options={"S_churn": 10, "num_steps": 30} if "stochastic" in solver else None)
    assert abs(x.mean().item() - mu) < 0.05 and abs(x.std().item() - s0) < 0.05


def test_legacy_precond_loss_and_patched_sampler():
    torch.manual_seed(0)
    net = EDMPrecond(img_resolution=16, img_channels=2, model_type="SongUNet", img_in_channels=2 + 3,
                     img_out_channels=2, model_channels=8, channel_mult=[1, 2], num_blocks=1, attn_resolutions=[])
    img, lr = torch.randn(2, 2, 16, 16), torch.randn(2, 3, 16, 16)
    loss = EDMLoss()(net, img, condition=lr)
    assert loss.shape == img.shape and torch.isfinite(loss).all()
    patching = GridPatching2D((16, 16), (16, 16))
    out = stochastic_sampler(net, torch.randn(2, 2, 16, 16), lr, patching=None, num_steps=4, sigma_max=10.0)
    assert out.shape == (2, 2, 16, 16) and torch.isfinite(out).all()
    rp = RandomPatching2D((16, 16), (8, 8), 3)
    assert rp.apply(img).shape == (6, 2, 8, 8) and rp.global_index().shape == (3, 2, 8, 8)
    assert patching.fuse(patching.apply(img), 2).allclose(img)


# ---- guidance, multi-diffusion, generate -----------------------------------------------------------------------------
def test_dps_guidance_matches_closed_form_gradient():
    from physicsnemo_b200.diffusion.guidance import DataConsistencyDPSGuidance, DPSGuidance, DPSScorePredictor, ModelConsistencyDPSGuidance

    torch.manual_seed(0)
    x, t = torch.randn(3, 2, 4, 4), torch.tensor([0.5, 1.0, 2.0])
    a = 0.7                                                       # x0 predictor: x0 = a x  ->  d/dx ||m (a x - y)||^2 = 2 a m (a x - y)
    predictor = lambda x, t: a * x  # noqa: E731
    mask = torch.rand(3, 2, 4, 4) > 0.5
    y = torch.randn(3, 2, 4, 4)
    g = DataConsistencyDPSGuidance(mask, y, std_y=0.3, gamma=0.5, sigma_fn=lambda t: t, alpha_fn=torch.ones_like,
                                   retain_graph=True)            # a second guidance walks the same graph afterwards
    assert isinstance(g, DPSGuidance)
    xr = x.clone().requires_grad_(True)
    got = g(xr, t, predictor(xr, t))
    rho = 1.0 / (2.0 * (0.3 ** 2 + 0.5 * t ** 2)).reshape(-1, 1, 1, 1)
    assert torch.allclose(got, -rho * 2 * a * mask * (a * x - y), atol=1e-6)
    op = lambda x0: x0.mean(dim=(2, 3))  # noqa: E731
    gm = ModelConsistencyDPSGuidance(op, torch.zeros(3, 2), std_y=1.0, norm=2)
    score = DPSScorePredictor(predictor, lambda x0, x, t: (x0 - x) / t.reshape(-1, 1, 1, 1) ** 2, [g, gm])
    out = score(x, t)
    xr = x.clone().requires_grad_(True)
    want = (a * x - x) / t.reshape(-1, 1, 1, 1) ** 2 + g(xr, t, predictor(xr, t))
    xr2 = x.clone().requires_grad_(True)
    want = want + gm(xr2, t, predictor(xr2, t))
    assert torch.allclose(out, want, atol=1e-6)
    with pytest.raises(ValueError):
        DataConsistencyDPSGuidance(mask, y, std_y=0.3, gamma=0.5)            # gamma > 0 needs sigma_fn
    with torch.inference_mode():
        with pytest.raises(RuntimeError):
            score(x, t)


class _PatchNet(torch.nn.Module):
    """Stand-in denoiser: scales x by a learnable gain and adds the mean of every spatial condition it is given."""

    def __init__(self):
        super().__init__()
        self.gain = torch.nn.Parameter(torch.tensor(0.5))
        self.seen = None

    def forward(self, x, t, condition=None):
        self.seen = condition
        out = self.gain * x
        if isinstance(condition, dict):
            for v in condition.values():
                if v.ndim == 4 and v.shape[-2:] == x.shape[-2:]:
                    out = out + 0 * v.mean(dim=1, keepdim=True)
        return out


def test_multi_diffusion_model_losses_and_predictor():
    from physicsnemo_b200.diffusion.multi_diffusion import (ConditionDict, MultiDiffusionModel2D, MultiDiffusionMSEDSMLoss,
                                                             MultiDiffusionPredictor, MultiDiffusionWeightedMSEDSMLoss)
    from physicsnemo_b200.diffusion.noise_schedulers import EDMNoiseScheduler

    torch.manual_seed(0)
    net = _PatchNet()
    md = MultiDiffusionModel2D(net, (16, 24), positional_embedding="sinusoidal", channels_positional_embedding=4,
                               condition_patch={"img": True}, condition_interp={"coarse": True})
    x = torch.randn(2, 3, 16, 24)
    t = torch.tensor([0.3, 0.9])
    cond = {"img": torch.randn(2, 1, 16, 24), "coarse": torch.randn(2, 2, 4, 6), "vec": torch.randn(2, 5)}
    with pytest.raises(RuntimeError):
        md.patch_x(x)
    md.set_random_patching((8, 8), patch_num=5)
    out = md(x, t, condition=cond)
    assert out.shape == (10, 3, 8, 8) and md.patch_shape == (8, 8)
    seen = net.seen
    assert isinstance(seen, ConditionDict) and seen.batch_size == [10]
    assert seen["img"].shape == (10, 1, 8, 8) and seen["coarse"].shape == (10, 2, 8, 8) and seen["vec"].shape == (10, 5)
    assert seen["positional_embedding"].shape == (10, 4, 8, 8)
    assert seen[2:6]["vec"].shape == (4, 5)
    sched = EDMNoiseScheduler()
    loss = MultiDiffusionMSEDSMLoss(md, sched)(x, condition=cond)
    loss.backward()
    assert loss.ndim == 0 and net.gain.grad is not None
    wl = MultiDiffusionWeightedMSEDSMLoss(md, sched, reduction="none")(x, torch.ones_like(x), condition=cond)
    assert wl.shape == (10, 3, 8, 8)
    # grid patching + fuse: a pointwise model commutes with patch / overlap-average
    md.set_grid_patching((8, 8), overlap_pix=2, boundary_pix=1)
    fused = md(x, t, condition=cond)
    assert fused.shape == x.shape and torch.allclose(fused, net.gain * x, atol=1e-5)
    pred = MultiDiffusionPredictor(md, condition=cond, chunk_size=4)
    with pytest.raises(RuntimeError):
        pred(x, t)
    pred.set_patching(overlap_pix=2, boundary_pix=1)
    with torch.no_grad():
        full = pred(x, t)
        assert torch.allclose(full, net.gain * x, atol=1e-5)
        pred.fuse = False
        patches = pred(x, t)
        assert patches.shape[1:] == (3, 8, 8) and torch.allclose(pred.fuse_fn(patches), full, atol=1e-6)
        starts = [s for s, *_ in pred.chunks(x, t)]
    assert starts == list(range(0, patches.shape[0], 4))


def test_multi_diffusion_patch_local_dps_guidance():
    """Chunked, patch-local DPS guidance: for a point-wise x0-predictor the streamed result equals the global formula."""
    from physicsnemo_b200.diffusion.multi_diffusion import (MultiDiffusionDataConsistencyDPSGuidance, MultiDiffusionDPSGuidance,
                                                             MultiDiffusionDPSScorePredictor, MultiDiffusionModel2D,
                                                             MultiDiffusionModelConsistencyDPSGuidance, MultiDiffusionPredictor)

    torch.manual_seed(0)
    net = _PatchNet()
    md = MultiDiffusionModel2D(net, (16, 24))
    pred = MultiDiffusionPredictor(md, chunk_size=4, fuse=False)
    pred.set_patching(overlap_pix=0, boundary_pix=0, patch_shape=(8, 8))
    x, t = torch.randn(2, 3, 16, 24), torch.tensor([0.5, 1.5])
    y = torch.randn(2, 3, 16, 24)
    mask = (torch.rand(2, 3, 16, 24) > 0.6).float()
    score_fn = lambda x0, xt, tt: (x0 - xt) / tt.reshape(-1, 1, 1, 1) ** 2                     # noqa: E731
    data = MultiDiffusionDataConsistencyDPSGuidance(pred, mask, y, std_y=0.3, gamma=0.5, sigma_fn=lambda s: s,
                                                    retain_graph=True)           # a second guidance differentiates the same chunk
    model = MultiDiffusionModelConsistencyDPSGuidance(pred, lambda z: 2.0 * z, y, std_y=0.5)
    assert isinstance(data, MultiDiffusionDPSGuidance) and isinstance(model, MultiDiffusionDPSGuidance)
    guided = MultiDiffusionDPSScorePredictor(pred, score_fn, [data, model])
    with torch.no_grad():
        got = guided(x, t)
    assert got.shape == x.shape and not got.requires_grad
    g = float(net.gain)                                              # the network is x0 = gain * x, pixel by pixel
    x0 = g * x
    tb = t.reshape(-1, 1, 1, 1)
    rho_d = 1.0 / (2.0 * (0.3 ** 2 + 0.5 * tb ** 2))
    want = (x0 - x) / tb ** 2 - rho_d * mask * 2 * (x0 - y) * g - (1.0 / (2 * 0.25)) * 2 * (2 * x0 - y) * 2 * g
    assert torch.allclose(got, want, atol=1e-4)
    with pytest.raises(ValueError):
        MultiDiffusionDPSScorePredictor(MultiDiffusionPredictor(md), score_fn, data)
    with pytest.raises(ValueError):
        MultiDiffusionDataConsistencyDPSGuidance(pred, mask, y, std_y=0.3, gamma=0.5)


def test_generate_steps_are_seeded():
    from physicsnemo_b200.diffusion.generate import diffusion_step, regression_step

    class Reg(torch.nn.Module):
        device = torch.device("cpu")

        def forward(self, x, img_lr, lead_time_label=None):
            return x + img_lr.mean(dim=1, keepdim=True).to(x.dtype)

    img_lr = torch.randn(1, 3, 8, 8)
    out = regression_step(Reg(), img_lr, (4, 1, 8, 8))
    assert out.shape == (4, 1, 8, 8) and torch.allclose(out[0], out[3])
    sampler = lambda net, latents, img_lr, randn_like=None, **kw: latents + 0 * randn_like(latents)  # noqa: E731
    lr2 = img_lr.expand(2, -1, -1, -1).contiguous()                # one conditioning image per seed of a batch
    a = diffusion_step(None, sampler, (8, 8), 2, [[1, 2], [3, 4]], lr2, rank=0, device="cpu")
    b = diffusion_step(None, sampler, (8, 8), 2, [[3, 4]], lr2, rank=0, device="cpu")
    assert a.shape == (4, 2, 8, 8) and torch.equal(a[2:], b) and not torch.equal(a[:2], b)
    with pytest.raises(ValueError):
        diffusion_step(None, sampler, (8, 8), 2, [[1]], img_lr, 0, "cpu", distribution="student_t")

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

"""Conditional diffusion with an EDM-preconditioned SongUNet: training and sampling.

The data are synthetic "downscaling" pairs: a smooth random field (sum of a few random plane waves)
is the target, its 8× block average is the condition, so the model learns to add the small scales
back.  Training minimises the denoising-score-matching loss of the EDM noise schedule; an
exponential moving average of the weights is kept for sampling, which integrates the probability-flow
ODE with the Heun solver.

    python train.py --steps 2000 --resolution 128
    python -m torch.distributed.run --nproc-per-node 4 train.py
    python train.py --smoke
"""
from __future__ import annotations

import argparse
import copy

import torch

from physicsnemo_b200.diffusion.metrics.losses import MSEDSMLoss
from physicsnemo_b200.diffusion.noise_schedulers import EDMNoiseScheduler
from physicsnemo_b200.diffusion.preconditioners import EDMPreconditioner
from physicsnemo_b200.diffusion.samplers import sample
from physicsnemo_b200.diffusion.utils.model_wrappers import ConcatConditionWrapper
from physicsnemo_b200.distributed import DistributedManager
from physicsnemo_b200.models.diffusion_unets import SongUNet
from physicsnemo_b200.utils.checkpoint import save_checkpoint
from physicsnemo_b200.utils.logging import PythonLogger


def make_pairs(batch: int, res: int, channels: int, generator: torch.Generator, device):
    """``(condition, target)``: random plane-wave fields and their 8× block averages, both ``[B, C, res, res]``."""
    y, x = torch.meshgrid(torch.linspace(0, 1, res), torch.linspace(0, 1, res), indexing="ij")
    k = torch.randint(1, 12, (batch, channels, 6, 2), generator=generator).float()
    phase = torch.rand(batch, channels, 6, generator=generator) * 6.2832
    amp = torch.randn(batch, channels, 6, generator=generator) / k.norm(dim=-1)
    arg = 6.2832 * (k[..., 0, None, None] * x + k[..., 1, None, None] * y) + phase[..., None, None]
    target = (amp[..., None, None] * torch.sin(arg)).sum(2)
    coarse = torch.nn.functional.avg_pool2d(target, 8)
    condition = torch.nn.functional.interpolate(coarse, size=res, mode="nearest")
    return condition.to(device), target.to(device)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--resolution", type=int, default=128)
    ap.add_argument("--channels", type=int, default=2)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--lr", type=float, default=2e-4)
    ap.add_argument("--ema", type=float, default=0.999)
    ap.add_argument("--sample-steps", type=int, default=18)
    ap.add_argument("--out", default="./outputs/edm_songunet")
    ap.add_argument("--smoke", action="store_true")
    a = ap.parse_args()
    if a.smoke:
        a.resolution, a.batch, a.steps, a.sample_steps = 16, 2, 3, 4

    DistributedManager.initialize()
    dist = DistributedManager()
    log = PythonLogger("edm_songunet")
    on_gpu = dist.device.type == "cuda"
    torch.manual_seed(0)
    unet = SongUNet(img_resolution=a.resolution, in_channels=2 * a.channels, out_channels=a.channels,
                    model_channels=32 if a.smoke else 128, channel_mult=[1, 2] if a.smoke else [1, 2, 2, 2],
                    num_blocks=1 if a.smoke else 2, attn_resolutions=[a.resolution // 2] if a.smoke else [16])
    model = EDMPreconditioner(ConcatConditionWrapper(unet), sigma_data=0.5).to(dist.device)
    ema = copy.deepcopy(model).requires_grad_(False)
    train_model = model
    if dist.world_size > 1:
        train_model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[dist.local_rank] if on_gpu else None)
    scheduler = EDMNoiseScheduler()
    loss_fn = MSEDSMLoss(train_model, scheduler)
    optimizer = torch.optim.Adam(model.parameters(), lr=a.lr)
    gen = torch.Generator().manual_seed(100 + dist.rank)

    for step in range(1, a.steps + 1):
        cond, target = make_pairs(a.batch, a.resolution, a.channels, gen, dist.device)
        optimizer.zero_grad(set_to_none=True)
        with torch.autocast(dist.device.type, dtype=torch.bfloat16, enabled=on_gpu):
            loss = loss_fn(target, condition=cond)
        loss.backward()
        optimizer.step()
        with torch.no_grad():
            for p_ema, p in zip(ema.parameters(), model.parameters()):
                p_ema.lerp_(p, 1.0 - a.ema)
        if dist.rank == 0 and (step % max(1, a.steps // 10) == 0 or step == a.steps):
            log.info(f"step {step}: loss {float(loss.detach()):.4f}")

    if dist.rank == 0:
        # sample: start from noise at the largest sigma and integrate down with the EMA weights
        cond, target = make_pairs(2, a.resolution, a.channels, torch.Generator().manual_seed(7), dist.device)
        with torch.no_grad():
            denoiser = scheduler.get_denoiser(x0_predictor=lambda x, t: ema(x, t, condition=cond).float())
            t_max = scheduler.timesteps(a.sample_steps, device=dist.device)[:1].expand(2)
            latents = scheduler.init_latents(tuple(target.shape[1:]), t_max, device=dist.device, dtype=torch.float32)
            generated = sample(denoiser, latents, scheduler, num_steps=a.sample_steps, solver="heun")
        coarse_err = (torch.nn.functional.avg_pool2d(generated, 8) - torch.nn.functional.avg_pool2d(target, 8)).abs().mean()
        log.info(f"sampled {tuple(generated.shape)}; mean error of the 8x block averages vs the condition: {float(coarse_err):.4f}")
        save_checkpoint(a.out, models=[model, ema], optimizer=optimizer, epoch=a.steps)
        log.success(f"saved to {a.out}")


if __name__ == "__main__":
    main()

"""FNO-2D on the CPU, fp32, single process (headline configuration 1: the plumbing check without a GPU).

Architecture: 1 input / 1 output channel, lift width 32, 4 Fourier layers with 12 × 12 retained modes, GELU, decoder MLP
32 → 128 → 1 (2,368,481 parameters).  Data: grid 64 × 64, batch 8, 100 steps of Adam (lr 1e-3) on the MSE loss.  Inputs
are piecewise-constant fields (12 where a Gaussian random field with covariance (−Δ + 9 I)⁻² is ≥ 0, else 3), targets a
smooth Gaussian random field.
"""
from __future__ import annotations

import os
import time

import torch


def make_data(batch: int = 8, n: int = 64, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    k = torch.fft.fftfreq(n, d=1.0 / n)
    k2 = (2 * torch.pi) ** 2 * (k[:, None] ** 2 + k[None, :] ** 2)
    amp = 1.0 / (k2 + 9.0)

    def grf():
        w = torch.randn(batch, n, n, generator=g)
        return torch.fft.ifft2(torch.fft.fft2(w) * amp).real

    a = grf()
    x = torch.where(a >= 0, torch.full_like(a, 12.0), torch.full_like(a, 3.0)).unsqueeze(1)
    y = grf()
    y = (y / y.std()).unsqueeze(1)
    return x.float(), y.float()


def run(args, rank: int, world: int, dev) -> dict:
    from ..models.fno import FNO

    torch.manual_seed(1234)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    model = FNO(in_channels=1, out_channels=1, decoder_layers=1, decoder_layer_size=128, dimension=2, latent_channels=32,
                num_fno_layers=4, num_fno_modes=12, padding=8, activation_fn="gelu")
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    x, y = make_data(8, 64, seed=0)
    steps = max(int(args.steps), 100)

    def step():
        opt.zero_grad(set_to_none=True)
        loss = torch.nn.functional.mse_loss(model(x), y)
        loss.backward()
        opt.step()
        return loss.item()

    for _ in range(3):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        loss = step()
    ms = (time.perf_counter() - t0) / steps * 1000.0
    return {"metric": "train samples/sec (CPU wall clock)", "value": 8 * 1000.0 / ms, "unit": "samples/s", "n_gpus": 0,
            "steps": steps, "warmup": 3, "ms_per_step": ms, "higher_is_better": True, "scaling": "none", "vs_baseline": None,
            "dtype": "fp32", "data": "synthetic (seeded Gaussian-random-field permeability / smooth target fields)",
            "config": {"model": "FNO-2D width 32, 4 layers, 12x12 modes, GELU, decoder 32-128-1", "global_batch": 8,
                       "seq_len": 64 * 64, "parallelism": "single CPU process", "threads": torch.get_num_threads(),
                       "parameters": sum(p.numel() for p in model.parameters())},
            "impl": "physicsnemo_b200", "loss": float(loss), "gpu_launches": 0}

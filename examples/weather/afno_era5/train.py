"""AFNO next-step forecaster on ERA5-style yearly arrays (the FourCastNet recipe in small).

Data: yearly ``.npy`` files ``[time, channel, lat, lon]`` plus ``stats/global_{means,stds}.npy``, the layout the
``ERA5Datapipe`` of the package reads (memory-mapped, batches staged in pinned buffers and copied on a side stream).
Without ``--data`` a small synthetic archive is generated first: travelling planetary waves with channel-dependent
phase speed, so that the 6-hour-ahead state is a learnable function of the current one.  Training is the usual
one-step latitude-weighted MSE; validation reports the latitude-weighted RMSE and anomaly correlation per channel.

    python train.py --epochs 5
    python -m torch.distributed.run --nproc-per-node 8 train.py --data /path/to/era5
    python train.py --smoke
"""
from __future__ import annotations

import argparse
import math
from pathlib import Path

import numpy as np
import torch

from physicsnemo_b200.datapipes.climate.era5 import ERA5Datapipe
from physicsnemo_b200.distributed import DistributedManager
from physicsnemo_b200.models.afno import AFNO
from physicsnemo_b200.utils.checkpoint import load_checkpoint, save_checkpoint
from physicsnemo_b200.utils.logging import PythonLogger


def write_synthetic_archive(root: Path, years: int, steps: int, channels: int, lat: int, lon: int, seed: int = 0) -> None:
    rng = np.random.default_rng(seed)
    y = np.linspace(-math.pi / 2, math.pi / 2, lat)[:, None]
    x = np.linspace(0, 2 * math.pi, lon, endpoint=False)[None, :]
    waves = [(int(rng.integers(1, 6)), rng.uniform(0.05, 0.3) * (1 + c), rng.uniform(0, 6.28)) for c in range(channels) for _ in range(3)]
    for split, n_years in (("train", years), ("test", 1)):
        (root / split).mkdir(parents=True, exist_ok=True)
        for year in range(n_years):
            t = (np.arange(steps) + year * steps)[:, None, None, None]
            field = np.zeros((steps, channels, lat, lon), np.float32)
            for i, (k, speed, phase) in enumerate(waves):
                c = i // 3
                field[:, c] += (np.cos(y) ** 2 * np.sin(k * x - speed * t[:, 0] + phase)).astype(np.float32)
            field += 0.02 * rng.standard_normal(field.shape).astype(np.float32)
            np.save(root / split / f"{2000 + year}.npy", field)
    (root / "stats").mkdir(exist_ok=True)
    sample = np.load(root / "train" / "2000.npy")
    np.save(root / "stats" / "global_means.npy", sample.mean((0, 2, 3), keepdims=True)[0:1].reshape(1, channels, 1, 1))
    np.save(root / "stats" / "global_stds.npy", sample.std((0, 2, 3), keepdims=True)[0:1].reshape(1, channels, 1, 1))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--data", default=None, help="archive with train/, test/ and stats/ (generated when omitted)")
    ap.add_argument("--grid", type=int, nargs=2, default=[64, 128])
    ap.add_argument("--channels", type=int, default=4)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--epochs", type=int, default=5)
    ap.add_argument("--embed", type=int, default=256)
    ap.add_argument("--depth", type=int, default=6)
    ap.add_argument("--lr", type=float, default=5e-4)
    ap.add_argument("--out", default="./outputs/afno_era5")
    ap.add_argument("--smoke", action="store_true")
    a = ap.parse_args()
    if a.smoke:
        a.grid, a.channels, a.batch, a.epochs, a.embed, a.depth = [16, 32], 2, 2, 2, 32, 2

    DistributedManager.initialize()
    dist = DistributedManager()
    log = PythonLogger("afno_era5")
    root = Path(a.data) if a.data else Path(a.out) / "synthetic_era5"
    if not a.data and dist.rank == 0 and not (root / "stats").exists():
        write_synthetic_archive(root, years=2, steps=24 if a.smoke else 120, channels=a.channels, lat=a.grid[0], lon=a.grid[1])
    if dist.world_size > 1:
        torch.distributed.barrier()
    pipe = dict(stats_dir=str(root / "stats"), batch_size=a.batch, num_steps=1, stride=1, device=dist.device)
    train = ERA5Datapipe(str(root / "train"), shuffle=True, process_rank=dist.rank, world_size=dist.world_size, **pipe)
    test = ERA5Datapipe(str(root / "test"), shuffle=False, **pipe)

    torch.manual_seed(0)
    model = AFNO(inp_shape=list(a.grid), in_channels=a.channels, out_channels=a.channels, patch_size=[4, 4] if a.smoke else [8, 8],
                 embed_dim=a.embed, depth=a.depth, num_blocks=4 if a.smoke else 8).to(dist.device)
    net = model
    on_gpu = dist.device.type == "cuda"
    if dist.world_size > 1:
        net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[dist.local_rank] if on_gpu else None)
    optimizer = torch.optim.AdamW(model.parameters(), lr=a.lr, weight_decay=1e-4)
    scheduler = torch.optim.lr_scheduler.CosineAnnealingLR(optimizer, T_max=a.epochs)
    first_epoch = load_checkpoint(a.out, models=model, optimizer=optimizer, scheduler=scheduler, device=dist.device) + 1
    lat = torch.linspace(-math.pi / 2, math.pi / 2, a.grid[0], device=dist.device)
    weight = (torch.cos(lat) / torch.cos(lat).mean()).reshape(1, 1, -1, 1)

    for epoch in range(first_epoch, a.epochs + 1):
        net.train()
        running, count = 0.0, 0
        for (batch,) in train:
            x, y = batch["invar"], batch["outvar"][:, 0]
            with torch.autocast(dist.device.type, dtype=torch.bfloat16, enabled=on_gpu):
                pred = net(x)
            loss = (weight * (pred.float() - y) ** 2).mean()
            optimizer.zero_grad(set_to_none=True)
            loss.backward()
            optimizer.step()
            running, count = running + float(loss.detach()), count + 1
        scheduler.step()
        net.eval()
        se = torch.zeros(a.channels, device=dist.device)
        cov = torch.zeros_like(se); var_p = torch.zeros_like(se); var_t = torch.zeros_like(se); n = 0
        with torch.no_grad():
            for (batch,) in test:
                x, y = batch["invar"], batch["outvar"][:, 0]
                with torch.autocast(dist.device.type, dtype=torch.bfloat16, enabled=on_gpu):
                    pred = model(x).float()
                se += (weight * (pred - y) ** 2).mean((0, 2, 3))
                cov += (weight * pred * y).mean((0, 2, 3)); var_p += (weight * pred ** 2).mean((0, 2, 3)); var_t += (weight * y ** 2).mean((0, 2, 3))
                n += 1
        if dist.rank == 0:
            rmse = (se / max(n, 1)).sqrt().tolist()
            acc = (cov / (var_p * var_t).sqrt().clamp_min(1e-12)).tolist()
            log.info(f"epoch {epoch}: train loss {running / max(count, 1):.4f}; test RMSE {[round(v, 3) for v in rmse]}, "
                     f"ACC {[round(v, 3) for v in acc]} (normalised units)")
            save_checkpoint(a.out, models=model, optimizer=optimizer, scheduler=scheduler, epoch=epoch)
    log.success("done")


if __name__ == "__main__":
    main()

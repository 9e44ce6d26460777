"""Transolver on an irregular point cloud, optionally sharded over points across GPUs.

The task is synthetic but shaped like external aerodynamics: points on a randomly stretched and
rotated ellipsoid, inputs = coordinates and normals, target = the surface pressure of potential
flow around the equivalent sphere mapped onto the body (a smooth function of the geometry and the
inflow direction).  With ``--domain-parallel`` every rank of the job holds ``N / world`` points of
each sample: slice tokens and gradients are reduced by the package's peer-memory kernels, the
parameters stay replicated.  Without it, ranks train data-parallel on different samples.

    python train.py --points 200000 --steps 200
    python -m torch.distributed.run --nproc-per-node 8 train.py --points 1000000 --domain-parallel
    python train.py --smoke
"""
from __future__ import annotations

import argparse
import math

import torch

from physicsnemo_b200.distributed import DistributedManager
from physicsnemo_b200.models.transolver import Transolver
from physicsnemo_b200.parallel.point_parallel import PointParallel
from physicsnemo_b200.utils.checkpoint import save_checkpoint
from physicsnemo_b200.utils.logging import PythonLogger


def make_case(n_points: int, generator: torch.Generator, device) -> tuple[torch.Tensor, torch.Tensor]:
    """One body: ``(features [N, 6], pressure coefficient [N, 1])``."""
    u = torch.randn(n_points, 3, generator=generator)
    sphere = u / u.norm(dim=1, keepdim=True)
    axes = 0.5 + torch.rand(3, generator=generator)
    q, _ = torch.linalg.qr(torch.randn(3, 3, generator=generator))
    points = (sphere * axes) @ q.T
    normals = torch.nn.functional.normalize((sphere / axes) @ q.T, dim=1)
    inflow = torch.tensor([1.0, 0.0, 0.0])
    cos = normals @ inflow
    cp = 1.0 - 2.25 * (1.0 - cos ** 2)                       # sphere potential flow, evaluated with the body's normals
    return torch.cat([points, normals], dim=1).to(device), cp[:, None].to(device)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--points", type=int, default=200_000)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=256)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--domain-parallel", action="store_true")
    ap.add_argument("--out", default="./outputs/transolver_point_cloud")
    ap.add_argument("--smoke", action="store_true")
    a = ap.parse_args()
    if a.smoke:
        a.points, a.steps, a.layers, a.hidden = 2048, 4, 2, 64

    DistributedManager.initialize()
    dist = DistributedManager()
    log = PythonLogger("transolver")
    on_gpu = dist.device.type == "cuda"
    torch.manual_seed(0)                                     # identical initial weights on every rank
    model = Transolver(functional_dim=3, out_dim=1, embedding_dim=3, n_layers=a.layers, n_hidden=a.hidden, n_head=8,
                       slice_num=32 if a.smoke else 64, mlp_ratio=4, use_te=False).to(dist.device)
    sharded = a.domain_parallel and dist.world_size > 1
    pp = PointParallel(model) if sharded else None
    if dist.world_size > 1 and not sharded:
        model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[dist.local_rank] if on_gpu else None)
    optimizer = torch.optim.Adam(model.parameters(), lr=a.lr)
    scheduler = torch.optim.lr_scheduler.OneCycleLR(optimizer, max_lr=a.lr, total_steps=a.steps)

    for step in range(1, a.steps + 1):
        # sharded: all ranks draw the same body and keep their slice of its points; otherwise one body per rank
        seed = step if sharded else step * dist.world_size + dist.rank
        x, y = make_case(a.points, torch.Generator().manual_seed(seed), dist.device)
        if sharded:
            share = a.points // dist.world_size
            x, y = x[dist.rank * share:(dist.rank + 1) * share], y[dist.rank * share:(dist.rank + 1) * share]
        pp.zero_grad() if pp else optimizer.zero_grad(set_to_none=True)
        with torch.autocast(dist.device.type, dtype=torch.bfloat16, enabled=on_gpu):
            pred = model(x[None, :, 3:], embedding=x[None, :, :3])       # features: normals; embedding: coordinates
        # the mean over all points of the body: a sharded rank contributes its share of the sum
        loss = (pred.float() - y[None]).square().sum() / a.points if sharded else (pred.float() - y[None]).square().mean()
        loss.backward()
        if pp:
            pp.reduce_gradients()
        optimizer.step()
        scheduler.step()
        if step % max(1, a.steps // 10) == 0 or step == a.steps:
            total = loss.detach().clone()
            if sharded:
                torch.distributed.all_reduce(total)
            if dist.rank == 0:
                log.info(f"step {step}: mse {float(total):.5f}  lr {scheduler.get_last_lr()[0]:.2e}")
    if dist.rank == 0:
        save_checkpoint(a.out, models=model, optimizer=optimizer, epoch=a.steps)
        log.success(f"saved to {a.out}")


if __name__ == "__main__":
    main()

"""Fourier neural operator on Darcy flow: permeability field → pressure field.

Data come from the Darcy generator of the package (random piecewise-constant permeability, multigrid
Jacobi solve, on the device when there is one).  The step is wrapped in ``StaticCaptureTraining``
(CUDA graph + AMP on a GPU), every epoch ends with a relative-L2 validation error and a checkpoint,
and a rerun with the same ``--out`` resumes from the last one.

    python train.py --epochs 20                      # one GPU
    python -m torch.distributed.run --nproc-per-node 4 train.py
    python train.py --smoke                          # a few CPU steps
"""
from __future__ import annotations

import argparse

import torch

from physicsnemo_b200.datapipes.benchmarks.darcy import Darcy2D
from physicsnemo_b200.distributed import DistributedManager
from physicsnemo_b200.models.fno import FNO
from physicsnemo_b200.utils.capture import StaticCaptureEvaluateNoGrad, StaticCaptureTraining
from physicsnemo_b200.utils.checkpoint import load_checkpoint, save_checkpoint
from physicsnemo_b200.utils.logging import LaunchLogger, PythonLogger


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--resolution", type=int, default=256)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--epochs", type=int, default=10)
    ap.add_argument("--steps-per-epoch", type=int, default=32)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--out", default="./outputs/darcy_fno")
    ap.add_argument("--smoke", action="store_true")
    a = ap.parse_args()
    if a.smoke:
        a.resolution, a.batch, a.epochs, a.steps_per_epoch = 16, 2, 2, 2

    DistributedManager.initialize()
    dist = DistributedManager()
    log = PythonLogger("darcy_fno")
    LaunchLogger.initialize()
    torch.manual_seed(1234 + dist.rank)

    model = FNO(in_channels=1, out_channels=1, decoder_layers=1, decoder_layer_size=32, dimension=2, latent_channels=32,
                num_fno_layers=4, num_fno_modes=4 if a.smoke else 12, padding=9).to(dist.device)
    if dist.world_size > 1:
        model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[dist.local_rank] if dist.cuda else None)
    optimizer = torch.optim.Adam(model.parameters(), lr=a.lr)
    scheduler = torch.optim.lr_scheduler.ExponentialLR(optimizer, gamma=0.95)
    solver = dict(max_iterations=100, iterations_per_convergence_check=50, nr_multigrids=2) if a.smoke else {}
    data = Darcy2D(resolution=a.resolution, batch_size=a.batch, device=dist.device, **solver)
    first_epoch = load_checkpoint(a.out, models=model, optimizer=optimizer, scheduler=scheduler, device=dist.device) + 1

    on_gpu = dist.device.type == "cuda"

    @StaticCaptureTraining(model=model, optim=optimizer, use_graphs=on_gpu, use_amp=on_gpu, amp_type=torch.bfloat16)
    def train_step(k, p):
        return torch.nn.functional.mse_loss(model(k), p)

    @StaticCaptureEvaluateNoGrad(model=model, use_graphs=False, use_amp=on_gpu, amp_type=torch.bfloat16)
    def predict(k):
        return model(k)

    batches = iter(data)
    for epoch in range(first_epoch, a.epochs + 1):
        with LaunchLogger("train", epoch=epoch, num_mini_batch=a.steps_per_epoch, epoch_alert_freq=1) as launch:
            for _ in range(a.steps_per_epoch):
                batch = next(batches)
                loss = train_step(batch["permeability"], batch["darcy"])
                launch.log_minibatch({"loss": float(loss.detach())})
        scheduler.step()
        batch = next(batches)
        pred = predict(batch["permeability"]).float()
        err = (pred - batch["darcy"]).norm() / batch["darcy"].norm()
        if dist.rank == 0:
            log.info(f"epoch {epoch}: validation relative L2 error {float(err):.4f}")
            save_checkpoint(a.out, models=model, optimizer=optimizer, scheduler=scheduler, epoch=epoch)
    log.success("done")


if __name__ == "__main__":
    main()

"""MeshGraphNet on unstructured 2-D meshes: flow past a circular obstacle in a channel.

Every sample is a Delaunay mesh of a channel with one obstacle of random size and position; node inputs are the
position and a one-hot boundary marker (interior / inlet / outlet / wall / obstacle), targets are the velocity and
pressure of the analytic potential-flow solution around the obstacle (standing in for a solver's output; the real
recipe reads ``.vtp`` files of Stokes solutions with the same dataset class).  Shows ``StokesDataset`` (statistics
fitted on the training split and reused for validation), per-graph batching of size one, activation checkpointing
of the processor and a denormalised validation error.

    python train.py --epochs 20 --samples 64
    python train.py --smoke
"""
from __future__ import annotations

import argparse
import math

import numpy as np
import torch

from physicsnemo_b200.datapipes.gnn import StokesDataset
from physicsnemo_b200.distributed import DistributedManager
from physicsnemo_b200.mesh.tessellation import delaunay_mesh_2d
from physicsnemo_b200.models.meshgraphnet import MeshGraphNet
from physicsnemo_b200.utils.checkpoint import save_checkpoint
from physicsnemo_b200.utils.logging import PythonLogger


def make_sample(rng: np.random.Generator, n_points: int) -> dict:
    """Channel ``[0, 3] × [0, 1]`` with a disc obstacle; fields of a uniform stream past the disc."""
    radius, cx, cy = rng.uniform(0.08, 0.2), rng.uniform(0.8, 1.6), rng.uniform(0.35, 0.65)
    ring = np.linspace(0, 2 * math.pi, 24, endpoint=False)
    obstacle = np.stack([cx + radius * np.cos(ring), cy + radius * np.sin(ring)], 1)
    edge = np.linspace(0, 1, 12)
    walls = np.concatenate([np.stack([3 * edge, 0 * edge], 1), np.stack([3 * edge, 0 * edge + 1], 1)])
    inlet, outlet = np.stack([0 * edge[1:-1], edge[1:-1]], 1), np.stack([0 * edge[1:-1] + 3, edge[1:-1]], 1)
    inner = rng.uniform([0, 0], [3, 1], (n_points, 2))
    inner = inner[np.hypot(inner[:, 0] - cx, inner[:, 1] - cy) > 1.15 * radius]
    pos = np.concatenate([inner, inlet, outlet, walls, obstacle]).astype(np.float32)
    marker = np.concatenate([np.zeros(len(inner)), np.ones(len(inlet)), 2 * np.ones(len(outlet)), 3 * np.ones(len(walls)),
                             4 * np.ones(len(obstacle))]).astype(np.int64)
    cells = delaunay_mesh_2d(torch.from_numpy(pos)).cells.numpy()
    centroid = pos[cells].mean(1)
    cells = cells[np.hypot(centroid[:, 0] - cx, centroid[:, 1] - cy) > radius]           # drop triangles inside the disc
    dx, dy = pos[:, 0] - cx, pos[:, 1] - cy
    r2 = np.maximum(dx ** 2 + dy ** 2, radius ** 2)
    u = 1 - radius ** 2 * (dx ** 2 - dy ** 2) / r2 ** 2
    v = -2 * radius ** 2 * dx * dy / r2 ** 2
    return dict(pos=pos, cells=cells, marker=marker, u=u, v=v, p=0.5 * (1 - u ** 2 - v ** 2))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--samples", type=int, default=32)
    ap.add_argument("--points", type=int, default=1500)
    ap.add_argument("--epochs", type=int, default=10)
    ap.add_argument("--layers", type=int, default=10)
    ap.add_argument("--hidden", type=int, default=128)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--out", default="./outputs/stokes_mgn")
    ap.add_argument("--smoke", action="store_true")
    a = ap.parse_args()
    if a.smoke:
        a.samples, a.points, a.epochs, a.layers, a.hidden = 4, 120, 2, 2, 32

    DistributedManager.initialize()
    dist = DistributedManager()
    log = PythonLogger("stokes_mgn")
    rng = np.random.default_rng(0)
    n_val = max(1, a.samples // 8)
    train = StokesDataset(samples=[make_sample(rng, a.points) for _ in range(a.samples)], num_samples=a.samples, stats_dir=a.out)
    valid = StokesDataset(samples=[make_sample(rng, a.points) for _ in range(n_val)], num_samples=n_val, split="validation",
                          stats_dir=a.out)
    torch.manual_seed(0)
    g0 = train[0]
    model = MeshGraphNet(input_dim_nodes=g0.x.shape[1], input_dim_edges=g0.edge_attr.shape[1], output_dim=g0.y.shape[1],
                         processor_size=a.layers, hidden_dim_processor=a.hidden, hidden_dim_node_encoder=a.hidden,
                         hidden_dim_edge_encoder=a.hidden, hidden_dim_node_decoder=a.hidden,
                         num_processor_checkpoint_segments=2 if a.layers % 2 == 0 and not a.smoke else 0).to(dist.device)
    optimizer = torch.optim.Adam(model.parameters(), lr=a.lr)
    scheduler = torch.optim.lr_scheduler.CosineAnnealingLR(optimizer, T_max=a.epochs)
    on_gpu = dist.device.type == "cuda"

    def run(graph, training: bool):
        graph = graph.to(dist.device)
        with torch.autocast(dist.device.type, dtype=torch.bfloat16, enabled=on_gpu), torch.set_grad_enabled(training):
            pred = model(graph.x, graph.edge_attr, graph)
        return pred.float(), graph.y

    for epoch in range(1, a.epochs + 1):
        model.train()
        order = torch.randperm(len(train), generator=torch.Generator().manual_seed(epoch)).tolist()
        total = 0.0
        for i in order[dist.rank::dist.world_size]:
            pred, target = run(train[i], True)
            loss = torch.nn.functional.mse_loss(pred, target)
            optimizer.zero_grad(set_to_none=True)
            loss.backward()
            if dist.world_size > 1:                       # graphs differ in size per rank: average the gradients by hand
                for p in model.parameters():
                    torch.distributed.all_reduce(p.grad)
                    p.grad /= dist.world_size
            optimizer.step()
            total += float(loss.detach())
        scheduler.step()
        model.eval()
        errs = []
        for i in range(len(valid)):
            pred, target = run(valid[i], False)
            p_phys, t_phys = valid.denormalize(pred.cpu(), target.cpu())
            errs.append(float((p_phys - t_phys).norm() / t_phys.norm()))
        if dist.rank == 0:
            log.info(f"epoch {epoch}: train mse {total / max(1, len(order) // dist.world_size):.4f}, "
                     f"validation relative L2 (physical units) {sum(errs) / len(errs):.4f}")
    if dist.rank == 0:
        save_checkpoint(a.out, models=model, optimizer=optimizer, scheduler=scheduler, epoch=a.epochs)
        log.success(f"saved to {a.out}")


if __name__ == "__main__":
    main()

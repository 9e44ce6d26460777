"""GLOBE on boundary meshes: potential flow past a cylinder, learned from the boundary alone.

Every sample is a circle of random radius and position inside a far-field ring, with a uniform inflow
of random direction.  The model sees the two boundary meshes (the wall carries no data, the far
field carries the inflow direction as a per-face vector) and predicts, at arbitrary query points,
the perturbation potential and the velocity of the exact solution
``phi = U·x (1 + R² / |x|²)``.  Because GLOBE is equivariant and works with nondimensional lengths, a
model trained on a handful of sizes transfers to other sizes, positions and directions; the script
reports the error on a rotated, shifted, rescaled case at the end.

    python train.py --steps 300
    python train.py --smoke
"""
from __future__ import annotations

import argparse
import math

import torch

from physicsnemo_b200.experimental.models.globe import GLOBE
from physicsnemo_b200.mesh.mesh import Mesh
from physicsnemo_b200.utils.checkpoint import save_checkpoint
from physicsnemo_b200.utils.logging import PythonLogger


def ring(n: int, radius: float, centre: torch.Tensor, outward: bool) -> tuple[torch.Tensor, torch.Tensor]:
    angle = torch.linspace(0, 2 * math.pi, n + 1)[:-1]
    pts = centre + radius * torch.stack([angle.cos(), angle.sin()], 1)
    nxt = (torch.arange(n) + 1) % n
    cells = torch.stack([torch.arange(n), nxt], 1)
    return pts, (cells if outward else cells.flip(1))


def make_case(generator: torch.Generator, n_wall: int, n_far: int, n_query: int, device, radius=None, centre=None, angle=None):
    radius = float(0.5 + torch.rand(1, generator=generator)) if radius is None else radius
    centre = (torch.rand(2, generator=generator) - 0.5) if centre is None else centre
    angle = float(torch.rand(1, generator=generator)) * 2 * math.pi if angle is None else angle
    inflow = torch.tensor([math.cos(angle), math.sin(angle)])
    wall_pts, wall_cells = ring(n_wall, radius, centre, outward=False)          # normals point into the fluid
    far_pts, far_cells = ring(n_far, 8.0 * radius, centre, outward=True)
    wall = Mesh(wall_pts.to(device), wall_cells.to(device))
    far = Mesh(far_pts.to(device), far_cells.to(device), cell_data={"inflow": inflow.expand(n_far, 2).clone().to(device)})
    r = radius * (1.05 + 4.0 * torch.rand(n_query, generator=generator))
    th = torch.rand(n_query, generator=generator) * 2 * math.pi
    rel = torch.stack([r * th.cos(), r * th.sin()], 1)
    ux = rel @ inflow
    phi = ux * radius ** 2 / r ** 2                                              # perturbation potential
    vel = inflow * (1 + radius ** 2 / r[:, None] ** 2) - 2 * radius ** 2 * ux[:, None] * rel / r[:, None] ** 4
    lengths = {"radius": torch.tensor(radius, device=device)}
    # nondimensional targets: potential in units of U·R, velocity in units of U (U = 1)
    return (centre + rel).to(device), {"wall": wall, "far": far}, lengths, (phi / radius).to(device), vel.to(device)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--faces", type=int, default=96)
    ap.add_argument("--queries", type=int, default=512)
    ap.add_argument("--lr", type=float, default=3e-3)
    ap.add_argument("--out", default="./outputs/globe_potential_flow")
    ap.add_argument("--smoke", action="store_true")
    a = ap.parse_args()
    if a.smoke:
        a.steps, a.faces, a.queries = 3, 24, 32
    device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    log = PythonLogger("globe")
    torch.manual_seed(0)
    model = GLOBE(n_spatial_dims=2, output_field_ranks={"phi": 0, "u": 1},
                  boundary_source_data_ranks={"wall": {}, "far": {"inflow": 1}}, reference_length_names=["radius"],
                  reference_area=1.0, n_communication_hyperlayers=1, n_latent_scalars=4, n_latent_vectors=2,
                  hidden_layer_sizes=[32, 32], theta=0.0, use_gradient_checkpointing=False).to(device)
    optimizer = torch.optim.Adam(model.parameters(), lr=a.lr)
    gen = torch.Generator().manual_seed(1)

    def evaluate(case):
        q, meshes, lengths, phi, vel = case
        # face measures are divided by reference_area: use the body's radius so that the sums are nondimensional
        model.reference_area.fill_(float(lengths["radius"]))
        out = model(q, meshes, lengths).point_data
        return (out["phi"] - phi).square().mean() + (out["u"] - vel).square().mean()

    for step in range(1, a.steps + 1):
        loss = evaluate(make_case(gen, a.faces, a.faces // 2, a.queries, device))
        optimizer.zero_grad(set_to_none=True)
        loss.backward()
        optimizer.step()
        if step % max(1, a.steps // 10) == 0 or step == a.steps:
            log.info(f"step {step}: loss {float(loss.detach()):.5f}")
    with torch.no_grad():
        model.eval()
        seen = evaluate(make_case(torch.Generator().manual_seed(5), a.faces, a.faces // 2, a.queries, device))
        moved = evaluate(make_case(torch.Generator().manual_seed(5), a.faces, a.faces // 2, a.queries, device, radius=3.0,
                                   centre=torch.tensor([20.0, -7.0]), angle=2.5))
    log.info(f"held-out case in the training range: {float(seen):.5f}; body 3x larger, far away, other inflow: {float(moved):.5f}")
    save_checkpoint(a.out, models=model, optimizer=optimizer, epoch=a.steps)
    log.success(f"saved to {a.out}")


if __name__ == "__main__":
    main()

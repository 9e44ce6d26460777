"""``KelvinHelmholtz2D``: endless generator of shear-layer instability sequences (2-D compressible Euler).

Parity: ``physicsnemo/datapipes/benchmarks/kelvin_helmholtz.py`` — random multi-frequency perturbation of two
counter-flowing bands, MUSCL-Hancock finite volumes with a Rusanov flux on a periodic unit square,
``nr_snapshots`` snapshots every ``iteration_per_snapshot`` steps, from which shuffled windows of length
``seq_length`` are served as ``{"density" [B,T,1,N,N], "velocity" [B,T,2,N,N], "pressure" [B,T,1,N,N]}``.

On CUDA the whole simulation of a batch is one cooperative launch (``csrc/pde_kh.cu``, two fused phases per
step); on CPU the same scheme runs with ``torch.roll``.
"""
import math
import sys
from dataclasses import dataclass
from typing import Dict, Tuple, Union

import torch

from ...ops import _lib
from ...ops import gemm as _g
from ..datapipe import Datapipe
from ..meta import DatapipeMetaData
from .darcy import _declare


@dataclass
class MetaData(DatapipeMetaData):
    name: str = "KelvinHelmholtz2D"
    auto_device: bool = True
    cuda_graphs: bool = True
    ddp_sharding: bool = False


def _rusanov(rl, rr, unl, unr, utl, utr, pl, pr, gamma):
    el = pl / (gamma - 1) + 0.5 * rl * (unl ** 2 + utl ** 2)
    er = pr / (gamma - 1) + 0.5 * rr * (unr ** 2 + utr ** 2)
    ra, mn, mt, ea = 0.5 * (rl + rr), 0.5 * (rl * unl + rr * unr), 0.5 * (rl * utl + rr * utr), 0.5 * (el + er)
    pa = (gamma - 1) * (ea - 0.5 * (mn ** 2 + mt ** 2) / ra)
    c = torch.maximum(torch.sqrt(gamma * pl / rl) + unl.abs(), torch.sqrt(gamma * pr / rr) + unr.abs())
    return (mn - c * 0.5 * (rl - rr), mn ** 2 / ra + pa - c * 0.5 * (rl * unl - rr * unr),
            mn * mt / ra - c * 0.5 * (rl * utl - rr * utr), (ea + pa) * mn / ra - c * 0.5 * (el - er))


def kh_simulate_torch(w, N, snapshots, steps, gamma, dx, dt, sigma):
    """Tensor formulation of the scheme; returns (rho [S,B,N,N], vel [S,B,N,N,2], p [S,B,N,N])."""
    B, nf = w.shape
    dev = w.device
    vol = dx * dx
    x = (torch.arange(N, device=dev) / N)[None, :, None]
    y = (torch.arange(N, device=dev) / N)[None, None, :]
    band = (y - 0.5).abs() < 0.25
    r = torch.where(band, 2.0, 1.0).expand(B, N, N).clone()
    ux = torch.where(band, 0.5, -0.5).expand(B, N, N).clone()
    env = torch.exp(-(y - 0.25) ** 2 / (2 * sigma ** 2)) + torch.exp(-(y - 0.75) ** 2 / (2 * sigma ** 2))
    ff = torch.arange(1, nf + 1, device=dev, dtype=w.dtype)
    uy = (ff[None, :, None, None] * w[:, :, None, None] * torch.sin(4.0 * 3.14159 * x[:, None] * ff[None, :, None, None])).sum(1) * env
    p = torch.full_like(r, 2.5)
    mass, mx, my = r * vol, ux * r * vol, uy * r * vol
    e = (p / (gamma - 1) + 0.5 * r * (ux ** 2 + uy ** 2)) * vol
    sx = lambda a, k: torch.roll(a, -k, 1)  # noqa: E731  value at i + k
    sy = lambda a, k: torch.roll(a, -k, 2)  # noqa: E731
    out_r, out_v, out_p = [], [], []
    for _ in range(snapshots):
        r = mass / vol
        u, v = mx / r / vol, my / r / vol
        p = (e / vol - 0.5 * r * (u ** 2 + v ** 2)) * (gamma - 1)
        out_r.append(r.clone()), out_v.append(torch.stack([u, v], -1)), out_p.append(p.clone())
        for _ in range(steps):
            r = mass / vol
            u, v = mx / r / vol, my / r / vol
            p = (e / vol - 0.5 * r * (u ** 2 + v ** 2)) * (gamma - 1)
            d = lambda a: ((sx(a, 1) - sx(a, -1)) / (2 * dx), (sy(a, 1) - sy(a, -1)) / (2 * dx))  # noqa: E731
            (rdx, rdy), (udx, udy), (vdx, vdy), (pdx, pdy) = d(r), d(u), d(v), d(p)
            h = 0.5 * dt
            r1 = r - h * (u * rdx + r * udx + v * rdy + r * vdy)
            u1 = u - h * (u * udx + v * udy + pdx / r)
            v1 = v - h * (u * vdx + v * vdy + pdy / r)
            p1 = p - h * (gamma * p * (udx + vdy) + u * pdx + v * pdy)
            hd = dx / 2
            face = lambda a, ax, ay: (a - ax * hd, a + ax * hd, a - ay * hd, a + ay * hd)  # noqa: E731
            rxl, rxr, ryl, ryr = face(r1, rdx, rdy)
            uxl, uxr, uyl, uyr = face(u1, udx, udy)
            vxl, vxr, vyl, vyr = face(v1, vdx, vdy)
            pxl, pxr, pyl, pyr = face(p1, pdx, pdy)
            fx = _rusanov(sx(rxl, 1), rxr, sx(uxl, 1), uxr, sx(vxl, 1), vxr, sx(pxl, 1), pxr, gamma)
            fy = _rusanov(sy(ryl, 1), ryr, sy(vyl, 1), vyr, sy(uyl, 1), uyr, sy(pyl, 1), pyr, gamma)
            k = dt * dx
            mass = mass + k * (-fx[0] + sx(fx[0], -1) - fy[0] + sy(fy[0], -1))
            mx = mx + k * (-fx[1] + sx(fx[1], -1) - fy[2] + sy(fy[2], -1))
            my = my + k * (-fx[2] + sx(fx[2], -1) - fy[1] + sy(fy[1], -1))
            e = e + k * (-fx[3] + sx(fx[3], -1) - fy[3] + sy(fy[3], -1))
    return torch.stack(out_r), torch.stack(out_v), torch.stack(out_p)


class KelvinHelmholtz2D(Datapipe):
    def __init__(self, resolution: int = 512, batch_size: int = 16, seq_length: int = 8, nr_perturbation_freq: int = 5,
                 perturbation_range: float = 0.1, nr_snapshots: int = 256, iteration_per_snapshot: int = 32,
                 gamma: float = 5.0 / 3.0, normaliser: Union[Dict[str, Tuple[float, float]], None] = None,
                 device: Union[str, torch.device] = "cuda"):
        super().__init__(meta=MetaData())
        self.resolution, self.batch_size, self.seq_length = resolution, batch_size, seq_length
        self.nr_perturbation_freq, self.perturbation_range = nr_perturbation_freq, perturbation_range
        self.nr_snapshots, self.iteration_per_snapshot, self.gamma = nr_snapshots, iteration_per_snapshot, gamma
        self.courant_fac = 0.4
        self.normaliser = normaliser
        if normaliser is not None and not {"density", "velocity", "pressure"}.issubset(normaliser.keys()):
            raise ValueError("normaliser need to have keys `density`, `velocity` and `pressure` with mean and std")
        self.device = torch.device(device)
        self.dx = 1.0 / resolution
        self.dt = self.courant_fac * self.dx / (math.sqrt(gamma * 5.0) + 2.0)
        self.vol = self.dx ** 2
        self.dim = (batch_size, resolution, resolution)
        z = lambda *s: torch.zeros(*s, dtype=torch.float32, device=self.device)  # noqa: E731
        self.w = z(batch_size, nr_perturbation_freq)
        self.seq_rho, self.seq_vel, self.seq_p = z(nr_snapshots, *self.dim), z(nr_snapshots, *self.dim, 2), z(nr_snapshots, *self.dim)
        if self.device.type == "cuda":
            self._cons, self._faces = z(4, *self.dim), z(16, *self.dim)
        self.output_rho = self.output_vel = self.output_p = None
        self._generator = None

    def set_generator(self, generator: torch.Generator) -> None:
        self._generator = generator

    def generate_batch(self) -> None:
        self.w.uniform_(-self.perturbation_range, self.perturbation_range, generator=self._generator)
        sigma = 0.05 / math.sqrt(2.0)
        if self.device.type == "cuda":
            lib = _lib.load(required=True)
            _declare(lib)
            err = lib.pnm_kh_simulate(self._cons.data_ptr(), self._faces.data_ptr(), self.w.data_ptr(), self.seq_rho.data_ptr(),
                                      self.seq_vel.data_ptr(), self.seq_p.data_ptr(), self.batch_size, self.resolution,
                                      self.nr_perturbation_freq, self.nr_snapshots, self.iteration_per_snapshot, self.gamma,
                                      self.dx, self.dt, sigma, torch.cuda.current_stream().cuda_stream)
            if err:
                raise RuntimeError(f"pnm_kh_simulate failed ({err})")
            _g.launch_count += 1
        else:
            r, v, p = kh_simulate_torch(self.w, self.resolution, self.nr_snapshots, self.iteration_per_snapshot, self.gamma,
                                        self.dx, self.dt, sigma)
            self.seq_rho.copy_(r), self.seq_vel.copy_(v), self.seq_p.copy_(p)

    def __iter__(self):
        B, T, S = self.batch_size, self.seq_length, self.nr_snapshots
        norm = self.normaliser
        while True:
            self.generate_batch()
            # an independent random order of window starts for every batch member
            starts = torch.stack([torch.randperm(S - T, device=self.device, generator=self._generator) for _ in range(B)])
            rows = torch.arange(B, device=self.device)[:, None]
            offs = torch.arange(T, device=self.device)[None, :]
            for step in range(S - T):
                t = starts[:, step, None] + offs                                  # [B, T]
                rho = self.seq_rho[t, rows].unsqueeze(2)                          # [B, T, 1, N, N]
                vel = self.seq_vel[t, rows].permute(0, 1, 4, 2, 3)                # [B, T, 2, N, N]
                p = self.seq_p[t, rows].unsqueeze(2)
                if norm is not None:
                    rho = (rho - norm["density"][0]) / norm["density"][1]
                    vel = (vel - norm["velocity"][0]) / norm["velocity"][1]
                    p = (p - norm["pressure"][0]) / norm["pressure"][1]
                if self.output_rho is None:
                    self.output_rho, self.output_vel, self.output_p = rho.clone(), vel.clone(), p.clone()
                else:
                    self.output_rho.copy_(rho), self.output_vel.copy_(vel), self.output_p.copy_(p)
                yield {"density": self.output_rho, "velocity": self.output_vel, "pressure": self.output_p}

    def __len__(self):
        return sys.maxsize

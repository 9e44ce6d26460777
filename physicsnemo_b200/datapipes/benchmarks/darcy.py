"""``Darcy2D``: endless generator of (permeability, pressure) pairs for ``−∇·(k∇u) = 1`` on the unit square.

Parity: ``physicsnemo/datapipes/benchmarks/darcy.py:53-322`` — random Fourier field thresholded to
``{min, max}_permeability``, multigrid Jacobi solve (coarse → fine, convergence checked every
``iterations_per_convergence_check`` sweeps against ``convergence_threshold × grid factor``), outputs
``{"permeability", "darcy"}`` of shape ``[B, 1, res, res]`` written into buffers that keep their address
(CUDA-graph friendly).

On CUDA the permeability is one kernel and the whole multigrid solve one cooperative launch with the
convergence test on the device (``csrc/pde_darcy.cu``); on CPU the same scheme runs as tensor operations.
"""
import ctypes
import sys
from dataclasses import dataclass
from typing import Dict, Tuple, Union

import torch

from ...ops import _lib
from ...ops import gemm as _g
from ..datapipe import Datapipe
from ..meta import DatapipeMetaData


@dataclass
class MetaData(DatapipeMetaData):
    name: str = "Darcy2D"
    auto_device: bool = True
    cuda_graphs: bool = True
    ddp_sharding: bool = False


def _declare(lib):
    if getattr(lib, "_pde_declared", False):
        return
    c = ctypes
    vp = c.c_void_p
    lib.pnm_darcy_permeability.argtypes = [vp, vp, c.c_int, c.c_int, c.c_int, c.c_float, c.c_float, vp]
    lib.pnm_darcy_solve.argtypes = [vp, vp, vp, vp, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_float, vp]
    lib.pnm_kh_simulate.argtypes = [vp] * 6 + [c.c_int] * 5 + [c.c_float] * 4 + [vp]
    for f in (lib.pnm_darcy_permeability, lib.pnm_darcy_solve, lib.pnm_kh_simulate):
        f.restype = c.c_int
    lib._pde_declared = True


def permeability_from_fourier(fourier: torch.Tensor, res: int, kmin: float, kmax: float) -> torch.Tensor:
    """``fourier``: [4, B, nf, nf] → [B, res+1, res+1] two-valued field (tensor formulation of the kernel)."""
    _, B, nf, _ = fourier.shape
    L = res + 1
    pos = 6.28318 / res * torch.arange(L, device=fourier.device, dtype=fourier.dtype)
    k = torch.arange(nf, device=fourier.device, dtype=fourier.dtype)
    s, c = torch.sin(pos[:, None] * k), torch.cos(pos[:, None] * k)                      # [L, nf]
    field = (torch.einsum("bij,xi,yj->bxy", fourier[0], s, s) + torch.einsum("bij,xi,yj->bxy", fourier[1], c, s)
             + torch.einsum("bij,xi,yj->bxy", fourier[2], s, c) + torch.einsum("bij,xi,yj->bxy", fourier[3], c, c)) / nf ** 2
    return torch.where(field < 0, torch.full_like(field, kmin), torch.full_like(field, kmax))


def _shift_zero(a, dx, dy):
    out = torch.zeros_like(a)
    L = a.shape[-1]
    xs = slice(max(dx, 0), L + min(dx, 0))
    xd = slice(max(-dx, 0), L + min(-dx, 0))
    ys = slice(max(dy, 0), L + min(dy, 0))
    yd = slice(max(-dy, 0), L + min(-dy, 0))
    out[:, xd, yd] = a[:, xs, ys]
    return out


def _shift_clamp(a, dx, dy):
    L = a.shape[-1]
    ix = (torch.arange(L, device=a.device) + dx).clamp(0, L - 1)
    iy = (torch.arange(L, device=a.device) + dy).clamp(0, L - 1)
    return a[:, ix][:, :, iy]


def darcy_multigrid_torch(perm: torch.Tensor, res: int, levels: int, max_iterations: int, check_every: int,
                          threshold: float) -> torch.Tensor:
    """Tensor formulation of the multigrid Jacobi solve (CPU path and oracle of the cooperative kernel)."""
    B, L, _ = perm.shape
    dx = 1.0 / (res + 1)
    u = torch.zeros_like(perm)
    for level in range(levels):
        f = 2 ** (levels - level - 1)
        n = res // f if f > 1 else L
        g = f * torch.arange(n, device=perm.device) + (f - 1)
        sel = (slice(None), g[:, None], g[None, :])
        gdx = dx * f
        for _ in range(max_iterations // check_every):
            prev = u
            for _ in range(check_every):
                d01, d21 = _shift_zero(u, -f, 0), _shift_zero(u, f, 0)
                d10, d12 = _shift_zero(u, 0, -f), _shift_zero(u, 0, f)
                p01, p21 = _shift_clamp(perm, -f, 0), _shift_clamp(perm, f, 0)
                p10, p12 = _shift_clamp(perm, 0, -f), _shift_clamp(perm, 0, f)
                t1 = perm * (d01 + d21 + d10 + d12) / gdx ** 2
                t2 = (p21 - p01) * (d21 - d01) / (2 * gdx)
                t3 = (p12 - p10) * (d12 - d10) / (2 * gdx)
                new = (t1 + t2 + t3 + 1.0) / (perm * 4.0 / gdx ** 2)
                prev = u
                u = u.clone()
                u[sel] = new[sel]
            if float((u[sel] - prev[sel]).abs().max()) < threshold * f:
                break
        if f > 1:
            idx = torch.arange(L, device=perm.device)
            r = (idx + 1) % f
            lo, hi = idx - r, idx + r
            w = (idx - lo).to(perm.dtype) / f

            def pick(ix, iy):
                okx, oky = (ix >= 0) & (ix < L), (iy >= 0) & (iy < L)
                v = u[:, ix.clamp(0, L - 1)][:, :, iy.clamp(0, L - 1)]
                return v * (okx[:, None] & oky[None, :])

            wx, wy = w[:, None], w[None, :]
            u = (1 - wy) * ((1 - wx) * pick(lo, lo) + wx * pick(hi, lo)) + wy * ((1 - wx) * pick(lo, hi) + wx * pick(hi, hi))
    return u


class Darcy2D(Datapipe):
    def __init__(self, resolution: int = 256, batch_size: int = 64, nr_permeability_freq: int = 5,
                 max_permeability: float = 2.0, min_permeability: float = 0.5, max_iterations: int = 30000,
                 convergence_threshold: float = 1e-6, iterations_per_convergence_check: int = 1000, nr_multigrids: int = 4,
                 normaliser: Union[Dict[str, Tuple[float, float]], None] = None, device: Union[str, torch.device] = "cuda"):
        super().__init__(meta=MetaData())
        self.resolution, self.batch_size = resolution, batch_size
        self.nr_permeability_freq = nr_permeability_freq
        self.max_permeability, self.min_permeability = max_permeability, min_permeability
        self.max_iterations, self.convergence_threshold = max_iterations, convergence_threshold
        self.iterations_per_convergence_check, self.nr_multigrids = iterations_per_convergence_check, nr_multigrids
        self.normaliser = normaliser
        if normaliser is not None and not {"permeability", "darcy"}.issubset(normaliser.keys()):
            raise ValueError("normaliser need to have keys permeability and darcy with mean and std")
        self.device = torch.device(device)
        if resolution % 2 ** (nr_multigrids - 1) != 0:
            raise ValueError("Resolution is incompatible with number of sub grids.")
        self.dx = 1.0 / (resolution + 1)
        self.dim = (batch_size, resolution + 1, resolution + 1)
        self.fourier_dim = (4, batch_size, nr_permeability_freq, nr_permeability_freq)
        z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=self.device)  # noqa: E731
        self.darcy0, self.darcy1, self.permeability = z(self.dim), z(self.dim), z(self.dim)
        self.rand_fourier = z(self.fourier_dim)
        self.inf_residual = z(2, dt=torch.int32)
        self.output_k = self.output_p = None
        self._generator = None
        self.sweeps_last_batch = 0

    def set_generator(self, generator: torch.Generator) -> None:
        self._generator = generator

    def initialize_batch(self) -> None:
        self.rand_fourier.uniform_(-1.0, 1.0, generator=self._generator)
        if self.device.type == "cuda":
            lib = _lib.load(required=True)
            _declare(lib)
            err = lib.pnm_darcy_permeability(self.rand_fourier.data_ptr(), self.permeability.data_ptr(), self.batch_size,
                                             self.resolution, self.nr_permeability_freq, self.min_permeability,
                                             self.max_permeability, torch.cuda.current_stream().cuda_stream)
            if err:
                raise RuntimeError(f"pnm_darcy_permeability failed ({err})")
            _g.launch_count += 1
        else:
            self.permeability.copy_(permeability_from_fourier(self.rand_fourier, self.resolution, self.min_permeability,
                                                              self.max_permeability))
        self.darcy0.zero_()
        self.darcy1.zero_()

    def generate_batch(self) -> None:
        self.initialize_batch()
        if self.device.type == "cuda":
            lib = _lib.load(required=True)
            self.inf_residual.zero_()
            err = lib.pnm_darcy_solve(self.darcy0.data_ptr(), self.darcy1.data_ptr(), self.permeability.data_ptr(),
                                      self.inf_residual.data_ptr(), self.batch_size, self.resolution, self.nr_multigrids,
                                      self.max_iterations, self.iterations_per_convergence_check,
                                      self.convergence_threshold, torch.cuda.current_stream().cuda_stream)
            if err:
                raise RuntimeError(f"pnm_darcy_solve failed ({err})")
            _g.launch_count += 1
        else:
            self.darcy0.copy_(darcy_multigrid_torch(self.permeability, self.resolution, self.nr_multigrids,
                                                    self.max_iterations, self.iterations_per_convergence_check,
                                                    self.convergence_threshold))

    def __iter__(self):
        r = self.resolution
        while True:
            self.generate_batch()
            k = self.permeability[:, None, :r, :r]
            p = self.darcy0[:, None, :r, :r]
            if self.normaliser is not None:
                k = (k - self.normaliser["permeability"][0]) / self.normaliser["permeability"][1]
                p = (p - self.normaliser["darcy"][0]) / self.normaliser["darcy"][1]
            if self.output_k is None:
                self.output_k, self.output_p = k.clone(), p.clone()
            else:
                self.output_k.copy_(k)
                self.output_p.copy_(p)
            yield {"permeability": self.output_k, "darcy": self.output_p}

    def __len__(self):
        return sys.maxsize

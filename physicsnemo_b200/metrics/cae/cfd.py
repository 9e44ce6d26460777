"""CFD post-processing metrics (parity: ``physicsnemo/metrics/cae/cfd.py``).

Only ``compute_frontal_area`` needs pyvista / shapely (imported when called); the force
coefficients, dominant frequency, velocity-gradient invariants and the TKE spectrum are plain
array code.  The TKE shell sums are one ``bincount`` instead of a triple Python loop.
"""
from typing import List, Tuple, Union

import numpy as np
import torch


def compute_frontal_area(mesh, direction: str = "x"):
    """Area of the union of the mesh triangles projected on the plane normal to ``direction``."""
    try:
        import shapely
    except ImportError:
        raise ImportError("These metrics require shapely, install it using `pip install shapely`.")
    planes = {"x": ((1, 0, 0), (1, 2)), "y": ((0, 1, 0), (0, 2)), "z": ((0, 0, 1), (0, 1))}
    if direction not in planes:
        raise ValueError("Direction must be x, y or z only")
    normal, (a, b) = planes[direction]
    flat = mesh.project_points_to_plane(origin=(0, 0, 0), normal=normal)
    pts = flat.points
    polys = [shapely.Polygon(np.stack([pts[tri, a], pts[tri, b]], axis=1)) for tri in flat.triangulate().regular_faces]
    return shapely.union_all(polys).area


def compute_force_coefficients(normals: np.ndarray, area: np.ndarray, coeff: float, p: np.ndarray, wss: np.ndarray,
                               force_direction: np.ndarray = np.array([1, 0, 0])):
    """``(c_total, c_pressure, c_friction)`` from cell normals, areas, pressure and wall shear stress."""
    c_p = coeff * np.sum((normals @ force_direction) * area * p)
    c_f = -coeff * np.sum((wss @ force_direction) * area)
    return c_p + c_f, c_p, c_f


def dominant_freq_calc(signal: List[Union[int, float]], sample_spacing: float = 1) -> float:
    """Frequency of the largest non-DC Fourier mode."""
    mag = np.abs(np.fft.fft(signal))
    mag[0] = 0
    return np.abs(np.fft.fftfreq(len(signal), sample_spacing)[np.argmax(mag)])


def compute_p_q_r(velocity_grad: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Normalised invariants of the velocity-gradient tensor ``[B, 3, 3, X, Y, Z]`` per grid point."""
    bs = velocity_grad.shape[0]
    J = velocity_grad.permute(0, 3, 4, 5, 1, 2).reshape(bs, -1, 3, 3)
    S = 0.5 * (J + J.transpose(-1, -2))
    J2 = J @ J
    tr = lambda m: m.diagonal(dim1=-2, dim2=-1).sum(-1)  # noqa: E731
    s2 = tr(S @ S)
    P = -tr(J) / torch.mean(s2 ** 0.5, dim=-1, keepdim=True)
    Q = -0.5 * tr(J2) / torch.mean(s2, dim=-1, keepdim=True)
    R = -tr(J @ J2) / 3 / torch.mean(s2 ** 1.5, dim=-1, keepdim=True)
    return P, Q, R


def compute_tke_spectrum(field: np.ndarray, length: float = None):
    """``(|k| sorted, E sorted, shell wavenumbers, shell-summed E)`` of a velocity field ``[3, X, Y, Z]``."""
    lx = ly = lz = 2 * np.pi if length is None else length
    u, v, w = field[0], field[1], field[2]
    nx, ny, nz = u.shape
    nt = nx * ny * nz
    E = 0.5 * sum(np.abs(np.fft.fftn(c) / nt) ** 2 for c in (u, v, w))
    kx, ky, kz = np.fft.fftfreq(nx, lx / nx), np.fft.fftfreq(ny, ly / ny), np.fft.fftfreq(nz, lz / nz)
    gx, gy, gz = np.meshgrid(kx, ky, kz, indexing="ij")
    mk = np.sqrt(gx ** 2 + gy ** 2 + gz ** 2).ravel()
    wave_numbers = np.arange(0, nx + 1) * 2 * np.pi
    ix, iy, iz = np.meshgrid(np.arange(nx), np.arange(ny), np.arange(nz), indexing="ij")
    shell = np.round(np.sqrt(ix * ix + iy * iy + iz * iz)).astype(np.int64).ravel()
    keep = shell < wave_numbers.size
    tke = np.bincount(shell[keep], weights=E.ravel()[keep], minlength=wave_numbers.size).astype(np.float64)
    order = mk.argsort()
    return mk[order], E.ravel()[order], wave_numbers, tke

"""Metadata features of observations: local solar time, offset from the analysis time, height / pressure, viewing angles.

Parity: ``physicsnemo/experimental/datapipes/healda/transforms/obs_features.py`` (28 features) and
``obs_features_ext.py`` (30 features, with latitude and a conventional / satellite split of the last
20 columns).  On a CUDA device the rows come from one kernel of the package library
(``csrc/obs_features.cu``); ``compute_unified_metadata_reference`` is the same formula in tensor
operations and serves the host path and the tests.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

N_FEATURES = 28
N_FEATURES_EXT = 30
_TWO_PI = 2 * math.pi


def local_solar_time(lon_deg: torch.Tensor, abs_time_ns: torch.Tensor) -> torch.Tensor:
    """Hours in ``[0, 24)``: UTC hour of the day plus ``lon / 15``."""
    utc_hours = ((abs_time_ns // 1_000_000_000) % 86400).float() / 3600.0
    return (utc_hours + lon_deg / 15.0) % 24.0


def _waves(angle: torch.Tensor, n: int) -> torch.Tensor:
    """``[sin(k a) for k = 1..n] + [cos(k a) for k = 1..n]`` along a new last axis."""
    k = torch.arange(1, n + 1, device=angle.device, dtype=angle.dtype)
    a = angle.unsqueeze(-1) * k
    return torch.cat([a.sin(), a.cos()], dim=-1)


def _nan_column(like: torch.Tensor) -> torch.Tensor:
    return torch.full_like(like, float("nan"), dtype=torch.float32)


def compute_unified_metadata_reference(target_time_sec, *, time, lon, lat=None, height=None, pressure=None, scan_angle=None,
                                       sat_zenith_angle=None, sol_zenith_angle=None, extended: bool = False) -> torch.Tensor:
    lonf = lon.float()
    n = lonf.shape[0]
    cols = [height, pressure, scan_angle, sat_zenith_angle, sol_zenith_angle]
    h, p, sc, zs, zo = [(_nan_column(lonf) if c is None else c.float()) for c in cols]
    lst = _waves(local_solar_time(lonf, time) / 24.0 * _TWO_PI, 2)
    dt = (time - target_time_sec * 1_000_000_000).float() * 1e-9 / 86400.0
    unit = lambda x, top: torch.clamp(x / top, 0.0, 1.0) * _TWO_PI  # noqa: E731
    if not extended:
        cz, so = torch.cos(torch.deg2rad(zs)), torch.deg2rad(zo)
        out = torch.cat([lst, dt[:, None], dt[:, None] ** 2, _waves(unit(h, 60000.0), 4), _waves(unit(p, 1100.0), 4),
                         (sc / 50.0)[:, None], (sc / 50.0)[:, None] ** 2, cz[:, None], cz[:, None] ** 2,
                         so.cos()[:, None], so.sin()[:, None]], dim=-1)
        return out.nan_to_num(0.0)
    if lat is None:
        raise ValueError("the extended feature set needs lat")
    out = torch.zeros(n, N_FEATURES_EXT, dtype=torch.float32, device=lonf.device)
    latr = torch.deg2rad(lat.float())
    out[:, :10] = torch.cat([lst, dt[:, None], dt[:, None] ** 2, _waves(dt, 1), latr.sin()[:, None], latr.cos()[:, None]], dim=-1)
    conv = ~torch.isnan(h)
    out[conv, 10:] = torch.cat([_waves(unit(h[conv], 60000.0), 5), _waves(unit(p[conv], 1100.0), 5)], dim=-1)
    sat = ~conv
    out[sat, 10:] = torch.cat([_waves(sc[sat] / 50.0 * _TWO_PI, 3), _waves(zs[sat] / 90.0 * _TWO_PI, 4),
                               _waves(zo[sat] / 180.0 * _TWO_PI, 3)], dim=-1)
    return out


def _lib_obs():
    from .....ops import _lib

    lib = _lib.load(required=True)
    if not getattr(lib, "_obs_declared", False):
        vp = ctypes.c_void_p
        lib.pnm_obs_metadata.argtypes = [vp] * 10 + [ctypes.c_longlong, ctypes.c_int, vp]
        lib.pnm_obs_metadata.restype = ctypes.c_int
        lib._obs_declared = True
    return lib


def compute_unified_metadata(target_time_sec: torch.Tensor, *, time: torch.Tensor, lon: torch.Tensor, lat: Optional[torch.Tensor] = None,
                             height: Optional[torch.Tensor] = None, pressure: Optional[torch.Tensor] = None,
                             scan_angle: Optional[torch.Tensor] = None, sat_zenith_angle: Optional[torch.Tensor] = None,
                             sol_zenith_angle: Optional[torch.Tensor] = None, extended: bool = False) -> torch.Tensor:
    """``(n, 28)`` or, with ``extended``, ``(n, 30)`` fp32 features.

    ``target_time_sec`` (int64 seconds) and ``time`` (int64 nanoseconds) are per observation; a missing
    column counts as all-NaN ("not reported"): zeros in the basic scheme, and in the extended scheme a
    NaN height marks a satellite observation.
    """
    if not lon.is_cuda:
        return compute_unified_metadata_reference(target_time_sec, time=time, lon=lon, lat=lat, height=height, pressure=pressure,
                                                  scan_angle=scan_angle, sat_zenith_angle=sat_zenith_angle,
                                                  sol_zenith_angle=sol_zenith_angle, extended=extended)
    if extended and lat is None:
        raise ValueError("the extended feature set needs lat")
    n = lon.shape[0]
    out = torch.empty(n, N_FEATURES_EXT if extended else N_FEATURES, dtype=torch.float32, device=lon.device)
    if n == 0:
        return out
    f32 = lambda t: (_nan_column(lon) if t is None else t.to(torch.float32)).contiguous()  # noqa: E731
    i64 = lambda t: t.to(torch.int64).expand(n).contiguous()  # noqa: E731
    cols = [f32(lat) if lat is not None else None, f32(lon), i64(time), i64(target_time_sec), f32(height), f32(pressure),
            f32(scan_angle), f32(sat_zenith_angle), f32(sol_zenith_angle)]
    ptrs = [None if c is None else c.data_ptr() for c in cols]
    rc = _lib_obs().pnm_obs_metadata(*ptrs, out.data_ptr(), n, int(extended), torch.cuda.current_stream(lon.device).cuda_stream)
    if rc != 0:
        raise RuntimeError(f"pnm_obs_metadata failed with status {rc}")
    return out

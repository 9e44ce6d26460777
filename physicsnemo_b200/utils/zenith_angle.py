"""Solar geometry for weather models: cosine of the zenith angle, azimuth, solar irradiance and accumulated top-of-atmosphere
radiation.

Parity: ``physicsnemo/utils/zenith_angle.py`` (``cos_zenith_angle``, ``cos_zenith_angle_from_timestamp``,
``zenith_azimuth_angles``, ``zenith_azimuth_angles_from_timestamp``, ``irradiance``,
``toa_incident_solar_radiation_accumulated``).  The Sun's apparent position follows the low-precision series of the
Astronomical Almanac (mean anomaly, mean longitude, equation of centre, obliquity polynomial) and Greenwich mean sidereal
time from the IAU-1982 polynomial.  Everything is evaluated in float64 tensors (so it runs on the GPU for on-the-fly
forcing channels) and returned in the dtype / container type of the inputs: tensors in → tensor out, arrays or floats in →
NumPy out.
"""
from __future__ import annotations

import datetime
import math
from typing import Tuple

import numpy as np
import torch

TIMESTAMP_2000 = datetime.datetime(2000, 1, 1, 12, 0, tzinfo=datetime.timezone.utc).timestamp()
_TWO_PI = 2 * math.pi


def _to_t(x, like: torch.Tensor | None = None) -> torch.Tensor:
    if isinstance(x, torch.Tensor):
        return x.to(torch.float64)
    return torch.as_tensor(np.asarray(x, dtype=np.float64), device=like.device if like is not None else None)


def _finish(out: torch.Tensor, *inputs):
    tens = [x for x in inputs if isinstance(x, torch.Tensor)]
    if tens:
        return out.to(tens[0].dtype if tens[0].is_floating_point() else torch.float32)
    arr = out.cpu().numpy().astype(np.float32)
    return arr if arr.ndim else np.float32(arr)


def _timestamp_of(time) -> np.ndarray:
    """POSIX seconds of a ``datetime`` (naive = UTC) or an array of them."""
    arr = np.asarray(time, dtype=object)
    conv = lambda d: d.replace(tzinfo=datetime.timezone.utc).timestamp() if isinstance(d, datetime.datetime) else _bad(d)  # noqa: E731
    return np.vectorize(conv, otypes=[np.float64])(arr)


def _bad(d):
    raise ValueError(f"model_time has an invalid date type. It must be datetime.datetime. Got {type(d)}.")


def _julian_century(ts: torch.Tensor) -> torch.Tensor:
    return (ts - TIMESTAMP_2000) / 86400.0 / 36525.0


def _gmst(T: torch.Tensor) -> torch.Tensor:
    theta = 67310.54841 + T * (876600 * 3600 + 8640184.812866 + T * (0.093104 - T * 6.2e-6))
    return torch.deg2rad(theta / 240.0) % _TWO_PI


def _sun_ra_dec(T: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    M = torch.deg2rad(357.5291 + 35999.0503 * T - 0.0001559 * T * T - 4.8e-7 * T ** 3)
    L = torch.deg2rad(280.46645 + 36000.76983 * T + 0.0003032 * T * T)
    centre = torch.deg2rad((1.9146 - 0.004817 * T - 1.4e-5 * T * T) * torch.sin(M) + (0.019993 - 0.000101 * T) * torch.sin(2 * M)
                           + 0.00029 * torch.sin(3 * M))
    lam = L + centre
    eps = torch.deg2rad(23.0 + 26.0 / 60 + 21.406 / 3600.0 - (46.836769 * T - 0.0001831 * T ** 2 + 0.0020034 * T ** 3 - 5.76e-7 * T ** 4
                                                                - 4.34e-8 * T ** 5) / 3600.0)
    x, y, z = torch.cos(lam), torch.cos(eps) * torch.sin(lam), torch.sin(eps) * torch.sin(lam)
    r = torch.sqrt(1.0 - z * z)
    return 2 * torch.atan2(y, x + r), torch.atan2(z, r)


def _angles(ts, lon, lat):
    ref = next((x for x in (lon, lat, ts) if isinstance(x, torch.Tensor)), None)
    lon_r, lat_r = torch.deg2rad(_to_t(lon, ref)), torch.deg2rad(_to_t(lat, ref))
    T = _julian_century(_to_t(ts, ref).to(lon_r.device))
    ra, dec = _sun_ra_dec(T)
    return lat_r, dec, _gmst(T) + lon_r - ra


def cos_zenith_angle_from_timestamp(timestamp, lon, lat):
    """Cosine of the solar zenith angle at POSIX time ``timestamp`` [s] and longitude / latitude [deg] (broadcast)."""
    lat_r, dec, h = _angles(timestamp, lon, lat)
    return _finish(torch.sin(lat_r) * torch.sin(dec) + torch.cos(lat_r) * torch.cos(dec) * torch.cos(h), lon, lat, timestamp)


def cos_zenith_angle(time, lon, lat):
    """Same for ``datetime`` objects (a single one or an array of them; naive datetimes are UTC)."""
    return cos_zenith_angle_from_timestamp(_timestamp_of(time), lon, lat)


def zenith_azimuth_angles_from_timestamp(timestamp, lon, lat, sin_zenith_epsilon: float = 1e-6):
    """``(sin zenith, cos zenith, sin azimuth, cos azimuth)``; the azimuth is measured from north through east."""
    lat_r, dec, h = _angles(timestamp, lon, lat)
    cz = (torch.sin(lat_r) * torch.sin(dec) + torch.cos(lat_r) * torch.cos(dec) * torch.cos(h)).clamp(-1, 1)
    sz = torch.sqrt(1.0 - cz * cz).clamp_min(sin_zenith_epsilon)
    sa = (-torch.sin(h) * torch.cos(dec) / sz).clamp(-1, 1)
    ca = ((torch.sin(dec) - cz * torch.sin(lat_r)) / (sz * torch.cos(lat_r))).clamp(-1, 1)
    return tuple(_finish(v, lon, lat, timestamp) for v in (sz, cz, sa, ca))


def zenith_azimuth_angles(time, lon, lat, sin_zenith_epsilon: float = 1e-6):
    return zenith_azimuth_angles_from_timestamp(_timestamp_of(time), lon, lat, sin_zenith_epsilon)


def _irradiance_t(t: torch.Tensor, S0, e, perihelion_longitude, mean_tropical_year, newton_iterations) -> torch.Tensor:
    year = mean_tropical_year * 86400.0
    equinox = datetime.datetime(2000, 3, 20, 7, 35, tzinfo=datetime.timezone.utc).timestamp()
    M = ((t - equinox) % year) / year * _TWO_PI - math.radians(perihelion_longitude)
    E = M
    for _ in range(newton_iterations):                      # Kepler's equation E − e sin E = M
        E = E - (E - e * torch.sin(E) - M) / (1 - e * torch.cos(E))
    return S0 / (1 - e * torch.cos(E)) ** 2


def irradiance(t, S0=1361, e=0.0167, perihelion_longitude=282.895, mean_tropical_year=365.2422, newton_iterations: int = 3):
    """Solar irradiance [W m⁻²] at POSIX time ``t`` from the Earth-Sun distance of a Kepler orbit."""
    return _finish(_irradiance_t(_to_t(t), S0, e, perihelion_longitude, mean_tropical_year, newton_iterations), t)


def toa_incident_solar_radiation_accumulated(t, lat, lon, interval=3600, S0=1361, e=0.0167, perihelion_longitude=282.895,
                                             mean_tropical_year=365.2422):
    """Top-of-atmosphere solar energy [J m⁻²] received during the ``interval`` seconds that end at ``t`` (the time integral
    of ``S · max(cos zenith, 0)`` in closed form over the hour angle)."""
    lat_r, dec, h1 = _angles(t, lon, lat)
    h0 = h1 - interval / 86400.0 * _TWO_PI
    A, B = torch.sin(lat_r) * torch.sin(dec), torch.cos(lat_r) * torch.cos(dec)
    A, B = torch.broadcast_tensors(A, B)
    hc = torch.acos(-A / B)                                  # NaN where the Sun never crosses the horizon during the day

    def seg(left, right):
        return A * (right - left) + B * (torch.sin(right) - torch.sin(left))

    def from_zero(a):
        root = _TWO_PI - hc
        n, a = torch.div(a, _TWO_PI, rounding_mode="floor"), a % _TWO_PI
        lit = seg(torch.zeros_like(a), torch.where(a < hc, a, hc)) + torch.where(root < a, seg(root, a), torch.zeros_like(a))
        return lit + (seg(torch.zeros_like(hc), hc) + seg(root, torch.full_like(hc, _TWO_PI))) * n

    integral = torch.where(torch.isnan(hc), seg(h0, h1).clamp_min(0), from_zero(h1) - from_zero(h0))
    S = _irradiance_t(_to_t(t).to(integral.device), S0, e, perihelion_longitude, mean_tropical_year, 3)
    return _finish(S * integral * (86400.0 / _TWO_PI), lon, lat, t)

"""Approximate insolation fields for DLWP-style forcing channels.

Parity: ``physicsnemo/utils/insolation.py`` (``insolation(dates, lat, lon, scale, daily, enforce_2d, clip_zero)``): solar
declination and Earth-Sun distance from a fixed-eccentricity orbit by day of year, hour angle from the fraction of the
day and the longitude; returns ``[time, *lat.shape]`` float32.
"""
from __future__ import annotations

import numpy as np


def insolation(dates, lat: np.ndarray, lon: np.ndarray, scale: float = 1.0, daily: bool = False, enforce_2d: bool = False,
               clip_zero: bool = True) -> np.ndarray:
    if lat.ndim != lon.ndim:
        raise ValueError("'lat' and 'lon' must have the same number of dimensions")
    if lat.ndim >= 2 and lat.shape != lon.shape:
        raise ValueError(f"shape mismatch between lat ({lat.shape} and lon ({lon.shape})")
    if lat.ndim == 1 and enforce_2d:
        lon, lat = np.meshgrid(lon, lat)
    eps, ecc, om = np.deg2rad(23.4441), 0.016715, np.deg2rad(282.7)
    beta = np.sqrt(1 - ecc ** 2)
    dates = np.asarray(dates, dtype="datetime64[us]")
    days = (dates - dates.astype("datetime64[Y]").astype("datetime64[us]")) / np.timedelta64(1, "D")
    days = days.reshape(days.shape + (1,) * lat.ndim)
    if daily:
        days, use_lon = 0.5 + np.round(days), np.zeros_like(lon, dtype=np.float32)
    else:
        use_lon = lon.astype(np.float32)
    lam_m = ecc * (1.0 + beta) * np.sin(om) + 2.0 * np.pi * (days - 80.5) / 365.0
    lam = lam_m + 2.0 * ecc * np.sin(lam_m - om)
    dec = np.arcsin(np.sin(eps) * np.sin(lam))
    h = 2 * np.pi * (days + use_lon / 360.0)
    rho = (1.0 - ecc ** 2) / (1.0 + ecc * np.cos(lam - om))
    lat_r = np.deg2rad(lat)[None, ...]
    sol = scale * (np.sin(lat_r) * np.sin(dec) - np.cos(lat_r) * np.cos(dec) * np.cos(h)) * rho ** (-2.0)
    if clip_zero:
        sol = np.maximum(sol, 0.0)
    return sol.astype(np.float32)

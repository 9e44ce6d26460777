"""Row filters of observation tables: finite values inside the channel's valid range, plausible height / pressure
for conventional observations, optional quality-control flags.

Parity: ``physicsnemo/experimental/datapipes/healda/transforms/obs_filtering.py`` (``filter_observations``).
Tables are mappings ``column → numpy array``; the per-row channel attributes (``min_valid``,
``max_valid``, ``is_conv``) are columns of the table, as after the reference's join with its channel
table.
"""
from __future__ import annotations

from typing import Dict, Sequence

import numpy as np

from ..configs import QCLimits, take_rows


def conventional_mask(table: Dict[str, np.ndarray], qc_filter: bool = False, uv_channels: Sequence[int] = (),
                      uv_in_situ_types: Sequence[int] = (), drop_channels: Sequence[int] = (),
                      gps_channel_limit: int = 2) -> np.ndarray:
    """Rows acceptable as conventional observations.

    Height must lie in ``[HEIGHT_MIN, HEIGHT_MAX]``; pressure in ``[min, PRESSURE_MAX]`` with the lower
    bound relaxed for GPS channels (local id ≤ ``gps_channel_limit``).  ``uv_channels`` with
    ``uv_in_situ_types`` keeps wind rows of in-situ report types only; ``drop_channels`` removes local
    channels altogether (e.g. the level-2 GPS retrievals).
    """
    height, pressure, local = (np.asarray(table[k]) for k in ("Height", "Pressure", "local_channel_id"))
    with np.errstate(invalid="ignore"):
        ok = np.isfinite(height) & (height >= QCLimits.HEIGHT_MIN) & (height <= QCLimits.HEIGHT_MAX)
        floor = np.where(local <= gps_channel_limit, QCLimits.PRESSURE_MIN_GPS, QCLimits.PRESSURE_MIN_DEFAULT)
        ok &= np.isfinite(pressure) & (pressure >= floor) & (pressure <= QCLimits.PRESSURE_MAX)
    if qc_filter and "Analysis_Use_Flag" in table:
        ok &= np.asarray(table["Analysis_Use_Flag"]) == 1
    if len(uv_channels):
        wind = np.isin(local, np.asarray(uv_channels))
        ok &= ~wind | np.isin(np.asarray(table["Observation_Type"]), np.asarray(uv_in_situ_types))
    if len(drop_channels):
        ok &= ~np.isin(local, np.asarray(drop_channels))
    return ok


def filter_observations(table: Dict[str, np.ndarray], qc_filter: bool = False, **conventional_options) -> Dict[str, np.ndarray]:
    """Keep rows with a finite observation inside ``[min_valid, max_valid]`` that pass their kind's checks."""
    obs = np.asarray(table["Observation"])
    with np.errstate(invalid="ignore"):
        ok = np.isfinite(obs) & (obs >= np.asarray(table["min_valid"])) & (obs <= np.asarray(table["max_valid"]))
    satellite_ok = np.ones_like(ok)
    if qc_filter and "QC_Flag" in table:
        satellite_ok = np.asarray(table["QC_Flag"]) == 0
    conv = np.asarray(table["is_conv"]).astype(bool)
    ok &= np.where(conv, conventional_mask(table, qc_filter, **conventional_options), satellite_ok)
    return take_rows(table, ok)

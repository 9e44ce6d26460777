"""Sensor registry, quality-control limits and the observation column schema.

Parity: ``physicsnemo/experimental/datapipes/healda/configs/{sensors,combined_schema,variable_configs}.py``.
The reference hard-codes the sensors of one observation archive; here a ``SensorRegistry`` is built
from the sensors a user declares (order = sensor id, channels = consecutive global channel ids,
platforms = union in declaration order), which keeps the id arithmetic and leaves the archive's
contents out of the source.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Sequence

import numpy as np

from .types import VariableConfig

#: columns of an observation table (a mapping ``name → 1-D array``), named as in the reference's parquet schema
OBS_COLUMNS = ("Latitude", "Longitude", "Observation", "Global_Channel_ID", "local_channel_id", "sensor_id", "Platform_ID",
               "Observation_Type", "Absolute_Obs_Time", "Height", "Pressure", "Scan_Angle", "Sat_Zenith_Angle", "Sol_Zenith_Angle")
OPTIONAL_OBS_COLUMNS = ("QC_Flag", "Analysis_Use_Flag")
_DTYPES = {"Global_Channel_ID": np.int64, "local_channel_id": np.int64, "sensor_id": np.int64, "Platform_ID": np.int64,
           "Observation_Type": np.int64, "Absolute_Obs_Time": "datetime64[ns]", "QC_Flag": np.int64, "Analysis_Use_Flag": np.int64}


def empty_table() -> Dict[str, np.ndarray]:
    return {c: np.empty(0, dtype=_DTYPES.get(c, np.float32)) for c in OBS_COLUMNS}


def concat_tables(tables: Iterable[Dict[str, np.ndarray]]) -> Dict[str, np.ndarray]:
    tables = [t for t in tables if len(t["Observation"])]
    if not tables:
        return empty_table()
    keys = [k for k in tables[0] if all(k in t for t in tables)]
    return {k: np.concatenate([np.asarray(t[k]) for t in tables]) for k in keys}


def take_rows(table: Dict[str, np.ndarray], rows) -> Dict[str, np.ndarray]:
    return {k: np.asarray(v)[rows] for k, v in table.items()}


class QCLimits:
    HEIGHT_MIN = 0
    HEIGHT_MAX = 60000
    PRESSURE_MIN_GPS = 0.5
    PRESSURE_MIN_DEFAULT = 200
    PRESSURE_MAX = 1100


@dataclass
class SensorConfig:
    """One instrument family: its platforms, channel count, valid range and per-channel normalisation."""

    name: str
    platforms: List[str]
    channels: int
    min_valid: float = 0.0
    max_valid: float = 400.0
    sensor_type: str = "microwave"            # "conventional" marks in-situ / GPS style observations
    means: np.ndarray = field(default=None)
    stds: np.ndarray = field(default=None)

    def __post_init__(self):
        self.means = np.zeros(self.channels) if self.means is None else np.asarray(self.means, dtype=float)
        self.stds = np.ones(self.channels) if self.stds is None else np.asarray(self.stds, dtype=float)
        if self.means.shape != (self.channels,) or self.stds.shape != (self.channels,):
            raise ValueError(f"sensor {self.name!r}: means / stds must have one entry per channel ({self.channels})")

    @property
    def is_conv(self) -> bool:
        return self.sensor_type == "conventional"


def _next_power_of_two(n: int) -> int:
    return 1 << max(n - 1, 0).bit_length()


class SensorRegistry:
    """Ids derived from a list of sensors: ``sensor_id`` = position, global channel = offset + local channel."""

    def __init__(self, sensors: Sequence[SensorConfig]):
        self.sensors = list(sensors)
        names = [s.name for s in self.sensors]
        if len(set(names)) != len(names):
            raise ValueError(f"duplicate sensor names in {names}")
        self.name_to_id = {n: i for i, n in enumerate(names)}
        self.offsets = dict(zip(names, np.concatenate([[0], np.cumsum([s.channels for s in self.sensors])[:-1]]).astype(int))) \
            if names else {}
        platforms: List[str] = []
        for s in self.sensors:
            platforms += [p for p in s.platforms if p not in platforms]
        self.platform_to_id = {p: i for i, p in enumerate(platforms)}
        self.n_platforms = _next_power_of_two(max(len(platforms), 64))
        self.n_channels = _next_power_of_two(max(sum(s.channels for s in self.sensors), 1024))

    def __getitem__(self, name: str) -> SensorConfig:
        return self.sensors[self.name_to_id[name]]

    def __contains__(self, name: str) -> bool:
        return name in self.name_to_id

    def global_channel(self, sensor: str, local_channel) -> np.ndarray:
        return (np.asarray(local_channel) + self.offsets[sensor]).astype(np.int64)

    def platform_lut(self, sensor: str) -> np.ndarray:
        """Global platform id → position of the platform in the sensor's own list (0 for foreign platforms)."""
        lut = np.zeros(self.n_platforms, dtype=np.int64)
        for local, p in enumerate(self[sensor].platforms):
            lut[self.platform_to_id[p]] = local
        return lut

    def channel_stats(self) -> Dict[str, np.ndarray]:
        """Per global channel: sensor id, local id, valid range, normalisation constants, conventional flag."""
        rows = [(i, c, s.min_valid, s.max_valid, s.means[c], s.stds[c], s.is_conv)
                for i, s in enumerate(self.sensors) for c in range(s.channels)]
        cols = list(zip(*rows)) if rows else [[]] * 7
        names = ("sensor_id", "local_channel_id", "min_valid", "max_valid", "mean", "stddev", "is_conv")
        return {n: np.asarray(c) for n, c in zip(names, cols)}


VARIABLE_CONFIGS = {
    "era5": VariableConfig(name="era5", variables_2d=["tcwv", "tas", "uas", "vas", "100u", "100v", "pres_msl", "sst", "sic"],
                           variables_3d=["U", "V", "T", "Z", "Q"],
                           levels=[1000, 925, 850, 700, 600, 500, 400, 300, 250, 200, 150, 100, 50],
                           variables_static=["orog", "lfrac"]),
}


def channel_names(config: VariableConfig) -> List[str]:
    """Pressure-level fields level by level, then the surface fields: the channel order of a state tensor."""
    return [f"{v}{lev}" for v in config.variables_3d for lev in config.levels] + list(config.variables_2d)

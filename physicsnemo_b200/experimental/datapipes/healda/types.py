"""Value types of the HealDA data pipeline.

Parity: ``physicsnemo/experimental/datapipes/healda/types.py`` (``TimeUnit``, ``VariableConfig``,
``BatchInfo``, ``UnifiedObservation``, ``Batch``, ``empty_batch``, ``split_by_sensor``).  A
``UnifiedObservation`` holds all observations of a batch as flat columns ordered sensor-major, then
by batch item, then by time frame; ``lengths[s, b, t]`` counts the rows of each group.
"""
from __future__ import annotations

import dataclasses
import json
from datetime import timedelta
from enum import Enum
from typing import Any, Optional, TypedDict

import numpy as np
import torch

N_FLOAT_METADATA = 28


class TimeUnit(Enum):
    HOUR = "h"
    DAY = "D"
    MINUTE = "min"
    SECOND = "s"

    def to_timedelta(self, steps: float) -> timedelta:
        key = {"h": "hours", "D": "days", "min": "minutes", "s": "seconds"}[self.value]
        return timedelta(**{key: steps})


@dataclasses.dataclass(frozen=True)
class VariableConfig:
    """Named selection of state variables: surface fields, pressure-level fields with their levels, static fields."""

    name: str
    variables_2d: list
    variables_3d: list
    levels: list
    variables_static: list = dataclasses.field(default_factory=list)


@dataclasses.dataclass
class BatchInfo:
    """Channel names, time step and normalisation constants of the state tensors in a batch."""

    channels: list
    time_step: int = 1
    time_unit: TimeUnit = TimeUnit.HOUR
    scales: Any = None
    center: Any = None

    def __post_init__(self):
        if isinstance(self.time_unit, str):
            raise ValueError("Time unit is a str. Should be a TimeUnit.")

    @staticmethod
    def loads(text: str) -> "BatchInfo":
        fields = json.loads(text)
        fields.pop("residual_normalization", None)
        if "time_unit" in fields:
            fields["time_unit"] = TimeUnit(fields["time_unit"])
        return BatchInfo(**fields)

    def asdict(self) -> dict:
        as_list = lambda v: None if v is None else np.asarray(v).tolist()  # noqa: E731
        return {"channels": self.channels, "time_step": self.time_step, "time_unit": self.time_unit.value,
                "scales": as_list(self.scales), "center": as_list(self.center)}

    def dumps(self) -> str:
        return json.dumps(self.asdict())

    def sel_channels(self, channels) -> "BatchInfo":
        channels = list(channels)
        where = np.array([self.channels.index(c) for c in channels], dtype=np.int64)
        take = lambda v: None if v is None else np.asarray(v)[where]  # noqa: E731
        return BatchInfo(channels=channels, time_step=self.time_step, time_unit=self.time_unit, scales=take(self.scales),
                         center=take(self.center))

    def denormalize(self, x: torch.Tensor) -> torch.Tensor:
        """``x · scales + center`` with the constants broadcast over ``(channel, time, pixel)``."""
        scales = torch.as_tensor(self.scales).to(x).view(-1, 1, 1)
        center = torch.as_tensor(self.center).to(x).view(-1, 1, 1)
        return x * scales + center

    def get_time_delta(self, t: int) -> timedelta:
        return self.time_unit.to_timedelta(t * self.time_step)


_OBS_COLUMNS = ("obs", "time", "float_metadata", "pix", "local_channel", "local_platform", "obs_type", "global_channel",
                "global_platform")


@dataclasses.dataclass
class UnifiedObservation:
    obs: torch.Tensor
    time: torch.Tensor
    float_metadata: torch.Tensor
    pix: torch.Tensor
    local_channel: torch.Tensor
    local_platform: torch.Tensor
    obs_type: torch.Tensor
    global_channel: torch.Tensor
    hpx_level: int
    global_platform: Optional[torch.Tensor] = None
    lengths: Optional[torch.Tensor] = None

    @classmethod
    def empty(cls, device="cpu", hpx_level: int = 8, batch_dims=(1, 1)) -> "UnifiedObservation":
        ids = lambda: torch.empty(0, dtype=torch.long, device=device)  # noqa: E731
        return cls(obs=torch.empty(0, device=device), time=ids(), float_metadata=torch.empty(0, N_FLOAT_METADATA, device=device),
                   pix=ids(), local_channel=ids(), local_platform=ids(), obs_type=ids(), global_channel=ids(),
                   global_platform=ids(), hpx_level=hpx_level,
                   lengths=torch.zeros(1, *batch_dims, dtype=torch.long, device=device))

    @property
    def batch_dims(self):
        return () if self.lengths is None else self.lengths.shape[-2:]

    def __repr__(self) -> str:
        return f"UnifiedObservation(nobs={self.obs.shape[0]!r}, batch_dims={self.batch_dims})"

    def columns(self) -> dict:
        return {name: getattr(self, name) for name in _OBS_COLUMNS if getattr(self, name) is not None}

    def to(self, device=None, dtype=None, non_blocking: bool = True) -> "UnifiedObservation":
        """Move every column; ``dtype`` applies to the floating columns only."""
        def move(t):
            if t is None:
                return None
            return t.to(device=device, dtype=dtype if t.is_floating_point() else None, non_blocking=non_blocking)

        moved = {f.name: move(getattr(self, f.name)) for f in dataclasses.fields(self) if f.name != "hpx_level"}
        return UnifiedObservation(hpx_level=self.hpx_level, **moved)


class Batch(TypedDict):
    target: torch.Tensor
    condition: torch.Tensor
    second_of_day: torch.Tensor
    day_of_year: torch.Tensor
    labels: torch.Tensor
    timestamp: torch.Tensor
    unified_obs: Optional[UnifiedObservation]


def empty_batch(*, batch_gpu: int, out_channels: int, condition_channels: int, time_length: int, x_size: int, device) -> Batch:
    """A batch of the right shapes with uninitialised states and no observations (for warm-up and shape inference)."""
    if x_size <= 0:
        raise ValueError(f"x_size must be positive, got {x_size}")
    per_frame = lambda **kw: torch.empty(batch_gpu, time_length, device=device, **kw)  # noqa: E731
    return {"target": torch.empty(batch_gpu, out_channels, time_length, x_size, device=device),
            "condition": torch.empty(batch_gpu, condition_channels, time_length, x_size, device=device),
            "second_of_day": per_frame(), "day_of_year": per_frame(), "labels": torch.empty(batch_gpu, 0, device=device),
            "timestamp": per_frame(dtype=torch.long),
            "unified_obs": UnifiedObservation.empty(device=device, batch_dims=(batch_gpu, time_length))}


def split_by_sensor(obs: UnifiedObservation, target_sensor_ids) -> dict:
    """One ``UnifiedObservation`` per sensor id; ids beyond the sensors present in ``lengths`` give empty sets."""
    if obs.lengths is None:
        raise ValueError("lengths is required for split_by_sensor")
    lengths = obs.lengths
    per_sensor = lengths.sum(dim=(1, 2)).tolist()
    if len(target_sensor_ids) < len(per_sensor):
        raise ValueError("target_sensor_ids must include the configured sensor order for split_by_sensor")
    pieces = {name: torch.split(col, per_sensor) for name, col in obs.columns().items()}
    out = {}
    for s, sensor_id in enumerate(target_sensor_ids):
        if s < len(per_sensor):
            cols = {name: parts[s] for name, parts in pieces.items()}
            lens = lengths[s:s + 1]
        else:
            cols = {name: col[:0] for name, col in obs.columns().items()}
            lens = torch.zeros((1,) + tuple(obs.batch_dims), dtype=lengths.dtype, device=lengths.device)
        cols.setdefault("global_platform", None)
        out[sensor_id] = UnifiedObservation(hpx_level=obs.hpx_level, lengths=lens, **cols)
    return out

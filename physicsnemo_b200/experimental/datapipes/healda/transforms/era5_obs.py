"""Two-stage batch transform: the host stage assembles flat columns, the device stage finishes the features.

Parity: ``physicsnemo/experimental/datapipes/healda/transforms/era5_obs.py`` (``ERA5ObsTransform``).

* ``transform(times, frames)`` (host, in the loader's worker): normalises and stacks the states to
  ``target [B, C, T, X]``, expands the static condition, encodes the frame times, and concatenates all
  observation tables ordered by (sensor, batch item, frame), recording ``lengths[s, b, t]``.
* ``device_transform(batch, device)`` (on the prefetch stream): copies the columns, locates every
  observation's HEALPix pixel, computes the metadata features on the device and maps platform ids to
  the sensor-local numbering, giving a :class:`~..types.UnifiedObservation`.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import numpy as np
import torch

from .....nn.module.hpx.tokenizer import healpix_lonlat_to_xy
from ..configs import SensorRegistry, concat_tables, take_rows
from ..time_utils import compute_day_of_year, compute_second_of_day, compute_timestamp
from ..types import BatchInfo, UnifiedObservation
from .obs_features import compute_unified_metadata

_FLOAT_COLUMNS = {"latitude": "Latitude", "longitude": "Longitude", "observation": "Observation", "height": "Height",
                  "pressure": "Pressure", "scan_angle": "Scan_Angle", "sat_zenith_angle": "Sat_Zenith_Angle",
                  "sol_zenith_angle": "Sol_Zenith_Angle"}
_INT_COLUMNS = {"global_channel_id": "Global_Channel_ID", "local_channel_id": "local_channel_id", "platform_id": "Platform_ID",
                "observation_type": "Observation_Type"}


class ERA5ObsTransform:
    def __init__(self, batch_info: BatchInfo, registry: Optional[SensorRegistry] = None, sensors: Sequence[str] = (),
                 hpx_level: int = 10, static_condition: Optional[torch.Tensor] = None, extended_features: bool = False,
                 pixel_reorder: Optional[torch.Tensor] = None):
        """``static_condition`` is ``[C_static, X]`` (already normalised); ``pixel_reorder`` optionally permutes the pixel axis
        of states and condition (e.g. from the archive's nested order to the model's face-row-column order)."""
        self.batch_info, self.registry, self.sensors = batch_info, registry, list(sensors)
        self.hpx_level, self.extended_features = hpx_level, extended_features
        self.mean = np.asarray(batch_info.center, dtype=np.float32)[:, None]
        self.std = np.asarray(batch_info.scales, dtype=np.float32)[:, None]
        self.static_condition, self.pixel_reorder = static_condition, pixel_reorder
        if self.sensors and registry is None:
            raise ValueError("a sensor registry is required when sensors are configured")
        self._sensor_ids = [registry.name_to_id[s] for s in self.sensors] if registry else []
        self._platform_luts = {registry.name_to_id[s]: torch.from_numpy(registry.platform_lut(s)) for s in self.sensors} \
            if registry else {}

    # ------------------------------------------------------------------ host
    def _reorder(self, x: torch.Tensor) -> torch.Tensor:
        return x if self.pixel_reorder is None else x.index_select(-1, self.pixel_reorder)

    def _process_obs(self, times, frames):
        if not self.sensors:
            raise ValueError("ERA5ObsTransform requires configured sensors.")
        B, T = len(frames), len(frames[0])
        tables, tags = [], []
        for b, sample in enumerate(frames):
            for t, frame in enumerate(sample):
                table = frame["obs"]
                n = len(table["Observation"])
                tables.append(table)
                tags.append(np.stack([np.full(n, b), np.full(n, t), np.full(n, compute_timestamp(times[b][t]))], 1).astype(np.int64))
        obs, tag = concat_tables(tables), (np.concatenate(tags) if tags else np.zeros((0, 3), np.int64))
        sensor = np.asarray(obs["sensor_id"]).astype(np.int64)
        rank = np.full(max(int(sensor.max()) + 1 if sensor.size else 0, max(self._sensor_ids, default=-1) + 1), len(self._sensor_ids))
        rank[self._sensor_ids] = np.arange(len(self._sensor_ids))
        slot = rank[sensor]
        keep = slot < len(self._sensor_ids)
        order = np.lexsort((tag[:, 1], tag[:, 0], slot))           # sensor-major, then batch item, then frame (stable)
        order = order[keep[order]]
        obs, tag, slot = take_rows(obs, order), tag[order], slot[order]
        lengths = torch.zeros(len(self._sensor_ids), B, T, dtype=torch.int32)
        if slot.size:
            flat = (slot * B + tag[:, 0]) * T + tag[:, 1]
            lengths = torch.from_numpy(np.bincount(flat, minlength=lengths.numel()).astype(np.int32)).reshape(lengths.shape)
        cols: Dict[str, torch.Tensor] = {k: torch.from_numpy(np.ascontiguousarray(obs[c], dtype=np.float32)) for k, c in _FLOAT_COLUMNS.items()}
        cols.update({k: torch.from_numpy(np.ascontiguousarray(obs[c], dtype=np.int64)) for k, c in _INT_COLUMNS.items()})
        when = np.asarray(obs["Absolute_Obs_Time"])
        when = when.astype("datetime64[ns]").view(np.int64) if when.dtype.kind == "M" else when.astype(np.int64)
        cols["absolute_obs_time"] = torch.from_numpy(np.ascontiguousarray(when))
        cols["target_time_sec"] = torch.from_numpy(np.ascontiguousarray(tag[:, 2]))
        return cols, lengths

    def _target(self, frames) -> torch.Tensor:
        state = np.stack([np.stack([(np.asarray(f["state"], dtype=np.float32) - self.mean) / self.std for f in sample])
                          for sample in frames])                                     # [B, T, C, X]
        return self._reorder(torch.from_numpy(state).permute(0, 2, 1, 3).contiguous())

    def transform(self, times, frames) -> dict:
        out = {}
        if "obs" in frames[0][0]:
            out["unified_obs"] = self._process_obs(times, frames)
        out["target"] = self._target(frames).float()
        encode = lambda fn, dtype: torch.tensor([[fn(t) for t in sample] for sample in times], dtype=dtype)  # noqa: E731
        out["second_of_day"] = encode(compute_second_of_day, torch.float32)
        out["day_of_year"] = encode(compute_day_of_year, torch.float32)
        out["timestamp"] = encode(compute_timestamp, torch.int64)
        B, _, T, X = out["target"].shape
        if self.static_condition is not None:
            cond = self._reorder(self.static_condition.float())[None, :, None, :]
            out["condition"] = cond.expand(B, -1, T, -1).clone()
        else:
            out["condition"] = torch.empty(B, 0, T, X)
        out["labels"] = torch.empty(B, 0)
        return out

    # ---------------------------------------------------------------- device
    def device_transform(self, batch: dict, device) -> dict:
        out = {}
        for key, value in batch.items():
            if key == "unified_obs":
                out[key] = self._device_obs(value[0], value[1], device)
            else:
                out[key] = value.to(device, non_blocking=True)
        return out

    def _local_platform(self, platform: torch.Tensor, lengths: torch.Tensor) -> torch.Tensor:
        local = torch.zeros_like(platform)
        end = 0
        for s, sensor_id in enumerate(self._sensor_ids):
            start, end = end, end + int(lengths[s].sum())
            if end > start:
                lut = self._platform_luts[sensor_id].to(platform.device)
                local[start:end] = lut[platform[start:end].clamp(0, lut.shape[0] - 1)]
        return local

    def _device_obs(self, cols: Dict[str, torch.Tensor], lengths: torch.Tensor, device) -> UnifiedObservation:
        per_sensor = lengths.sum(dim=(1, 2))                        # read on the host before the copy
        c = {k: v.to(device, non_blocking=True) for k, v in cols.items()}
        pix = healpix_lonlat_to_xy(c["longitude"], c["latitude"], self.hpx_level)
        meta = compute_unified_metadata(c["target_time_sec"], time=c["absolute_obs_time"], lon=c["longitude"], lat=c["latitude"],
                                        height=c["height"], pressure=c["pressure"], scan_angle=c["scan_angle"],
                                        sat_zenith_angle=c["sat_zenith_angle"], sol_zenith_angle=c["sol_zenith_angle"],
                                        extended=self.extended_features)
        local_platform = self._local_platform(c["platform_id"], per_sensor.reshape(-1, 1, 1))
        return UnifiedObservation(obs=c["observation"], time=c["absolute_obs_time"], float_metadata=meta, pix=pix,
                                  local_channel=c["local_channel_id"], local_platform=local_platform,
                                  obs_type=c["observation_type"], global_channel=c["global_channel_id"],
                                  global_platform=c["platform_id"], hpx_level=self.hpx_level,
                                  lengths=lengths.to(device, non_blocking=True))

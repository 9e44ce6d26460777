"""Synthetic weather data for benchmarking forecast models without any file IO.

Parity: ``physicsnemo/datapipes/climate/synthetic.py`` (``SyntheticWeatherDataset``, ``SyntheticWeatherDataLoader``): a
"temperature" field = base + lapse rate per channel + meridional gradient + annual cycle + noise, served as
``[{"invar": x_t, "outvar": x_{t+1 … t+num_steps}}]``.  The field is generated directly on the target device from
broadcasting tensors (the dense ``[days, channels, lat, lon]`` array is the only large allocation).
"""
from __future__ import annotations

import math
from typing import Any, List, Sequence, Tuple

import torch
from torch.utils.data import DataLoader, Dataset


class SyntheticWeatherDataset(Dataset):
    def __init__(self, channels: Sequence[int], num_samples_per_year: int, num_steps: int, device: str | torch.device = "cuda",
                 grid_size: Tuple[int, int] = (721, 1440), base_temp: float = 15, amplitude: float = 10, noise_level: float = 2, seed: int | None = None,
                 **kwargs: Any):
        self.num_days, self.num_steps, self.num_channels = num_samples_per_year, num_steps, len(channels)
        if self.num_days <= self.num_steps:
            raise ValueError("num_samples_per_year must exceed num_steps")
        self.device = torch.device(device if (str(device) != "cuda" or torch.cuda.is_available()) else "cpu")
        self.grid_size = tuple(grid_size)
        self.temperatures = self.generate_data(self.num_days, self.num_channels, self.grid_size, base_temp, amplitude, noise_level, seed)
        self.extra_args = kwargs

    def generate_data(self, num_days, num_channels, grid_size, base_temp, amplitude, noise_level, seed=None) -> torch.Tensor:
        lat, lon = grid_size
        dev = self.device
        gen = torch.Generator(device=dev)
        if seed is not None:
            gen.manual_seed(seed)
        altitude = (-0.5 * torch.arange(num_channels, device=dev, dtype=torch.float32)).reshape(1, -1, 1, 1)
        meridional = torch.linspace(-amplitude, amplitude, lat, device=dev).reshape(1, 1, -1, 1)
        season = torch.sin(2 * math.pi * torch.arange(num_days, device=dev, dtype=torch.float32) / 365).reshape(-1, 1, 1, 1)
        noise = torch.randn(num_days, num_channels, lat, lon, device=dev, generator=gen) * noise_level
        return noise.add_(base_temp + altitude + meridional + season)

    def __len__(self) -> int:
        return self.num_days - self.num_steps

    def __getitem__(self, idx: int) -> List[dict]:
        return [{"invar": self.temperatures[idx], "outvar": self.temperatures[idx + 1:idx + self.num_steps + 1]}]


class SyntheticWeatherDataLoader(DataLoader):
    """``DataLoader`` over ``SyntheticWeatherDataset``; loader options (``batch_size``, ``shuffle`` …) ride in the kwargs."""

    def __init__(self, *args, **kwargs):
        opts = {k: kwargs.pop(k) for k in ("batch_size", "shuffle", "num_workers", "pin_memory", "drop_last") if k in kwargs}
        dataset = SyntheticWeatherDataset(*args, **kwargs)
        opts.setdefault("batch_size", 1)
        if dataset.device.type == "cuda":
            opts["pin_memory"] = False            # samples already live on the device
            opts["num_workers"] = 0
        super().__init__(dataset=dataset, **opts)

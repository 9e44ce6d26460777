"""Interfaces a user implements to plug own observation sources or transforms into the pipeline.

Parity: ``physicsnemo/experimental/datapipes/healda/protocols.py``.
"""
from __future__ import annotations

from typing import Any, Protocol, runtime_checkable

import torch


@runtime_checkable
class ObsLoader(Protocol):
    """Asynchronous observation source: ``sel_time(times)`` → ``{"obs": [one table per time, …], …}``."""

    async def sel_time(self, times) -> dict:
        ...


class Transform(Protocol):
    """Host-side stage: per-sample frame lists → one batch dictionary of (pinned) host tensors."""

    def transform(self, times: list, frames: list) -> dict:
        ...


class DeviceTransform(Protocol):
    """Device-side stage: moves a host batch to ``device`` and finishes the features there."""

    def device_transform(self, batch: dict, device: torch.device) -> dict:
        ...

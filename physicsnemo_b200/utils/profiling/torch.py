"""``torch.profiler`` back end: CPU + CUDA activities, shapes, memory, flops; writes
``cpu_time.txt``, ``gpu_time.txt`` and ``trace.json`` per rank."""
from __future__ import annotations

from pathlib import Path
from typing import Optional

import torch
from torch.profiler import ProfilerActivity, profile

from .core import PhysicsNeMoProfilerWrapper


class TorchProfileWrapper(PhysicsNeMoProfilerWrapper):
    def __init__(self, **config):
        super().__init__(**config)
        self._profiler = None

    def _standup(self):
        activities = [ProfilerActivity.CPU]
        if torch.cuda.is_available():
            activities.append(ProfilerActivity.CUDA)
        cfg = dict(activities=activities, record_shapes=True, profile_memory=True, with_flops=True, with_stack=False)
        cfg.update(self._config)
        self._profiler = profile(**cfg)
        self._initialized = True

    def __enter__(self):
        if self._profiler is None:
            self._standup()
        self._profiler.__enter__()
        return self

    def __exit__(self, *exc):
        self._profiler.__exit__(*exc)
        return False

    def step(self):
        if self._profiler is not None:
            self._profiler.step()

    def finalize(self, output_top: Optional[Path] = None):
        if self._profiler is None or self._finalized:
            return
        out = self.output_dir(Path(output_top or self._output_top or "physicsnemo_profiling_outputs"))
        try:
            from ...distributed.manager import DistributedManager

            if DistributedManager.is_initialized() and DistributedManager().distributed:
                out = out / f"rank_{DistributedManager().rank}"
                out.mkdir(parents=True, exist_ok=True)
        except Exception:
            pass
        avg = self._profiler.key_averages()
        (out / "cpu_time.txt").write_text(avg.table(sort_by="cpu_time_total", row_limit=50))
        if torch.cuda.is_available():
            (out / "gpu_time.txt").write_text(avg.table(sort_by="cuda_time_total", row_limit=50))
        self._profiler.export_chrome_trace(str(out / "trace.json"))
        self._finalized = True

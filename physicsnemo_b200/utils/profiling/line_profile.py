"""``line_profiler`` back end (optional dependency): per-line timings of decorated functions."""
from __future__ import annotations

from pathlib import Path
from typing import Optional

from .core import PhysicsNeMoProfilerWrapper


class LineProfileWrapper(PhysicsNeMoProfilerWrapper):
    _is_decorator = True

    def __init__(self, **config):
        super().__init__(**config)
        try:
            from line_profiler import LineProfiler

            self._profiler = LineProfiler()
        except ImportError:
            self._profiler = None

    @property
    def available(self) -> bool:
        return self._profiler is not None

    def __call__(self, fn):
        if self._profiler is None:
            return fn
        return self._profiler(fn)

    def finalize(self, output_top: Optional[Path] = None):
        if self._profiler is None or self._finalized:
            return
        out = self.output_dir(Path(output_top or self._output_top or "physicsnemo_profiling_outputs"))
        with open(out / "profiler_stats.txt", "w") as f:
            self._profiler.print_stats(stream=f)
        self._finalized = True

"""Profiling tools.

Parity: ``physicsnemo/utils/profiling`` — singleton ``Profiler`` multiplexing registered
back ends (``interface.py:33-374``), ``TorchProfileWrapper`` (``torch.py:28-180``),
``LineProfileWrapper`` (``line_profile.py:29-107``, optional), ``profile`` / ``annotate``
decorators.  Added here: ``DeviceTimer`` (CUDA-event timing, max over ranks) and
``ExposedCommMeter`` (communication time not covered by compute) used by the benchmarks.
"""
from .core import ProfileRegistry, _Profiler_Singleton
from .interface import Profiler, annotate, profile
from .timing import DeviceTimer, ExposedCommMeter

__all__ = ["Profiler", "profile", "annotate", "ProfileRegistry", "DeviceTimer", "ExposedCommMeter"]

"""Profiler back-end protocol, registry and the singleton metaclass."""
from __future__ import annotations

import threading
from pathlib import Path
from typing import Dict, Optional


class _Profiler_Singleton(type):
    """Metaclass: one instance per class, created under a lock."""

    _instances: Dict[type, object] = {}
    _lock = threading.Lock()

    def __call__(cls, *args, **kwargs):
        with cls._lock:
            if cls not in cls._instances:
                cls._instances[cls] = super().__call__(*args, **kwargs)
        return cls._instances[cls]


class PhysicsNeMoProfilerWrapper:
    """Base of a profiling back end: context manager with ``step`` / ``finalize`` / ``__call__`` (decorator)."""

    _is_context = True
    _is_decorator = False

    def __init__(self, **config):
        self._config = config
        self._initialized = False
        self._finalized = False
        self.enabled = False
        self._output_top: Optional[Path] = None

    def _standup(self):
        self._initialized = True

    def initialize(self, output_top: Optional[Path] = None):
        self._output_top = output_top
        if not self._initialized:
            self._standup()

    def output_dir(self, top: Path) -> Path:
        out = Path(top) / type(self).__name__.replace("Wrapper", "").lower()
        out.mkdir(parents=True, exist_ok=True)
        return out

    def step(self):
        pass

    def finalize(self, output_top: Optional[Path] = None):
        self._finalized = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False

    def __call__(self, fn):
        return fn


class ProfileRegistry:
    """Name → back-end class table; instances are singletons of their class."""

    _classes: Dict[str, type] = {}
    _instances: Dict[str, PhysicsNeMoProfilerWrapper] = {}

    @classmethod
    def register_profiler(cls, key: str, klass: type):
        cls._classes[key] = klass

    @classmethod
    def get_profiler(cls, key: str) -> PhysicsNeMoProfilerWrapper:
        if key not in cls._instances:
            if key not in cls._classes:
                raise KeyError(f"No profiler registered under '{key}'; available: {sorted(cls._classes)}")
            cls._instances[key] = cls._classes[key]()
        return cls._instances[key]

    @classmethod
    def clear(cls):
        cls._instances.clear()

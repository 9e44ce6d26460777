"""``Profiler`` singleton, ``profile`` decorator and ``annotate`` (NVTX ranges).

``Profiler().enable("torch")`` / ``enable("line_profiler")`` select back ends;
``initialize()`` stands them up, ``with Profiler(): ...`` activates them, ``step()`` marks
iteration boundaries and ``finalize()`` writes the reports.  Functions decorated with
``@profile`` before the profiler is initialised are recorded and wrapped later (zero cost
while profiling is off).
"""
from __future__ import annotations

import atexit
import functools
import sys
from contextlib import ContextDecorator, ExitStack
from pathlib import Path
from typing import Callable, List, Optional, Tuple

import torch

from .core import ProfileRegistry, _Profiler_Singleton
from .line_profile import LineProfileWrapper
from .torch import TorchProfileWrapper

ProfileRegistry.register_profiler("torch", TorchProfileWrapper)
ProfileRegistry.register_profiler("line_profiler", LineProfileWrapper)
ProfileRegistry.register_profiler("line_profile", LineProfileWrapper)


class annotate(ContextDecorator):
    """NVTX range as context manager / decorator: ``with annotate("step"): ...`` or ``@annotate("fn")``."""

    def __init__(self, message: Optional[str] = None, color: Optional[str] = None, domain: Optional[str] = None,
                 category: Optional[str] = None):
        self.message = message

    def __call__(self, fn):
        if self.message is None:
            self.message = getattr(fn, "__qualname__", "fn")
        return super().__call__(fn)

    def __enter__(self):
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_push(self.message or "range")
        return self

    def __exit__(self, *exc):
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()
        return False


class Profiler(metaclass=_Profiler_Singleton):
    """Multiplexes the enabled profiling back ends."""

    def __init__(self):
        self._profilers: List = []
        self._deferred: List[Tuple[Callable, str]] = []
        self._decorated = {}
        self._initialized = False
        self._finalized = False
        self._output_top = Path("./physicsnemo_profiling_outputs/")
        self._stack: Optional[ExitStack] = None
        atexit.register(self.finalize)

    # ----------------------------------------------------------- configuration
    @property
    def output_path(self) -> Path:
        return self._output_top

    @output_path.setter
    def output_path(self, path):
        self._output_top = Path(path)

    @property
    def initialized(self) -> bool:
        return self._initialized

    @property
    def enabled(self) -> bool:
        return len(self._profilers) > 0

    def enable(self, profiler):
        if isinstance(profiler, str):
            profiler = ProfileRegistry.get_profiler(profiler)
        if profiler not in self._profilers:
            profiler.enabled = True
            self._profilers.append(profiler)
        return profiler

    def get(self, key: str):
        return ProfileRegistry.get_profiler(key)

    def initialize(self):
        for p in self._profilers:
            p.initialize(self._output_top)
        self._initialized = True
        for fn, name in self._deferred:
            self._late_wrap(fn)
        self._deferred.clear()

    def finalize(self):
        if self._finalized:
            return
        for p in self._profilers:
            try:
                p.finalize(self._output_top)
            except Exception:  # interpreter teardown: best effort
                pass
        self._finalized = True

    def step(self):
        for p in self._profilers:
            p.step()

    # -------------------------------------------------------- context manager
    def __enter__(self):
        if not self._initialized:
            self.initialize()
        self._stack = ExitStack()
        for p in self._profilers:
            if p._is_context:
                self._stack.enter_context(p)
        return self

    def __exit__(self, *exc):
        if self._stack is not None:
            self._stack.close()
            self._stack = None
        return False

    # ------------------------------------------------------------- decoration
    def _wrap_now(self, fn: Callable) -> Callable:
        wrapped = fn
        for p in self._profilers:
            if p._is_decorator and p.enabled:
                wrapped = p(wrapped)
        return wrapped

    def _late_wrap(self, fn: Callable):
        """Replace ``fn`` in its defining module (or ``__main__``) by the wrapped version."""
        wrapped = self._wrap_now(fn)
        if wrapped is fn:
            return
        holder = self._decorated.get(fn)
        if holder is not None:
            holder["target"] = wrapped
        mod = sys.modules.get(getattr(fn, "__module__", ""), None)
        name = getattr(fn, "__name__", None)
        if mod is not None and name and getattr(mod, name, None) is holder.get("proxy") if holder else False:
            pass

    def __call__(self, fn: Callable) -> Callable:
        """Decorator form: ``@Profiler()`` / ``@profile``."""
        holder = {"target": fn}

        @functools.wraps(fn)
        def proxy(*args, **kwargs):
            return holder["target"](*args, **kwargs)

        holder["proxy"] = proxy
        self._decorated[fn] = holder
        if self._initialized:
            holder["target"] = self._wrap_now(fn)
        else:
            self._deferred.append((fn, getattr(fn, "__qualname__", "fn")))
        return proxy

    @classmethod
    def _clear_instance(cls):
        _Profiler_Singleton._instances.pop(cls, None)


def profile(fn: Optional[Callable] = None):
    """``@profile``: profile ``fn`` with every decorator-style back end once profiling is enabled."""
    if fn is None:
        return Profiler()
    return Profiler()(fn)

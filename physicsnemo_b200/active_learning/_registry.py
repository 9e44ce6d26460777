"""Name → class registry used to rebuild strategies from a checkpoint.

Parity: ``physicsnemo/active_learning/_registry.py`` (``ActiveLearningRegistry``: ``register``
decorator, ``construct`` with signature validation, ``get_class`` with an import-path fallback).
"""
from __future__ import annotations

import importlib
import inspect
from typing import Any, Callable
from warnings import warn

__all__ = ["registry", "ActiveLearningRegistry"]

_VARIADIC = (inspect.Parameter.VAR_KEYWORD, inspect.Parameter.VAR_POSITIONAL)


class ActiveLearningRegistry:
    def __init__(self) -> None:
        self._registry: dict[str, type] = {}

    def register(self, cls_name: str) -> Callable[[type], type]:
        def decorator(cls: type) -> type:
            if cls_name in self._registry:
                raise ValueError(f"Protocol '{cls_name}' is already registered. "
                                 f"Existing class: {self._registry[cls_name].__name__}")
            self._registry[cls_name] = cls
            return cls

        return decorator

    def get_class(self, cls_name: str, module_path: str | None = None) -> type:
        if cls_name in self._registry:
            return self._registry[cls_name]
        if not module_path:
            raise NameError(f"Class {cls_name} not found in registry, and no module path was provided.")
        cls = getattr(importlib.import_module(module_path), cls_name, None)
        if cls is None:
            raise NameError(f"Class {cls_name} not found in module {module_path}")
        return cls

    def construct(self, cls_name: str, module_path: str | None = None, **kwargs: Any):
        cls = self.get_class(cls_name, module_path)
        try:
            params = {n: p for n, p in inspect.signature(cls.__init__).parameters.items() if n != "self"}
        except (ValueError, TypeError) as e:
            raise TypeError(f"Could not inspect signature of {cls.__name__}.__init__: {e}")
        named = {n: p for n, p in params.items() if p.kind not in _VARIADIC}
        missing = [n for n, p in named.items() if p.default is inspect.Parameter.empty and n not in kwargs]
        if missing:
            raise TypeError(f"Missing required arguments for {cls.__name__}: {', '.join(missing)}")
        if not any(p.kind is inspect.Parameter.VAR_KEYWORD for p in params.values()):
            unexpected = [n for n in kwargs if n not in named]
            if unexpected:
                warn(f"Unexpected arguments for {cls.__name__}: {', '.join(unexpected)}. "
                     f"Valid parameters: {', '.join(sorted(named))}")
        return cls(**kwargs)

    def __getitem__(self, cls_name: str) -> type:
        if cls_name not in self._registry:
            available = ", ".join(self._registry) if self._registry else "none"
            raise KeyError(f"Protocol '{cls_name}' is not registered. Available protocols: {available}")
        return self._registry[cls_name]

    def is_registered(self, cls_name: str) -> bool:
        return cls_name in self._registry

    @property
    def registered_names(self) -> list[str]:
        return sorted(self._registry)


registry = ActiveLearningRegistry()

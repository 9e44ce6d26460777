"""Name → class registry of datapipe components (parity: ``physicsnemo/datapipes/registry.py``), with an OmegaConf
resolver ``${dp:Name}`` that expands to the import path when OmegaConf is installed."""
from __future__ import annotations

from typing import Callable, Type, TypeVar

T = TypeVar("T")


class ComponentRegistry:
    def __init__(self, name: str) -> None:
        self.name = name
        self._components: dict[str, Type] = {}

    def register(self, name: str | None = None) -> Callable[[Type[T]], Type[T]]:
        def decorator(cls: Type[T]) -> Type[T]:
            key = name or cls.__name__
            if key in self._components and self._components[key] is not cls:
                raise ValueError(f"Component '{key}' is already registered in {self.name} registry")
            self._components[key] = cls
            return cls

        return decorator

    def get(self, name: str) -> Type:
        if name not in self._components:
            raise KeyError(f"Component '{name}' not found in {self.name} registry. Available: {sorted(self._components)}")
        return self._components[name]

    def list(self) -> list[str]:
        return sorted(self._components)

    def __contains__(self, name: str) -> bool:
        return name in self._components

    def __len__(self) -> int:
        return len(self._components)

    def __repr__(self) -> str:
        return f"ComponentRegistry(name={self.name!r}, components={self.list()})"


COMPONENT_REGISTRY = ComponentRegistry("datapipes")


def register(name: str | None = None):
    return COMPONENT_REGISTRY.register(name)


def _resolve_component(name: str) -> str:
    cls = COMPONENT_REGISTRY.get(name)
    return f"{cls.__module__}.{cls.__qualname__}"


def register_resolvers() -> None:
    try:
        from omegaconf import OmegaConf
    except ImportError:
        return
    if not OmegaConf.has_resolver("dp"):
        OmegaConf.register_new_resolver("dp", _resolve_component)

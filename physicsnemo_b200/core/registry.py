"""Model registry backed by entry points.

Parity: ``physicsnemo/core/registry.py:49-193`` — a process-wide shared-state
registry that lists entry points of the groups ``physicsnemo.models`` and
``modulus.models`` lazily and lets classes be registered at run time.
"""
from __future__ import annotations

from importlib.metadata import EntryPoint, entry_points
from typing import Dict, List, Union
import warnings

_GROUPS = ("physicsnemo.models", "physicsnemo_b200.models", "modulus.models")


def _pyproject_entry_points() -> Dict[str, str]:
    """``{name: "module:Class"}`` of the ``physicsnemo.models`` group in the repository's ``pyproject.toml`` (if present)."""
    from pathlib import Path

    path = Path(__file__).resolve().parents[2] / "pyproject.toml"
    if not path.exists():
        return {}
    try:
        import tomllib

        with open(path, "rb") as fh:
            data = tomllib.load(fh)
        return dict(data.get("project", {}).get("entry-points", {}).get("physicsnemo.models", {}))
    except Exception:  # noqa: BLE001  (a malformed file must not break imports)
        return {}


class ModelRegistry:
    """Shared-state ("Borg") registry: every instance sees the same table."""

    _shared: dict = {}

    def __new__(cls):
        obj = super().__new__(cls)
        obj.__dict__ = cls._shared
        if "_table" not in cls._shared:
            cls._shared["_table"] = cls._scan_entry_points()
        return obj

    @staticmethod
    def _scan_entry_points() -> Dict[str, Union[EntryPoint, type]]:
        table: Dict[str, Union[EntryPoint, type]] = {}
        for group in _GROUPS:
            try:
                eps = entry_points(group=group)
            except Exception:  # pragma: no cover - metadata backend problems
                continue
            for ep in eps:
                table.setdefault(ep.name, ep)
        if not any(getattr(ep, "value", "").startswith("physicsnemo_b200.") for ep in table.values()):
            # source checkout that was never pip-installed: read the entry-point table from pyproject.toml
            for name, value in _pyproject_entry_points().items():
                table.setdefault(name, EntryPoint(name=name, value=value, group="physicsnemo.models"))
        return table

    # -- public API ---------------------------------------------------------
    def register(self, model: type, name: str | None = None) -> None:
        """Register ``model`` (a ``Module`` subclass) under ``name``."""
        from .module import Module

        if not (isinstance(model, type) and issubclass(model, Module)):
            raise ValueError(
                f"Only subclasses of physicsnemo Module can be registered, got {model!r}"
            )
        name = name or model.__name__
        if name in self._table and self._resolve(name) is not model:
            raise ValueError(f"Name {name} already in use")
        self._table[name] = model

    def _resolve(self, name: str):
        item = self._table[name]
        if isinstance(item, EntryPoint):
            try:
                item = item.load()
            except Exception as exc:  # keep the registry usable
                warnings.warn(f"entry point {name} failed to load: {exc}")
                raise
            self._table[name] = item
        return item

    def factory(self, name: str) -> type:
        """Return the class registered under ``name``."""
        if name in self._table:
            return self._resolve(name)
        raise KeyError(f"No model is registered under the name {name}")

    def list_models(self) -> List[str]:
        return list(self._table.keys())

    def __clear_registry__(self):
        self._table.clear()

    def __restore_registry__(self):
        self._shared["_table"] = self._scan_entry_points()

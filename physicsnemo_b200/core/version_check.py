"""Version gating and lazy optional imports.

Parity: ``physicsnemo/core/version_check.py`` (``check_version_spec`` ``:380``,
``require_version_spec`` ``:455``, ``OptionalImport`` ``:609-763``,
``get_physicsnemo_pkg_info``).
"""
from __future__ import annotations

import functools
import importlib
import importlib.metadata
import importlib.util
import subprocess
from pathlib import Path

from packaging.specifiers import SpecifierSet
from packaging.version import Version

__version__ = "2.2.0a0"


def get_physicsnemo_pkg_info() -> dict:
    """Version (and git hash when run from a checkout) of this package."""
    git_hash = "unknown"
    try:
        root = Path(__file__).resolve().parents[2]
        if (root / ".git").exists():
            git_hash = subprocess.run(
                ["git", "-C", str(root), "rev-parse", "HEAD"], capture_output=True, text=True, timeout=5
            ).stdout.strip() or "unknown"
    except Exception:
        pass
    return {"version": __version__, "git_hash": git_hash}


def get_installed_version(name: str) -> str | None:
    """Installed distribution / module version, or ``None`` when absent."""
    try:
        return importlib.metadata.version(name)
    except importlib.metadata.PackageNotFoundError:
        pass
    try:
        if importlib.util.find_spec(name) is None:
            return None
        mod = importlib.import_module(name)
        return getattr(mod, "__version__", "0")
    except Exception:
        return None


def check_version_spec(name: str, spec: str = "", *, error_msg: str | None = None, hard_fail: bool = False) -> bool:
    """True when ``name`` is importable and its version satisfies ``spec``."""
    version = get_installed_version(name)
    ok = version is not None
    if ok and spec:
        spec_set = SpecifierSet(spec if spec[0] in "<>=!~" else f">={spec}")
        try:
            ok = Version(version.split("+")[0]) in spec_set
        except Exception:
            ok = False
    if not ok and hard_fail:
        raise ImportError(error_msg or f"{name}{spec} is required but not available (found {version})")
    return ok


def require_version_spec(name: str, spec: str = ""):
    """Decorator: calling the function raises ``ImportError`` unless ``name``/``spec`` holds."""

    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            check_version_spec(name, spec, hard_fail=True)
            return fn(*args, **kwargs)

        return wrapper

    return deco


def ensure_available(name: str, spec: str = "") -> None:
    check_version_spec(name, spec, hard_fail=True)


class OptionalImport:
    """Proxy that imports ``name`` on first attribute access.

    ``bool(proxy)`` / ``proxy.available`` tell whether the import works; using
    a missing package raises an ``ImportError`` carrying an install hint.
    """

    def __init__(self, name: str, spec: str = "", hint: str | None = None):
        self._name, self._spec, self._hint = name, spec, hint
        self._mod = None

    @property
    def available(self) -> bool:
        return check_version_spec(self._name, self._spec)

    def __bool__(self):
        return self.available

    def _load(self):
        if self._mod is None:
            if not self.available:
                raise ImportError(
                    f"Optional dependency '{self._name}{self._spec}' is not installed. "
                    + (self._hint or f"Install it with `pip install {self._name}`.")
                )
            self._mod = importlib.import_module(self._name)
        return self._mod

    def __getattr__(self, item):
        return getattr(self._load(), item)

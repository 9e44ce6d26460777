"""File-system helpers: local / fsspec back ends, download cache, ``Package``.

Parity: ``physicsnemo/core/filesystem.py`` — ``_get_fs`` (``:50-54``),
``_download_cached`` with a sha256-of-URL cache directory under
``$LOCAL_CACHE`` or ``~/.cache/physicsnemo`` (``:198-307``) and ``Package``
(``:310-346``).  ``fsspec`` / ``s3fs`` / ``requests`` are optional here: plain
paths and ``file://`` URLs work with the standard library alone.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import urllib.parse
import urllib.request
from pathlib import Path


def _cache_dir() -> str:
    root = os.environ.get("LOCAL_CACHE") or os.path.join(os.path.expanduser("~"), ".cache", "physicsnemo")
    os.makedirs(root, exist_ok=True)
    return root


class _LocalFS:
    """Minimal stand-in for an fsspec file system on local paths."""

    protocol = "file"

    def put(self, src, dst):
        src, dst = str(src), _strip_file_scheme(str(dst))
        parent = os.path.dirname(os.path.abspath(dst))
        os.makedirs(parent, exist_ok=True)
        tmp = dst + ".tmp-write"
        shutil.copyfile(src, tmp)
        os.replace(tmp, dst)  # atomic on POSIX: readers never see a partial file

    def get(self, src, dst):
        shutil.copyfile(_strip_file_scheme(str(src)), str(dst))

    def exists(self, path):
        return os.path.exists(_strip_file_scheme(str(path)))

    def open(self, path, mode="rb"):
        return open(_strip_file_scheme(str(path)), mode)

    def glob(self, pattern):
        import glob

        return sorted(glob.glob(_strip_file_scheme(str(pattern))))

    def makedirs(self, path, exist_ok=True):
        os.makedirs(_strip_file_scheme(str(path)), exist_ok=exist_ok)

    def ls(self, path, detail=False):
        p = _strip_file_scheme(str(path))
        return sorted(os.path.join(p, f) for f in os.listdir(p))

    def rm(self, path):
        os.remove(_strip_file_scheme(str(path)))


def _strip_file_scheme(path: str) -> str:
    return path[len("file://") :] if path.startswith("file://") else path


def _scheme(path: str) -> str:
    parsed = urllib.parse.urlparse(str(path))
    return parsed.scheme if len(parsed.scheme) > 1 else ""


def _get_fs(path):
    """Return a file-system object able to ``put/get/open/exists`` ``path``."""
    scheme = _scheme(str(path))
    if scheme in ("", "file"):
        return _LocalFS()
    try:
        import fsspec
    except ImportError as exc:  # pragma: no cover - optional dependency
        raise ImportError(f"fsspec is required for '{scheme}://' paths") from exc
    return fsspec.filesystem(scheme)


def _download_cached(path: str, recursive: bool = False, local_cache_path: str | None = None) -> str:
    """Return a local path for ``path``; remote objects are cached by URL hash."""
    path = str(path)
    scheme = _scheme(path)
    if scheme in ("", "file"):
        return _strip_file_scheme(path)
    cache = local_cache_path or _cache_dir()
    target = os.path.join(cache, hashlib.sha256(path.encode()).hexdigest())
    if os.path.exists(target):
        return target
    tmp = target + f".tmp{os.getpid()}"
    if scheme in ("http", "https"):
        with urllib.request.urlopen(path) as resp, open(tmp, "wb") as out:  # noqa: S310
            shutil.copyfileobj(resp, out)
    elif scheme == "ngc":
        raise NotImplementedError("NGC downloads need network access and an NGC_API_KEY")
    else:
        fs = _get_fs(path)
        fs.get(path, tmp, recursive=recursive) if recursive else fs.get(path, tmp)
    os.replace(tmp, target)
    return target


class Package:
    """A directory-like bundle of files, possibly remote.

    ``Package(root, seperator="/")``; ``get(relative)`` returns a local path.
    """

    def __init__(self, root: str, seperator: str = "/"):
        self.root = root
        self.seperator = seperator

    def get(self, path: str, recursive: bool = False) -> str:
        return _download_cached(self._fullpath(path), recursive=recursive)

    def _fullpath(self, path: str) -> str:
        return self.root + self.seperator + path

    def __repr__(self):
        return f"Package(root={self.root!r})"

"""File-system helpers: local / fsspec back ends, download cache, ``Package``.

Parity: ``physicsnemo/core/filesystem.py`` — ``_get_fs`` (``:50-54``),
``_download_cached`` with a sha256-of-URL cache directory under
``$LOCAL_CACHE`` or ``~/.cache/physicsnemo`` (``:198-307``) and ``Package``
(``:310-346``), plus the SHA-256 digest check (``_file_sha256``,
``_validate_checksum``, ``_install_in_cache`` at ``:155-196``): a download is
staged beside its cache entry, verified, and only then renamed into place.
``fsspec`` / ``s3fs`` / ``requests`` are optional here: plain paths, ``file://``
and ``http(s)://`` URLs work with the standard library alone; ``s3://``,
``msc://`` and other protocols go through fsspec when it is installed.
"""
from __future__ import annotations

import hashlib
import logging
import os
import re
import shutil
import tempfile
import urllib.parse
import urllib.request
import warnings
from pathlib import Path

logger = logging.getLogger(__name__)


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


_SHA256_HEX = re.compile(r"[0-9a-fA-F]{64}")


def _file_sha256(path) -> str:
    """Hex SHA-256 of a file, read in 1 MiB pieces."""
    h = hashlib.sha256()
    with open(path, "rb") as f:
        while True:
            block = f.read(1 << 20)
            if not block:
                break
            h.update(block)
    return h.hexdigest()


def _check_digest_format(checksum: str) -> None:
    if not isinstance(checksum, str) or _SHA256_HEX.fullmatch(checksum) is None:
        raise ValueError("checksum must be a 64-character SHA-256 hex digest")


def _validate_checksum(path, checksum: str) -> None:
    """Raise ``ValueError`` unless the file's SHA-256 equals ``checksum``."""
    _check_digest_format(checksum)
    got = _file_sha256(path)
    if got.lower() != checksum.lower():
        raise ValueError(f"Checksum mismatch for {path}: expected {checksum}, got {got}")


def _install_in_cache(fetch, target: str, checksum: str | None) -> None:
    """Run ``fetch(tmp)`` into a sibling of ``target`` and rename it into place.

    The rename happens only after the optional digest check, so a reader of the
    shared cache sees either the previous file or a complete verified one.
    """
    fd, tmp = tempfile.mkstemp(dir=os.path.dirname(target) or ".", prefix=os.path.basename(target) + ".")
    os.close(fd)
    try:
        fetch(tmp)
        if checksum is not None:
            _validate_checksum(tmp, checksum)
        os.replace(tmp, target)
    finally:
        if os.path.exists(tmp):
            os.remove(tmp)


def _fetch_http(url: str, dest: str, timeout: float = 5.0) -> None:
    secure = url.startswith("https://")
    with urllib.request.urlopen(url, timeout=timeout) as resp, open(dest, "wb") as out:  # noqa: S310
        final = getattr(resp, "url", None) or resp.geturl()
        if secure and _scheme(final) != "https":
            raise ValueError("HTTPS download redirected to a non-HTTPS URL")
        shutil.copyfileobj(resp, out)


def _download_cached(
    path: str,
    recursive: bool = False,
    local_cache_path: str | None = None,
    checksum: str | None = None,
) -> str:
    """Return a local path for ``path``; remote objects are cached by URL hash.

    ``checksum`` (SHA-256 hex) is verified for single files: local paths are
    checked in place, a cached copy that fails the check is fetched again, and
    a download that fails it never enters the cache.
    """
    path = str(path)
    scheme = _scheme(path)
    if checksum is not None:
        if recursive:
            raise ValueError("checksum verification is only supported for individual files")
        _check_digest_format(checksum)
        if scheme == "ngc" and path.endswith(".zip"):
            raise ValueError("checksum verification is not supported for automatically extracted NGC archives")
    if scheme in ("", "file"):
        local = _strip_file_scheme(path)
        if checksum is not None:
            _validate_checksum(local, checksum)
        return local
    cache = str(local_cache_path) if local_cache_path else _cache_dir()
    os.makedirs(cache, exist_ok=True)
    target = os.path.join(cache, hashlib.sha256(path.encode()).hexdigest())
    if os.path.exists(target):
        if checksum is None:
            return target
        try:
            _validate_checksum(target, checksum)
            return target
        except ValueError:
            logger.warning("Refetching cached file with an unexpected checksum: %s", path)
    if scheme == "http":
        warnings.warn(
            "Downloading over plain HTTP; prefer HTTPS. A checksum can verify file integrity.",
            UserWarning,
            stacklevel=2,
        )
    if scheme in ("http", "https"):
        _install_in_cache(lambda tmp: _fetch_http(path, tmp), target, checksum)
    elif scheme == "ngc":
        raise NotImplementedError("NGC downloads need network access and an NGC_API_KEY")
    else:
        fs = _get_fs(path)  # s3://, msc:// and any other fsspec protocol
        if recursive:
            fs.get(path, target, recursive=True)
        else:
            _install_in_cache(lambda tmp: fs.get(path, tmp), target, checksum)
    return target


class Package:
    """A directory-like bundle of files, possibly remote.

    ``Package(root, seperator="/")``; ``get(relative)`` returns a local path.
    """

    def __init__(self, root: str, seperator: str = "/"):
        self.root = root
        self.seperator = seperator

    def get(self, path: str, recursive: bool = False, checksum: str | None = None) -> str:
        return _download_cached(self._fullpath(path), recursive=recursive, checksum=checksum)

    def _fullpath(self, path: str) -> str:
        return self.root + self.seperator + path

    def __repr__(self):
        return f"Package(root={self.root!r})"

"""Download cache, digest verification and ``Package`` (CPU only).

Mirrors the coverage of the reference's ``test/core/test_filesystem.py``:
local paths, ``file://`` URLs, an HTTP server on the loopback interface and an
in-memory fsspec protocol stand in for the remote back ends.
"""
import hashlib
import http.server
import os
import threading

import pytest

from physicsnemo_b200.core import filesystem as fsmod


def _digest(data: bytes) -> str:
    return hashlib.sha256(data).hexdigest()


@pytest.fixture()
def http_root(tmp_path):
    root = tmp_path / "www"
    root.mkdir()

    class Quiet(http.server.SimpleHTTPRequestHandler):
        def __init__(self, *a, **k):
            super().__init__(*a, directory=str(root), **k)

        def log_message(self, *a):
            pass

    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), Quiet)
    t = threading.Thread(target=srv.serve_forever, daemon=True)
    t.start()
    yield root, f"http://127.0.0.1:{srv.server_address[1]}"
    srv.shutdown()
    srv.server_close()


def test_local_path_and_file_url_checksum(tmp_path):
    f = tmp_path / "a.bin"
    f.write_bytes(b"abc" * 1000)
    good = _digest(b"abc" * 1000)
    assert fsmod._file_sha256(f) == good
    assert fsmod._download_cached(str(f), checksum=good) == str(f)
    assert fsmod._download_cached(f"file://{f}", checksum=good.upper()) == str(f)
    with pytest.raises(ValueError, match="Checksum mismatch"):
        fsmod._download_cached(str(f), checksum="0" * 64)
    with pytest.raises(ValueError, match="64-character"):
        fsmod._download_cached(str(f), checksum="abc")
    with pytest.raises(ValueError, match="individual files"):
        fsmod._download_cached(str(f), recursive=True, checksum=good)
    with pytest.raises(ValueError, match="NGC archives"):
        fsmod._download_cached("ngc://models/org/m@1/w.zip", checksum=good)


def test_http_download_cache_and_refetch(http_root, tmp_path):
    root, base = http_root
    (root / "w.bin").write_bytes(b"first")
    cache = tmp_path / "cache"
    url = base + "/w.bin"
    with pytest.warns(UserWarning, match="plain HTTP"):
        p = fsmod._download_cached(url, local_cache_path=str(cache), checksum=_digest(b"first"))
    assert open(p, "rb").read() == b"first"
    assert os.path.basename(p) == hashlib.sha256(url.encode()).hexdigest()
    # a second call is served from the cache although the origin has changed
    (root / "w.bin").write_bytes(b"second")
    assert open(fsmod._download_cached(url, local_cache_path=str(cache)), "rb").read() == b"first"
    # a stale cached copy fails its digest and is replaced by a verified download
    with pytest.warns(UserWarning):
        p2 = fsmod._download_cached(url, local_cache_path=str(cache), checksum=_digest(b"second"))
    assert p2 == p and open(p, "rb").read() == b"second"
    # a download that fails the check never replaces the cached file, and leaves no temp file
    with pytest.warns(UserWarning), pytest.raises(ValueError, match="Checksum mismatch"):
        fsmod._download_cached(url, local_cache_path=str(cache), checksum="1" * 64)
    assert open(p, "rb").read() == b"second"
    assert sorted(os.listdir(cache)) == [os.path.basename(p)]


def test_fsspec_protocol_and_package(tmp_path, monkeypatch):
    fsspec = pytest.importorskip("fsspec")
    mem = fsspec.filesystem("memory")
    mem.pipe("/bundle/x/weights.bin", b"payload")
    monkeypatch.setenv("LOCAL_CACHE", str(tmp_path / "c"))
    pkg = fsmod.Package("memory://bundle", seperator="/")
    p = pkg.get("x/weights.bin", checksum=_digest(b"payload"))
    assert open(p, "rb").read() == b"payload"
    assert os.path.dirname(p) == str(tmp_path / "c")
    with pytest.raises(ValueError, match="Checksum mismatch"):
        fsmod.Package("memory://bundle").get("x/weights.bin", checksum="2" * 64)
    assert open(p, "rb").read() == b"payload"


def test_install_in_cache_cleans_up_after_failed_fetch(tmp_path):
    target = tmp_path / "t"

    def boom(tmp):
        open(tmp, "wb").write(b"partial")
        raise RuntimeError("link dropped")

    with pytest.raises(RuntimeError):
        fsmod._install_in_cache(boom, str(target), None)
    assert os.listdir(tmp_path) == []

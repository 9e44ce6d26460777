"""Loader / builder of the in-tree sm_100a kernel library ``libpnm_b200.so``.

The library is plain C ABI (see ``csrc/pnm_api.h``) bound through ``ctypes``: every
call passes raw device pointers and the current CUDA stream.  ``build()`` compiles the
single translation unit ``csrc/pnm_lib.cu`` with
``nvcc -gencode arch=compute_100a,code=sm_100a`` (cross-compiles without a GPU).
On a machine with a CUDA device a missing library is an error, never a silent
fallback.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import threading
from pathlib import Path

_PKG_DIR = Path(__file__).resolve().parents[1]
_REPO = _PKG_DIR.parent
_SRC_DIR = _REPO / "csrc"
_LIB_DIR = _PKG_DIR / "lib"
_LIB_PATH = _LIB_DIR / "libpnm_b200.so"
_lock = threading.Lock()
_lib = None
_load_error: str | None = None

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def lib_path() -> Path:
    return _LIB_PATH


def _sources():
    return sorted(list(_SRC_DIR.glob("*.cu")) + list(_SRC_DIR.glob("*.cuh")) + list(_SRC_DIR.glob("*.h")))


def needs_build() -> bool:
    if not _LIB_PATH.exists():
        return True
    built = _LIB_PATH.stat().st_mtime
    return any(s.stat().st_mtime > built for s in _sources())


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the kernel library in-tree; returns the path of the ``.so``."""
    if not _SRC_DIR.exists():
        raise FileNotFoundError(f"kernel sources not found at {_SRC_DIR}")
    if not force and not needs_build():
        return _LIB_PATH
    _LIB_DIR.mkdir(parents=True, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    tmp_out = _LIB_DIR / f".libpnm_b200.{os.getpid()}.so.tmp"     # built aside, then moved into place in one step
    cmd = [nvcc, *NVCC_FLAGS, "-o", str(tmp_out), *[str(p) for p in sorted(_SRC_DIR.glob("*.cu"))]]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        if tmp_out.exists():
            tmp_out.unlink()
        raise RuntimeError(f"nvcc failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp_out, _LIB_PATH)
    if verbose:
        print(proc.stderr)
    return _LIB_PATH


def _declare(lib):
    c = ctypes
    vp, i32, i64, f32 = c.c_void_p, c.c_int, c.c_longlong, c.c_float
    sigs = {
        "pnm_version": ([], i32),
        "pnm_num_sms": ([], i32),
        "pnm_get_error": ([], i32),
        "pnm_reset_error": ([], i32),
        "pnm_gemm_tn": ([vp, i32, vp, i32, vp, i32, vp, i32, vp, i32, vp, i32, vp, i32, i32, i32, i32, i32, i32, vp, vp, vp,
                         i32, i32, i32, i32, i32, vp], i32),
        "pnm_gemm_nt": ([vp, i32, vp, i32, vp, i32, vp, i32, i32, i32, i32, vp], i32),
        "pnm_gemm_tn_stacked": ([vp, i32, vp, i32, vp, i32, vp, i32, i32, i32, i32, i32, vp, i32, i32, i32, vp], i32),
        "pnm_gemm_nt_stacked": ([vp, i32, vp, i32, vp, vp, i32, i32, i32, i32, i32, vp], i32),
        "pnm_layernorm_fwd": ([vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, f32, vp], i32),
        "pnm_gather_rows": ([vp, i32, vp, vp, vp, i32, i64, i32, vp], i32),
        "pnm_segment_sum": ([vp, i32, vp, vp, vp, i32, i64, i32, i32, i32, vp], i32),
        "pnm_layernorm_bwd_scratch_floats": ([i64, i32], i64),
        "pnm_layernorm_bwd": ([vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, vp], i32),
    }
    for name, (argtypes, restype) in sigs.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue
        fn.argtypes = argtypes
        fn.restype = restype
    # optional symbols (added by later kernels) declare themselves in their wrappers


def load(required: bool = False):
    """Return the ctypes handle (or ``None`` when unavailable and not required)."""
    global _lib, _load_error
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        try:
            if not _LIB_PATH.exists():
                raise FileNotFoundError(f"{_LIB_PATH} not built; run `python -c 'import __graft_entry__ as g; g.build()'`")
            lib = ctypes.CDLL(str(_LIB_PATH))
            _declare(lib)
            _lib = lib
        except Exception as exc:  # noqa: BLE001
            _load_error = str(exc)
            if required:
                raise RuntimeError(f"sm_100a kernel library unavailable: {exc}") from exc
            return None
    return _lib


def available() -> bool:
    return load() is not None


def load_error() -> str | None:
    return _load_error

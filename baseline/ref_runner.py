"""Import the unmodified reference package from ``baseline/_ref`` for the reference arm.

The reference is pure Python; the directory holds an untouched copy of its ``physicsnemo``
package.  Some of its import-time dependencies are third-party packages that are not part
of the reference and are not installed in this image (warp, tensordict, treelib, s3fs,
...).  They are only needed by code paths the benchmark does not execute, so for the
duration of the reference arm they are replaced by inert stub modules; nothing of the
reference itself is patched and none of this repository's code runs on that path.
"""
from __future__ import annotations

import importlib
import os
import importlib.abc
import importlib.machinery
import importlib.util
import sys
import types
from unittest import mock

_OPTIONAL_THIRD_PARTY = (
    "warp", "tensordict", "treelib", "s3fs", "nvtx", "termcolor", "hydra", "omegaconf", "timm", "h5py", "onnx",
    "cftime", "mlflow", "wandb", "jaxtyping", "fsspec", "onnxruntime", "netCDF4", "zarr", "vtk", "pyvista",
    "torch_geometric", "torch_scatter", "transformer_engine", "apex", "natten", "cuml", "cupy", "nvfuser", "dgl",
    "line_profiler", "xarray", "tqdm_joblib", "einops_exts", "importlib_metadata", "rmm", "tensorstore", "stl",
    "shapely", "trimesh", "pylibraft", "cuvs", "moviepy", "numba", "scikit_image", "skimage", "matplotlib",
)


class _StubModule(types.ModuleType):
    """Module whose every attribute is a permissive mock; sub-modules resolve too."""

    def __getattr__(self, name):
        if name.startswith("__") and name.endswith("__"):
            raise AttributeError(name)
        value = mock.MagicMock(name=f"{self.__name__}.{name}")
        setattr(self, name, value)
        return value


class _StubFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def __init__(self, roots):
        self.roots = set(roots)

    def find_spec(self, fullname, path=None, target=None):
        root = fullname.split(".")[0]
        if root in self.roots:
            return importlib.machinery.ModuleSpec(fullname, self, is_package=True)
        return None

    def create_module(self, spec):
        mod = _StubModule(spec.name)
        mod.__path__ = []
        mod.__version__ = "0.0.0"
        return mod

    def exec_module(self, module):
        if module.__name__ == "tensordict":
            # the reference tests ``isinstance(x, TensorDict)`` on plain tensors: the names must be real classes
            for n in ("TensorDict", "TensorDictBase", "TensorClass", "LazyStackedTensorDict"):
                setattr(module, n, type(n, (dict,), {}))
            module.tensorclass = lambda *a, **k: (a[0] if a and isinstance(a[0], type) else (lambda cls: cls))
        if module.__name__ == "jaxtyping":
            # type-annotation helpers used as ``Float[torch.Tensor, "..."]``
            class _Sub:
                def __class_getitem__(cls, item):
                    return item[0] if isinstance(item, tuple) else item

            for n in ("Float", "Int", "Bool", "Shaped", "Num", "Integer", "Complex", "Inexact", "Real", "UInt8"):
                setattr(module, n, _Sub)
            module.jaxtyped = lambda *a, **k: (a[0] if a and callable(a[0]) else (lambda f: f))


def import_reference(ref_dir: str):
    """Put ``ref_dir`` first on ``sys.path``, stub missing third-party packages, import."""
    missing = []
    for name in _OPTIONAL_THIRD_PARTY:
        try:
            if importlib.util.find_spec(name) is None:
                missing.append(name)
        except (ImportError, ValueError):
            missing.append(name)
    if missing:
        sys.meta_path.append(_StubFinder(missing))
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    loaded = sys.modules.get("physicsnemo")
    if loaded is not None and str(getattr(loaded, "__file__", "")).startswith(os.path.abspath(ref_dir)):
        return loaded          # already the reference: keep its state (its DistributedManager holds the process group)
    for key in [k for k in sys.modules if k == "physicsnemo" or k.startswith("physicsnemo.")]:
        del sys.modules[key]
    return importlib.import_module("physicsnemo")

"""``Module``: the base class of every model, with ``.mdlus`` checkpoints.

Parity with ``physicsnemo/core/module.py:87-1321``:

* constructor arguments are captured when the object is created so that a
  checkpoint can rebuild the model (``__new__`` at ``:193-224``);
* ``save`` writes an uncompressed zip (or a legacy tar) holding ``model.pt``
  (``torch.save`` of the state dict), ``args.json`` and ``metadata.json``
  (``:440-635``); nested ``Module`` arguments are hoisted to the top level of
  ``args.json`` under keys ``__physicsnemo.Module__.<arg>[.<arg>...]``;
* ``from_checkpoint`` rebuilds (class lookup: caller class, registry, import
  path, with ``modulus.`` paths mapped to ``physicsnemo``), applies permitted
  overrides and loads the weights (``:794-1117``);
* ``from_torch`` wraps a plain ``torch.nn.Module`` class (``:1119-1303``).

The on-disk layout is byte-compatible in structure: a file written here opens
with the reference and vice versa (module paths ``physicsnemo.*`` and
``physicsnemo_b200.*`` are mapped onto each other when a class is looked up).
"""
from __future__ import annotations

import importlib
import inspect
import io
import json
import keyword
import logging
import os
import tarfile
import tempfile
import zipfile
from pathlib import Path
from typing import Any, Dict, Optional, Set, Union

import torch

from .meta import ModelMetaData
from .registry import ModelRegistry
from .filesystem import _download_cached, _get_fs
from .version_check import get_physicsnemo_pkg_info

_NESTED = "__physicsnemo.Module__"
_PKG = "physicsnemo_b200"
_FILES = ("model.pt", "args.json", "metadata.json")


def _drop_device_buffer_keys(module, incompatible_keys):
    """Old checkpoints stored the zero-size ``device_buffer``; ignore it."""
    for bucket in (incompatible_keys.missing_keys, incompatible_keys.unexpected_keys):
        for key in [k for k in bucket if k.split(".")[-1] == "device_buffer"]:
            bucket.remove(key)


def _candidate_module_paths(path: str):
    """Module paths to try for a class recorded at ``path`` in a checkpoint."""
    seen = []
    for p in (
        path,
        path.replace("modulus.", "physicsnemo.", 1) if path.startswith("modulus.") else path,
    ):
        for q in (p, p.replace("physicsnemo.", _PKG + ".", 1) if p.startswith("physicsnemo.") else p):
            if q not in seen:
                seen.append(q)
    return seen


def _flatten_nested(root: "Module"):
    """Return (args, metadata_extra): nested Module args replaced by placeholders."""
    args: Dict[str, Any] = {k: v for k, v in root._args.items()}
    meta_extra: Dict[str, Any] = {}

    def visit(owner: "Module", slot: str, prefix: str):
        record = args[slot] if slot else args
        flat = dict(record["__args__"])
        for name, value in flat.items():
            if isinstance(value, Module):
                key = f"{prefix or _NESTED}.{name}"
                args[key] = dict(value._args)
                flat[name] = key
                meta_extra[f"{key}.mdlus_file_version"] = value.__model_checkpoint_version__
                visit(value, key, key)
            elif isinstance(value, torch.nn.Module):
                raise TypeError(
                    f"Argument '{name}' of {type(owner).__name__} is a plain torch "
                    "module; wrap its class with Module.from_torch before saving."
                )
        record = dict(record)
        record["__args__"] = flat
        if slot:
            args[slot] = record
        else:
            args.update(record)

    visit(root, "", "")
    return args, meta_extra


class Module(torch.nn.Module):
    """Drop-in ``torch.nn.Module`` with argument capture and ``.mdlus`` I/O.

    Constructor arguments must be JSON serialisable, or themselves ``Module``
    instances (arbitrarily nested).
    """

    _file_extension = ".mdlus"
    __model_checkpoint_version__ = "0.1.0"
    __supported_model_checkpoint_version__: Dict[str, str] = {}
    _overridable_args: Set[str] = set()

    def __new__(cls, *args, **kwargs):
        obj = super().__new__(cls)
        sig = inspect.signature(cls.__init__)
        bound = sig.bind_partial(None, *args, **kwargs)
        bound.apply_defaults()
        captured: Dict[str, Any] = {}
        for name, value in bound.arguments.items():
            if name == "self":
                continue
            if sig.parameters[name].kind is inspect.Parameter.VAR_KEYWORD:
                captured.update(value)
            else:
                captured[name] = value
        obj._args = {
            "__name__": cls.__name__,
            "__module__": cls.__module__,
            "__args__": captured,
        }
        return obj

    def __init__(self, meta: Union[ModelMetaData, None] = None):
        super().__init__()
        self.meta = meta
        self.register_buffer("device_buffer", torch.empty(0), persistent=False)
        self.logger = logging.getLogger("core.module")
        if not self.logger.handlers:
            handler = logging.StreamHandler()
            handler.setFormatter(
                logging.Formatter("[%(asctime)s - %(levelname)s] %(message)s", datefmt="%H:%M:%S")
            )
            self.logger.addHandler(handler)
        self.logger.setLevel(logging.WARNING)
        self.register_load_state_dict_post_hook(_drop_device_buffer_keys)

    def __init_subclass__(cls, *, register: bool = False, **kwargs):
        super().__init_subclass__(**kwargs)
        if register:
            ModelRegistry().register(cls, cls.__name__)

    # ------------------------------------------------------------------ misc
    def debug(self):
        """Switch the model logger to debug verbosity."""
        self.logger.handlers.clear()
        handler = logging.StreamHandler()
        handler.setFormatter(
            logging.Formatter(
                f"[%(asctime)s - %(levelname)s - {self.meta.name if self.meta else ''}] %(message)s",
                datefmt="%Y-%m-%d %H:%M:%S",
            )
        )
        self.logger.addHandler(handler)
        self.logger.setLevel(logging.DEBUG)

    @property
    def device(self) -> torch.device:
        """Device of the model (tracked through a zero-size buffer)."""
        return self.device_buffer.device

    def num_parameters(self) -> int:
        """Total number of learnable parameter elements."""
        return sum(p.numel() for p in self.parameters())

    # ------------------------------------------------------- backward compat
    @classmethod
    def _backward_compat_arg_mapper(cls, version: str, args: Dict[str, Any]) -> Dict[str, Any]:
        """Hook for subclasses: map constructor args of an older checkpoint version."""
        return args

    @classmethod
    def _override_args(cls, args: Dict[str, Any], override: Dict[str, Any]) -> None:
        for key, value in override.items():
            if key not in cls._overridable_args:
                raise ValueError(
                    f"Argument '{key}' cannot be overridden for {cls.__name__}; "
                    f"overridable: {sorted(cls._overridable_args)}"
                )
            args[key] = value

    # ---------------------------------------------------------- construction
    @classmethod
    def _lookup_class(cls, record: Dict[str, Any]) -> type:
        name, path = record["__name__"], record["__module__"]
        if cls.__name__ == name and cls is not Module:
            return cls
        registry = ModelRegistry()
        if name in registry.list_models():
            try:
                return registry.factory(name)
            except Exception:
                pass
        last_err = None
        for mod_path in _candidate_module_paths(path):
            try:
                return getattr(importlib.import_module(mod_path), name)
            except (ImportError, AttributeError) as exc:
                last_err = exc
        raise AttributeError(
            f"Cannot locate class {name} (recorded module {path}): {last_err}"
        )

    @classmethod
    def instantiate(cls, arg_dict: Dict[str, Any]) -> "Module":
        """Build a model from ``{"__name__", "__module__", "__args__"}``."""
        klass = cls._lookup_class(arg_dict)
        return klass(**arg_dict["__args__"])

    # ------------------------------------------------------------------ save
    def save(
        self,
        file_name: Path | str | None = None,
        verbose: bool = False,
        legacy_format: bool = False,
        _state_dict: dict | None = None,
    ) -> None:
        """Write the model to a ``.mdlus`` file (zip by default, tar if legacy)."""
        if file_name is not None:
            file_name = str(file_name)
            if not file_name.endswith(self._file_extension):
                raise ValueError(f"File name must end with {self._file_extension} extension")
        else:
            file_name = f"{type(self).__name__}{self._file_extension}"

        pkg = get_physicsnemo_pkg_info()
        metadata = {
            "physicsnemo_version": pkg["version"],
            "mdlus_file_version": self.__model_checkpoint_version__,
        }
        if verbose:
            metadata["git_hash"] = pkg["git_hash"]
        args, extra = _flatten_nested(self)
        metadata.update(extra)

        state = _state_dict if _state_dict is not None else self.state_dict()
        blob = io.BytesIO()
        torch.save(state, blob)
        payload = {
            "model.pt": blob.getvalue(),
            "args.json": json.dumps(args).encode(),
            "metadata.json": json.dumps(metadata).encode(),
        }
        fs = _get_fs(file_name)
        fd, tmp_path = tempfile.mkstemp(suffix=".tar" if legacy_format else ".zip")
        os.close(fd)
        try:
            if legacy_format:
                with tarfile.open(tmp_path, "w") as tar:
                    for member, data in payload.items():
                        info = tarfile.TarInfo(member)
                        info.size = len(data)
                        tar.addfile(info, io.BytesIO(data))
            else:
                with zipfile.ZipFile(tmp_path, "w", zipfile.ZIP_STORED) as archive:
                    for member, data in payload.items():
                        archive.writestr(member, data)
            fs.put(tmp_path, file_name)
        finally:
            if os.path.exists(tmp_path):
                os.remove(tmp_path)

    # ------------------------------------------------------------------ read
    @staticmethod
    def _detect_checkpoint_format(file_path: str) -> str:
        """``"tar"`` or ``"zip"``; tar is probed first like the reference."""
        if tarfile.is_tarfile(file_path):
            return "tar"
        if zipfile.is_zipfile(file_path):
            return "zip"
        raise IOError(f"{file_path} is neither a tar nor a zip .mdlus checkpoint")

    @staticmethod
    def _read_members(local_path: str, names=_FILES) -> Dict[str, bytes]:
        fmt = Module._detect_checkpoint_format(local_path)
        out: Dict[str, bytes] = {}
        if fmt == "zip":
            with zipfile.ZipFile(local_path, "r") as archive:
                present = set(archive.namelist())
                for n in names:
                    if n in present:
                        out[n] = archive.read(n)
        else:
            with tarfile.open(local_path, "r") as tar:
                for member in tar.getmembers():
                    base = os.path.basename(member.name)
                    # refuse anything that is not a plain file at the top level
                    if not member.isfile() or member.name.startswith(("/", "..")) or ".." in Path(member.name).parts:
                        continue
                    if base in names:
                        out[base] = tar.extractfile(member).read()
        return out

    @staticmethod
    def _check_checkpoint(local_path: str) -> None:
        members = Module._read_members(local_path)
        for n in _FILES:
            if n not in members:
                raise IOError(f"Checkpoint is missing '{n}'")

    def load(
        self,
        file_name: Path | str,
        map_location: Union[None, str, torch.device] = None,
        strict: bool = True,
    ) -> None:
        """Load weights from a ``.mdlus`` file into this (already built) model."""
        file_name = str(file_name)
        local = _download_cached(file_name)
        if not Path(local).exists():
            raise IOError(f"Model checkpoint {file_name} not found")
        members = self._read_members(local)
        if "model.pt" not in members:
            raise IOError("Checkpoint is missing 'model.pt'")
        device = map_location if map_location is not None else self.device
        state = torch.load(io.BytesIO(members["model.pt"]), map_location=device, weights_only=False)
        result = self.load_state_dict(state, strict=strict)
        if result.missing_keys:
            self.logger.warning(f"missing keys: {result.missing_keys}")
        if result.unexpected_keys:
            self.logger.warning(f"unexpected keys: {result.unexpected_keys}")

    @classmethod
    def from_checkpoint(
        cls,
        file_name: Path | str,
        override_args: Optional[Dict[str, Any]] = None,
        strict: bool = True,
    ) -> "Module":
        """Rebuild a model from a ``.mdlus`` file and load its weights.

        ``override_args`` may replace constructor arguments listed in the
        class attribute ``_overridable_args``; nested modules use dotted keys
        (``"submodule.arg"``).
        """
        override_args = dict(override_args or {})
        for key in override_args:
            if not isinstance(key, str):
                raise ValueError(f"override_args keys must be strings, got {type(key)}")
            parts = key.split(".")
            if not all(p and p.isidentifier() and not keyword.iskeyword(p) for p in parts):
                raise ValueError(f"Key {key} in override_args is not of the form a.b.c")

        file_name = str(file_name)
        local = _download_cached(file_name)
        if not Path(local).exists():
            raise IOError(f"Model checkpoint {file_name} not found")
        members = cls._read_members(local)
        for n in _FILES:
            if n not in members:
                raise IOError(f"Checkpoint is missing '{n}'")
        args = json.loads(members["args.json"])
        metadata = json.loads(members["metadata.json"])

        def build(caller: type, slot: str) -> "Module":
            record = args if slot == "" else args[slot]
            version_key = "mdlus_file_version" if slot == "" else f"{slot}.mdlus_file_version"
            version = metadata.get(version_key, caller.__model_checkpoint_version__)
            klass = caller._lookup_class(record)
            ctor_args = dict(record["__args__"])
            if version != klass.__model_checkpoint_version__:
                if version in klass.__supported_model_checkpoint_version__:
                    klass_logger = logging.getLogger("core.module")
                    klass_logger.warning(klass.__supported_model_checkpoint_version__[version])
                    ctor_args = klass._backward_compat_arg_mapper(version, ctor_args)
                else:
                    raise IOError(
                        f"Model checkpoint version {version} is not compatible with "
                        f"{klass.__name__} version {klass.__model_checkpoint_version__}"
                    )
            # nested modules first
            for name, value in list(ctor_args.items()):
                if isinstance(value, str) and value.startswith(_NESTED) and value in args:
                    ctor_args[name] = build(Module, value)
            # overrides addressed to this level
            depth_prefix = "" if slot == "" else slot[len(_NESTED) + 1 :] + "."
            here = {}
            for key, value in override_args.items():
                if key.startswith(depth_prefix):
                    rest = key[len(depth_prefix) :]
                    if "." not in rest:
                        here[rest] = value
            if here:
                klass._override_args(ctor_args, here)
                for rest in here:
                    consumed.add(depth_prefix + rest)
            return klass(**ctor_args)

        consumed: set = set()
        model = build(cls, "")
        leftover = set(override_args) - consumed
        if leftover:
            raise ValueError(f"override_args keys {sorted(leftover)} match no module argument")

        state = torch.load(io.BytesIO(members["model.pt"]), map_location=model.device, weights_only=False)
        result = model.load_state_dict(state, strict=strict)
        if result.missing_keys:
            model.logger.warning(f"missing keys: {result.missing_keys}")
        if result.unexpected_keys:
            model.logger.warning(f"unexpected keys: {result.unexpected_keys}")
        return model

    # ------------------------------------------------------------ from_torch
    @staticmethod
    def from_torch(
        torch_model_class: type,
        meta: ModelMetaData | None = None,
        name: str | None = None,
        register: bool = False,
    ) -> type:
        """Make a ``Module`` subclass whose ``inner_model`` is ``torch_model_class``.

        The generated class has the same constructor signature as the wrapped
        class, forwards ``forward`` to it, and can be saved / re-loaded when it
        is registered (``register=True``).
        """
        if not (isinstance(torch_model_class, type) and issubclass(torch_model_class, torch.nn.Module)):
            raise TypeError("from_torch expects a torch.nn.Module subclass")
        name = name or torch_model_class.__name__
        init_sig = inspect.signature(torch_model_class.__init__)

        def __init__(self, *args, **kwargs):
            Module.__init__(self, meta=meta)
            self.inner_model = torch_model_class(*args, **kwargs)

        __init__.__signature__ = init_sig

        def forward(self, *args, **kwargs):
            return self.inner_model(*args, **kwargs)

        wrapped = type(
            name,
            (Module,),
            {
                "__init__": __init__,
                "forward": forward,
                "__module__": torch_model_class.__module__,
                "__doc__": torch_model_class.__doc__,
            },
        )
        if register:
            registry = ModelRegistry()
            if name in registry.list_models():
                try:
                    existing = registry.factory(name)
                except Exception:
                    existing = None
                if existing is not None and existing is not wrapped:
                    registry._table[name] = wrapped
            else:
                registry.register(wrapped, name)
        return wrapped

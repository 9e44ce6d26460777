"""``TensorDict``: the container every datapipe stage exchanges.

The reference depends on the ``tensordict`` package; when it is importable it is used as is.  Otherwise this
module provides the subset the datapipes need — an ordered mapping ``str → Tensor | TensorDict`` with a shared
``batch_size``, device moves (``non_blocking``), ``select`` / ``exclude`` / ``update``, nested keys, ``stack`` and
``cat``.
"""
from __future__ import annotations

from typing import Any, Iterable, Iterator, Mapping, Sequence

import torch

try:  # pragma: no cover - exercised only where the package exists
    from tensordict import TensorDict, is_tensor_collection  # type: ignore
except ImportError:

    class TensorDict(dict):  # type: ignore[no-redef]
        def __init__(self, source: Mapping[str, Any] | None = None, batch_size: Sequence[int] | None = None,
                     device: torch.device | str | None = None):
            super().__init__()
            self.batch_size = torch.Size(batch_size or [])
            self._device = torch.device(device) if device is not None else None
            for k, v in (source or {}).items():
                self[k] = v

        def __setitem__(self, key, value):
            if isinstance(key, tuple):
                if len(key) == 1:
                    key = key[0]
                else:
                    sub = dict.get(self, key[0])
                    if sub is None:
                        sub = TensorDict({}, batch_size=self.batch_size, device=self._device)
                        dict.__setitem__(self, key[0], sub)
                    sub[key[1:]] = value
                    return
            if isinstance(value, Mapping) and not isinstance(value, TensorDict):
                value = TensorDict(value, batch_size=self.batch_size, device=self._device)
            elif not isinstance(value, (torch.Tensor, TensorDict)):
                value = torch.as_tensor(value)
            if self._device is not None and isinstance(value, (torch.Tensor, TensorDict)) and _dev(value) != self._device:
                value = value.to(self._device)
            dict.__setitem__(self, key, value)

        def __getitem__(self, key):
            if isinstance(key, tuple):
                out = self
                for k in key:
                    out = dict.__getitem__(out, k)
                return out
            if isinstance(key, str):
                return dict.__getitem__(self, key)
            # tensor-style indexing of the batch dimensions
            return TensorDict({k: v[key] for k, v in self.items()}, device=self._device)

        @property
        def device(self):
            return self._device

        def to(self, device=None, non_blocking: bool = False, **kw):
            device = torch.device(device) if device is not None else None
            out = TensorDict({}, batch_size=self.batch_size, device=None)
            for k, v in self.items():
                dict.__setitem__(out, k, v.to(device, non_blocking=non_blocking, **kw) if device is not None else v.to(**kw))
            out._device = device if device is not None else self._device
            return out

        def keys(self, include_nested: bool = False, leaves_only: bool = False):  # type: ignore[override]
            if not include_nested:
                return dict.keys(self)
            return [k for k, _ in self._walk(leaves_only)]

        def values(self, include_nested: bool = False, leaves_only: bool = False):  # type: ignore[override]
            if not include_nested:
                return dict.values(self)
            return [v for _, v in self._walk(leaves_only)]

        def items(self, include_nested: bool = False, leaves_only: bool = False):  # type: ignore[override]
            if not include_nested:
                return dict.items(self)
            return list(self._walk(leaves_only))

        def _walk(self, leaves_only, prefix=()) -> Iterator:
            for k, v in dict.items(self):
                if isinstance(v, TensorDict):
                    if not leaves_only:
                        yield (prefix + (k,) if prefix else k), v
                    yield from v._walk(leaves_only, prefix + (k,))
                else:
                    yield (prefix + (k,) if prefix else k), v

        def select(self, *keys, strict: bool = True):
            missing = [k for k in keys if k not in self]
            if missing and strict:
                raise KeyError(f"keys {missing} not found in TensorDict with keys {list(self.keys())}")
            return TensorDict({k: self[k] for k in keys if k in self}, batch_size=self.batch_size, device=self._device)

        def exclude(self, *keys):
            return TensorDict({k: v for k, v in self.items() if k not in keys}, batch_size=self.batch_size, device=self._device)

        def clone(self, recurse: bool = True):
            return TensorDict({k: (v.clone() if recurse else v) for k, v in self.items()}, batch_size=self.batch_size,
                              device=self._device)

        def apply(self, fn):
            return TensorDict({k: (v.apply(fn) if isinstance(v, TensorDict) else fn(v)) for k, v in self.items()},
                              batch_size=self.batch_size, device=self._device)

        def pin_memory(self):
            return self.apply(lambda t: t.pin_memory())

        def update(self, other=None, **kw):  # type: ignore[override]
            for k, v in dict(other or {}, **kw).items():
                self[k] = v
            return self

        def rename_key_(self, old: str, new: str):
            dict.__setitem__(self, new, dict.pop(self, old))
            return self

        def to_dict(self):
            return {k: (v.to_dict() if isinstance(v, TensorDict) else v) for k, v in self.items()}

        def __repr__(self):
            body = ", ".join(f"{k}: {tuple(v.shape) if isinstance(v, torch.Tensor) else v}" for k, v in self.items())
            return f"TensorDict({{{body}}}, batch_size={tuple(self.batch_size)}, device={self._device})"

    def is_tensor_collection(obj) -> bool:  # type: ignore[no-redef]
        return isinstance(obj, TensorDict)


def _dev(v):
    return v.device if isinstance(v, torch.Tensor) else v.device


def stack_tensordicts(items: Sequence["TensorDict"], dim: int = 0) -> "TensorDict":
    first = items[0]
    out = {}
    for k in first.keys():
        vals = [it[k] for it in items]
        out[k] = stack_tensordicts(vals, dim) if is_tensor_collection(vals[0]) else torch.stack(vals, dim=dim)
    return TensorDict(out, batch_size=[len(items)], device=first.device)


def cat_tensordicts(items: Sequence["TensorDict"], dim: int = 0) -> "TensorDict":
    first = items[0]
    out = {}
    for k in first.keys():
        vals = [it[k] for it in items]
        out[k] = cat_tensordicts(vals, dim) if is_tensor_collection(vals[0]) else torch.cat(vals, dim=dim)
    return TensorDict(out, device=first.device)

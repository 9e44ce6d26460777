"""One collective for many tensors.

Parity: ``physicsnemo/distributed/fused_all_reduce.py`` — pack leaves of a tensor / mapping /
sequence (sorted keys for mappings: deterministic order on every rank) into one buffer of the
promoted dtype (≥ fp32 for 16-bit floats; integer + float mixes are refused unless
``buffer_dtype`` is given), run **one** all-reduce, unpack into the caller's container type.
``async_op=True`` returns ``(container, work)`` whose ``work.wait()`` performs the deferred
unpack.  Without an initialised multi-rank group the call returns exact clones.
"""
from __future__ import annotations

import functools
from collections.abc import Mapping, Sequence

import torch
import torch.distributed as dist


class _FusedAllReduceWork:
    """Handle of an asynchronous fused all-reduce; ``wait()`` unpacks into the outputs."""

    def __init__(self, work=None, buffer=None, outputs=None, numels=None):
        self._work, self._buffer, self._outputs, self._numels = work, buffer, outputs, numels
        self._done = work is None

    def is_completed(self) -> bool:
        return self._done or (self._work is not None and self._work.is_completed())

    def wait(self) -> bool:
        if self._done:
            return True
        self._work.wait()
        offset = 0
        for out, n in zip(self._outputs, self._numels):
            out.copy_(self._buffer[offset:offset + n].reshape(out.shape))
            offset += n
        self._done = True
        self._buffer = None
        return True


def _flatten(obj, prefix=()):
    """Leaves of a (possibly nested) mapping / sequence in deterministic order."""
    if isinstance(obj, torch.Tensor):
        return [(prefix, obj)]
    if isinstance(obj, Mapping) or hasattr(obj, "keys") and hasattr(obj, "__getitem__") and not isinstance(obj, (str, bytes)):
        out = []
        for k in sorted(obj.keys(), key=str):
            out += _flatten(obj[k], prefix + (k,))
        return out
    if isinstance(obj, Sequence) and not isinstance(obj, (str, bytes)):
        out = []
        for i, v in enumerate(obj):
            out += _flatten(v, prefix + (i,))
        return out
    raise TypeError(f"fused_all_reduce cannot handle leaves of type {type(obj)}")


def _rebuild(template, values: dict, prefix=()):
    if isinstance(template, torch.Tensor):
        return values[prefix]
    if isinstance(template, Mapping) or hasattr(template, "keys") and hasattr(template, "__getitem__"):
        items = {k: _rebuild(template[k], values, prefix + (k,)) for k in template.keys()}
        if isinstance(template, dict):
            return type(template)(items) if type(template) is not dict else items
        try:  # TensorDict-like containers
            out = template.clone(recurse=False) if hasattr(template, "clone") else dict(items)
            for k, v in items.items():
                out[k] = v
            return out
        except Exception:
            return items
    seq = [_rebuild(v, values, prefix + (i,)) for i, v in enumerate(template)]
    if isinstance(template, tuple):
        return type(template)(*seq) if hasattr(template, "_fields") else tuple(seq)
    return seq


@torch.no_grad()
def _fused_reduce_tensors(tensors, *, op, group, buffer_dtype, device, async_op=False):
    if not tensors:
        return [], (_FusedAllReduceWork() if async_op else None)
    detached = [t.detach() for t in tensors]
    if buffer_dtype is not None:
        work_dtype = buffer_dtype
    else:
        work_dtype = functools.reduce(torch.promote_types, (t.dtype for t in detached))
        if work_dtype.is_floating_point:
            if any(not t.dtype.is_floating_point for t in detached):
                raise ValueError(
                    "fused_all_reduce would cast integer/bool leaves into a "
                    f"{work_dtype} buffer, silently corrupting large or index-like values. Reduce integer "
                    "leaves on their own, or pass buffer_dtype= to opt in to the cast."
                )
            if work_dtype.itemsize < 4:
                work_dtype = torch.float32
    if not (dist.is_available() and dist.is_initialized() and dist.get_world_size(group=group) > 1):
        return [t.clone() for t in detached], (_FusedAllReduceWork() if async_op else None)
    buffer_device = torch.device(device) if device is not None else detached[0].device
    flats = [t.reshape(-1).to(device=buffer_device, dtype=work_dtype) for t in detached]
    numels = [f.numel() for f in flats]
    buffer = torch.cat(flats)
    if async_op:
        outputs = [s.clone() for s in detached]
        work = dist.all_reduce(buffer, op=op, group=group, async_op=True)
        return outputs, _FusedAllReduceWork(work, buffer, outputs, numels)
    dist.all_reduce(buffer, op=op, group=group)
    reduced, offset = [], 0
    for src, n in zip(detached, numels):
        chunk = buffer[offset:offset + n].reshape(src.shape)
        reduced.append(chunk.to(device=src.device, dtype=src.dtype, copy=True))
        offset += n
    return reduced, None


@torch.no_grad()
def fused_all_reduce(tensors, *, op=dist.ReduceOp.SUM, group=None, buffer_dtype=None, device=None, async_op=False):
    """All-reduce every leaf of ``tensors`` with a single collective, preserving the container."""
    leaves = _flatten(tensors)
    reduced, work = _fused_reduce_tensors([t for _, t in leaves], op=op, group=group, buffer_dtype=buffer_dtype,
                                          device=device, async_op=async_op)
    values = {path: r for (path, _), r in zip(leaves, reduced)}
    out = _rebuild(tensors, values)
    return (out, work) if async_op else out

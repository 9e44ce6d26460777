"""Training checkpoints: model files + one training-state file per step index.

Parity: ``physicsnemo/utils/checkpoint.py`` — ``save_checkpoint`` (``:724-947``),
``load_checkpoint`` (``:950-1167``), ``load_model_weights`` (``:1170-1237``),
``get_checkpoint_dir`` (``:1495-1521``), file naming ``{Class}{id}.{mp_rank}.{epoch}.mdlus|.pt``
and ``checkpoint.{mp_rank}.{epoch}.pt`` with "next free / latest" index discovery
(``_get_checkpoint_filename`` ``:570-674``), unwrapping of DDP / ``torch.compile`` wrappers
(``:84-102, 677-721``), static-capture scaler states (``:929-930, 1156-1158``).

Models whose parameters are sharded (FSDP / DTensor / ShardTensor) are gathered to full
tensors collectively and written by rank 0 as a topology-agnostic file; on load rank 0
reads and the state is broadcast and re-sharded by ``load_state_dict`` of each rank.
The optimizer's per-parameter state (Adam moments, ...) of sharded parameters is gathered
the same way and re-distributed with the layout of the loading run's parameters.
A training-state file that cannot be read (truncated write) makes ``load_checkpoint``
fall back to the previous index, and the model files of that same index are loaded.
"""
from __future__ import annotations

import io
import logging
import os
import re
from pathlib import Path, PurePath
from typing import Any, Dict, List, Optional, Union

import torch
import torch.distributed as dist

from ..core.filesystem import _download_cached, _get_fs
from ..core.module import Module
from ..distributed.manager import DistributedManager

checkpoint_logging = logging.getLogger("checkpoint")


def _manager() -> DistributedManager:
    if not DistributedManager.is_initialized():
        checkpoint_logging.warning(
            "`DistributedManager` not initialized already. Initializing now, but this might lead to unexpected errors"
        )
        DistributedManager.initialize()
    return DistributedManager()


def _unwrap(model: torch.nn.Module) -> torch.nn.Module:
    """Strip DistributedDataParallel / DataParallel / torch.compile wrappers."""
    while True:
        if isinstance(model, (torch.nn.parallel.DistributedDataParallel, torch.nn.DataParallel)):
            model = model.module
        elif hasattr(model, "_orig_mod") and isinstance(getattr(model, "_orig_mod"), torch.nn.Module):
            model = model._orig_mod
        else:
            return model


def _is_distributed_model(model: torch.nn.Module) -> bool:
    try:
        from torch.distributed.tensor import DTensor
    except Exception:  # pragma: no cover
        DTensor = ()
    if type(model).__name__ in ("FullyShardedDataParallel", "FSDPModule"):
        return True
    for p in model.parameters():
        if DTensor and isinstance(p, DTensor):
            return True
        if type(p.data).__name__ == "ShardTensor" or type(p).__name__ == "ShardTensor":
            return True
    return False


def _unique_model_names(models: List[torch.nn.Module], loading: bool = False) -> Dict[str, torch.nn.Module]:
    groups: Dict[str, List[torch.nn.Module]] = {}
    for m in models:
        inner = _unwrap(m)
        groups.setdefault(type(inner).__name__, []).append(inner)
    out: Dict[str, torch.nn.Module] = {}
    for name, lst in groups.items():
        if len(lst) > 1:
            for i, m in enumerate(lst):
                out[f"{name}{i}"] = m
        else:
            out[name] = lst[0]
    return out


def _indices(path: str, base_name: str, mp_rank: int, ext: str) -> List[int]:
    fs = _get_fs(path)
    pattern = rf"^{re.escape(base_name)}\.{mp_rank}\.(\d+){re.escape(ext)}$"
    out = []
    try:
        names = fs.glob(f"{path}/{base_name}.{mp_rank}*{ext}")
    except FileNotFoundError:
        names = []
    for fname in names:
        m = re.match(pattern, PurePath(fname).name)
        if m:
            out.append(int(m.group(1)))
    return sorted(out)


def _get_checkpoint_filename(path: str, base_name: str = "checkpoint", index: Optional[int] = None,
                             saving: bool = False, model_type: str = "mdlus", distributed: bool = False) -> str:
    """``{path}/{base_name}.{mp_rank}.{index}{ext}``; without ``index`` the latest (loading) or next (saving)."""
    m = _manager()
    mp_rank = 0 if distributed else (m.group_rank("model_parallel") if "model_parallel" in m.group_names else 0)
    if "://" not in str(path):
        path = str(Path(path).resolve())
    ext = ".mdlus" if model_type == "mdlus" else ".pt"
    stem = f"{path}/{base_name}.{mp_rank}"
    if index is not None:
        return f"{stem}.{index}{ext}"
    found = _indices(path, base_name, mp_rank, ext)
    if found:
        return f"{stem}.{found[-1] + 1 if saving else found[-1]}{ext}"
    return f"{stem}.0{ext}"


def get_checkpoint_dir(base_dir: Union[str, Path], model_name: str) -> str:
    """``{base_dir}/checkpoints_{model_name}`` (keeps URL schemes such as ``msc://`` intact)."""
    base_dir = str(base_dir)
    top = f"checkpoints_{model_name}"
    if base_dir.startswith("msc://") or "://" in base_dir:
        return base_dir.rstrip("/") + "/" + top
    return os.path.join(base_dir, top)


def _full_state_dict(model: torch.nn.Module) -> dict:
    """Gather sharded parameters into full CPU tensors (collective)."""
    out = {}
    for k, v in model.state_dict().items():
        if hasattr(v, "full_tensor"):
            v = v.full_tensor()
        out[k] = v.detach().cpu() if isinstance(v, torch.Tensor) else v
    return out


def _is_sharded_tensor(v) -> bool:
    return isinstance(v, torch.Tensor) and hasattr(v, "full_tensor") and hasattr(v, "placements")


def _optimizer_is_sharded(optimizer) -> bool:
    if optimizer is None:
        return False
    return any(_is_sharded_tensor(p) for g in optimizer.param_groups for p in g["params"])


def _full_optimizer_state(optimizer) -> dict:
    """``optimizer.state_dict()`` with every sharded state tensor (the moments of DTensor / ShardTensor parameters)
    gathered to a full CPU tensor — collective; the result does not depend on how the parameters were sharded
    (reference: ``get_optimizer_state_dict(..., StateDictOptions(full_state_dict=True))``)."""
    sd = optimizer.state_dict()
    out_state = {}
    for idx in sorted(sd["state"]):                       # same order on every rank: the gathers are collectives
        out_state[idx] = {}
        for k, v in sd["state"][idx].items():
            if _is_sharded_tensor(v):
                v = v.full_tensor()
            out_state[idx][k] = v.detach().cpu() if isinstance(v, torch.Tensor) else v
    return {"state": out_state, "param_groups": sd["param_groups"]}


def _reshard_optimizer_state(optimizer, full: dict) -> dict:
    """A full optimizer state dict laid out for THIS run's parameters: state tensors that have the global shape of a
    sharded parameter are distributed with that parameter's mesh and placements (``set_optimizer_state_dict`` with
    ``full_state_dict`` in the reference)."""
    params = [p for g in optimizer.param_groups for p in g["params"]]
    saved_ids = [i for g in full["param_groups"] for i in g["params"]]
    state = {}
    for pos, idx in enumerate(saved_ids):
        if idx not in full["state"]:
            continue
        p = params[pos] if pos < len(params) else None
        entry = {}
        for k, v in full["state"][idx].items():
            if p is not None and _is_sharded_tensor(p) and isinstance(v, torch.Tensor) and tuple(v.shape) == tuple(p.shape):
                v = _distribute_like(v, p)
            entry[k] = v
        state[idx] = entry
    return {"state": state, "param_groups": full["param_groups"]}


def _distribute_like(full: torch.Tensor, like) -> torch.Tensor:
    local_dev = like.to_local().device
    if hasattr(like, "copy_full_"):                       # ShardTensor: same layout as the parameter
        out = torch.zeros_like(like)
        out.copy_full_(full.to(local_dev))
        return out
    from torch.distributed.tensor import distribute_tensor

    return distribute_tensor(full.to(local_dev), like.device_mesh, like.placements)


def save_checkpoint(path: Union[Path, str], models=None, optimizer=None, scheduler=None, scaler=None,
                    epoch: Optional[int] = None, metadata: Optional[Dict[str, Any]] = None,
                    optimizer_model: Optional[torch.nn.Module] = None) -> None:
    """Write model files and the training-state file of one step into directory ``path``."""
    path = str(path)
    fs = _get_fs(path)
    if "://" not in path or path.startswith("file://"):
        Path(path[len("file://"):] if path.startswith("file://") else path).mkdir(parents=True, exist_ok=True)
    m = _manager()
    model_list = [] if models is None else (models if isinstance(models, list) else [models])
    named = _unique_model_names(model_list)
    any_dist = any(_is_distributed_model(mod) for mod in named.values()) or _optimizer_is_sharded(optimizer) or (
        optimizer_model is not None and _is_distributed_model(_unwrap(optimizer_model)))
    for name, model in named.items():
        is_pn = isinstance(model, Module)
        model_type = "mdlus" if is_pn else "pt"
        distributed = _is_distributed_model(model)
        file_name = _get_checkpoint_filename(path, name, index=epoch, saving=True, model_type=model_type,
                                             distributed=distributed)
        if distributed:
            state = _full_state_dict(model)  # collective: every rank takes part
            if m.rank != 0:
                continue
            if is_pn:
                model.save(file_name, _state_dict=state)
            else:
                _torch_save(state, file_name, fs)
        else:
            if is_pn:
                model.save(file_name)
            else:
                _torch_save(model.state_dict(), file_name, fs)
        checkpoint_logging.info(f"Saved model state dictionary: {file_name}")
    state: Dict[str, Any] = {}
    if optimizer is not None:
        # sharded parameters: gather the moments (collective, every rank) so that rank 0's file holds all of them
        state["optimizer_state_dict"] = _full_optimizer_state(optimizer) if any_dist else optimizer.state_dict()
    if scheduler is not None:
        state["scheduler_state_dict"] = scheduler.state_dict()
    if scaler is not None:
        state["scaler_state_dict"] = scaler.state_dict()
    from .capture import _StaticCapture

    if _StaticCapture._amp_scalers:
        state["static_capture_state_dict"] = _StaticCapture.state_dict()
    if state or metadata is not None or epoch is not None:
        file_name = _get_checkpoint_filename(path, index=epoch, saving=True, model_type="pt", distributed=any_dist)
        state["epoch"] = epoch
        state["metadata"] = metadata
        if not any_dist or m.rank == 0:
            _torch_save(state, file_name, fs)
            checkpoint_logging.info(f"Saved training checkpoint: {file_name}")
    if any_dist and dist.is_initialized():
        dist.barrier()


def _torch_save(obj, file_name: str, fs) -> None:
    buf = io.BytesIO()
    torch.save(obj, buf)
    local = file_name[len("file://"):] if file_name.startswith("file://") else file_name
    if "://" not in local:
        tmp = local + ".tmp-write"
        with open(tmp, "wb") as f:
            f.write(buf.getvalue())
        os.replace(tmp, local)
    else:
        with fs.open(file_name, "wb") as f:
            f.write(buf.getvalue())


def _load_plain(file_name: str, device) -> Any:
    local = _download_cached(file_name)
    return torch.load(local, map_location=device, weights_only=False)


def load_model_weights(model: torch.nn.Module, weights_path: str, device: Union[str, torch.device] = "cpu") -> None:
    """Load one ``.mdlus`` / ``.pt`` file into ``model`` (collective for sharded models)."""
    inner = _unwrap(model)
    if _is_distributed_model(inner):
        m = _manager()
        payload = [None]
        if m.rank == 0:
            payload[0] = _read_state(weights_path, "cpu")
        if dist.is_initialized():
            dist.broadcast_object_list(payload, src=0)
        _load_into_sharded(inner, payload[0])
        return
    if isinstance(inner, Module) and str(weights_path).endswith(".mdlus"):
        inner.load(weights_path, map_location=device)
    else:
        inner.load_state_dict(_read_state(weights_path, device))


def _read_state(file_name: str, device) -> dict:
    if str(file_name).endswith(".mdlus"):
        members = Module._read_members(_download_cached(str(file_name)), names=("model.pt",))
        return torch.load(io.BytesIO(members["model.pt"]), map_location=device, weights_only=False)
    return _load_plain(str(file_name), device)


def _load_into_sharded(model: torch.nn.Module, full_state: dict) -> None:
    """Copy a full state dict into a model with sharded (DTensor-like) parameters."""
    own = model.state_dict()
    for k, v in own.items():
        if k not in full_state:
            continue
        src = full_state[k]
        if hasattr(v, "_local_tensor") and hasattr(v, "copy_full_"):
            v.copy_full_(src)
        elif hasattr(v, "device_mesh") and hasattr(v, "placements"):
            from torch.distributed.tensor import distribute_tensor

            v.copy_(distribute_tensor(src.to(v.device), v.device_mesh, v.placements))
        else:
            v.copy_(src.to(v.device))


def load_checkpoint(path: Union[Path, str], models=None, optimizer=None, scheduler=None, scaler=None,
                    epoch: Optional[int] = None, metadata_dict: Optional[Dict[str, Any]] = {},
                    device: Union[str, torch.device] = "cpu",
                    optimizer_model: Optional[torch.nn.Module] = None) -> int:
    """Restore models / optimizer / scheduler / scaler from ``path``; returns the stored epoch (0 if none)."""
    path = str(path)
    fs = _get_fs(path)
    if not fs.exists(path):
        checkpoint_logging.warning(f"Provided checkpoint directory {path} does not exist, skipping load")
        return 0
    model_list = [] if models is None else (models if isinstance(models, list) else [models])
    named = _unique_model_names(model_list, loading=True)
    any_dist = any(_is_distributed_model(mod) for mod in named.values()) or _optimizer_is_sharded(optimizer) or (
        optimizer_model is not None and _is_distributed_model(_unwrap(optimizer_model)))
    # training state first: newest readable index (falls back when the newest file is damaged); the model files are then
    # taken from the SAME index, so that weights and optimizer state always belong to one step
    m = _manager()
    mp_rank = 0 if any_dist else (m.group_rank("model_parallel") if "model_parallel" in m.group_names else 0)
    resolved = str(Path(path).resolve()) if "://" not in path else path
    candidates = [epoch] if epoch is not None else list(reversed(_indices(resolved, "checkpoint", mp_rank, ".pt")))
    state, used = None, epoch
    for idx in candidates:
        file_name = _get_checkpoint_filename(path, index=idx, model_type="pt", distributed=any_dist)
        if not fs.exists(file_name):
            continue
        try:
            state = _load_plain(file_name, device)
            used = idx
            checkpoint_logging.info(f"Loaded checkpoint file {file_name} to device {device}")
            break
        except Exception as exc:  # noqa: BLE001 - damaged / partial file: try the previous index
            checkpoint_logging.warning(f"Checkpoint file {file_name} is unreadable ({exc}); trying an older one")
    for name, model in named.items():
        model_type = "mdlus" if isinstance(model, Module) else "pt"
        file_name = _get_checkpoint_filename(path, name, index=used if state is not None else epoch, model_type=model_type,
                                             distributed=_is_distributed_model(model))
        if not fs.exists(file_name):
            checkpoint_logging.error(f"Could not find valid model file {file_name}, skipping load")
            continue
        load_model_weights(model, file_name, device)
        checkpoint_logging.info(f"Loaded model state dictionary {file_name} to device {device}")
    if state is None:
        checkpoint_logging.warning("Could not find valid checkpoint file, skipping load")
        return 0
    if optimizer is not None and "optimizer_state_dict" in state:
        osd = state["optimizer_state_dict"]
        if _optimizer_is_sharded(optimizer):
            osd = _reshard_optimizer_state(optimizer, osd)
        optimizer.load_state_dict(osd)
    if scheduler is not None and "scheduler_state_dict" in state:
        scheduler.load_state_dict(state["scheduler_state_dict"])
    if scaler is not None and "scaler_state_dict" in state:
        scaler.load_state_dict(state["scaler_state_dict"])
    if "static_capture_state_dict" in state:
        from .capture import _StaticCapture

        _StaticCapture.load_state_dict(state["static_capture_state_dict"])
    if metadata_dict is not None:
        metadata_dict.update(state.get("metadata") or {})
    return state.get("epoch") or 0

"""Optional unified GPU memory pool shared by PyTorch and CuPy / RAPIDS through RMM.

Parity: ``physicsnemo/utils/memory.py``: accessing ``unified_gpu_memory`` once (``from ... import unified_gpu_memory``)
re-initialises RMM with a pool on this rank's device and routes the PyTorch and CuPy allocators through it; set
``PHYSICSNEMO_DISABLE_RMM=1`` to switch it off.  Without ``rmm`` installed the attribute access is a no-op.
"""
from __future__ import annotations

import importlib
import importlib.util
import os


def srt2bool(val) -> bool:
    if isinstance(val, bool):
        return val
    if str(val).lower() in ("true", "1", "yes", "y"):
        return True
    if str(val).lower() in ("false", "0", "no", "n"):
        return False
    raise ValueError(f"Invalid boolean value: {val}")


RMM_AVAILABLE = importlib.util.find_spec("rmm") is not None
CUPY_AVAILABLE = importlib.util.find_spec("cupy") is not None
DISABLE_RMM = srt2bool(os.environ.get("PHYSICSNEMO_DISABLE_RMM", False))


def _local_rank() -> int:
    method = os.environ.get("PHYSICSNEMO_DISTRIBUTED_INITIALIZATION_METHOD")
    names = {"ENV": ["LOCAL_RANK"], "SLURM": ["SLURM_LOCALID"], "OPENMPI": ["OMPI_COMM_WORLD_LOCAL_RANK"],
             None: ["LOCAL_RANK", "OMPI_COMM_WORLD_LOCAL_RANK", "SLURM_LOCALID"]}
    if method not in names:
        raise ValueError(f"Unknown initialization method: {method}")
    for n in names[method]:
        if os.environ.get(n) is not None:
            return int(os.environ[n])
    return 0


def _setup_unified_gpu_memory():
    if not RMM_AVAILABLE or DISABLE_RMM:
        return None
    import torch

    rmm = importlib.import_module("rmm")
    alloc = importlib.import_module("rmm.allocators.torch")
    rmm.reinitialize(pool_allocator=True, devices=_local_rank(), initial_pool_size="1024MB")
    if torch.cuda.is_available():
        torch.cuda.memory.change_current_allocator(alloc.rmm_torch_allocator)
    if CUPY_AVAILABLE:
        cupy = importlib.import_module("cupy")
        cupy.cuda.set_allocator(importlib.import_module("rmm.allocators.cupy").rmm_cupy_allocator)
    return True


def __getattr__(name):
    if name == "unified_gpu_memory":
        return _setup_unified_gpu_memory()
    raise AttributeError(f"module '{__name__}' has no attribute '{name}'")

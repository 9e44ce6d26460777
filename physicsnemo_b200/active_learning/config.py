"""Configuration dataclasses of the active-learning driver.

Parity: ``physicsnemo/active_learning/config.py`` (``OptimizerConfig``, ``TrainingConfig``,
``StrategiesConfig``, ``DriverConfig``; validation in ``__post_init__``, ``to_dict`` / ``from_dict``
and ``to_json`` / ``from_json`` for checkpoints; data pools, collate functions and the
distributed manager are never serialised and are re-supplied on load).
"""
from __future__ import annotations

import json
import math
import uuid
from dataclasses import dataclass, field, fields
from pathlib import Path
from typing import Any, Callable
from warnings import warn

import torch
from torch import distributed as dist
from torch.optim import AdamW

from ..distributed import DistributedManager
from . import protocols as p
from ._registry import registry
from .loop import DefaultTrainingLoop


def _class_ref(cls: type) -> dict[str, str]:
    return {"__name__": cls.__name__, "__module__": cls.__module__}


def _args_of(obj: Any, what: str) -> dict:
    if not hasattr(obj, "_args"):
        raise ValueError(
            f"{what} {obj} does not have an `_args` attribute which is required for serialization. Make sure it "
            "either subclasses `ActiveLearningProtocol` or implements the `__new__` method to capture object arguments.")
    return obj._args


def _rebuild(entry: dict):
    return registry.construct(entry["__name__"], module_path=entry["__module__"], **entry["__args__"])


@dataclass
class OptimizerConfig:
    optimizer_cls: type = AdamW
    optimizer_kwargs: dict[str, Any] = field(default_factory=lambda: {"lr": 1e-4})
    scheduler_cls: type | None = None
    scheduler_kwargs: dict[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        lr = self.optimizer_kwargs.get("lr")
        if "lr" in self.optimizer_kwargs and (not isinstance(lr, (int, float)) or lr <= 0):
            raise ValueError(f"Learning rate must be positive, got {lr}")
        if self.scheduler_kwargs and self.scheduler_cls is None:
            raise ValueError("scheduler_kwargs provided but scheduler_cls is None. "
                             "Provide a scheduler_cls or remove scheduler_kwargs.")

    def to_dict(self) -> dict[str, Any]:
        return {"optimizer_cls": _class_ref(self.optimizer_cls), "optimizer_kwargs": self.optimizer_kwargs,
                "scheduler_cls": _class_ref(self.scheduler_cls) if self.scheduler_cls else None,
                "scheduler_kwargs": self.scheduler_kwargs}

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "OptimizerConfig":
        opt = registry.get_class(data["optimizer_cls"]["__name__"], data["optimizer_cls"]["__module__"])
        s = data.get("scheduler_cls")
        sched = registry.get_class(s["__name__"], s["__module__"]) if s is not None else None
        return cls(optimizer_cls=opt, optimizer_kwargs=data["optimizer_kwargs"], scheduler_cls=sched,
                   scheduler_kwargs=data["scheduler_kwargs"])


@dataclass
class TrainingConfig:
    train_datapool: Any
    max_training_epochs: int
    val_datapool: Any = None
    optimizer_config: OptimizerConfig = field(default_factory=OptimizerConfig)
    max_fine_tuning_epochs: int | None = None
    train_loop_fn: Any = field(default_factory=DefaultTrainingLoop)

    def __post_init__(self) -> None:
        if not hasattr(self.train_datapool, "__len__"):
            raise ValueError("train_datapool must implement __len__")
        if self.val_datapool is not None and not hasattr(self.val_datapool, "__len__"):
            raise ValueError("val_datapool must implement __len__")
        if not callable(self.train_loop_fn):
            raise ValueError("train_loop_fn must be callable")
        if self.max_fine_tuning_epochs is None:
            self.max_fine_tuning_epochs = self.max_training_epochs

    def to_dict(self) -> dict[str, Any]:
        warn("The `train_datapool` and `val_datapool` attributes are not supported for serialization and will be "
             "excluded from the ``TrainingConfig`` dictionary. You must re-provide these datapools when deserializing.")
        return {"max_training_epochs": self.max_training_epochs, "max_fine_tuning_epochs": self.max_fine_tuning_epochs,
                "optimizer_config": self.optimizer_config.to_dict(),
                "train_loop_fn": _args_of(self.train_loop_fn, "Training loop")}

    @classmethod
    def from_dict(cls, data: dict[str, Any], **kwargs: Any) -> "TrainingConfig":
        if "train_datapool" not in kwargs:
            raise ValueError("``train_datapool`` must be provided in kwargs when deserializing TrainingConfig, "
                             "as datapools are not serialized.")
        try:
            return cls(max_training_epochs=data["max_training_epochs"],
                       max_fine_tuning_epochs=data.get("max_fine_tuning_epochs"),
                       optimizer_config=OptimizerConfig.from_dict(data["optimizer_config"]),
                       train_loop_fn=_rebuild(data["train_loop_fn"]), **kwargs)
        except Exception as e:
            raise ValueError("Failed to construct ``TrainingConfig`` from dictionary.") from e


@dataclass
class StrategiesConfig:
    query_strategies: list
    queue_cls: type
    label_strategy: Any = None
    metrology_strategies: list | None = None
    unlabeled_datapool: Any = None

    def __post_init__(self) -> None:
        if not self.query_strategies:
            raise ValueError("At least one query strategy must be provided. "
                             "Active learning requires a mechanism to select data.")
        for s in self.query_strategies:
            if not callable(s):
                raise ValueError(f"Query strategy {s} must be callable")
        if self.label_strategy is not None and not callable(self.label_strategy):
            raise ValueError("label_strategy must be callable")
        if self.metrology_strategies is not None:
            if not self.metrology_strategies:
                raise ValueError("metrology_strategies is an empty list. "
                                 "Either provide strategies or set to None to skip metrology.")
            for s in self.metrology_strategies:
                if not callable(s):
                    raise ValueError(f"Metrology strategy {s} must be callable")
        if not callable(self.queue_cls):
            raise ValueError("queue_cls must be a callable class")

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"query_strategies": [_args_of(s, "Query strategy") for s in self.query_strategies]}
        if self.label_strategy is not None:
            out["label_strategy"] = _args_of(self.label_strategy, "Label strategy")
        out["queue_cls"] = _class_ref(self.queue_cls)
        if self.metrology_strategies is not None:
            out["metrology_strategies"] = [_args_of(s, "Metrology strategy") for s in self.metrology_strategies]
        if self.unlabeled_datapool is not None:
            warn("The `unlabeled_datapool` attribute is not supported for serialization and will be excluded from "
                 "the ``StrategiesConfig`` dictionary.")
        return out

    @classmethod
    def from_dict(cls, data: dict[str, Any], **kwargs: Any) -> "StrategiesConfig":
        expected = {f.name for f in fields(cls)}
        extra = set(data) - expected
        if extra:
            raise ValueError(f"Unexpected keys in data: {extra}. Expected keys are {expected}.")
        built: dict[str, Any] = {"query_strategies": [_rebuild(e) for e in data["query_strategies"]]}
        if "metrology_strategies" in data:
            built["metrology_strategies"] = [_rebuild(e) for e in data["metrology_strategies"]]
        if "label_strategy" in data:
            built["label_strategy"] = _rebuild(data["label_strategy"])
        built["queue_cls"] = registry.get_class(data["queue_cls"]["__name__"], data["queue_cls"]["__module__"])
        built.update(kwargs)
        try:
            return cls(**built)
        except Exception as e:
            raise ValueError("Failed to construct ``StrategiesConfig`` from dictionary.") from e


_UNSERIALISED = ("dist_manager", "collate_fn", "root_log_dir", "device", "dtype")
_METADATA = ("default_dtype", "world_size", "dist_manager_init_method", "log_dir")
_DTYPES = {str(t): t for t in (torch.float32, torch.float64, torch.float16, torch.bfloat16, torch.int32, torch.int64,
                               torch.int8, torch.uint8)}


@dataclass
class DriverConfig:
    batch_size: int
    max_active_learning_steps: int | float | None = None
    run_id: str = field(default_factory=lambda: str(uuid.uuid4()))
    fine_tuning_lr: float | None = None
    reset_optim_states: bool = True
    skip_training: bool = False
    skip_metrology: bool = False
    skip_labeling: bool = False
    checkpoint_interval: int = 1
    checkpoint_on_training: bool = False
    checkpoint_on_metrology: bool = False
    checkpoint_on_query: bool = False
    checkpoint_on_labeling: bool = True
    model_checkpoint_frequency: int = 0
    root_log_dir: str | Path = field(default_factory=lambda: Path.cwd() / "active_learning_logs")
    dist_manager: DistributedManager | None = None
    collate_fn: Callable | None = None
    num_dataloader_workers: int = 0
    device: str | torch.device | None = None
    dtype: torch.dtype | None = None

    def __post_init__(self) -> None:
        if self.max_active_learning_steps is None:
            self.max_active_learning_steps = float("inf")
        if self.max_active_learning_steps <= 0:
            raise ValueError("`max_active_learning_steps` must be a positive integer or None.")
        if not math.isfinite(self.batch_size) or self.batch_size <= 0:
            raise ValueError("`batch_size` must be a positive integer.")
        if not math.isfinite(self.checkpoint_interval) or self.checkpoint_interval < 0:
            raise ValueError("`checkpoint_interval` must be a non-negative integer. Use 0 to disable checkpointing.")
        if self.fine_tuning_lr is not None and self.fine_tuning_lr <= 0:
            raise ValueError("`fine_tuning_lr` must be positive if provided.")
        if self.num_dataloader_workers < 0:
            raise ValueError("`num_dataloader_workers` must be non-negative.")
        if self.model_checkpoint_frequency < 0:
            raise ValueError("`model_checkpoint_frequency` must be non-negative.")
        self.root_log_dir = Path(self.root_log_dir)
        if self.collate_fn is not None and not callable(self.collate_fn):
            raise ValueError("`collate_fn` must be callable if provided.")
        if self.device is None and not self.dist_manager:
            self.device = torch.get_default_device()
        if self.dtype is None:
            self.dtype = torch.get_default_dtype()

    def to_json(self) -> str:
        out = {k: v for k, v in self.__dict__.items() if k not in _UNSERIALISED}
        if out["max_active_learning_steps"] == float("inf"):
            out["max_active_learning_steps"] = None
        out["default_dtype"] = str(torch.get_default_dtype())
        out["log_dir"] = str(self.root_log_dir)
        out["dtype"] = str(self.dtype) if self.dtype is not None else None
        if self.dist_manager is not None:
            out["world_size"] = self.dist_manager.world_size
            out["device"] = self.dist_manager.device.type
            out["dist_manager_init_method"] = getattr(self.dist_manager, "_initialization_method", None)
        else:
            out["world_size"] = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
            out["device"] = str(self.device) if self.device is not None else torch.get_default_device().type
            out["dist_manager_init_method"] = None
        out["collate_fn"] = getattr(self.collate_fn, "__name__", None) if self.collate_fn is not None else None
        return json.dumps(out, indent=2)

    @classmethod
    def from_json(cls, json_str: str, **kwargs: Any) -> "DriverConfig":
        try:
            data = json.loads(json_str)
        except json.JSONDecodeError as e:
            raise ValueError(f"Invalid JSON string: {e}") from e
        cfg = {k: v for k, v in data.items() if k not in _METADATA + _UNSERIALISED}
        if "log_dir" in data:
            cfg["root_log_dir"] = Path(data["log_dir"])
        if data.get("device") is not None:
            cfg["device"] = torch.device(data["device"])
        if data.get("dtype") is not None:
            if data["dtype"] in _DTYPES:
                cfg["dtype"] = _DTYPES[data["dtype"]]
            else:
                warn(f"Unknown dtype string '{data['dtype']}' in JSON. Using default dtype instead.")
        cfg.update(kwargs)
        try:
            return cls(**cfg)
        except Exception as e:
            raise ValueError("Failed to construct ``DriverConfig`` from JSON string.") from e

"""Structural interfaces of the active-learning loop.

Parity: ``physicsnemo/active_learning/protocols.py`` — phases (``ActiveLearningPhase``), containers
(``AbstractQueue``, ``DataPool``), strategies (``QueryStrategy``, ``LabelStrategy``,
``MetrologyStrategy``), step callables (``TrainingProtocol``, ``ValidationProtocol``,
``InferenceProtocol``, ``TrainingLoop``), ``LearnerProtocol`` and ``DriverProtocol``.

Every strategy records the arguments it was constructed with in ``_args`` (name, module, keyword
dictionary) so that a driver checkpoint can rebuild it; ``capture_init_args`` is the one helper
that does this for strategies and training loops alike.
"""
from __future__ import annotations

import inspect
import logging
from enum import Enum
from logging import Logger
from pathlib import Path
from typing import Any, Callable, Iterator, Protocol, TypeVar

import torch

T = TypeVar("T")
S = TypeVar("S")


class ActiveLearningPhase(str, Enum):
    TRAINING = "training"
    METROLOGY = "metrology"
    QUERY = "query"
    LABELING = "labeling"
    DATA_INTEGRATION = "data_integration"

    def __str__(self) -> str:
        return self.value

    def __format__(self, spec: str) -> str:
        return format(self.value, spec)


def capture_init_args(cls: type, args: tuple, kwargs: dict, encode: Callable[[str, Any], Any] | None = None) -> dict:
    """``{"__name__", "__module__", "__args__"}`` describing ``cls(*args, **kwargs)`` with defaults applied."""
    sig = inspect.signature(cls.__init__)
    bound = sig.bind_partial(None, *args, **kwargs)
    bound.apply_defaults()
    captured: dict[str, Any] = {}
    for name, value in bound.arguments.items():
        if name == "self":
            continue
        kind = sig.parameters[name].kind
        if kind is inspect.Parameter.VAR_KEYWORD:
            captured.update(value)
        elif kind is inspect.Parameter.VAR_POSITIONAL:
            continue
        else:
            captured[name] = encode(name, value) if encode else value
    return {"__name__": cls.__name__, "__module__": cls.__module__, "__args__": captured}


class AbstractQueue(Protocol[T]):
    def put(self, item: T) -> None: ...

    def get(self) -> T: ...

    def empty(self) -> bool: ...


class DataPool(Protocol[T]):
    def __getitem__(self, index: int) -> T: ...

    def __len__(self) -> int: ...

    def __iter__(self) -> Iterator[T]: ...

    def append(self, item: T) -> None: ...


class ActiveLearningProtocol(Protocol):
    """Base of all strategies: argument capture, attachment to a driver, per-strategy logger and folders."""

    __protocol_name__: str
    __protocol_type__: ActiveLearningPhase
    _args: dict[str, Any]

    def __new__(cls, *args: Any, **kwargs: Any):
        out = super().__new__(cls)
        out._args = capture_init_args(cls, args, kwargs)
        return out

    def attach(self, other: object) -> None:
        """Default: remember the driver; strategies may override to grab pools or the learner."""
        self.driver = other

    @property
    def is_attached(self) -> bool:
        return getattr(self, "driver", None) is not None

    @property
    def logger(self) -> Logger:
        if not hasattr(self, "_logger"):
            self._setup_logger()
        return self._logger

    @logger.setter
    def logger(self, logger: Logger) -> None:
        self._logger = logger

    def _setup_logger(self) -> None:
        name = getattr(self, "__protocol_name__", type(self).__name__)
        self._logger = logging.getLogger(f"core.active_learning.{name}")
        self._logger.setLevel(logging.WARNING)

    def _require_driver(self):
        if not self.is_attached:
            raise RuntimeError(f"{self.__class__.__name__} is not attached to a driver yet.")
        return self.driver

    @property
    def strategy_dir(self) -> Path:
        path = self._require_driver().log_dir / str(self.__protocol_type__) / self.__class__.__name__
        path.mkdir(parents=True, exist_ok=True)
        return path

    @property
    def checkpoint_dir(self) -> Path:
        driver = self._require_driver()
        path = driver.log_dir / "checkpoints" / f"step_{driver.active_learning_step_idx}"
        path.mkdir(parents=True, exist_ok=True)
        return path


class QueryStrategy(ActiveLearningProtocol):
    """Selects samples worth labelling and puts them on the query queue."""

    max_samples: int
    __protocol_type__ = ActiveLearningPhase.QUERY

    def sample(self, query_queue: AbstractQueue[T], *args: Any, **kwargs: Any) -> None: ...

    def __call__(self, query_queue: AbstractQueue[T], *args: Any, **kwargs: Any) -> None:
        self.sample(query_queue, *args, **kwargs)


class LabelStrategy(ActiveLearningProtocol):
    """Turns queried samples into labelled ones (a solver, an oracle, a database lookup)."""

    __is_external_process__: bool
    __provides_fields__: set[str] | None = None
    __protocol_type__ = ActiveLearningPhase.LABELING

    def label(self, queue_to_label: AbstractQueue[T], serialize_queue: AbstractQueue[T], *args: Any, **kwargs: Any) -> None: ...

    def __call__(self, queue_to_label: AbstractQueue[T], serialize_queue: AbstractQueue[T], *args: Any, **kwargs: Any) -> None:
        self.label(queue_to_label, serialize_queue, *args, **kwargs)


class MetrologyStrategy(ActiveLearningProtocol):
    """Measures the learner between training and querying; keeps a list of records."""

    records: list
    __protocol_type__ = ActiveLearningPhase.METROLOGY

    def append(self, record: S) -> None:
        self.records.append(record)

    def __len__(self) -> int:
        return len(self.records)

    def serialize_records(self, path: Path | None = None, *args: Any, **kwargs: Any) -> None: ...

    def load_records(self, path: Path | None = None, *args: Any, **kwargs: Any) -> None: ...

    def compute(self, *args: Any, **kwargs: Any) -> None: ...

    def __call__(self, *args: Any, **kwargs: Any) -> None:
        self.compute(*args, **kwargs)

    def reset(self) -> None:
        self.records = []


class TrainingProtocol(Protocol):
    def __call__(self, model, data: T, *args: Any, **kwargs: Any) -> torch.Tensor: ...


class ValidationProtocol(Protocol):
    def __call__(self, model, data: T, *args: Any, **kwargs: Any) -> None: ...


class InferenceProtocol(Protocol):
    def __call__(self, model, data: S, *args: Any, **kwargs: Any) -> Any: ...


class TrainingLoop(Protocol):
    def __call__(self, model, optimizer, train_dataloader, validation_dataloader=None, train_step_fn=None,
                 validate_step_fn=None, max_epochs: int | None = None, max_train_steps: int | None = None,
                 max_val_steps: int | None = None, lr_scheduler=None, device=None, dtype=None,
                 *args: Any, **kwargs: Any) -> None: ...


class LearnerProtocol:
    """A model that carries its own step logic (alternative to passing step functions to the driver)."""

    def training_step(self, data: T, *args: Any, **kwargs: Any) -> None: ...

    def validation_step(self, data: T, *args: Any, **kwargs: Any) -> None: ...

    def inference_step(self, data: T | S, *args: Any, **kwargs: Any) -> None: ...

    @property
    def parameters(self) -> Iterator[torch.Tensor]: ...

    def forward(self, *args: Any, **kwargs: Any) -> Any: ...


class DriverProtocol:
    learner: LearnerProtocol
    query_strategies: list
    query_queue: AbstractQueue
    label_strategy: LabelStrategy | None
    label_queue: AbstractQueue | None
    metrology_strategies: list | None
    training_pool: DataPool
    validation_pool: DataPool | None
    unlabeled_pool: DataPool | None

    def active_learning_step(self, *args: Any, **kwargs: Any) -> None: ...

    def _setup_logger(self) -> None: ...

    def attach_strategies(self) -> None:
        for strategy in self.query_strategies:
            strategy.attach(self)
        if self.label_strategy:
            self.label_strategy.attach(self)
        for strategy in self.metrology_strategies or []:
            strategy.attach(self)

"""Active-learning orchestration: train → measure → query → label, with phase-level resume.

Parity: ``physicsnemo/active_learning/driver.py`` (``Driver``, ``ActiveLearningCheckpoint``): phase
queue built per step from the config's skip flags and the phase a checkpoint was taken in,
optimizer / scheduler construction with signature validation, optimizer-state reset between
steps, fine-tuning learning rate and epoch budget after the first step, distributed sampler +
DDP wrapping when a ``DistributedManager`` is active, queue (de)serialisation, model saved as
``<Class>.mdlus`` or a ``state_dict``.
"""
from __future__ import annotations

import inspect
import pickle
from contextlib import contextmanager
from copy import deepcopy
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Generator

import torch
from torch import distributed as dist
from torch.nn.parallel import DistributedDataParallel
from torch.utils.data import DataLoader, DistributedSampler

from .. import __version__ as physicsnemo_version
from ..core import Module
from . import protocols as p
from .config import DriverConfig, StrategiesConfig, TrainingConfig
from .logger import ActiveLearningLoggerAdapter, setup_active_learning_logger
from .loop import DefaultTrainingLoop

_RESERVED_PT = {"checkpoint.pt", "query_queue.pt", "label_queue.pt", "training_state.pt"}


@dataclass
class ActiveLearningCheckpoint:
    driver_config: Any
    strategies_config: Any
    active_learning_step_idx: int
    active_learning_phase: p.ActiveLearningPhase
    physicsnemo_version: str = physicsnemo_version
    training_config: Any = None
    optimizer_state: dict[str, Any] | None = None
    lr_scheduler_state: dict[str, Any] | None = None
    has_query_queue: bool = False
    has_label_queue: bool = False


def _core_module(learner):
    """The ``Module`` inside ``learner`` (itself, or what a DDP wrapper holds), else ``None``."""
    if isinstance(learner, Module):
        return learner
    inner = getattr(learner, "module", None)
    return inner if isinstance(inner, Module) else None


class Driver(p.DriverProtocol):
    _PHASE_ORDER = [p.ActiveLearningPhase.TRAINING, p.ActiveLearningPhase.METROLOGY, p.ActiveLearningPhase.QUERY,
                    p.ActiveLearningPhase.LABELING]

    def __init__(self, config: DriverConfig, learner, strategies_config: StrategiesConfig,
                 training_config: TrainingConfig | None = None, inference_fn=None) -> None:
        self.config = config
        self.learner = learner
        self.strategies_config = strategies_config
        self.training_config = training_config
        self.inference_fn = inference_fn
        self.active_learning_step_idx = 0
        self.current_phase: p.ActiveLearningPhase | None = None
        self._last_checkpoint_path: Path | None = None
        self._validate_config_consistency()
        self._setup_logger()
        self.attach_strategies()
        self.query_queue = strategies_config.queue_cls()
        self.label_queue = strategies_config.queue_cls()

    # ---- configuration views --------------------------------------------------------------------------
    def _validate_config_consistency(self) -> None:
        cfg = self.config
        if not cfg.skip_training and self.training_config is None:
            raise ValueError("`training_config` must be provided when `skip_training` is False.")
        if not cfg.skip_labeling:
            if self.strategies_config.label_strategy is None:
                raise ValueError("`label_strategy` must be provided in strategies_config when `skip_labeling` is False.")
            if self.training_config is None or self.training_config.train_datapool is None:
                raise ValueError("`train_datapool` must be provided in training_config when `skip_labeling` is False "
                                 "(labeled data is appended to it).")
        if cfg.fine_tuning_lr is not None and cfg.skip_training:
            raise ValueError("`fine_tuning_lr` has no effect when `skip_training` is True.")

    query_strategies = property(lambda self: self.strategies_config.query_strategies)
    label_strategy = property(lambda self: self.strategies_config.label_strategy)
    metrology_strategies = property(lambda self: self.strategies_config.metrology_strategies)
    unlabeled_datapool = property(lambda self: self.strategies_config.unlabeled_datapool)
    train_datapool = property(lambda self: self.training_config.train_datapool if self.training_config else None)
    val_datapool = property(lambda self: self.training_config.val_datapool if self.training_config else None)
    train_loop_fn = property(lambda self: self.training_config.train_loop_fn if self.training_config else None)
    run_id = property(lambda self: self.config.run_id)
    short_run_id = property(lambda self: self.run_id[:8])
    log_dir = property(lambda self: self.config.root_log_dir / self.short_run_id)
    last_checkpoint = property(lambda self: self._last_checkpoint_path)
    dist_manager = property(lambda self: self.config.dist_manager)

    def _dist_active(self) -> bool:
        return self.dist_manager is not None and self.dist_manager.is_initialized()

    @property
    def device(self) -> torch.device:
        return self.dist_manager.device if self._dist_active() else torch.get_default_device()

    @property
    def active_learning_step_idx(self) -> int:
        return self._active_learning_step_idx

    @active_learning_step_idx.setter
    def active_learning_step_idx(self, value: int) -> None:
        if value < 0:
            raise ValueError("Active learning step index must be non-negative.")
        self._active_learning_step_idx = value

    # ---- optimizer ------------------------------------------------------------------------------------
    def configure_optimizer(self) -> None:
        self.optimizer = self.lr_scheduler = None
        if self.training_config is None:
            return
        oc = self.training_config.optimizer_config
        if oc.optimizer_cls is None:
            return
        try:
            inspect.signature(oc.optimizer_cls).bind(self.learner.parameters(), **oc.optimizer_kwargs)
        except TypeError as e:
            raise ValueError(f"Invalid optimizer kwargs for {oc.optimizer_cls}; {e}")
        self.optimizer = oc.optimizer_cls(self.learner.parameters(), **oc.optimizer_kwargs)
        if oc.scheduler_cls is not None:
            try:
                inspect.signature(oc.scheduler_cls).bind(self.optimizer, **oc.scheduler_kwargs)
            except TypeError as e:
                raise ValueError(f"Invalid LR scheduler kwargs for {oc.scheduler_cls}; {e}")
            self.lr_scheduler = oc.scheduler_cls(self.optimizer, **oc.scheduler_kwargs)
        if self.config.reset_optim_states:
            self._original_optim_state = deepcopy(self.optimizer.state_dict())

    is_optimizer_configured = property(lambda self: getattr(self, "optimizer", None) is not None)
    is_lr_scheduler_configured = property(lambda self: getattr(self, "lr_scheduler", None) is not None)

    def _setup_logger(self) -> None:
        base = setup_active_learning_logger("core.active_learning", run_id=self.run_id, log_dir=self.log_dir)
        self.logger = ActiveLearningLoggerAdapter(base, driver_ref=self)

    # ---- checkpoints ----------------------------------------------------------------------------------
    def _should_checkpoint_at_step(self) -> bool:
        k = self.config.checkpoint_interval
        return k != 0 and self.active_learning_step_idx % k == 0

    def _serialize_queue(self, queue, file_path: Path) -> bool:
        try:
            if callable(getattr(queue, "to_list", None)):
                torch.save({"type": "list", "data": queue.to_list()}, file_path)
            else:
                torch.save({"type": "torch", "data": queue}, file_path)
            return True
        except (TypeError, AttributeError, pickle.PicklingError, RuntimeError) as e:
            if file_path.exists():
                file_path.unlink()
            self.logger.warning(f"Failed to serialize queue to {file_path}: {e}. Queue state will not be saved. "
                                "Consider implementing to_list()/from_list() methods for custom serialization.")
            return False

    def _deserialize_queue(self, queue, file_path: Path) -> None:
        if not file_path.exists():
            return
        try:
            blob = torch.load(file_path, map_location="cpu", weights_only=False)
            if blob["type"] == "list":
                if callable(getattr(queue, "from_list", None)):
                    queue.from_list(blob["data"])
                else:
                    for item in blob["data"]:
                        queue.put(item)
            else:
                restored = blob["data"]
                while not restored.empty():
                    queue.put(restored.get())
        except Exception as e:  # noqa: BLE001
            self.logger.warning(f"Failed to deserialize queue from {file_path}: {e}. Queue will be empty.")

    def _save_learner(self, folder: Path) -> None:
        core = _core_module(self.learner)
        if core is not None:
            core.save(str(folder / f"{type(core).__name__}.mdlus"))
        else:
            torch.save(self.learner.state_dict(), folder / f"{type(self.learner).__name__}.pt")

    @staticmethod
    def _restore_learner(learner, folder: Path) -> None:
        core = _core_module(learner)
        if core is not None:
            path = folder / f"{type(core).__name__}.mdlus"
            candidates = [path] if path.exists() else sorted(folder.glob("*.mdlus"))
            if candidates:
                core.load(str(candidates[0]))
            return
        path = folder / f"{type(learner).__name__}.pt"
        candidates = [path] if path.exists() else [f for f in sorted(folder.glob("*.pt")) if f.name not in _RESERVED_PT]
        if candidates:
            learner.load_state_dict(torch.load(candidates[0], map_location="cpu"))

    def save_checkpoint(self, path: str | Path | None = None, training_epoch: int | None = None) -> Path | None:
        if path is None:
            folder = (self.log_dir / "checkpoints" / f"step_{self.active_learning_step_idx}"
                      / str(self.current_phase if self.current_phase else "init"))
            if training_epoch is not None:
                folder = folder / f"epoch_{training_epoch}"
        else:
            folder = Path(path)
        folder.mkdir(parents=True, exist_ok=True)
        if self._dist_active() and self.dist_manager.rank != 0:
            return None
        ckpt = ActiveLearningCheckpoint(
            driver_config=self.config.to_json(), strategies_config=self.strategies_config.to_dict(),
            active_learning_step_idx=self.active_learning_step_idx,
            active_learning_phase=self.current_phase or p.ActiveLearningPhase.TRAINING,
            training_config=self.training_config.to_dict() if self.training_config else None,
            has_query_queue=self._serialize_queue(self.query_queue, folder / "query_queue.pt"),
            has_label_queue=self._serialize_queue(self.label_queue, folder / "label_queue.pt"))
        blob: dict[str, Any] = {"checkpoint": ckpt}
        if training_epoch is not None:
            blob["training_epoch"] = training_epoch
        torch.save(blob, folder / "checkpoint.pt")
        self._save_learner(folder)
        self._last_checkpoint_path = folder
        self.logger.info(f"Saved checkpoint at step {self.active_learning_step_idx}, phase {self.current_phase}: {folder}")
        return folder

    @classmethod
    def load_checkpoint(cls, checkpoint_path: str | Path, learner=None, train_datapool=None, val_datapool=None,
                        unlabeled_datapool=None, **kwargs: Any) -> "Driver":
        folder = Path(checkpoint_path)
        if not (folder / "checkpoint.pt").exists():
            raise FileNotFoundError(f"Checkpoint file not found: {folder / 'checkpoint.pt'}")
        blob = torch.load(folder / "checkpoint.pt", map_location="cpu", weights_only=False)
        ckpt: ActiveLearningCheckpoint = blob["checkpoint"]
        config = DriverConfig.from_json(ckpt.driver_config, **kwargs.get("driver_config_overrides", {}))
        strategies = StrategiesConfig.from_dict(ckpt.strategies_config, unlabeled_datapool=unlabeled_datapool,
                                                **kwargs.get("strategies_config_overrides", {}))
        training = None
        if ckpt.training_config is not None:
            training = TrainingConfig.from_dict(ckpt.training_config, train_datapool=train_datapool,
                                                val_datapool=val_datapool, **kwargs.get("training_config_overrides", {}))
        if learner is None:
            saved = sorted(folder.glob("*.mdlus"))
            if not saved:
                raise ValueError("No learner provided and unable to reconstruct from checkpoint. "
                                 "Please provide a learner instance.")
            learner = Module.from_checkpoint(str(saved[0]))
        else:
            cls._restore_learner(learner, folder)
        driver = cls(config=config, learner=learner, strategies_config=strategies, training_config=training,
                     inference_fn=kwargs.get("inference_fn"))
        driver.active_learning_step_idx = ckpt.active_learning_step_idx
        driver.current_phase = ckpt.active_learning_phase
        driver._last_checkpoint_path = folder
        if driver.training_config is not None:
            driver.configure_optimizer()
            DefaultTrainingLoop.load_training_checkpoint(folder, driver.learner, driver.optimizer,
                                                         getattr(driver, "lr_scheduler", None))
        if ckpt.has_query_queue:
            driver._deserialize_queue(driver.query_queue, folder / "query_queue.pt")
        if ckpt.has_label_queue:
            driver._deserialize_queue(driver.label_queue, folder / "label_queue.pt")
        driver.logger.info(f"Loaded checkpoint from {folder} at step {ckpt.active_learning_step_idx}, "
                           f"phase {ckpt.active_learning_phase}")
        if blob.get("training_epoch") is not None:
            driver.logger.info(f"Resuming from training epoch {blob['training_epoch']}")
        return driver

    # ---- distributed plumbing -------------------------------------------------------------------------
    def barrier(self) -> None:
        if not (dist.is_available() and dist.is_initialized()):
            return
        if self.dist_manager is not None and self.dist_manager.device.type == "cuda":
            dist.barrier(device_ids=[self.dist_manager.local_rank])
        elif torch.get_default_device().type == "cuda":
            dist.barrier(device_ids=[torch.cuda.current_device()])
        else:
            dist.barrier()

    def _configure_model(self) -> None:
        if self._dist_active():
            dm = self.dist_manager
            if dm.world_size > 1 and not isinstance(self.learner, DistributedDataParallel):
                on_gpu = dm.device.type == "cuda"
                self.learner = DistributedDataParallel(
                    self.learner, device_ids=[dm.local_rank] if on_gpu else None,
                    output_device=dm.device if on_gpu else None, broadcast_buffers=dm.broadcast_buffers,
                    find_unused_parameters=dm.find_unused_parameters)
        elif self.config.device is not None:
            self.learner = self.learner.to(self.config.device, self.config.dtype)
        if not self.config.skip_training and not self.is_optimizer_configured:
            self.configure_optimizer()
        if self.is_optimizer_configured and self.config.reset_optim_states:
            self.optimizer.load_state_dict(self._original_optim_state)

    def _construct_dataloader(self, pool, shuffle: bool = False, drop_last: bool = False) -> DataLoader:
        sampler = None
        pin = False
        if self._dist_active():
            dm = self.dist_manager
            sampler = DistributedSampler(pool, num_replicas=dm.world_size, rank=dm.rank, shuffle=shuffle,
                                         drop_last=drop_last)
            shuffle = None
            pin = dm.device.type == "cuda"
        workers = self.config.num_dataloader_workers
        return DataLoader(pool, shuffle=shuffle, sampler=sampler, collate_fn=self.config.collate_fn,
                          batch_size=self.config.batch_size, num_workers=workers, persistent_workers=workers > 0,
                          pin_memory=pin)

    # ---- the step -------------------------------------------------------------------------------------
    def _get_phase_index(self, phase) -> int:
        if phase is None:
            return 0
        try:
            return self._PHASE_ORDER.index(p.ActiveLearningPhase(phase))
        except ValueError:
            self.logger.warning(f"Unknown phase {phase}, defaulting to start from beginning")
            return 0

    def _build_phase_queue(self, train_step_fn, validate_step_fn, args: tuple, kwargs: dict) -> list:
        cfg = self.config
        plan = [
            (p.ActiveLearningPhase.TRAINING, lambda: self._training_phase(train_step_fn, validate_step_fn, *args, **kwargs),
             not cfg.skip_training),
            (p.ActiveLearningPhase.METROLOGY, lambda: self._metrology_phase(*args, **kwargs),
             not cfg.skip_metrology and bool(self.metrology_strategies)),
            (p.ActiveLearningPhase.QUERY, lambda: self._query_phase(*args, **kwargs), True),
            (p.ActiveLearningPhase.LABELING, lambda: self._labeling_phase(*args, **kwargs), not cfg.skip_labeling),
        ]
        start = self._get_phase_index(self.current_phase)
        if start > 0:
            self.logger.info(f"Resuming AL step {self.active_learning_step_idx} from {self.current_phase}")
        queue = []
        for idx, (phase, fn, enabled) in enumerate(plan):
            if idx < start:
                self.logger.debug(f"Skipping {phase} (already completed in this AL step)")
            elif enabled:
                queue.append(fn)
            else:
                self.logger.debug(f"Skipping {phase} (disabled in config)")
        return queue

    def active_learning_step(self, train_step_fn=None, validate_step_fn=None, *args: Any, **kwargs: Any) -> None:
        self._setup_active_learning_step()
        for phase_fn in self._build_phase_queue(train_step_fn, validate_step_fn, args, kwargs):
            phase_fn()
        self.current_phase = None
        self.logger.debug("Entering barrier for synchronization.")
        self.barrier()
        self.active_learning_step_idx += 1
        self.logger.info(f"Completed active learning step {self.active_learning_step_idx}")

    def _setup_active_learning_step(self) -> None:
        if self.dist_manager is not None and not self.dist_manager.is_initialized():
            self.logger.info("Distributed manager configured but not initialized; initializing.")
            self.dist_manager.initialize()
        self._configure_model()
        self.logger.info(f"Starting active learning step {self.active_learning_step_idx}")

    def _remaining_epochs(self, target: int) -> tuple[int, int]:
        """(first epoch to run, number of epochs left) given the last checkpoint's ``training_state.pt``."""
        last = self._last_checkpoint_path
        if last and (last / "training_state.pt").exists():
            state = torch.load(last / "training_state.pt", map_location="cpu", weights_only=False)
            done = state.get("training_epoch") or 0
            if done > 0:
                return done + 1, target - done
        return 1, target

    def _training_phase(self, train_step_fn, validate_step_fn, *args: Any, **kwargs: Any) -> None:
        self._validate_training_requirements(train_step_fn, validate_step_fn)
        with self._phase_context(p.ActiveLearningPhase.TRAINING, call_barrier=False):
            train_loader = self._construct_dataloader(self.train_datapool, shuffle=True)
            self.logger.info(f"There are {len(train_loader)} batches in the training loader.")
            val_loader = None
            if self.val_datapool is not None:
                if validate_step_fn or hasattr(self.learner, "validation_step"):
                    val_loader = self._construct_dataloader(self.val_datapool, shuffle=False)
                else:
                    self.logger.warning("Validation data is available, but no `validate_step_fn` or "
                                        "`validation_step` method in Learner is provided.")
            later = self.active_learning_step_idx > 0
            if later and self.config.fine_tuning_lr is not None:
                self.optimizer.param_groups[0]["lr"] = self.config.fine_tuning_lr
            tc = self.training_config
            target = tc.max_fine_tuning_epochs if later else tc.max_training_epochs
            start_epoch, todo = self._remaining_epochs(target)
            if start_epoch > 1:
                self.logger.info(f"Resuming training from epoch {start_epoch} ({todo} epochs remaining)")
            if todo <= 0:
                self.logger.info(f"Training already complete ({target} epochs), skipping training phase")
                return
            loop = self.train_loop_fn
            if hasattr(loop, "checkpoint_base_dir") and hasattr(loop, "checkpoint_frequency"):
                loop.checkpoint_base_dir = (self.log_dir / "checkpoints" / f"step_{self.active_learning_step_idx}"
                                            / "training")
                loop.checkpoint_frequency = self.config.model_checkpoint_frequency
            loop(self.learner, self.optimizer, train_step_fn=train_step_fn, validate_step_fn=validate_step_fn,
                 train_dataloader=train_loader, validation_dataloader=val_loader, lr_scheduler=self.lr_scheduler,
                 max_epochs=todo, device=self.dist_manager.device if self.dist_manager is not None else self.config.device,
                 dtype=self.config.dtype, **kwargs)

    def _metrology_phase(self, *args: Any, **kwargs: Any) -> None:
        with self._phase_context(p.ActiveLearningPhase.METROLOGY):
            for strategy in self.metrology_strategies or []:
                name = type(strategy).__name__
                self.logger.info(f"Running metrology strategy: {name}")
                strategy(*args, **kwargs)
                self.logger.info(f"Completed metrics for strategy: {name}")
                strategy.serialize_records(*args, **kwargs)

    def _query_phase(self, *args: Any, **kwargs: Any) -> None:
        with self._phase_context(p.ActiveLearningPhase.QUERY):
            for strategy in self.query_strategies:
                self.logger.info(f"Running query strategy: {type(strategy).__name__}")
                strategy(self.query_queue, *args, **kwargs)
            if self.query_queue.empty():
                self.logger.warning("Querying strategies produced no samples this iteration.")

    def _labeling_phase(self, *args: Any, **kwargs: Any) -> None:
        self._validate_labeling_requirements()
        if self.query_queue.empty():
            self.logger.warning("No samples to label. Skipping labeling phase.")
            return
        with self._phase_context(p.ActiveLearningPhase.LABELING):
            try:
                self.label_strategy(self.query_queue, self.label_queue, *args, **kwargs)
            except Exception as e:  # noqa: BLE001
                self.logger.error(f"Exception encountered during labeling: {e}")
            self.logger.info("Labeling completed. Now appending to training pool.")
            added = 0
            while not self.label_queue.empty():
                self.train_datapool.append(self.label_queue.get())
                added += 1
            self.logger.info(f"Appended {added} samples to training pool.")

    def _validate_training_requirements(self, train_step_fn, validate_step_fn) -> None:
        if self.training_config is None:
            raise ValueError("`training_config` must be provided if `skip_training` is False.")
        if self.train_loop_fn is None:
            raise ValueError("`train_loop_fn` must be provided in training_config.")
        if self.train_datapool is None:
            raise ValueError("`train_datapool` must be provided in training_config.")
        if not train_step_fn and not hasattr(self.learner, "training_step") \
                and getattr(self.train_loop_fn, "train_step_fn", None) is None:
            raise ValueError("`train_step_fn` must be provided if the model does not implement the "
                             "`training_step` method.")
        if validate_step_fn and self.val_datapool is None:
            raise ValueError("`val_datapool` must be provided in training_config if `validate_step_fn` is provided.")

    def _validate_labeling_requirements(self) -> None:
        if self.label_strategy is None:
            raise ValueError("`label_strategy` must be provided in strategies_config if `skip_labeling` is False.")
        if self.training_config is None or self.train_datapool is None:
            raise ValueError("`train_datapool` must be provided in training_config for labeling, as data will be "
                             "appended to it.")

    @contextmanager
    def _phase_context(self, phase_name, call_barrier: bool = True) -> Generator[None, Any, None]:
        phase = p.ActiveLearningPhase(phase_name)
        self.current_phase = phase
        if phase is not p.ActiveLearningPhase.TRAINING:
            if getattr(self.config, f"checkpoint_on_{phase.value}", False) and self._should_checkpoint_at_step():
                self.save_checkpoint()
        try:
            yield
        except Exception as e:
            self.logger.error(f"Exception encountered during {phase}: {e}")
            raise
        finally:
            if call_barrier:
                self.logger.debug("Entering barrier for synchronization.")
                self.barrier()

    def run(self, train_step_fn=None, validate_step_fn=None, *args: Any, **kwargs: Any) -> None:
        while self.active_learning_step_idx < self.config.max_active_learning_steps:
            self.active_learning_step(train_step_fn, validate_step_fn, *args, **kwargs)

    def __call__(self, train_step_fn=None, validate_step_fn=None, *args: Any, **kwargs: Any) -> None:
        self.run(train_step_fn, validate_step_fn, *args, **kwargs)

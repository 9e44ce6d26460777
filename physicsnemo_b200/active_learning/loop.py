"""Default epoch loop used by the active-learning driver.

Parity: ``physicsnemo/active_learning/loop.py`` (``DefaultTrainingLoop``: optional static capture of
the step functions, device / dtype casting of nested batches, ``LaunchLogger`` epochs, periodic
training checkpoints ``model.mdlus`` / ``model_state.pt`` + ``training_state.pt``).

When static capture is on, the captured step owns backward and the optimizer step (forward,
backward and update replay as one CUDA graph on a GPU); the loop then only advances the
scheduler.  Without capture the loop calls ``backward`` and ``optimizer.step`` itself.
Batches are moved with ``non_blocking=True`` so a pinned-memory loader overlaps the copy of
batch *i+1* with the step of batch *i*.
"""
from __future__ import annotations

from pathlib import Path
from typing import Any

import torch

from ..core import Module
from ..distributed import DistributedManager
from ..utils.capture import StaticCaptureEvaluateNoGrad, StaticCaptureTraining
from ..utils.logging import LaunchLogger
from . import protocols as p

__all__ = ["DefaultTrainingLoop"]


def _recursive_data_device_cast(data: Any, device=None, dtype=None, **kwargs: Any) -> Any:
    """Move every tensor-like leaf of a nested dict / list / tuple; floating tensors also change dtype."""
    kwargs.setdefault("non_blocking", True)
    if isinstance(data, torch.Tensor):
        return data.to(device=device, dtype=dtype if data.is_floating_point() else None, **kwargs)
    if hasattr(data, "to"):
        return data.to(device=device, dtype=dtype, **kwargs)
    if isinstance(data, dict):
        return {k: _recursive_data_device_cast(v, device, dtype, **kwargs) for k, v in data.items()}
    if isinstance(data, list):
        return [_recursive_data_device_cast(v, device, dtype, **kwargs) for v in data]
    if isinstance(data, tuple):
        return tuple(_recursive_data_device_cast(v, device, dtype, **kwargs) for v in data)
    return data


def _progress(iterable, enabled: bool, **kw):
    if not enabled:
        return iterable
    try:
        from tqdm import tqdm
    except ImportError:
        return iterable
    return tqdm(iterable, leave=False, **kw)


def _encode_arg(name: str, value: Any) -> Any:
    if name in ("device", "dtype") and isinstance(value, (torch.device, torch.dtype)):
        return str(value)
    return value


class DefaultTrainingLoop(p.TrainingLoop):
    def __new__(cls, *args: Any, **kwargs: Any):
        out = object.__new__(cls)
        out._args = p.capture_init_args(cls, args, kwargs, encode=_encode_arg)
        return out

    def __init__(self, train_step_fn=None, validate_step_fn=None, enable_static_capture: bool = True,
                 use_progress_bars: bool = True, device=None, dtype=None, checkpoint_frequency: int = 0,
                 **capture_kwargs: Any) -> None:
        self.train_step_fn = train_step_fn
        self.validate_step_fn = validate_step_fn
        self.enable_static_capture = enable_static_capture
        if isinstance(device, str):
            device = torch.device(device)
        if device is None and DistributedManager.is_initialized():
            device = DistributedManager().device
        self.device = device
        if isinstance(dtype, str):
            dtype = getattr(torch, dtype.replace("torch.", ""))
        self.dtype = dtype if dtype is not None else torch.get_default_dtype()
        self.capture_kwargs = capture_kwargs
        self.use_progress_bars = use_progress_bars
        self.capture_functions: dict[int, Any] = {}
        self.checkpoint_frequency = checkpoint_frequency
        self.checkpoint_base_dir: Path | None = None

    # ---- checkpoints --------------------------------------------------------------------------------
    def save_training_checkpoint(self, checkpoint_dir: Path, model, optimizer, lr_scheduler=None,
                                 training_epoch: int | None = None) -> None:
        checkpoint_dir.mkdir(parents=True, exist_ok=True)
        if isinstance(model, Module):
            model.save(str(checkpoint_dir / "model.mdlus"))
        else:
            torch.save(model.state_dict(), checkpoint_dir / "model_state.pt")
        torch.save({"optimizer_state": optimizer.state_dict(),
                    "lr_scheduler_state": lr_scheduler.state_dict() if lr_scheduler else None,
                    "training_epoch": training_epoch}, checkpoint_dir / "training_state.pt")

    @staticmethod
    def load_training_checkpoint(checkpoint_dir: Path, model, optimizer, lr_scheduler=None) -> int | None:
        if isinstance(model, Module):
            if (checkpoint_dir / "model.mdlus").exists():
                model.load(str(checkpoint_dir / "model.mdlus"))
        elif (checkpoint_dir / "model_state.pt").exists():
            model.load_state_dict(torch.load(checkpoint_dir / "model_state.pt", map_location="cpu"))
        path = checkpoint_dir / "training_state.pt"
        if not path.exists():
            return None
        state = torch.load(path, map_location="cpu", weights_only=False)
        if "optimizer_state" in state:
            optimizer.load_state_dict(state["optimizer_state"])
        if lr_scheduler and state.get("lr_scheduler_state"):
            lr_scheduler.load_state_dict(state["lr_scheduler_state"])
        return state.get("training_epoch")

    # ---- capture ------------------------------------------------------------------------------------
    @property
    def amp_type(self) -> torch.dtype:
        return self.dtype if self.dtype in (torch.float16, torch.bfloat16) else torch.float16

    def _captured(self, fn, factory):
        key = id(fn)
        if key not in self.capture_functions:
            try:
                self.capture_functions[key] = factory()(fn)
            except Exception as e:
                raise RuntimeError(f"Failed to create static capture for `{getattr(fn, '__name__', fn)}`. ") from e
        return self.capture_functions[key]

    def _create_capture_functions(self, model, optimizer, train_step_fn=None, validate_step_fn=None):
        train_step_fn = train_step_fn or self.train_step_fn
        train = self._captured(train_step_fn, lambda: StaticCaptureTraining(
            model=model, optim=optimizer, amp_type=self.amp_type, **self.capture_kwargs))
        validate_step_fn = validate_step_fn or self.validate_step_fn
        validate = None
        if validate_step_fn:
            validate = self._captured(validate_step_fn, lambda: StaticCaptureEvaluateNoGrad(
                model=model, amp_type=self.amp_type, **self.capture_kwargs))
        return train, validate

    # ---- the loop -----------------------------------------------------------------------------------
    def __call__(self, model, optimizer, train_dataloader, max_epochs: int, validation_dataloader=None,
                 train_step_fn=None, validate_step_fn=None, lr_scheduler=None, device=None, dtype=None,
                 *args: Any, **kwargs: Any) -> None:
        train_step_fn = train_step_fn or self.train_step_fn
        validate_step_fn = validate_step_fn or self.validate_step_fn
        if train_step_fn is None:
            raise RuntimeError("No training step function: pass `train_step_fn` to the loop or to its constructor.")
        device = device or self.device or torch.get_default_device()
        dtype = dtype or self.dtype or torch.get_default_dtype()
        if device and torch.device(device) != getattr(model, "device", None):
            model = model.to(device)
        captured = self.enable_static_capture
        if captured:
            train_step_fn, validate_step_fn = self._create_capture_functions(model, optimizer, train_step_fn,
                                                                             validate_step_fn)
        for epoch in _progress(range(1, max_epochs + 1), self.use_progress_bars, desc="Epoch", position=0):
            model.train()
            with LaunchLogger("train", epoch=epoch, num_mini_batch=len(train_dataloader)) as log:
                for batch in _progress(train_dataloader, self.use_progress_bars, desc="Training step", unit="batch"):
                    batch = _recursive_data_device_cast(batch, device=device, dtype=dtype)
                    if not captured:
                        model.zero_grad(set_to_none=True)
                    loss = train_step_fn(model, batch, *args, **kwargs)
                    if not captured:
                        loss.backward()
                        optimizer.step()
                    log.log_minibatch({"train_loss": loss.detach().item()})
                    if lr_scheduler:
                        lr_scheduler.step()
            if validate_step_fn and validation_dataloader:
                model.eval()
                with LaunchLogger("validation", epoch=epoch, num_mini_batch=len(validation_dataloader)):
                    for batch in _progress(validation_dataloader, self.use_progress_bars, desc="Validation step",
                                           unit="batch"):
                        batch = _recursive_data_device_cast(batch, device=device, dtype=dtype)
                        if captured:
                            validate_step_fn(model, batch, *args, **kwargs)
                        else:
                            with torch.no_grad():
                                validate_step_fn(model, batch, *args, **kwargs)
            if self.checkpoint_base_dir and self.checkpoint_frequency > 0 and epoch % self.checkpoint_frequency == 0:
                self.save_training_checkpoint(self.checkpoint_base_dir / f"epoch_{epoch}", model, optimizer,
                                              lr_scheduler, training_epoch=epoch)

"""Static capture of training / evaluation steps: CUDA graphs + AMP + gradient scaling.

Parity: ``physicsnemo/utils/capture.py`` — ``_StaticCapture`` (``:35-338``),
``StaticCaptureTraining`` (``:341-435``), ``StaticCaptureEvaluateNoGrad`` (``:438-``): a decorator
around the forward(+loss) function; the first ``cuda_graph_warmup`` calls run eagerly on a
side stream, then forward + backward are captured into one CUDA graph and replayed; the
optimizer step (through the ``GradScaler``) stays outside the graph.  Scaler states are
kept per ``label`` so that checkpoints can restore them (``:270-338``).

CUDA graphs, not a tracing compiler, are this framework's way of removing launch overhead
from inner loops, so the ``compile`` flag is accepted and ignored.
"""
from __future__ import annotations

import functools
import logging
import os
import time
from contextlib import nullcontext
from logging import Logger
from typing import Any, Callable, Dict, NewType, Optional, Union

import torch

from ..core.module import Module

float16 = NewType("float16", torch.float16)
bfloat16 = NewType("bfloat16", torch.bfloat16)


class _StaticCapture:
    """Base of the capture decorators."""

    _amp_scalers: Dict[str, Any] = {}
    _amp_scaler_checkpoints: Dict[str, Any] = {}
    _logger = logging.getLogger("capture")

    def __new__(cls, *args, **kwargs):
        obj = super().__new__(cls)
        obj.amp_scalers = cls._amp_scalers
        obj.amp_scaler_checkpoints = cls._amp_scaler_checkpoints
        obj.logger = cls._logger
        return obj

    def __init__(self, model, optim=None, logger: Optional[Logger] = None, use_graphs: bool = True,
                 use_autocast: bool = True, use_gradscaler: bool = True, compile: bool = False,
                 cuda_graph_warmup: int = 11, amp_type=torch.float16, gradient_clip_norm: Optional[float] = None,
                 label: Optional[str] = None):
        self.logger = logger if logger else self.logger
        self.label = label if label else f"scaler_{len(self.amp_scalers.keys())}"
        if not isinstance(model, Module) and hasattr(model, "module"):
            model = model.module
        if not isinstance(model, Module):
            self.logger.error("Model not a PhysicsNeMo Module!")
            raise ValueError("Model not a PhysicsNeMo Module!")
        self.model, self.optim = model, optim
        self.eval = self.no_grad = False
        self.gradient_clip_norm = gradient_clip_norm
        if amp_type not in (torch.float16, torch.bfloat16):
            raise ValueError("AMP type must be torch.float16 or torch.bfloat16")
        meta = model.meta
        if "cuda" in str(model.device):
            if use_graphs and not (meta and meta.cuda_graphs):
                self.logger.warning(f"Model {type(model).__name__} does not support CUDA graphs, turning off")
                use_graphs = False
            self.cuda_graphs_enabled = use_graphs
            if not (meta and meta.amp_gpu):
                self.logger.warning(f"Model {type(model).__name__} does not support AMP on GPUs, turning off")
                use_autocast = use_gradscaler = False
            self.use_gradscaler, self.use_autocast, self.amp_device = use_gradscaler, use_autocast, "cuda"
            if amp_type == torch.bfloat16 and not torch.cuda.is_bf16_supported():
                amp_type = torch.float16
            self.amp_dtype = amp_type
            self.scaler = self._init_amp_scaler(use_gradscaler and amp_type == torch.float16, self.logger)
            self.replay_stream = torch.cuda.Stream(model.device)
        else:
            self.cuda_graphs_enabled = False
            if use_autocast and not (meta and meta.amp_cpu):
                self.logger.warning(f"Model {type(model).__name__} does not support AMP on CPUs, turning off")
                use_autocast = False
            self.use_autocast, self.amp_device = use_autocast, "cpu"
            self.amp_dtype = torch.bfloat16
            self.scaler = self._init_amp_scaler(False, self.logger)
            self.replay_stream = None
        if self.cuda_graphs_enabled:
            self.graph = torch.cuda.CUDAGraph()
        self.output = None
        self.iteration = 0
        self.cuda_graph_warmup = cuda_graph_warmup

    def __call__(self, fn: Callable) -> Callable:
        self.function = fn

        @functools.wraps(fn)
        def decorated(*args, **kwds):
            with torch.no_grad() if self.no_grad else nullcontext():
                if self.cuda_graphs_enabled:
                    self._cuda_graph_forward(*args, **kwds)
                else:
                    self._zero_grads()
                    self.output = self._amp_forward(*args, **kwds)
                if not self.eval:
                    self.scaler.step(self.optim)
                    self.scaler.update()
            return self.output

        return decorated

    def _cuda_graph_forward(self, *args, **kwargs):
        if self.iteration < self.cuda_graph_warmup:
            self.replay_stream.wait_stream(torch.cuda.current_stream())
            self._zero_grads()
            with torch.cuda.stream(self.replay_stream):
                output = self._amp_forward(*args, **kwargs)
                self.output = output.detach() if isinstance(output, torch.Tensor) else output
            torch.cuda.current_stream().wait_stream(self.replay_stream)
        elif self.iteration == self.cuda_graph_warmup:
            torch.cuda.synchronize()
            if torch.distributed.is_initialized():
                torch.distributed.barrier()
            delay = os.environ.get("PHYSICSNEMO_CUDA_GRAPH_CAPTURE_DELAY", "10")
            time.sleep(int(delay))
            with torch.cuda.graph(self.graph):
                output = self._amp_forward(*args, **kwargs)
                self.output = output.detach() if isinstance(output, torch.Tensor) else output
            self.graph.replay()
        else:
            self.graph.replay()
        self.iteration += 1

    def _zero_grads(self):
        if self.eval:
            return
        try:
            self.optim.zero_grad(set_to_none=True)
        except Exception:
            if self.optim:
                self.optim.zero_grad()
        self.model.zero_grad(set_to_none=True)

    def _amp_forward(self, *args, **kwargs) -> Any:
        with torch.autocast(self.amp_device, enabled=self.use_autocast, dtype=self.amp_dtype):
            output = self.function(*args, **kwargs)
        if not self.eval:
            self.scaler.scale(output).backward()
            if self.gradient_clip_norm is not None:
                self.scaler.unscale_(self.optim)
                torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.gradient_clip_norm)
        return output

    def _init_amp_scaler(self, scaler_enabled: bool, logger: Logger):
        if self.label in self.amp_scalers:
            raise ValueError(f"Static capture with label {self.label} already exists; labels must be unique")
        scaler = torch.amp.GradScaler(self.amp_device if self.amp_device == "cuda" else "cpu", enabled=scaler_enabled)
        self.amp_scalers[self.label] = scaler
        if self.label in self.amp_scaler_checkpoints:
            try:
                scaler.load_state_dict(self.amp_scaler_checkpoints[self.label])
                del self.amp_scaler_checkpoints[self.label]
            except Exception as exc:  # noqa: BLE001
                logger.error(f"Failed to load grad scaler state for {self.label}: {exc}")
        return scaler

    @classmethod
    def state_dict(cls) -> Dict[str, Any]:
        return {k: v.state_dict() for k, v in cls._amp_scalers.items()}

    @classmethod
    def load_state_dict(cls, state_dict: Dict[str, Any]) -> None:
        for key, value in state_dict.items():
            cls._amp_scaler_checkpoints[key] = value
            if key in cls._amp_scalers:
                try:
                    cls._amp_scalers[key].load_state_dict(value)
                    del cls._amp_scaler_checkpoints[key]
                except Exception as exc:  # noqa: BLE001
                    cls._logger.warning(f"Failed to load scaler state for {key}: {exc}")

    @classmethod
    def reset_state(cls):
        cls._amp_scalers = {}
        cls._amp_scaler_checkpoints = {}


class StaticCaptureTraining(_StaticCapture):
    """Decorator for a function that returns the loss; runs forward, backward and the optimizer step."""

    def __init__(self, model, optim, logger: Optional[Logger] = None, use_graphs: bool = True, use_amp: bool = True,
                 compile: bool = False, cuda_graph_warmup: int = 11, amp_type=torch.float16,
                 gradient_clip_norm: Optional[float] = None, label: Optional[str] = None):
        super().__init__(model, optim, logger, use_graphs, use_amp, use_amp, compile, cuda_graph_warmup, amp_type,
                         gradient_clip_norm, label)


class StaticCaptureEvaluateNoGrad(_StaticCapture):
    """Decorator for an inference function; no gradients, no optimizer."""

    def __init__(self, model, logger: Optional[Logger] = None, use_graphs: bool = True, use_amp: bool = True,
                 compile: bool = False, cuda_graph_warmup: int = 11, amp_type=torch.float16,
                 label: Optional[str] = None):
        super().__init__(model, None, logger, use_graphs, use_amp, False, compile, cuda_graph_warmup, amp_type,
                         None, label)
        self.eval = True
        self.no_grad = True


class GraphedStep:
    """A whole training step — forward, backward, gradient reduction, optimizer — as one CUDA graph.

    ``step_fn(*inputs)`` is run ``warmup`` times on a side stream, then captured once with the tensors in
    ``static_inputs`` as its arguments; calling the object copies new inputs into those tensors (from pinned host
    memory this is an asynchronous copy on the current stream), replays the graph and returns the captured outputs
    (static tensors, overwritten by the next replay).  One replay costs one launch on the host, so steps whose
    kernels are shorter than the per-launch host overhead (small shards, many ranks) stop being host-bound.

    Requirements on ``step_fn``: no host synchronisation and no host-computed scalar that changes from step to step
    (use ``FusedAdam(capturable=True)``; the peer collectives keep their call counter on the device).
    """

    def __init__(self, step_fn: Callable, static_inputs, warmup: int = 3, pool=None):
        if not torch.cuda.is_available():
            raise RuntimeError("GraphedStep needs a CUDA device")
        self.step_fn = step_fn
        self.static_inputs = list(static_inputs)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(int(warmup), 1)):
                step_fn(*self.static_inputs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, pool=pool):
            self.static_outputs = step_fn(*self.static_inputs)
        self.replays = 0

    def __call__(self, *inputs):
        if inputs:
            if len(inputs) != len(self.static_inputs):
                raise ValueError(f"expected {len(self.static_inputs)} inputs, got {len(inputs)}")
            for dst, src in zip(self.static_inputs, inputs):
                if src is not dst:
                    dst.copy_(src, non_blocking=True)
        self.graph.replay()
        self.replays += 1
        return self.static_outputs

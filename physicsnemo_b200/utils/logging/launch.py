"""``LaunchLogger``: per-namespace epoch / mini-batch logging context manager.

Parity: ``physicsnemo/utils/logging/launch.py:35-449`` — ``log_minibatch``, ``log_epoch``, epoch
timing with CUDA events, cross-rank averaging of mini-batch losses through ``reduce_loss``,
optional back ends (console always; Weights & Biases / MLflow when installed and
initialised), ``profile=True`` wrapping the epoch in NVTX emission, ``toggle_*`` class methods.
"""
from __future__ import annotations

import re
import sys
import time
from os import getcwd, makedirs
from os.path import abspath, exists, join
from typing import Dict, Tuple, Union

import torch

from ...distributed.manager import DistributedManager
from ...distributed.utils import reduce_loss
from .console import PythonLogger


class LaunchLogger:
    _instances: Dict[str, "LaunchLogger"] = {}
    console_backend = True
    wandb_backend = False
    mlflow_backend = False
    tensorboard_backend = False
    enable_profiling = False
    mlflow_run = None
    mlflow_client = None

    def __new__(cls, name_space, *args, **kwargs):
        if name_space in cls._instances:
            return cls._instances[name_space]
        self = super().__new__(cls)
        cls._instances[name_space] = self
        self.pyLogger = PythonLogger(name_space)
        self.total_iteration_index = None
        self.root = True
        if DistributedManager.is_initialized():
            self.root = DistributedManager().rank == 0
        self.mini_batch_log_freq = 100
        self._initialized = False
        return self

    def __init__(self, name_space: str, epoch: int = 1, num_mini_batch: Union[int, None] = None,
                 profile: bool = False, mini_batch_log_freq: int = 100, epoch_alert_freq: Union[int, None] = None):
        self.name_space = name_space
        self.mini_batch_index = 0
        self.minibatch_losses: Dict[str, float] = {}
        self.epoch_losses: Dict[str, float] = {}
        self.mini_batch_log_freq = mini_batch_log_freq
        self.epoch_alert_freq = epoch_alert_freq
        self.epoch = epoch
        self.num_mini_batch = num_mini_batch
        self.profile = profile
        if self.total_iteration_index is None:
            self.total_iteration_index = 0 if num_mini_batch is None else (epoch - 1) * num_mini_batch
        self.device = DistributedManager().device if DistributedManager.is_initialized() else torch.device("cpu")
        self.max_memory = 0

    def log_minibatch(self, losses: Dict[str, float]):
        self.mini_batch_index += 1
        self.total_iteration_index += 1
        for name, value in losses.items():
            self.minibatch_losses[name] = self.minibatch_losses.get(name, 0.0) + float(value)
        if self.mini_batch_index % self.mini_batch_log_freq == 0:
            mb_metrics = {n: v / self.mini_batch_index for n, v in self.minibatch_losses.items()}
            msg = f"Mini-Batch Losses:"
            for n, v in mb_metrics.items():
                msg += f" {n} = {v:10.3e},"
            self.pyLogger.log(f"Epoch {self.epoch} [{self.mini_batch_index}" + (f"/{self.num_mini_batch}" if self.num_mini_batch else "") + f"] {msg}")
            self._log_backends(mb_metrics, step=("mini_batch", self.total_iteration_index))

    def log_epoch(self, losses: Dict[str, float]):
        for name, value in losses.items():
            self.epoch_losses[name] = float(value)

    def __enter__(self):
        self.mini_batch_index = 0
        self.minibatch_losses = {}
        self.epoch_losses = {}
        if self.profile and torch.cuda.is_available():
            self.profiler = torch.autograd.profiler.emit_nvtx(enabled=self.enable_profiling)
            self.profiler.__enter__()
            torch.cuda.profiler.start()
        if torch.cuda.is_available() and self.device.type == "cuda":
            self.start_event = torch.cuda.Event(enable_timing=True)
            self.end_event = torch.cuda.Event(enable_timing=True)
            self.start_event.record()
        else:
            self.start_event = time.time()
        return self

    def __exit__(self, exc_type, exc_value, exc_tb):
        metrics = dict(self.epoch_losses)
        if self.mini_batch_index > 0:
            for name, value in self.minibatch_losses.items():
                mean = value / self.mini_batch_index
                if DistributedManager.is_initialized() and DistributedManager().distributed and torch.distributed.is_initialized():
                    reduced = reduce_loss(mean, dst_rank=0, mean=True)
                    mean = reduced if reduced is not None else mean
                metrics[name] = mean
        if self.profile and torch.cuda.is_available():
            self.profiler.__exit__(exc_type, exc_value, exc_tb)
            torch.cuda.profiler.stop()
        if isinstance(self.start_event, float):
            epoch_time = time.time() - self.start_event
        else:
            self.end_event.record()
            torch.cuda.synchronize()
            epoch_time = self.start_event.elapsed_time(self.end_event) / 1000.0
            self.max_memory = torch.cuda.max_memory_allocated(self.device) / (1024.0 ** 3)
        if self.root:
            msg = f"Epoch {self.epoch} Metrics:"
            for n, v in metrics.items():
                msg += f" {n} = {v:10.3e},"
            self.pyLogger.info(msg)
            t = f"Epoch Execution Time: {epoch_time:10.3e}s"
            if self.mini_batch_index > 0:
                t += f", Time/Iter: {epoch_time / self.mini_batch_index * 1000:10.3e}ms"
            self.pyLogger.info(t)
            if self.max_memory:
                self.pyLogger.info(f"GPU memory allocated: {self.max_memory:10.3e} GB")
            self._log_backends(metrics, step=("epoch", self.epoch))
        if self.epoch_alert_freq and self.root and self.epoch % self.epoch_alert_freq == 0 and self.wandb_backend:
            from .wandb import alert

            alert(title=f"{sys.argv[0]} training progress report", text=f"Run reached epoch {self.epoch}")

    def _log_backends(self, metric_dict: Dict[str, float], step: Tuple[str, int] = None):
        if self.wandb_backend:
            import wandb

            d = {f"{self.name_space}/{k}": v for k, v in metric_dict.items()}
            if step:
                d[step[0]] = step[1]
            wandb.log(d)
        if self.mlflow_backend and self.mlflow_client is not None:
            for k, v in metric_dict.items():
                name = re.sub(r"[^a-zA-Z0-9_\-\.\s/]+", "", f"{self.name_space}/{k}")
                self.mlflow_client.log_metric(self.mlflow_run.info.run_id, key=name, value=v, step=step[1] if step else 0)

    def log_figure(self, figure, artifact_file: str = "artifact", plot_dir: str = "./", log_to_file: bool = False):
        dist_rank = DistributedManager().rank if DistributedManager.is_initialized() else 0
        if dist_rank != 0:
            return
        if self.wandb_backend:
            import wandb

            wandb.log({artifact_file: wandb.Image(figure)})
        if log_to_file:
            plot_dir = abspath(join(getcwd(), plot_dir))
            if not exists(plot_dir):
                makedirs(plot_dir)
            figure.savefig(join(plot_dir, artifact_file + ".png"))

    @classmethod
    def toggle_wandb(cls, value: bool):
        cls.wandb_backend = value

    @classmethod
    def toggle_mlflow(cls, value: bool):
        cls.mlflow_backend = value

    @staticmethod
    def initialize(use_wandb: bool = False, use_mlflow: bool = False):
        """Enable the optional back ends when their packages are importable."""
        if use_wandb:
            try:
                import wandb  # noqa: F401

                LaunchLogger.toggle_wandb(wandb.run is not None)
            except ImportError:
                PythonLogger().warning("WandB not installed; logging to console only")
        if use_mlflow:
            LaunchLogger.toggle_mlflow(LaunchLogger.mlflow_run is not None and LaunchLogger.mlflow_client is not None)

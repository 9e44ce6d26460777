"""Timing, clock sampling and bookkeeping shared by the benchmark configurations."""
from __future__ import annotations

import statistics
import subprocess
import threading
import time
from typing import Callable, Optional

import torch


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def timed_loop(step_fn: Callable[[], None], steps: int, warmup: int, world: int, dev, flush_buf: Optional[torch.Tensor] = None):
    """``warmup`` untimed calls, then ``steps`` calls each bracketed by CUDA events; returns (ms per step as the max over
    ranks, wall seconds of the timed region).  ``flush_buf`` (larger than L2) is rewritten between timed iterations."""
    import torch.distributed as dist

    for _ in range(warmup):
        step_fn()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    t0 = time.perf_counter()
    for i in range(steps):
        if flush_buf is not None:
            flush_buf.add_(1.0)  # evict L2 between timed iterations (outside the event pair)
        ev[i][0].record()
        step_fn()
        ev[i][1].record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    ms = sum(a.elapsed_time(b) for a, b in ev)
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item() / steps, wall


def flush_buffer(dev) -> torch.Tensor:
    """256 MB of fp32 (> the 126 MB L2)."""
    return torch.empty(256 * 1024 * 1024 // 4, device=dev)


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """max |a - b| / max |b| in fp32 (0 when both vanish)."""
    a, b = a.detach().float(), b.detach().float()
    den = b.abs().max().item()
    num = (a - b).abs().max().item()
    return num / den if den > 0 else num


def base_line(metric_value: float, ms: float, world: int, args, scaling: str, data: str, config: dict, clocks, e2e: dict,
              launches_per_step: int, extra: Optional[dict] = None) -> dict:
    out = {
        "metric": "train samples/sec (device-timed, max over ranks)", "value": metric_value, "unit": "samples/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": scaling, "vs_baseline": None, "dtype": "bf16", "data": data, "config": config, "clocks": clocks,
        "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "gpu_launches_per_step": launches_per_step,
        "impl": "physicsnemo_b200",
    }
    if extra:
        out.update(extra)
    return out


def domain_mesh(world: int):
    """The 1-D ``("domain",)`` device mesh over all ranks (created once per process through ``DistributedManager``)."""
    from ..distributed import DistributedManager

    if not DistributedManager.is_initialized():
        DistributedManager.initialize()
    dm = DistributedManager()
    mesh = getattr(dm, "_global_mesh", None)
    if mesh is None:
        mesh = dm.initialize_mesh((world,), ("domain",))
    return mesh

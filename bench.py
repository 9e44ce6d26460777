"""Training-throughput benchmark on B200 (samples / s, device-timed, max over ranks).

``python bench.py --gpus N --steps K --warmup W [--config NAME] [--impl reference] [--no-extras]``; for N > 1 launch
with ``python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...``.  Rank 0 prints ONE JSON line.

The headline line is the Transolver configuration (1 M points, points sharded over the GPUs).  The other headline
configurations — ``songunet`` (EDM SongUNet 1024², height-sharded through ShardTensor), ``mgn`` (MeshGraphNet 2 M
nodes, partitioned graph), ``afno`` (AFNO 720×1440, distributed spectral filter), ``fno`` (FNO-2D on the CPU) — run
with ``--config NAME``; without ``--config`` they are measured after the headline with a few steps each and reported
in ``extra_configs`` of the same JSON line (``--no-extras`` skips them).

``value`` is device-timed (CUDA events, max over ranks) with the inputs resident on the GPU; ``e2e.value`` times
the same step through the public API including the host→device copy of that step's inputs from pinned memory and
the device→host read of the loss; ``exposed_comm_ms`` is the step time minus the time of the same step with all
peer traffic switched off.
"""
from __future__ import annotations

import argparse
import copy
import json
import os
import sys
import time
import traceback

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
EXTRA_ORDER = ("songunet", "afno", "mgn", "fno")
EXTRA_STEPS = {"songunet": 3, "afno": 4, "mgn": 4, "fno": 100}


def _run_config(name: str, impl: str, args, rank: int, world: int, dev):
    import importlib

    if impl == "reference":
        from baseline import ref_bench

        return ref_bench.run(name, args, rank, world, dev, ROOT)
    mod = importlib.import_module(f"physicsnemo_b200.benchmarks.{name}")
    return mod.run(args, rank, world, dev)


def _arm_watchdog(line: dict, extras: dict, rank: int, seconds: float) -> None:
    """The headline number must reach stdout even if an extra configuration stalls: after ``seconds`` every rank leaves,
    rank 0 first printing the headline line with the extras finished so far."""
    import threading

    def fire():
        if rank == 0:
            out = dict(line)
            out["extra_configs"] = dict(extras, watchdog=f"extra configurations still running after {seconds:.0f} s; cut off")
            print(json.dumps(out), flush=True)
        os._exit(0)

    t = threading.Timer(seconds + (0.0 if rank == 0 else 5.0), fire)
    t.daemon = True
    t.start()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default=None, choices=["transolver", "songunet", "mgn", "afno", "fno"])
    ap.add_argument("--no-extras", action="store_true", help="only the headline configuration")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from the host instead of replaying a CUDA graph")
    ap.add_argument("--points", type=int, default=None,
                    help="Transolver configuration only: number of points (default 1 M, the headline size); smaller values "
                         "measure the per-GPU work of an N-way shard on one GPU")
    ap.add_argument("--micro-batch", type=int, default=None,
                    help="images per micro-step of the SongUNet configuration (default: one image-equivalent of rows per GPU)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    sys.path.insert(0, ROOT)
    name = args.config or "transolver"
    if name == "fno":                                     # the CPU plumbing configuration needs no device
        if rank == 0:
            print(json.dumps(_run_config("fno", args.impl, args, 0, 1, torch.device("cpu"))))
        return
    if not torch.cuda.is_available():
        if rank == 0:
            print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device"}))
        return
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if args.impl != "reference":          # the reference's own DistributedManager brings up the group of its arm
            dist.init_process_group("nccl", device_id=dev)
    t_start = time.time()
    try:
        line = _run_config(name, args.impl, args, rank, world, dev)
        extras = {}
        if args.config is None and not args.no_extras and isinstance(line, dict) and "unavailable" not in line:
            budget_s = float(os.environ.get("PNM_BENCH_EXTRAS_SECONDS", "420"))
            _arm_watchdog(line, extras, rank, budget_s + 240.0)
            for extra in EXTRA_ORDER:
                if time.time() - t_start > budget_s:
                    extras[extra] = {"skipped": "time budget of the extra configurations used up"}
                    continue
                eargs = copy.copy(args)
                eargs.steps = EXTRA_STEPS[extra]
                try:
                    torch.cuda.empty_cache()
                    if extra == "fno":
                        res = _run_config("fno", args.impl, eargs, 0, 1, torch.device("cpu")) if rank == 0 else None
                    else:
                        res = _run_config(extra, args.impl, eargs, rank, world, dev)
                    extras[extra] = res
                except Exception as exc:  # noqa: BLE001  (an extra configuration must never take the headline down)
                    extras[extra] = {"error": f"{type(exc).__name__}: {exc}"[:400],
                                     "where": traceback.format_exc().strip().splitlines()[-3:]}
            line["extra_configs"] = extras
        if rank == 0:
            print(json.dumps(line))
    finally:
        if world > 1:
            import torch.distributed as dist

            try:
                if dist.is_initialized():
                    dist.destroy_process_group()
            except Exception:  # noqa: BLE001
                pass


if __name__ == "__main__":
    main()

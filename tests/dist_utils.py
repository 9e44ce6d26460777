"""Helpers to run a function on N CPU ranks (gloo) as child processes."""
import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, args, errq):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    os.environ["CUDA_VISIBLE_DEVICES"] = ""
    torch.set_num_threads(1)
    try:
        from physicsnemo_b200.distributed import DistributedManager

        DistributedManager.initialize()
        fn(rank, world, *args)
        dist.barrier()
    except Exception:  # noqa: BLE001
        errq.put((rank, traceback.format_exc()))
    finally:
        try:
            from physicsnemo_b200.distributed import DistributedManager

            DistributedManager.cleanup()
        except Exception:
            pass


def run_ranks(fn, world: int = 2, args=(), timeout: float = 120.0):
    """Run ``fn(rank, world, *args)`` on ``world`` gloo ranks; raise if any rank failed."""
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn, args, errq)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()
    errors = []
    while not errq.empty():
        errors.append(errq.get())
    if alive:
        raise RuntimeError(f"{len(alive)} rank(s) timed out; errors so far: {errors}")
    if errors:
        raise RuntimeError("\n".join(f"[rank {r}]\n{tb}" for r, tb in errors))
    bad = [p.exitcode for p in procs if p.exitcode != 0]
    if bad:
        raise RuntimeError(f"rank exit codes {bad}")

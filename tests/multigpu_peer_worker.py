"""Worker run under torchrun on 2+ GPUs: peer-memory all-reduce against NCCL, and the
point-sharded Transolver step against the single-GPU step (collective asserts)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from physicsnemo_b200.parallel.peer import PeerRuntime
    from physicsnemo_b200.parallel.point_parallel import PointParallel
    from physicsnemo_b200.models.transolver import Transolver

    ok = True
    rt = PeerRuntime(capacity_floats=1 << 23)
    for n, two in [(5, False), (16500, False), (70001, True), (6_000_000, True), (6_000_000, False)]:
        for rep in range(3):
            torch.manual_seed(rank * 100 + rep)
            x = torch.randn(n, device=dev)
            ref = x.clone()
            dist.all_reduce(ref)
            out = rt.all_reduce(x, two_shot=two)
            torch.cuda.synchronize()
            err = (out - ref).abs().max().item()
            if err > 1e-4 * max(1.0, ref.abs().max().item()):
                ok = False
                print(f"[rank {rank}] all_reduce n={n} two_shot={two} rep={rep} max err {err}", flush=True)
    rt.check()
    # timing of the small reduction the physics attention issues (67 KB)
    x = torch.randn(8 * 64 * 33, device=dev)
    for fn, name in ((lambda: rt.all_reduce(x), "peer"), (lambda: dist.all_reduce(x), "nccl")):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(50):
            fn()
        e1.record()
        torch.cuda.synchronize()
        if rank == 0:
            print(f"all_reduce 16896 floats via {name}: {e0.elapsed_time(e1) / 50 * 1000:.1f} us", flush=True)

    # sharded Transolver step == single-GPU step
    torch.manual_seed(0)
    cfg = dict(functional_dim=3, out_dim=4, embedding_dim=3, n_layers=2, n_hidden=256, n_head=8, slice_num=64, use_te=False)
    full = Transolver(**cfg).to(dev)
    shard = Transolver(**cfg).to(dev)
    shard.load_state_dict(full.state_dict())
    n = 4096 * world
    g = torch.Generator(device="cpu").manual_seed(1)
    fx, emb, tgt = (torch.randn(1, n, c, generator=g).to(dev) for c in (3, 3, 4))
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out_full = full(fx, embedding=emb)
    (((out_full.float() - tgt) ** 2).sum() / tgt.numel()).backward()
    pp = PointParallel(shard, backend="peer")
    sl = slice(rank * (n // world), (rank + 1) * (n // world))
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out_sh = shard(fx[:, sl], embedding=emb[:, sl])
    (((out_sh.float() - tgt[:, sl]) ** 2).sum() / tgt.numel()).backward()
    pp.reduce_gradients()
    torch.cuda.synchronize()
    rel = ((out_sh.float() - out_full[:, sl].float()).norm() / out_full[:, sl].float().norm()).item()
    if rel > 3e-2:
        ok = False
        print(f"[rank {rank}] sharded forward rel err {rel}", flush=True)
    worst = 0.0
    for (name, p), (_, q) in zip(shard.named_parameters(), full.named_parameters()):
        r = ((p.grad - q.grad).norm() / (q.grad.norm() + 1e-12)).item()
        worst = max(worst, r)
        if r > 0.15:
            ok = False
            print(f"[rank {rank}] grad {name} rel err {r}", flush=True)
    flag = torch.tensor([1.0 if ok else 0.0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"forward rel {rel:.4f}, worst grad rel {worst:.4f}")
        print("MULTIGPU_PEER_OK" if flag.item() == 1.0 else "MULTIGPU_PEER_FAILED", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1.0 else 1)


if __name__ == "__main__":
    main()

"""Worker run under torchrun on 2+ GPUs (launched by ``tests/test_multigpu.py``): every check compares a peer-memory /
sharded path against NCCL or against the unsharded computation and ends in a collective verdict."""
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _rel(a, b):
    return float((a.float() - b.float()).abs().max()) / max(float(b.float().abs().max()), 1e-12)


def check_allreduce(rank, world, dev, report):
    from physicsnemo_b200.parallel.peer import PeerRuntime

    rt = PeerRuntime(capacity_floats=1 << 23, budget_s=20.0)
    for n, two in [(5, False), (16500, False), (70001, True), (6_000_000, True), (6_000_000, False), (4099, True)]:
        for rep in range(3):
            torch.manual_seed(rank * 100 + rep)
            x = torch.randn(n, device=dev)
            ref = x.clone()
            dist.all_reduce(ref)
            out = rt.all_reduce(x, two_shot=two)
            report(f"allreduce fp32 n={n} two_shot={two}", _rel(out, ref), 1e-5)
    # back-to-back calls with different data and no synchronisation in between (slot parity protocol)
    xs = [torch.randn(33000, device=dev) + i for i in range(6)]
    outs = [rt.all_reduce(x) for x in xs]
    for x, o in zip(xs, outs):
        ref = x.clone()
        dist.all_reduce(ref)
        report("allreduce back-to-back", _rel(o, ref), 1e-5)
    # bf16 wire, in place, with scale
    for n in (8, 4096, 1_000_000 + 8, 5_969_736):
        torch.manual_seed(rank + 7)
        x = torch.randn(n, device=dev)
        ref = (x * 0.5).to(torch.bfloat16).float()
        dist.all_reduce(ref)
        rt.all_reduce_bf16_(x, scale=0.5)
        report(f"allreduce bf16 n={n}", _rel(x, ref), 1.2e-2)
    rt.check()
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
    g = torch.randn(12_000_000, device=dev)
    for fn, name in ((lambda: rt.all_reduce_bf16_(g, max_ctas=0), "peer bf16 wire"), (lambda: dist.all_reduce(g), "nccl fp32")):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            fn()
        e1.record()
        torch.cuda.synchronize()
        if rank == 0:
            print(f"gradient all_reduce 12 M floats via {name}: {e0.elapsed_time(e1) / 10:.3f} ms", flush=True)
    audit = rt.audit_flags()          # hundreds of calls of every kind later: no stray, future-dated or diverging flags
    report("flag audit after the all-reduce traffic", 0.0 if audit["calls"] >= max(audit["max_per_peer"]) > 0 else 1.0, 0.5)
    return rt


def check_timeout_and_recovery(rank, world, dev, report):
    """A rank that arrives late (host sleep between steps) makes the others' bounded wait run out: they must raise
    ``PeerTimeoutError``, and after ``recover()`` on every rank the next all-reduce must be correct again."""
    from physicsnemo_b200.parallel.peer import PeerRuntime, PeerTimeoutError

    rt = PeerRuntime(capacity_floats=1 << 16, budget_s=0.05)
    x = torch.full((1024,), float(rank + 1), device=dev)
    torch.cuda.synchronize()
    dist.barrier()
    if rank == world - 1:
        time.sleep(1.0)                       # late by far more than the 50 ms budget; nothing of this rank is in flight
    out = rt.all_reduce(x)
    torch.cuda.synchronize()
    raised = False
    try:
        rt.check()
    except PeerTimeoutError:
        raised = True
    timed_out_somewhere = torch.tensor([1.0 if raised else 0.0], device=dev)
    dist.all_reduce(timed_out_somewhere, op=dist.ReduceOp.MAX)
    report("timeout detected on a waiting rank", 0.0 if timed_out_somewhere.item() == 1.0 else 1.0, 0.5)
    if raised:
        report("timed-out output is NaN, not stale data", 0.0 if torch.isnan(out).any().item() else 1.0, 0.5)
    rt.recover()
    rt.budget_s = 20.0
    ref = x.clone()
    dist.all_reduce(ref)
    out = rt.all_reduce(x)
    report("allreduce after recover()", _rel(out, ref), 1e-6)
    rt.check()
    audit = rt.audit_flags()                      # no stray, future-dated or diverging flags after the traffic above
    report("flag audit", 0.0 if len(audit["max_per_peer"]) == world and audit["calls"] >= max(audit["max_per_peer"]) else 1.0, 0.5)


def check_sharded_conv_gn(rank, world, dev, report):
    """F.conv2d / GroupNorm on a height-sharded ShardTensor (the fused halo + peer-moment kernels) vs the gathered image."""
    from physicsnemo_b200.distributed import DistributedManager
    from physicsnemo_b200.nn.module.group_norm import GroupNorm
    from physicsnemo_b200.parallel import Shard, ShardTensor
    from physicsnemo_b200.parallel.halo_conv import get_halo_runtime
    from physicsnemo_b200 import ops

    mesh = DistributedManager().global_mesh
    torch.manual_seed(0)
    for (n, cin, cout, hl, w) in [(2, 64, 128, 16, 40), (1, 16, 64, 8, 32), (2, 128, 4, 24, 48)]:
        h = hl * world
        xg = torch.randn(n, cin, h, w, device=dev)
        wt = torch.randn(cout, cin, 3, 3, device=dev) / (9 * cin) ** 0.5
        b = torch.randn(cout, device=dev)
        dyg = torch.randn(n, cout, h, w, device=dev)
        sl = slice(rank * hl, (rank + 1) * hl)
        for it in range(2):
            x = (xg[:, :, sl] * (1 + it)).clone().requires_grad_(True)
            wl, bl = wt.clone().requires_grad_(True), b.clone().requires_grad_(True)
            before = ops.kernel_launches()
            with torch.autocast("cuda", dtype=torch.bfloat16):
                xs = ShardTensor.from_local(x, mesh, [Shard(2)], sharding_shapes="chunk", global_shape=xg.shape)
                ys = torch.nn.functional.conv2d(xs, wl, bl, padding=1)
            assert ops.kernel_launches() > before, "the fused halo path was not taken"
            y = ys.to_local()
            y.backward(dyg[:, :, sl].to(y.dtype))
            xr = (xg * (1 + it)).clone().requires_grad_(True)
            wr, br = wt.clone().requires_grad_(True), b.clone().requires_grad_(True)
            ref = torch.nn.functional.conv2d(xr, wr, br, padding=1)
            ref.backward(dyg)
            tag = f"halo conv {cin}->{cout} it{it}"
            report(tag + " fwd", _rel(y, ref[:, :, sl]), 2e-2)
            report(tag + " dgrad", _rel(x.grad, xr.grad[:, :, sl]), 2e-2)
            report(tag + " wgrad", _rel(wl.grad, wr.grad), 2e-2)       # per-use reduction: already summed over ranks
            report(tag + " bgrad", _rel(bl.grad, br.grad), 2e-2)
    get_halo_runtime(mesh.get_group()).check()
    for (n, c, hl, w, silu, dt) in [(2, 128, 16, 40, True, torch.bfloat16), (3, 64, 8, 24, False, torch.float32)]:
        h = hl * world
        xg = (torch.randn(n, c, h, w, device=dev) * 2 + 0.5).to(dt)
        gn_s = GroupNorm(c, act="silu" if silu else None).to(dev)
        gn_r = GroupNorm(c, act="silu" if silu else None).to(dev)
        with torch.no_grad():
            gn_s.weight.copy_(torch.randn(c, device=dev) * 0.5 + 1)
            gn_s.bias.copy_(torch.randn(c, device=dev) * 0.2)
        gn_r.load_state_dict(gn_s.state_dict())
        sl = slice(rank * hl, (rank + 1) * hl)
        dyg = torch.randn(n, c, h, w, device=dev)
        x = xg[:, :, sl].contiguous(memory_format=torch.channels_last).clone().requires_grad_(True)
        xs = ShardTensor.from_local(x, mesh, [Shard(2)], sharding_shapes="chunk", global_shape=xg.shape)
        before = ops.kernel_launches()
        ys = gn_s(xs)
        assert ops.kernel_launches() > before, "the sharded GroupNorm kernels were not used"
        ys.to_local().backward(dyg[:, :, sl].to(dt))
        xr = xg.float().clone().requires_grad_(True)
        gn_r.float()
        yr = torch.nn.functional.group_norm(xr, gn_r.num_groups, gn_r.weight, gn_r.bias, gn_r.eps)
        yr = torch.nn.functional.silu(yr) if silu else yr
        yr.backward(dyg)
        tol = 3e-2 if dt == torch.bfloat16 else 3e-4
        tag = f"sharded GN c={c} {str(dt)[6:]}"
        report(tag + " fwd", _rel(ys.to_local(), yr[:, :, sl]), tol)
        report(tag + " dx", _rel(x.grad, xr.grad[:, :, sl]), tol)
        report(tag + " dgamma", _rel(gn_s.weight.grad, gn_r.weight.grad), tol)
        report(tag + " dbeta", _rel(gn_s.bias.grad, gn_r.bias.grad), tol)


def check_grad_reducer(rank, world, dev, report):
    from physicsnemo_b200.parallel.grad_reducer import GradBucketReducer

    torch.manual_seed(3)
    model = torch.nn.Sequential(torch.nn.Linear(300, 517), torch.nn.GELU(), torch.nn.Linear(517, 1031), torch.nn.GELU(),
                                torch.nn.Linear(1031, 7)).to(dev)
    ref = torch.nn.Sequential(torch.nn.Linear(300, 517), torch.nn.GELU(), torch.nn.Linear(517, 1031), torch.nn.GELU(),
                              torch.nn.Linear(1031, 7)).to(dev)
    ref.load_state_dict(model.state_dict())
    red = GradBucketReducer(model.parameters(), bucket_mb=0.5, scale=1.0 / world, wire="bf16")
    for step in range(3):
        torch.manual_seed(10 * step + rank)
        x = torch.randn(64, 300, device=dev)
        red.zero_grad()
        model(x).square().mean().backward()
        red.finish()
        ref.zero_grad(set_to_none=True)
        ref(x).square().mean().backward()
        for (name, p), q in zip(model.named_parameters(), ref.parameters()):
            g = q.grad.clone() / world
            dist.all_reduce(g)
            report(f"bucketed bf16 reduction {name}", _rel(p.grad, g), 2e-2)
    torch.cuda.synchronize()


def check_transolver(rank, world, dev, report):
    from physicsnemo_b200.models.transolver import Transolver
    from physicsnemo_b200.parallel.point_parallel import PointParallel

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
    pp = PointParallel(shard, backend="peer", wire="fp32")
    pp.zero_grad()
    sl = slice(rank * (n // world), (rank + 1) * (n // world))
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out_sh = shard(fx[:, sl], embedding=emb[:, sl])
    (((out_sh.float() - tgt[:, sl]) ** 2).sum() / tgt.numel()).backward()
    pp.reduce_gradients()
    torch.cuda.synchronize()
    rel = ((out_sh.float() - out_full[:, sl].float()).norm() / out_full[:, sl].float().norm()).item()
    report("point-sharded Transolver forward", rel, 1e-2)
    # every gradient within 2 % of its own norm; tensors whose gradient nearly cancels (norm ~1e-3 of the model's total
    # gradient norm, e.g. the slice projections at initialisation, which differ by that much between two runs of the SAME
    # unsharded model) are held to an absolute floor of 2e-4 of the total norm instead
    total = torch.sqrt(sum(q.grad.float().pow(2).sum() for q in full.parameters())).item()
    for (name, p), (_, q) in zip(shard.named_parameters(), full.named_parameters()):
        d = (p.grad - q.grad).norm().item()
        report(f"point-sharded Transolver grad {name}", d / (q.grad.norm().item() + 1e-2 * total), 2e-2)


def check_sharded_attention(rank, world, dev, report):
    """F.scaled_dot_product_attention on sequence-sharded ShardTensors (peer-staged K / V, GEMM + softmax kernels) vs
    fp32 attention over the gathered sequence, forward and the gradients of q, k, v."""
    import math

    from physicsnemo_b200 import ops
    from physicsnemo_b200.distributed import DistributedManager
    from physicsnemo_b200.parallel import Shard, ShardTensor

    mesh = DistributedManager().global_mesh
    torch.manual_seed(3)
    for (b, hh, sl, d) in [(1, 1, 1024, 512), (2, 2, 264, 64)]:
        s = sl * world
        full = [torch.randn(b, hh, s, d, device=dev).to(torch.bfloat16) for _ in range(3)]
        do = torch.randn(b, hh, s, d, device=dev).to(torch.bfloat16)
        for t in full + [do]:
            dist.broadcast(t, src=0)
        sel = slice(rank * sl, (rank + 1) * sl)
        for it in range(2):
            loc = [t[:, :, sel].clone().requires_grad_(True) for t in full]
            st = [ShardTensor.from_local(t, mesh, [Shard(2)], sharding_shapes="chunk", global_shape=full[0].shape) for t in loc]
            before = ops.kernel_launches()
            out = torch.nn.functional.scaled_dot_product_attention(*st)
            assert ops.kernel_launches() > before, "the peer-staged attention path was not taken"
            out.to_local().backward(do[:, :, sel])
            ref_in = [t.float().requires_grad_(True) for t in full]
            sc = (ref_in[0] @ ref_in[1].transpose(-1, -2)) / math.sqrt(d)
            ref = torch.softmax(sc, dim=-1) @ ref_in[2]
            ref.backward(do.float())
            tag = f"sharded attention S={s} D={d} it{it}"
            report(tag + " fwd", _rel(out.to_local(), ref[:, :, sel]), 1.5e-2)
            for name, a, r in zip("qkv", loc, ref_in):
                report(tag + f" d{name}", _rel(a.grad, r.grad[:, :, sel]), 2.5e-2)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from physicsnemo_b200.distributed import DistributedManager

    DistributedManager.initialize()
    DistributedManager().initialize_mesh((world,), ("domain",))
    failures = []

    def report(what, err, tol):
        if not (err <= tol):
            failures.append(f"[rank {rank}] {what}: {err:.3e} > {tol:.1e}")

    which = sys.argv[1:] or ["allreduce", "timeout", "conv_gn", "reducer", "attention", "transolver"]
    table = {"allreduce": check_allreduce, "timeout": check_timeout_and_recovery, "conv_gn": check_sharded_conv_gn,
             "reducer": check_grad_reducer, "attention": check_sharded_attention, "transolver": check_transolver}
    for name in which:
        t0 = time.time()
        table[name](rank, world, dev, report)
        torch.cuda.synchronize()
        dist.barrier()
        if rank == 0:
            print(f"check {name}: done in {time.time() - t0:.1f} s", flush=True)
    for line in failures[:40]:
        print(line, flush=True)
    flag = torch.tensor([0.0 if failures else 1.0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("MULTIGPU_OK" if flag.item() == 1.0 else "MULTIGPU_FAILED", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1.0 else 1)


if __name__ == "__main__":
    main()

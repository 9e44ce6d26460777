"""EDM SongUNet at 1024 × 1024, bf16, height-sharded through ``ShardTensor`` (headline configuration 4).

Model: ``SongUNet(img_resolution=1024, in_channels=16, out_channels=4, model_channels=128, channel_mult=[1,2,2,4],
num_blocks=2, attn_resolutions=[64])`` (73.8 M parameters; 12 conditioning + 4 noisy-target input channels) inside
``EDMPreconditioner``; loss ``MSEDSMLoss`` with the EDM log-normal noise levels (P_mean −1.2, P_std 1.2); Adam.
Global batch 8.  On N ranks every image is split into N height slabs; the batch is processed in micro-batches of
``min(8, 4 N)`` images (at most four image-equivalents of activations per GPU; ``--micro-batch`` overrides) with gradient
accumulation, one optimizer step.  Micro-batches of one image leave the 128² and 256² levels of the U-Net with fewer
tiles than SMs; four images per micro-step measured 10 % faster at one GPU (1051 → 950 ms per step).

Sharded path: every 3×3 convolution is the halo-fused tcgen05 kernel (boundary rows read from the neighbours'
mailboxes inside the kernel), its weight gradient the split-reduction kernel on saved halo rows, GroupNorm(+SiLU)
takes its moments across ranks inside the normalising kernel, the parameter gradients go through the bucketed
bf16 peer all-reduce on a side stream.  ``sharded_vs_single_rel_err`` compares one forward + backward of the sharded
model at 512² against the unsharded model on rank 0.
"""
from __future__ import annotations

import torch

from .common import ClockSampler, base_line, flush_buffer, rel_err, timed_loop

RES = 1024
BATCH = 8
CFG = dict(img_resolution=RES, in_channels=16, out_channels=4, model_channels=128, channel_mult=[1, 2, 2, 4], num_blocks=2,
           attn_resolutions=[64], dropout=0.0, amp_mode=True)
DESC = ("SongUNet 1024^2: base 128, mult [1,2,2,4], 2 blocks/level, bottleneck self-attention (1 head x 512), GroupNorm, SiLU; "
        "EDM preconditioner + DSM loss (P_mean -1.2, P_std 1.2); dropout 0")


def make_batch(batch: int, res: int, seed: int = 0):
    """Seeded synthetic sample: 12 conditioning channels and 4 target channels, N(0, 1)."""
    g = torch.Generator().manual_seed(seed)
    cond = torch.randn(batch, 12, res, res, generator=g)
    x0 = torch.randn(batch, 4, res, res, generator=g)
    return cond, x0


def build_model(dev, res: int = RES):
    from ..diffusion.preconditioners import EDMPreconditioner
    from ..diffusion.utils.model_wrappers import ConcatConditionWrapper
    from ..models.diffusion_unets import SongUNet

    torch.manual_seed(1234)
    cfg = dict(CFG, img_resolution=res)
    return EDMPreconditioner(ConcatConditionWrapper(SongUNet(**cfg)), sigma_data=0.5).to(dev)


def _shard(t: torch.Tensor, mesh, global_h: int):
    from ..parallel import Shard, ShardTensor

    shape = list(t.shape)
    shape[2] = global_h
    return ShardTensor.from_local(t, mesh, [Shard(2)], sharding_shapes="chunk", global_shape=shape)


def _correctness(rank, world, dev, mesh):
    """Forward + every parameter gradient of the sharded model against the unsharded model (512², batch 1)."""
    import torch.distributed as dist

    from ..parallel import defer_param_grad_reduction

    res = 512
    model = build_model(dev, res)
    with torch.no_grad():                      # the zero-initialised output convolutions would hide forward errors
        gen = torch.Generator(device=dev).manual_seed(99)
        for p in model.parameters():
            p.add_(torch.randn(p.shape, generator=gen, device=dev) * 0.02)
    cond, x0 = make_batch(1, res, seed=7)
    sigma = torch.tensor([0.7])
    noise = torch.randn(1, 4, res, res, generator=torch.Generator().manual_seed(11))
    xt = x0 + sigma.view(-1, 1, 1, 1) * noise
    hl = res // world
    sl = slice(rank * hl, (rank + 1) * hl)
    defer_param_grad_reduction(False)      # per-use reduction: the gradients below are complete on every rank
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out_s = model(_shard(xt[:, :, sl].to(dev), mesh, res), sigma.to(dev), condition=_shard(cond[:, :, sl].to(dev), mesh, res))
        loss = ((out_s - _shard(x0[:, :, sl].to(dev), mesh, res)) ** 2).mean()
    loss.backward()
    full = out_s.full_tensor().float()
    grads = {n: p.grad.detach().clone() for n, p in model.named_parameters() if p.grad is not None}
    model.zero_grad(set_to_none=True)
    fwd_err = grad_err = 0.0
    worst = ""
    if rank == 0:
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out_1 = model(xt.to(dev), sigma.to(dev), condition=cond.to(dev))
            loss1 = ((out_1 - x0.to(dev)) ** 2).mean()
        loss1.backward()
        fwd_err = rel_err(full, out_1.float())
        for n, p in model.named_parameters():
            if p.grad is None or n not in grads:
                continue
            e = rel_err(grads[n], p.grad)
            if e > grad_err:
                grad_err, worst = e, n
        model.zero_grad(set_to_none=True)
    res_t = torch.tensor([fwd_err, grad_err], device=dev, dtype=torch.float64)
    dist.broadcast(res_t, src=0)
    del model
    torch.cuda.empty_cache()
    return {"forward": float(res_t[0]), "worst_param_grad": float(res_t[1]), "worst_param": worst,
            "at": "512^2, batch 1, vs the unsharded model on rank 0"}


def run(args, rank: int, world: int, dev) -> dict:
    import torch.distributed as dist

    from .. import ops
    from ..diffusion.metrics.losses import MSEDSMLoss
    from ..diffusion.noise_schedulers import DomainParallelNoiseScheduler, EDMNoiseScheduler
    from ..optim import FusedAdam
    from ..parallel import defer_param_grad_reduction
    from ..parallel.grad_reducer import GradBucketReducer
    from ..parallel.peer import set_loopback

    if RES % (8 * world):
        raise ValueError("the height must split into slabs that are multiples of 8 rows")
    mesh = None
    check = None
    if world > 1:
        from .common import domain_mesh

        mesh = domain_mesh(world)
        check = _correctness(rank, world, dev, mesh)
    model = build_model(dev)
    params = [p for p in model.parameters() if p.requires_grad]
    reducer = None
    if world > 1:
        defer_param_grad_reduction(True)
        reducer = GradBucketReducer(params, group=mesh.get_group(), scale=1.0, wire="bf16")
    opt = FusedAdam(params, lr=1e-4)
    base = EDMNoiseScheduler(P_mean=-1.2, P_std=1.2) if _accepts_p(EDMNoiseScheduler) else EDMNoiseScheduler()
    sched = DomainParallelNoiseScheduler(base, mesh, shard_dim=2) if world > 1 else base
    loss_fn = MSEDSMLoss(model, sched)
    micro = min(BATCH, 4 * world)              # images per micro-batch: four image-equivalents of rows per GPU
    if getattr(args, "micro_batch", None):
        micro = int(args.micro_batch)
        if BATCH % micro:
            raise ValueError(f"--micro-batch must divide the batch of {BATCH}")
    accum = BATCH // micro
    hl = RES // world
    cond, x0 = make_batch(BATCH, RES, seed=0)
    sl = slice(rank * hl, (rank + 1) * hl)
    host = [cond[:, :, sl].contiguous().pin_memory(), x0[:, :, sl].contiguous().pin_memory()]
    del cond, x0
    dev_in = [t.to(dev, non_blocking=True) for t in host]
    torch.cuda.synchronize()
    loss_host = torch.zeros(1, pin_memory=True)
    state = {}

    def train_step(cond_d, x0_d):
        if reducer is not None:
            reducer.zero_grad()
        else:
            opt.zero_grad(set_to_none=True)
        total = None
        for a in range(accum):
            c, x = cond_d[a * micro:(a + 1) * micro], x0_d[a * micro:(a + 1) * micro]
            if world > 1:
                c, x = _shard(c, mesh, RES), _shard(x, mesh, RES)
                reducer.sync = a == accum - 1
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = loss_fn(x, condition=c) / accum
            loss.backward()
            lv = loss.detach()
            lv = lv.to_local() if hasattr(lv, "to_local") else lv
            total = lv if total is None else total + lv
        if reducer is not None:
            reducer.finish()
        opt.step()
        state["loss"] = total

    def step_resident():
        train_step(*dev_in)

    def step_e2e():
        c, x = (t.to(dev, non_blocking=True) for t in host)
        train_step(c, x)
        loss_host.copy_(state["loss"].reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    flush = flush_buffer(dev)
    step_resident()
    torch.cuda.synchronize()
    before = ops.kernel_launches()
    step_resident()
    torch.cuda.synchronize()
    launches = ops.kernel_launches() - before
    sampler = ClockSampler(dev.index or 0)
    if rank == 0:
        sampler.start()
    ms, wall = timed_loop(step_resident, args.steps, max(args.warmup - 2, 1), world, dev, flush)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e, _ = timed_loop(step_e2e, max(2, args.steps // 2), 1, world, dev, flush)
    exposed = None
    if world > 1:
        set_loopback(True)
        ms_loop, _ = timed_loop(step_resident, max(2, args.steps // 2), 1, world, dev, flush)
        set_loopback(False)
        exposed = max(0.0, ms - ms_loop)
        step_resident()          # leave the state consistent (a real reduction after the communication-free steps)
    err = ops.device_error()
    if world > 1:
        total = loss_host.to(dev)
        dist.all_reduce(total)
        loss_host.copy_(total)
    h2d = sum(t.numel() * t.element_size() for t in host)
    return base_line(
        BATCH * 1000.0 / ms, ms, world, args, "strong",
        "synthetic (seeded N(0,1) conditioning and target fields, random-init weights)",
        {"model": DESC, "global_batch": BATCH, "seq_len": RES * RES, "parallelism": f"height sharded x{world} via ShardTensor",
         "micro_batch": micro, "grad_accumulation": accum, "optimizer": "Adam (fused)", "cuda_graph": False,
         "l2": "256 MB buffer rewritten between timed steps; activations are GBs (>> 126 MB L2)"},
        clocks,
        {"value": BATCH * 1000.0 / ms_e2e, "unit": "samples/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d,
         "d2h_bytes_per_step": 4},
        launches,
        {"exposed_comm_ms": exposed, "sharded_vs_single_rel_err": check, "device_error_word": err,
         "loss": float(loss_host.item()), "wall_s_timed_region": wall,
         "peak_memory_gb": round(torch.cuda.max_memory_allocated(dev) / 2 ** 30, 1),
         "exposed_comm_how": "step time minus the time of the same step with all peer traffic switched off (loopback)"})


def _accepts_p(cls) -> bool:
    import inspect

    return "P_mean" in inspect.signature(cls.__init__).parameters

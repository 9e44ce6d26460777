"""Reference arm of ``bench.py``: the unmodified reference package (``baseline/_ref/physicsnemo``) through its own public
API and stock eager code path, for the same configurations and the same timing protocol as this repository's arm.

None of this repository's models, kernels or engine is imported here: only ``baseline.ref_runner`` (which stubs the
third-party packages the reference imports but that are not installed) and the timing helpers below.  A configuration
that the reference cannot run prints ``{"impl": "reference", "unavailable": "<the actual exception>"}``.
"""
from __future__ import annotations

import os
import statistics
import subprocess
import threading
import time
import traceback

import torch


# ----------------------------------------------------------------------------- shared protocol (kept independent)
class _Clocks:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: [self.lines.append(line.strip()) for line in self.proc.stdout], daemon=True).start()
        except Exception:  # noqa: BLE001
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:  # noqa: BLE001
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


def _timed(step_fn, steps, warmup, world, dev, flush):
    import torch.distributed as dist

    for _ in range(warmup):
        step_fn()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    t0 = time.perf_counter()
    for i in range(steps):
        flush.add_(1.0)
        ev[i][0].record()
        step_fn()
        ev[i][1].record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    t = torch.tensor([sum(a.elapsed_time(b) for a, b in ev)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item() / steps, wall


def _line(value, ms, ms_e2e, value_e2e, world, args, config, clocks, h2d, loss, wall, extra=None):
    out = {"metric": "train samples/sec (device-timed, max over ranks)", "value": value, "unit": "samples/s", "n_gpus": world,
           "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
           "vs_baseline": None, "dtype": "bf16", "data": config.pop("_data"), "config": config, "clocks": clocks,
           "e2e": {"value": value_e2e, "unit": "samples/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d,
                   "d2h_bytes_per_step": 4},
           "impl": "reference", "loss": loss, "wall_s_timed_region": wall}
    if extra:
        out.update(extra)
    return out


def _unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": " ".join(why.split())[:600]}


def _ref_mesh(world):
    """The reference's own bring-up: DistributedManager -> 1-D domain mesh (flow of its ShardTensor training example)."""
    from physicsnemo.distributed import DistributedManager  # type: ignore

    if not DistributedManager.is_initialized():
        DistributedManager.initialize()
    dm = DistributedManager()
    mesh = getattr(dm, "_bench_mesh", None)
    if mesh is None:
        mesh = dm.initialize_mesh((world,), ("domain",))
        dm._bench_mesh = mesh
    return mesh


# ----------------------------------------------------------------------------------------------- Transolver
def _transolver(args, rank, world, dev):
    from physicsnemo.models.transolver import Transolver as RefTransolver  # type: ignore

    n_points = 1_000_000
    cfg = dict(functional_dim=3, out_dim=4, embedding_dim=3, n_layers=8, n_hidden=256, n_head=8, slice_num=64, mlp_ratio=4,
               use_te=False)
    g = torch.Generator().manual_seed(0)
    axes = torch.rand(3, generator=g) * 2.0 + 0.5
    u = torch.randn(n_points, 3, generator=g)
    u = u / u.norm(dim=1, keepdim=True)
    xyz, nrm = u * axes, u / axes
    nrm = nrm / nrm.norm(dim=1, keepdim=True)
    tgt = torch.randn(n_points, 4, generator=g)
    torch.manual_seed(1234)
    model = RefTransolver(**cfg).to(dev)
    opt = torch.optim.Adam(model.parameters(), lr=1e-3, fused=True)
    n_local = n_points // world
    sl = slice(rank * n_local, (rank + 1) * n_local)
    host = [t[sl].float().unsqueeze(0).contiguous().pin_memory() for t in (xyz, nrm, tgt)]
    dev_in = [t.to(dev, non_blocking=True) for t in host]
    denom = float(n_points * 4)
    loss_host = torch.zeros(1, pin_memory=True)
    state = {}
    wrap = lambda t: t  # noqa: E731
    if world > 1:
        from torch.distributed.tensor.placement_types import Shard

        from physicsnemo.domain_parallel import ShardTensor  # type: ignore

        mesh = _ref_mesh(world)
        def wrap(t):        # equal point shards: the global shape follows from the local one
            shape = list(t.shape)
            shape[1] *= world
            return ShardTensor.from_local(t, mesh, (Shard(1),), sharding_shapes="chunk", global_shape=tuple(shape))

    def train_step(emb, fx, target):
        opt.zero_grad(set_to_none=True)
        emb, fx, target = wrap(emb), wrap(fx), wrap(target)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out = model(fx, embedding=emb)
        loss = ((out.float() - target) ** 2).sum() / denom
        loss.backward()
        opt.step()
        lv = loss.detach()
        state["loss"] = lv.full_tensor() if hasattr(lv, "full_tensor") else lv

    def resident():
        train_step(*dev_in)

    def e2e():
        emb, fx, target = (t.to(dev, non_blocking=True) for t in host)
        train_step(emb, fx, target)
        loss_host.copy_(state["loss"].reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    flush = torch.empty(256 * 1024 * 1024 // 4, device=dev)
    sampler = _Clocks(dev.index or 0)
    resident()
    torch.cuda.synchronize()
    if rank == 0:
        sampler.start()
    ms, wall = _timed(resident, args.steps, max(args.warmup - 1, 1), world, dev, flush)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e, _ = _timed(e2e, args.steps, 1, world, dev, flush)
    h2d = sum(t.numel() * t.element_size() for t in host)
    return _line(1000.0 / ms, ms, ms_e2e, 1000.0 / ms_e2e, world, args,
                 {"model": "Transolver 8 blocks / hidden 256 / 8 heads / 64 slices / mlp_ratio 4", "global_batch": 1,
                  "seq_len": n_points, "parallelism": f"points sharded x{world}" + (" via the reference's ShardTensor" if world > 1 else ""),
                  "optimizer": "Adam (fused)", "cuda_graph": False, "use_te": False,
                  "_data": "synthetic (seeded ellipsoid point cloud, random-init weights)"},
                 clocks, h2d, float(loss_host.item()), wall)


# ------------------------------------------------------------------------------------------------- SongUNet
def _songunet(args, rank, world, dev):
    from physicsnemo.diffusion.metrics.losses import MSEDSMLoss  # type: ignore
    from physicsnemo.diffusion.noise_schedulers import EDMNoiseScheduler  # type: ignore
    from physicsnemo.diffusion.preconditioners import EDMPreconditioner  # type: ignore
    from physicsnemo.models.diffusion_unets import SongUNet  # type: ignore
    import physicsnemo  # type: ignore

    res, batch = 1024, 8
    torch.manual_seed(1234)
    net = SongUNet(img_resolution=res, in_channels=16, out_channels=4, model_channels=128, channel_mult=[1, 2, 2, 4],
                   num_blocks=2, attn_resolutions=[64], dropout=0.0, amp_mode=True)

    class Concat(physicsnemo.Module):  # glue only: image-like condition concatenated to the noisy state along channels
        def __init__(self, model):
            super().__init__()
            self.model = model

        def forward(self, x, t, condition=None, **kw):
            return self.model(torch.cat([x, condition.to(x.dtype)], dim=1), t, **kw)

    model = EDMPreconditioner(Concat(net), sigma_data=0.5).to(dev)
    opt = torch.optim.Adam(model.parameters(), lr=1e-4, fused=True)
    sched = EDMNoiseScheduler(P_mean=-1.2, P_std=1.2)
    hl = res // world
    wrap = lambda t: t  # noqa: E731
    if world > 1:
        from torch.distributed.tensor.placement_types import Shard

        from physicsnemo.diffusion.noise_schedulers import DomainParallelNoiseScheduler  # type: ignore
        from physicsnemo.domain_parallel import ShardTensor  # type: ignore

        mesh = _ref_mesh(world)
        sched = DomainParallelNoiseScheduler(sched, mesh, shard_dim=2) if _takes(DomainParallelNoiseScheduler, "shard_dim") \
            else DomainParallelNoiseScheduler(sched, mesh)
        def wrap(t):        # equal height slabs
            shape = list(t.shape)
            shape[2] *= world
            return ShardTensor.from_local(t, mesh, (Shard(2),), sharding_shapes="chunk", global_shape=tuple(shape))
    loss_fn = MSEDSMLoss(model, sched)
    g = torch.Generator().manual_seed(0)
    cond = torch.randn(batch, 12, res, res, generator=g)
    x0 = torch.randn(batch, 4, res, res, generator=g)
    sl = slice(rank * hl, (rank + 1) * hl)
    host = [cond[:, :, sl].contiguous().pin_memory(), x0[:, :, sl].contiguous().pin_memory()]
    del cond, x0
    dev_in = [t.to(dev, non_blocking=True) for t in host]
    micro = world if world > 1 else 1
    accum = batch // micro
    loss_host = torch.zeros(1, pin_memory=True)
    state = {}

    def train_step(cond_d, x0_d):
        opt.zero_grad(set_to_none=True)
        total = None
        for a in range(accum):
            c, x = wrap(cond_d[a * micro:(a + 1) * micro]), wrap(x0_d[a * micro:(a + 1) * micro])
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = loss_fn(x, condition=c) / accum
            loss.backward()
            lv = loss.detach()
            lv = lv.full_tensor() if hasattr(lv, "full_tensor") else lv
            total = lv if total is None else total + lv
        opt.step()
        state["loss"] = total

    def resident():
        train_step(*dev_in)

    def e2e():
        c, x = (t.to(dev, non_blocking=True) for t in host)
        train_step(c, x)
        loss_host.copy_(state["loss"].reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    flush = torch.empty(256 * 1024 * 1024 // 4, device=dev)
    sampler = _Clocks(dev.index or 0)
    resident()
    torch.cuda.synchronize()
    if rank == 0:
        sampler.start()
    ms, wall = _timed(resident, args.steps, max(args.warmup - 2, 1), world, dev, flush)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e, _ = _timed(e2e, max(2, args.steps // 2), 1, world, dev, flush)
    h2d = sum(t.numel() * t.element_size() for t in host)
    return _line(batch * 1000.0 / ms, ms, ms_e2e, batch * 1000.0 / ms_e2e, world, args,
                 {"model": "SongUNet 1024^2: base 128, mult [1,2,2,4], 2 blocks/level, bottleneck self-attention (1 head x 512), "
                           "GroupNorm, SiLU; EDM preconditioner + DSM loss (P_mean -1.2, P_std 1.2); dropout 0",
                  "global_batch": batch, "seq_len": res * res,
                  "parallelism": f"height sharded x{world}" + (" via the reference's ShardTensor" if world > 1 else ""),
                  "micro_batch": micro, "grad_accumulation": accum, "optimizer": "Adam (fused)", "cuda_graph": False,
                  "_data": "synthetic (seeded N(0,1) conditioning and target fields, random-init weights)"},
                 clocks, h2d, float(loss_host.item()), wall)


def _takes(cls, name):
    import inspect

    try:
        return name in inspect.signature(cls.__init__).parameters
    except (TypeError, ValueError):
        return False


# ------------------------------------------------------------------------------------------------------ FNO (CPU)
def _fno(args, rank, world, dev):
    from physicsnemo.models.fno import FNO  # type: ignore

    torch.manual_seed(1234)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    model = FNO(in_channels=1, out_channels=1, decoder_layers=1, decoder_layer_size=128, dimension=2, latent_channels=32,
                num_fno_layers=4, num_fno_modes=12, padding=8, activation_fn="gelu")
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    x, y = _fno_data(8, 64, seed=0)
    steps = max(args.steps, 100)
    for _ in range(3):
        _fno_step(model, opt, x, y)
    t0 = time.perf_counter()
    for _ in range(steps):
        loss = _fno_step(model, opt, x, y)
    dt = time.perf_counter() - t0
    ms = dt / steps * 1000.0
    return {"metric": "train samples/sec (CPU wall clock)", "value": 8 * 1000.0 / ms, "unit": "samples/s", "n_gpus": 0,
            "steps": steps, "warmup": 3, "ms_per_step": ms, "higher_is_better": True, "scaling": "none", "vs_baseline": None,
            "dtype": "fp32", "data": "synthetic (seeded Gaussian-random-field permeability / smooth target fields)",
            "config": {"model": "FNO-2D width 32, 4 layers, 12x12 modes, GELU, decoder 32-128-1", "global_batch": 8,
                       "seq_len": 64 * 64, "parallelism": "single CPU process", "threads": torch.get_num_threads()},
            "impl": "reference", "loss": float(loss)}


def _fno_data(batch, n, seed):
    """Inputs: 12 where a Gaussian random field with covariance (-Laplace + 9 I)^-2 is >= 0, else 3; targets: a smooth GRF."""
    g = torch.Generator().manual_seed(seed)
    k = torch.fft.fftfreq(n, d=1.0 / n)
    k2 = (2 * torch.pi) ** 2 * (k[:, None] ** 2 + k[None, :] ** 2)
    amp = 1.0 / (k2 + 9.0)
    def grf():
        w = torch.randn(batch, n, n, generator=g)
        return torch.fft.ifft2(torch.fft.fft2(w) * amp).real
    a = grf()
    x = torch.where(a >= 0, torch.full_like(a, 12.0), torch.full_like(a, 3.0)).unsqueeze(1)
    y = grf()
    y = (y / y.std()).unsqueeze(1)
    return x.float(), y.float()


def _fno_step(model, opt, x, y):
    opt.zero_grad(set_to_none=True)
    loss = torch.nn.functional.mse_loss(model(x), y)
    loss.backward()
    opt.step()
    return loss.item()


# -------------------------------------------------------------------------------------------------------- AFNO
def _afno(args, rank, world, dev):
    """Stock ``AFNO`` on one GPU; ``DistributedAFNO`` (channel parallel over the group "model_parallel") on several."""
    import math

    batch = 2
    cfg = dict(inp_shape=[720, 1440], in_channels=73, out_channels=73, patch_size=[8, 8], embed_dim=768, depth=12, num_blocks=8,
               sparsity_threshold=0.01)
    x, y = _sh_fields(batch, 73, 720, 1440, seed=0)
    torch.manual_seed(1234)
    if world == 1:
        from physicsnemo.models.afno import AFNO  # type: ignore

        model = AFNO(**cfg).to(dev)
        para = "single GPU"
    else:
        from physicsnemo.distributed import DistributedManager  # type: ignore
        from physicsnemo.models.afno import DistributedAFNO  # type: ignore

        if not DistributedManager.is_initialized():
            DistributedManager.initialize()
        dm = DistributedManager()
        if "model_parallel" not in dm.group_names:
            DistributedManager.create_process_subgroup("model_parallel", world, verbose=False)
        model = DistributedAFNO(inp_shape=(720, 1440), in_channels=73, out_channels=73, patch_size=8, embed_dim=768, depth=12,
                                num_blocks=8, channel_parallel_inputs=False, channel_parallel_outputs=False).to(dev)
        para = f"channel parallel x{world} (the reference's DistributedAFNO)"
    opt = torch.optim.Adam(model.parameters(), lr=5e-4, fused=True)
    host = [x.pin_memory(), y.pin_memory()]
    dev_in = [t.to(dev, non_blocking=True) for t in host]
    denom = float(y.numel())
    loss_host = torch.zeros(1, pin_memory=True)
    state = {}

    def train_step(xb, yb):
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out = model(xb)
        loss = ((out.float() - yb) ** 2).sum() / denom
        loss.backward()
        opt.step()
        state["loss"] = loss.detach()

    def resident():
        train_step(*dev_in)

    def e2e():
        a, b = (t.to(dev, non_blocking=True) for t in host)
        train_step(a, b)
        loss_host.copy_(state["loss"].reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    flush = torch.empty(256 * 1024 * 1024 // 4, device=dev)
    sampler = _Clocks(dev.index or 0)
    resident()
    torch.cuda.synchronize()
    if rank == 0:
        sampler.start()
    ms, wall = _timed(resident, args.steps, max(args.warmup - 2, 1), world, dev, flush)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e, _ = _timed(e2e, max(2, args.steps // 2), 1, world, dev, flush)
    h2d = sum(t.numel() * t.element_size() for t in host)
    return _line(batch * 1000.0 / ms, ms, ms_e2e, batch * 1000.0 / ms_e2e, world, args,
                 {"model": "AFNO 720x1440: patch 8x8, embed 768, depth 12, 8 blocks, mlp ratio 4, soft-shrink 0.01",
                  "global_batch": batch, "seq_len": 90 * 180, "parallelism": para, "optimizer": "Adam (fused)", "cuda_graph": False,
                  "_data": "synthetic (seeded spherical-harmonic random fields, spectrum l^-2, N(0,1)-normalised; random-init weights)"},
                 clocks, h2d, float(loss_host.item()), wall)


def _sh_fields(batch, channels, nlat, nlon, lmax=64, seed=0):
    """Two ``[batch, channels, nlat, nlon]`` tensors of band-limited spherical-harmonic random fields, power ~ l^-2."""
    import math

    n_fields = 2 * batch * channels
    g = torch.Generator().manual_seed(seed)
    theta = (torch.arange(nlat, dtype=torch.float64) + 0.5) * math.pi / nlat
    x, s = torch.cos(theta), torch.sin(theta)
    spec = torch.zeros(n_fields, nlat, nlon // 2 + 1, dtype=torch.complex128)
    pmm = torch.full((nlat,), math.sqrt(1.0 / (4 * math.pi)), dtype=torch.float64)
    for m in range(lmax + 1):
        if m > 0:
            pmm = -math.sqrt((2 * m + 1) / (2 * m)) * s * pmm
        p2, p1 = None, pmm
        for l in range(m, lmax + 1):
            if l == m:
                p = pmm
            elif l == m + 1:
                p = math.sqrt(2 * m + 3) * x * pmm
            else:
                a = math.sqrt((4 * l * l - 1) / (l * l - m * m))
                b = math.sqrt(((l - 1) ** 2 - m * m) / (4 * (l - 1) ** 2 - 1))
                p = a * (x * p1 - b * p2)
            p2, p1 = p1, p
            if l == 0:
                continue
            re = torch.randn(n_fields, generator=g, dtype=torch.float64)
            im = torch.randn(n_fields, generator=g, dtype=torch.float64) if m > 0 else torch.zeros(n_fields, dtype=torch.float64)
            spec[:, :, m] += (torch.complex(re, im) / l)[:, None] * p[None, :]
    f = torch.fft.irfft(spec, n=nlon, dim=-1)
    f = f - f.mean(dim=(1, 2), keepdim=True)
    f = (f / f.std(dim=(1, 2), keepdim=True)).float().reshape(2, batch, channels, nlat, nlon)
    return f[0].contiguous(), f[1].contiguous()


# ------------------------------------------------------------------------------------------------- MeshGraphNet
def _mgn(args, rank, world, dev):
    if world > 1:
        return _unavailable("the reference cannot run MeshGraphNet on a partitioned graph: its distributed graph is not wired into "
                            "MeshGraphNet.forward and graph partitioning raises NotImplementedError with its PyG backend "
                            "(models/graphcast/graph_cast_net.py:288-296)")
    import importlib

    for name in ("torch_geometric", "torch_scatter"):
        spec = importlib.util.find_spec(name)
        if spec is None or getattr(spec.loader, "__class__", type(None)).__name__ == "_StubFinder":
            return _unavailable(f"the reference MeshGraphNet needs {name} (gnn_layers/utils.py:83-84, torch_scatter.scatter at :276), "
                                "which is neither installed in this image nor in the offline wheelhouse")
    return _unavailable("reference MeshGraphNet arm not reached")


_RUNNERS = {"transolver": _transolver, "songunet": _songunet, "fno": _fno, "afno": _afno, "mgn": _mgn}


def run(name, args, rank, world, dev, root):
    try:
        from baseline.ref_runner import import_reference

        import_reference(os.path.join(root, "baseline", "_ref"))
    except Exception as exc:  # noqa: BLE001
        return _unavailable(f"reference import failed: {type(exc).__name__}: {exc}")
    fn = _RUNNERS.get(name)
    if fn is None:
        return _unavailable(f"no reference arm for configuration '{name}'")
    try:
        return fn(args, rank, world, dev)
    except Exception as exc:  # noqa: BLE001
        tb = traceback.format_exc().strip().splitlines()
        where = " | ".join(line.strip() for line in tb[-6:])
        return _unavailable(f"reference run failed: {type(exc).__name__}: {exc} @ {where}")

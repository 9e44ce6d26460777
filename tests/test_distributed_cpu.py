"""Distributed primitives on CPU (gloo) ranks against single-process oracles."""
import pytest
import torch
import torch.distributed as dist

from tests.dist_utils import run_ranks


def _collectives(rank, world):
    from physicsnemo_b200.distributed import (DistributedManager, all_gather_v, gather_v, indexed_all_to_all_v,
                                              scatter_v, fused_all_reduce)
    from physicsnemo_b200.distributed.utils import compute_split_shapes

    m = DistributedManager()
    assert m.rank == rank and m.world_size == world
    torch.manual_seed(0)
    sizes = [3 + r for r in range(world)]
    full = torch.randn(sum(sizes), 4)
    chunks = list(full.split(sizes))
    # all_gather_v fwd + bwd
    x = chunks[rank].clone().requires_grad_(True)
    y = all_gather_v(x, sizes)
    assert torch.allclose(y, full)
    w = torch.arange(y.numel(), dtype=torch.float32).reshape(y.shape)
    (y * w).sum().backward()
    assert torch.allclose(x.grad, world * w.split(sizes)[rank])
    # gather_v / scatter_v
    g = gather_v(chunks[rank], sizes, dst=0)
    if rank == 0:
        assert torch.allclose(g, full)
    s = scatter_v(full if rank == 1 % world else torch.empty(0, 4), sizes, src=1 % world)
    assert torch.allclose(s, chunks[rank])
    # indexed all-to-all-v: rank i sends rows idx[i][j] to rank j
    gen = torch.Generator().manual_seed(1)
    idx_all = [[torch.randint(0, sizes[i], (2 + (i + j) % 3,), generator=gen) for j in range(world)] for i in range(world)]
    send_sizes = [[len(idx_all[i][j]) for j in range(world)] for i in range(world)]
    x = chunks[rank].clone().requires_grad_(True)
    out = indexed_all_to_all_v(x, idx_all[rank], send_sizes)
    ref = torch.cat([chunks[i][idx_all[i][rank]] for i in range(world)])
    assert torch.allclose(out, ref)
    out.sum().backward()
    gref = torch.zeros_like(chunks[rank])
    for j in range(world):
        gref.index_add_(0, idx_all[rank][j], torch.ones(len(idx_all[rank][j]), 4))
    assert torch.allclose(x.grad, gref)
    # fused all reduce keeps structure
    bundle = {"b": torch.ones(3) * (rank + 1), "a": [torch.ones(2, 2), torch.tensor(float(rank))]}
    red = fused_all_reduce(bundle)
    tot = sum(range(1, world + 1))
    assert torch.allclose(red["b"], torch.ones(3) * tot) and torch.allclose(red["a"][0], torch.ones(2, 2) * world)
    assert compute_split_shapes(10, 4) == [3, 3, 3, 1] and compute_split_shapes(9, 4) == [2, 2, 2, 3]


def test_collectives_two_ranks():
    run_ranks(_collectives, world=2)


def test_collectives_three_ranks():
    run_ranks(_collectives, world=3)


def _dist_fft(rank, world):
    from physicsnemo_b200.distributed import DistributedManager
    from physicsnemo_b200.distributed.fft import DistributedIRFFT2, DistributedRFFT2

    m = DistributedManager()
    m.initialize_mesh((world,), ("spatial_parallel",))
    torch.manual_seed(0)
    x = torch.randn(2, 3, 8, 12, dtype=torch.float64)
    ref = torch.fft.rfft2(x, dim=(-2, -1), norm="ortho")
    xl = x.chunk(world, dim=-1)[rank].clone().requires_grad_(True)
    y = DistributedRFFT2.apply(xl, (None, None), (-2, -1), "ortho")
    assert torch.allclose(y, ref.chunk(world, dim=-2)[rank], atol=1e-10)
    back = DistributedIRFFT2.apply(y, (x.shape[-2], x.shape[-1]), (-2, -1), "ortho")
    assert torch.allclose(back, x.chunk(world, dim=-1)[rank], atol=1e-10)
    (y.real.sum() + y.imag.sum()).backward()
    xr = x.clone().requires_grad_(True)
    yr = torch.fft.rfft2(xr, dim=(-2, -1), norm="ortho")
    (yr.real.sum() + yr.imag.sum()).backward()
    assert torch.allclose(xl.grad, xr.grad.chunk(world, dim=-1)[rank], atol=1e-10)


def test_distributed_fft_two_ranks():
    run_ranks(_dist_fft, world=2)


def test_process_group_config_tree():
    from physicsnemo_b200.distributed import ProcessGroupConfig, ProcessGroupNode

    cfg = ProcessGroupConfig(ProcessGroupNode("world"))
    cfg.add_node(ProcessGroupNode("model_parallel"), parent="world")
    cfg.add_node(ProcessGroupNode("data_parallel"), parent="world")
    cfg.add_node(ProcessGroupNode("spatial_parallel"), parent="model_parallel")
    cfg.add_node(ProcessGroupNode("channel_parallel"), parent="model_parallel")
    assert sorted(cfg.leaf_groups()) == ["channel_parallel", "data_parallel", "spatial_parallel"]
    cfg.set_leaf_group_sizes({"spatial_parallel": 2, "channel_parallel": 2, "data_parallel": 4})
    assert cfg.get_node("model_parallel").size == 4 and cfg.get_node("world").size == 16


def _dist_afno(rank, world):
    import torch
    import torch.distributed as dist

    from physicsnemo_b200.distributed import DistributedManager
    from physicsnemo_b200.models.afno.distributed import DistributedAFNO

    DistributedManager.create_process_subgroup("model_parallel", world)
    torch.manual_seed(0)                       # same seed: identical replicated parameters, identical shards
    net = DistributedAFNO(inp_shape=(16, 32), in_channels=3, out_channels=2, patch_size=4, embed_dim=16, depth=2, num_blocks=4)
    assert net._impl.blocks[0].filter.w1.shape[0] == 4 // world and net._impl.pos_embed.shape[1] == 16 // world
    torch.manual_seed(1)
    x = torch.randn(2, 3, 16, 32)
    y = net(x)
    assert y.shape == (2, 2, 16, 32) and torch.isfinite(y).all()
    gathered = [torch.empty_like(y) for _ in range(world)]
    dist.all_gather(gathered, y.detach())
    for g in gathered:                         # the gathered channels and the broadcast head make every rank agree
        assert torch.allclose(g, gathered[0], atol=1e-6)
    y.square().mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in net.parameters())


def test_distributed_afno_two_ranks():
    run_ranks(_dist_afno, world=2)


def _dist_graph(rank, world):
    import torch

    from physicsnemo_b200.nn.module.gnn_layers.distributed_graph import DistributedGraph, partition_graph_nodewise

    torch.manual_seed(0)
    n, e = 40, 200
    dst = torch.randint(0, n, (e,)).sort().values
    src = torch.randint(0, n, (e,))
    src[0] = n - 1                                           # make sure the largest id occurs
    offsets = torch.zeros(n + 1, dtype=torch.long)
    offsets[1:] = torch.bincount(dst, minlength=n).cumsum(0)
    for decomp in (False, True):
        gp = partition_graph_nodewise(offsets, src, world, rank, torch.device("cpu"), matrix_decomp=decomp)
        g = DistributedGraph(offsets, src, world, graph_partition=gp)
        feats = torch.arange(n, dtype=torch.float32)[:, None] * torch.tensor([[1.0, 10.0]])
        part = g.get_src_node_features_in_partition(feats).clone().requires_grad_(True)
        local = g.get_src_node_features_in_local_graph(part)
        # local graph: edge j of this rank reads row local_indices[j]; it must be the feature of its global source
        edge_ids = gp.map_partitioned_edge_ids_to_global.long()
        assert torch.equal(local[gp.local_indices.long()], feats[src[edge_ids]])
        assert gp.local_offsets[-1] == edge_ids.numel() == gp.num_local_indices
        # aggregate onto the local destinations and compare with the global aggregation
        agg = torch.zeros(gp.num_local_dst_nodes, 2).index_add_(
            0, torch.repeat_interleave(torch.arange(gp.num_local_dst_nodes), gp.local_offsets.diff().long()),
            local[gp.local_indices.long()])
        ref = torch.zeros(n, 2).index_add_(0, dst, feats[src])
        assert torch.allclose(agg, ref[gp.map_partitioned_dst_ids_to_global.long()])
        assert torch.allclose(g.get_global_dst_node_features(agg), ref)
        local.sum().backward()                               # gradient of the halo gather = how often a row was sent
        assert part.grad.shape == part.shape and float(part.grad.sum()) == 2.0 * sum(row[r] for row in [gp.sizes[rank]] for r in range(world))
        ef = torch.arange(e, dtype=torch.float32)[:, None]
        assert torch.equal(g.get_global_edge_features(g.get_edge_features_in_partition(ef)), ef)


def test_distributed_graph_two_ranks():
    run_ranks(_dist_graph, world=2)


def _healda_resharding(rank, world):
    import torch
    import torch.distributed as dist

    from physicsnemo_b200.experimental.models.healda.sharding import shard_t, shard_x

    B, T, X, C = 2, 2 * world, 3 * world, 4
    full = torch.arange(B * T * X * C, dtype=torch.float32).view(B, T, X, C)
    t_local = full[:, rank * (T // world):(rank + 1) * (T // world)].clone().requires_grad_(True)
    x_local = shard_x(t_local, dist.group.WORLD)
    assert torch.equal(x_local, full[:, :, rank * (X // world):(rank + 1) * (X // world)])
    back = shard_t(x_local, dist.group.WORLD)
    assert torch.equal(back, t_local)
    # the all-to-all is differentiable: the gradient of sum(w * round_trip) is w itself
    w = torch.randn_like(back)
    (back * w).sum().backward()
    assert torch.allclose(t_local.grad, w)


def test_healda_time_space_resharding():
    run_ranks(_healda_resharding, world=2)


def _rank_that_raises(rank, world):
    import datetime

    import torch
    import torch.distributed as dist

    if rank == 1:
        raise RuntimeError("injected failure before the collective")      # this rank never joins
    # the surviving rank must get a host-side error within the process-group timeout, not hang
    t = torch.ones(4)
    try:
        work = dist.all_reduce(t, async_op=True)
        ok = work.wait(timeout=datetime.timedelta(seconds=3))
        raise AssertionError(f"collective completed although a rank never joined (ok={ok})")
    except AssertionError:
        raise
    except Exception as exc:  # noqa: BLE001  (timeout / connection error raised on the host)
        print(f"survivor saw: {type(exc).__name__}")


def test_failed_rank_gives_host_side_error_not_a_hang():
    """One rank raises before a collective; the other's wait ends with an error on the host inside the time limit."""
    import time

    from tests.dist_utils import run_ranks

    t0 = time.time()
    with pytest.raises(RuntimeError) as err:
        run_ranks(_rank_that_raises, world=2, timeout=60)
    assert "injected failure" in str(err.value)
    assert time.time() - t0 < 60


def _partitioned_mgn(rank, world):
    """MeshGraphNet on a destination-owned graph partition == MeshGraphNet on the whole graph (forward + gradients)."""
    import numpy as np

    from physicsnemo_b200.models.meshgraphnet import MeshGraphNet
    from physicsnemo_b200.nn.module.gnn_layers.graph_types import Graph
    from physicsnemo_b200.parallel.graph_partition import PartitionedGraph, plan_partition, spatial_order

    rng = np.random.default_rng(0)
    n = 300
    pts = rng.random((n, 2))
    src = rng.integers(0, n, 1500)
    dst = rng.integers(0, n, 1500)
    keep = src != dst
    src, dst = src[keep], dst[keep]
    order = spatial_order(pts)
    inv = np.empty(n, dtype=np.int64)
    inv[order] = np.arange(n)
    src, dst = inv[src], inv[dst]                       # spatially sorted numbering
    torch.manual_seed(0)
    nfeat = torch.randn(n, 6, dtype=torch.float64)
    efeat = torch.randn(len(src), 3, dtype=torch.float64)
    target = torch.randn(n, 3, dtype=torch.float64)
    model = MeshGraphNet(6, 3, 3, processor_size=3, hidden_dim_processor=16, hidden_dim_node_encoder=16,
                         hidden_dim_edge_encoder=16, hidden_dim_node_decoder=16, mlp_activation_fn="silu").double()
    full = model(nfeat, efeat, Graph(torch.from_numpy(np.stack([src, dst])), num_nodes=n))
    ((full - target) ** 2).sum().backward()
    ref = {k: p.grad.clone() for k, p in model.named_parameters()}
    model.zero_grad()
    plan = plan_partition(np.stack([src, dst]), n, world, rank)
    pg = PartitionedGraph(plan, "cpu", group=None)
    lo, hi = plan.node_range
    out = model(nfeat[lo:hi], efeat[torch.from_numpy(plan.edge_ids)], pg)
    assert torch.allclose(out, full[lo:hi], atol=1e-9), float((out - full[lo:hi]).abs().max())
    ((out - target[lo:hi]) ** 2).sum().backward()
    for k, p in model.named_parameters():
        g = p.grad.clone()
        dist.all_reduce(g)
        assert torch.allclose(g, ref[k], atol=1e-8, rtol=1e-7), (k, float((g - ref[k]).abs().max()))
    assert plan.n_halo > 0 and len(plan.send_idx) > 0


def test_partitioned_meshgraphnet_three_ranks():
    run_ranks(_partitioned_mgn, world=3, timeout=240)


def _sharded_optimizer_checkpoint(rank, world, tmp):
    """Adam on DTensor-sharded parameters: save on two ranks (Shard(0)), reload with another layout (Shard(1)) and compare
    the moments; the file is also read back by a single process afterwards."""
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor

    from physicsnemo_b200.utils.checkpoint import load_checkpoint, save_checkpoint

    mesh = init_device_mesh("cpu", (world,))

    def build(dim):
        torch.manual_seed(0)
        lin = torch.nn.Linear(6, 4)
        lin.weight = torch.nn.Parameter(distribute_tensor(lin.weight.detach(), mesh, [Shard(dim)]))
        return lin

    model = build(0)
    opt = torch.optim.Adam(model.parameters(), lr=1e-2)
    torch.manual_seed(1)
    for _ in range(3):
        x = torch.randn(5, 6)
        y = torch.nn.functional.linear(x, model.weight.full_tensor(), model.bias)
        opt.zero_grad()
        y.square().sum().backward()
        opt.step()
    want = {k: opt.state[model.weight][k].full_tensor().clone() for k in ("exp_avg", "exp_avg_sq")}
    want_w = model.weight.full_tensor().clone()
    save_checkpoint(tmp, models=model, optimizer=opt, epoch=3)
    if rank == 0:
        torch.save({"w": want_w, **want, "bias_avg": opt.state[model.bias]["exp_avg"].clone()}, tmp + "/expected.pt")
    # other layout, same job
    model2 = build(1)
    with torch.no_grad():
        model2.weight.mul_(0.0)
    opt2 = torch.optim.Adam(model2.parameters(), lr=1e-2)
    assert load_checkpoint(tmp, models=model2, optimizer=opt2) == 3
    st = opt2.state[model2.weight]
    assert st["exp_avg"].placements == model2.weight.placements          # re-sharded like the new parameter
    for k in ("exp_avg", "exp_avg_sq"):
        assert torch.allclose(st[k].full_tensor(), want[k])
    assert torch.allclose(model2.weight.full_tensor(), want_w)
    assert int(st["step"]) == 3


def test_sharded_optimizer_state_checkpoint(tmp_path):
    from physicsnemo_b200.utils.checkpoint import load_checkpoint

    run_ranks(_sharded_optimizer_checkpoint, world=2, args=(str(tmp_path),))
    # a single process (no sharding at all) resumes from the same files
    exp = torch.load(str(tmp_path / "expected.pt"))
    torch.manual_seed(0)
    lin = torch.nn.Linear(6, 4)
    opt = torch.optim.Adam(lin.parameters(), lr=1e-2)
    assert load_checkpoint(str(tmp_path), models=lin, optimizer=opt) == 3
    assert torch.allclose(lin.weight, exp["w"])
    assert torch.allclose(opt.state[lin.weight]["exp_avg"], exp["exp_avg"])
    assert torch.allclose(opt.state[lin.weight]["exp_avg_sq"], exp["exp_avg_sq"])
    assert torch.allclose(opt.state[lin.bias]["exp_avg"], exp["bias_avg"])

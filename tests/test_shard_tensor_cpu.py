"""Domain-parallel oracle: the same module on gathered data (one process) and on sharded
data (gloo ranks) must agree in outputs, input gradients and parameter gradients."""
import copy

import torch
import torch.distributed as dist

from tests.dist_utils import run_ranks


def _check(name, a, b, tol=1e-5):
    err = (a - b).abs().max().item()
    assert err <= tol * max(1.0, b.abs().max().item()), f"{name}: max err {err}"


def _numerical_check(mesh, module, full_inputs, shard_dims, tol=1e-5, sizes=None):
    """Run ``module`` on full inputs and on ShardTensors; compare forward and all gradients."""
    from physicsnemo_b200.parallel import Replicate, Shard, ShardTensor, reduce_param_grads

    rank, world = dist.get_rank(), dist.get_world_size()
    ref = copy.deepcopy(module)
    full = [t.clone().requires_grad_(t.is_floating_point()) for t in full_inputs]
    out_ref = ref(*full)
    out_ref.float().mean().backward()
    shards = []
    for t, d in zip(full_inputs, shard_dims):
        if d is None:
            shards.append(ShardTensor.from_local(t.clone(), mesh, [Replicate()]))
            continue
        if sizes is None:
            pieces = t.tensor_split(world, dim=d)
        else:
            pieces = t.split(sizes, dim=d)
        loc = pieces[rank].clone().requires_grad_(t.is_floating_point())
        shards.append(ShardTensor.from_local(loc, mesh, [Shard(d)]))
    out = module(*shards)
    assert isinstance(out, ShardTensor), type(out)
    _check("forward", out.full_tensor().detach(), out_ref.detach(), tol)
    loss = out.float().mean()
    loss.backward()
    for (n, p), (_, q) in zip(module.named_parameters(), ref.named_parameters()):
        assert p.grad is not None, n
        _check(f"grad {n}", p.grad, q.grad, tol * 10)
    for s, f, d in zip(shards, full, shard_dims):
        if d is None or not f.is_floating_point():
            continue
        pieces = f.grad.tensor_split(world, dim=d) if sizes is None else f.grad.split(sizes, dim=d)
        _check("input grad", s.grad.to_local(), pieces[rank], tol * 10)


def _conv_norm_pool(rank, world):
    from physicsnemo_b200.distributed import DistributedManager

    mesh = DistributedManager().initialize_mesh((world,), ("domain",))
    torch.manual_seed(0)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.c1 = torch.nn.Conv2d(3, 8, 3, padding=1)
            self.gn = torch.nn.GroupNorm(4, 8)
            self.c2 = torch.nn.Conv2d(8, 8, 3, padding=1, stride=2)
            self.c3 = torch.nn.Conv2d(8, 4, 1)
            self.up = torch.nn.ConvTranspose2d(4, 4, 2, stride=2)

        def forward(self, x):
            x = torch.nn.functional.silu(self.gn(self.c1(x)))
            x = self.c2(x)
            x = torch.nn.functional.avg_pool2d(x, 2)
            x = self.up(self.c3(x))
            x = torch.nn.functional.interpolate(x, scale_factor=2, mode="nearest")
            return torch.nn.functional.pad(x, (1, 1, 2, 2))

    x = torch.randn(2, 3, 16 * world, 12, dtype=torch.float64)
    _numerical_check(mesh, Net().double(), [x], [2], tol=1e-9)
    # uneven shards, valid convolution (no padding), bilinear up-sampling
    class Net2(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.c = torch.nn.Conv2d(2, 3, 5, padding=0)

        def forward(self, x):
            return torch.nn.functional.interpolate(self.c(x), scale_factor=2, mode="bilinear")

    sizes = [7 + r for r in range(world)]
    x = torch.randn(1, 2, sum(sizes), 9, dtype=torch.float64)
    _numerical_check(mesh, Net2().double(), [x], [2], tol=1e-9, sizes=sizes)


def test_conv_norm_pool_two_ranks():
    run_ranks(_conv_norm_pool, world=2)


def test_conv_norm_pool_three_ranks():
    run_ranks(_conv_norm_pool, world=3)


def _attention_and_transolver(rank, world):
    from physicsnemo_b200.distributed import DistributedManager
    from physicsnemo_b200.models.transolver import Transolver
    from physicsnemo_b200.parallel import Replicate, Shard, ShardTensor

    mesh = DistributedManager().initialize_mesh((world,), ("domain",))
    torch.manual_seed(0)

    class Attn(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.qkv = torch.nn.Linear(16, 48)

        def forward(self, x):
            B, N, _ = x.shape
            q, k, v = self.qkv(x).reshape(B, N, 3, 2, 8).permute(2, 0, 3, 1, 4).unbind(0)
            o = torch.nn.functional.scaled_dot_product_attention(q, k, v)
            return o.transpose(1, 2).reshape(B, N, 16)

    x = torch.randn(2, 6 * world + 1, 16, dtype=torch.float64)
    sizes = [6] * (world - 1) + [7]
    _numerical_check(mesh, Attn().double(), [x], [1], tol=1e-9, sizes=sizes)
    model = Transolver(functional_dim=2, out_dim=3, embedding_dim=3, n_layers=2, n_hidden=32, n_head=4, slice_num=8,
                       use_te=False).double()
    fx = torch.randn(1, 10 * world, 2, dtype=torch.float64)
    emb = torch.randn(1, 10 * world, 3, dtype=torch.float64)

    class Wrap(torch.nn.Module):
        def __init__(self, m):
            super().__init__()
            self.m = m

        def forward(self, fx, emb):
            return self.m(fx, embedding=emb)

    _numerical_check(mesh, Wrap(model), [fx, emb], [1, 1], tol=1e-8)


def test_ring_attention_and_transolver_two_ranks():
    run_ranks(_attention_and_transolver, world=2)


def _redistribute_and_scatter(rank, world):
    from physicsnemo_b200.distributed import DistributedManager
    from physicsnemo_b200.parallel import Partial, Replicate, Shard, ShardTensor, scatter_tensor, sync_module_over_mesh

    mesh = DistributedManager().initialize_mesh((world,), ("domain",))
    torch.manual_seed(0)
    full = torch.randn(5, 7, 4)
    st = scatter_tensor(full if rank == 0 else None, 0, mesh, (Shard(1),))
    assert tuple(st.shape) == (5, 7, 4)
    assert torch.equal(st.full_tensor(), full)
    moved = st.redistribute(placements=[Shard(0)])
    assert torch.equal(moved.full_tensor(), full) and moved.placements[0] == Shard(0)
    part = ShardTensor.from_local(torch.ones(3) * (rank + 1), mesh, [Partial("sum")])
    assert torch.equal(part.full_tensor(), torch.ones(3) * sum(range(1, world + 1)))
    s = st.sum(dim=1)
    assert isinstance(s.placements[0], Partial) and torch.allclose(s.full_tensor(), full.sum(1), atol=1e-5)
    assert abs(st.mean().item() - full.mean().item()) < 1e-6
    assert torch.allclose(st.amax(dim=1).full_tensor(), full.amax(1))
    lin = torch.nn.Linear(4, 4)
    sync_module_over_mesh(lin, mesh, verify=True)
    w = lin.weight.detach().clone()
    dist.broadcast(w, src=0)
    assert torch.equal(w, lin.weight)


def test_redistribute_scatter_sync_three_ranks():
    run_ranks(_redistribute_and_scatter, world=3)


def _sharded_preconditioner(rank, world):
    """EDM preconditioner on a height-sharded activation: the per-sample coefficients are plain tensors, also when the
    noise level arrives as a replicated ShardTensor, and the result matches the unsharded call."""
    from physicsnemo_b200.core.module import Module
    from physicsnemo_b200.diffusion.preconditioners import EDMPreconditioner
    from physicsnemo_b200.distributed import DistributedManager
    from physicsnemo_b200.parallel import Replicate, Shard, ShardTensor

    mesh = DistributedManager().initialize_mesh((world,), ("domain",))

    class Net(Module):
        def __init__(self):
            super().__init__()
            self.conv = torch.nn.Conv2d(2, 2, 3, padding=1)

        def forward(self, x, noise_labels):
            return self.conv(x) * noise_labels.reshape(-1, 1, 1, 1).to(x.dtype)

    torch.manual_seed(0)
    net = EDMPreconditioner(Net(), sigma_data=[0.5, 0.8])
    x = torch.randn(3, 2, 8, 6)
    t = torch.tensor([0.3, 1.0, 4.0])
    want = net(x, t)
    rows = x.tensor_split(world, dim=2)[rank].clone()
    xs = ShardTensor.from_local(rows, mesh, [Shard(2)])
    for level in (t, ShardTensor.from_local(t.clone(), mesh, [Replicate()])):
        got = net(xs, level)
        assert isinstance(got, ShardTensor)
        _check("preconditioned output", got.full_tensor(), want)
    c = net._coefficients_for(xs, ShardTensor.from_local(t.clone(), mesh, [Replicate()]))
    assert all(type(v) is torch.Tensor for v in c)


def test_preconditioner_on_shard_tensor_two_ranks():
    run_ranks(_sharded_preconditioner, world=2)


def _shard_tensor_api(rank, world):
    """DTensor bridge, gradient layouts of ``to_local``, the async flag of ``redistribute`` and the flatten protocol."""
    from torch.distributed.tensor import DTensor, Partial, Replicate, Shard, distribute_tensor

    from physicsnemo_b200.distributed import DistributedManager
    from physicsnemo_b200.parallel import ShardTensor

    mesh = DistributedManager().initialize_mesh((world,), ("domain",))
    torch.manual_seed(0)
    full = torch.randn(7, 5)
    # DTensor -> ShardTensor -> DTensor, uneven chunks included (7 rows over the ranks)
    dt = distribute_tensor(full, mesh, [Shard(0)])
    st = ShardTensor.from_dtensor(dt)
    assert isinstance(st, ShardTensor) and tuple(st.shape) == (7, 5)
    assert torch.equal(st.to_local(), dt.to_local()) and torch.equal(st.full_tensor(), full)
    back = st.to_dtensor()
    assert isinstance(back, DTensor) and torch.equal(back.full_tensor(), full)
    rep = ShardTensor.from_dtensor(distribute_tensor(full, mesh, [Replicate()]))
    assert rep._spec.is_replicated()
    # to_local(grad_placements=[Partial()]) on a replicated tensor: the ranks' gradient shares are summed
    leaf = full.clone().requires_grad_(True)
    r = ShardTensor.from_local(leaf, mesh, [Replicate()])
    loc = r.to_local(grad_placements=[Partial()])
    (loc * float(rank + 1)).sum().backward()
    want = float(sum(range(1, world + 1)))
    assert torch.allclose(leaf.grad, torch.full_like(full, want))
    leaf2 = full.clone().requires_grad_(True)
    ShardTensor.from_local(leaf2, mesh, [Replicate()]).to_local().sum().backward()          # default: no reduction
    assert torch.allclose(leaf2.grad, torch.ones_like(full))
    # redistribute(async_op=True) gives the same values (on CPU it completes synchronously)
    g = st.redistribute(placements=[Replicate()], async_op=True)
    assert torch.equal(g.to_local(), full)
    # wrapper-subclass protocol used by tracing
    names, meta = st.__tensor_flatten__()
    again = ShardTensor.__tensor_unflatten__({n: getattr(st, n) for n in names}, meta, tuple(st.shape), None)
    assert torch.equal(again.to_local(), st.to_local()) and again._spec is st._spec


def test_shard_tensor_api_three_ranks():
    run_ranks(_shard_tensor_api, world=3)


def _ring_neighbor_search(rank, world):
    """kNN and capped radius search with points and queries sharded (uneven shards) against the single-process result."""
    from physicsnemo_b200.distributed import DistributedManager
    from physicsnemo_b200.nn.functional.neighbors.knn import knn
    from physicsnemo_b200.nn.functional.neighbors.radius_search import radius_search
    from physicsnemo_b200.parallel import Replicate, Shard, ShardTensor

    mesh = DistributedManager().initialize_mesh((world,), ("domain",))
    torch.manual_seed(0)
    pts, qry = torch.rand(101, 3), torch.rand(37, 3)
    p_loc = pts.tensor_split(world)[rank].clone()
    q_loc = qry.tensor_split(world)[rank].clone().requires_grad_(True)
    ps = ShardTensor.from_local(p_loc, mesh, [Shard(0)])
    qs = ShardTensor.from_local(q_loc, mesh, [Shard(0)])
    want_i, want_d = knn(pts, qry, 5)
    got_i, got_d = knn(ps, qs, 5)
    assert isinstance(got_i, ShardTensor) and torch.equal(got_i.full_tensor(), want_i)
    _check("knn distances", got_d.full_tensor().detach(), want_d)
    got_d.to_local().sum().backward()                     # distances are differentiable in the queries
    assert q_loc.grad is not None and torch.isfinite(q_loc.grad).all()
    # sharded points, replicated queries
    ri, rd = knn(ps, ShardTensor.from_local(qry.clone(), mesh, [Replicate()]), 4)
    wi, wd = knn(pts, qry, 4)
    assert torch.equal(ri.to_local(), wi)
    # replicated points, sharded queries: purely local
    li, _ = knn(ShardTensor.from_local(pts.clone(), mesh, [Replicate()]), qs, 3)
    assert torch.equal(li.full_tensor(), knn(pts, qry, 3)[0])
    # ball query, at most 6 neighbours per query: same neighbour sets and distances
    want = radius_search(pts, qry, 0.25, 6, True, True)
    got = radius_search(ps, qs, 0.25, 6, True, True)
    gi, gp, gd = (t.full_tensor() for t in got)
    wd_sorted, _ = torch.sort(torch.where(want[2] > 0, want[2], torch.full_like(want[2], 9.0)), dim=1)
    gd_sorted, _ = torch.sort(torch.where(gd > 0, gd, torch.full_like(gd, 9.0)), dim=1)
    _check("ball query distances", gd_sorted.detach(), wd_sorted)
    found = gd > 0
    assert torch.allclose(gp[found], pts[gi[found]])


def test_ring_knn_and_ball_query_three_ranks():
    run_ranks(_ring_neighbor_search, world=3)


def _sharded_sdf(rank, world):
    from physicsnemo_b200.distributed import DistributedManager
    from physicsnemo_b200.nn.functional.geometry.sdf import signed_distance_field
    from physicsnemo_b200.parallel import Shard, ShardTensor

    mesh = DistributedManager().initialize_mesh((world,), ("domain",))
    verts = torch.tensor([[0.0, 0, 0], [1, 0, 0], [0, 1, 0], [0, 0, 1]])
    faces = torch.tensor([[0, 2, 1], [0, 1, 3], [0, 3, 2], [1, 2, 3]], dtype=torch.int32)
    torch.manual_seed(0)
    pts = torch.rand(23, 3) * 1.5 - 0.25
    want = signed_distance_field(verts, faces, pts)
    loc = pts.tensor_split(world)[rank].clone()
    got = signed_distance_field(ShardTensor.from_local(verts.tensor_split(world)[rank].clone(), mesh, [Shard(0)]),
                                ShardTensor.from_local(faces.tensor_split(world)[rank].clone(), mesh, [Shard(0)]),
                                ShardTensor.from_local(loc, mesh, [Shard(0)]))
    want = want if isinstance(want, tuple) else (want,)
    got = got if isinstance(got, tuple) else (got,)
    for w, g in zip(want, got):
        assert isinstance(g, ShardTensor)
        _check("sdf output", g.full_tensor().float(), w.float())


def test_sharded_sdf_two_ranks():
    run_ranks(_sharded_sdf, world=2)


def _fsdp2_with_domain_parallel(rank, world):
    """2-D mesh: FSDP2 (``fully_shard``) shards the parameters over "dp" and splits the batch, ShardTensor splits the
    image height over "domain".  Forward and parameter gradients match the single-process model on the whole batch."""
    from torch.distributed.fsdp import fully_shard

    from physicsnemo_b200.distributed import DistributedManager
    from physicsnemo_b200.parallel import Shard, ShardTensor

    mesh = DistributedManager().initialize_mesh((2, 2), ("dp", "domain"))
    dp, dom = mesh["dp"], mesh["domain"]
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Conv2d(3, 8, 3, padding=1), torch.nn.GroupNorm(2, 8), torch.nn.SiLU(),
                              torch.nn.Conv2d(8, 4, 3, padding=1))
    ref = copy.deepcopy(net)
    fully_shard(net, mesh=dp)
    x = torch.randn(4, 3, 8, 6)
    dp_r, dom_r = dp.get_local_rank(), dom.get_local_rank()
    rows = x.tensor_split(2, dim=0)[dp_r].tensor_split(2, dim=2)[dom_r].clone()
    y = net(ShardTensor.from_local(rows, dom, [Shard(2)]))
    assert isinstance(y, ShardTensor)
    y.float().square().mean().backward()
    yr = ref(x)
    yr.square().mean().backward()
    _check("forward", y.full_tensor().detach(), yr.tensor_split(2, dim=0)[dp_r].detach(), 1e-5)
    for (name, p), (_, q) in zip(net.named_parameters(), ref.named_parameters()):
        assert hasattr(p.grad, "full_tensor"), name                  # FSDP2 keeps parameters and gradients as DTensors
        _check(f"grad {name}", p.grad.full_tensor(), q.grad, 1e-4)


def test_fsdp2_coexists_with_shard_tensor_four_ranks():
    run_ranks(_fsdp2_with_domain_parallel, world=4)


def _sharded_natten(rank, world):
    """2-D neighbourhood attention on a height-sharded token grid vs the whole grid (output and q / k / v gradients)."""
    from physicsnemo_b200.distributed import DistributedManager
    from physicsnemo_b200.nn.functional.natten import na2d
    from physicsnemo_b200.parallel import Shard, ShardTensor

    mesh = DistributedManager().initialize_mesh((world,), ("domain",))
    torch.manual_seed(0)
    full = [torch.randn(1, 12, 7, 2, 8) for _ in range(3)]
    dy = torch.randn(1, 12, 7, 2, 8)
    for kernel, dilation in ((3, 1), (5, 1), (3, 2)):
        ref_in = [t.clone().requires_grad_(True) for t in full]
        ref = na2d(*ref_in, kernel, dilation=dilation)
        ref.backward(dy)
        loc = [t.tensor_split(world, dim=1)[rank].clone().requires_grad_(True) for t in full]
        st = [ShardTensor.from_local(t, mesh, [Shard(1)]) for t in loc]
        out = na2d(*st, kernel, dilation=dilation)
        assert isinstance(out, ShardTensor)
        _check(f"natten k={kernel} d={dilation}", out.full_tensor().detach(), ref.detach(), 1e-5)
        out.to_local().backward(dy.tensor_split(world, dim=1)[rank])
        for a, b in zip(loc, ref_in):
            _check("natten input grad", a.grad, b.grad.tensor_split(world, dim=1)[rank], 1e-4)


def test_sharded_neighbourhood_attention_two_ranks():
    run_ranks(_sharded_natten, world=2)


def _spec_hashes(rank, world):
    from physicsnemo_b200.distributed import DistributedManager
    from physicsnemo_b200.parallel import Replicate, Shard, ShardTensor

    mesh = DistributedManager().initialize_mesh((world,), ("domain",))
    even = ShardTensor.from_local(torch.zeros(4, 3), mesh, [Shard(0)])
    uneven = ShardTensor.from_local(torch.zeros(5 if rank == 0 else 3, 3), mesh, [Shard(0)])
    again = ShardTensor.from_local(torch.ones(4, 3), mesh, [Shard(0)])
    repl = ShardTensor.from_local(torch.zeros(8, 3), mesh, [Replicate()])
    digests = {n: t._spec._stable_hash() for n, t in (("even", even), ("uneven", uneven), ("again", again), ("repl", repl))}
    assert digests["even"] == digests["again"] and len({digests["even"], digests["uneven"], digests["repl"]}) == 3
    # equal on every rank for the even layout (same local shape), different for the uneven one (local shapes differ)
    gathered = [None] * world
    dist.all_gather_object(gathered, digests)
    assert gathered[0]["even"] == gathered[1]["even"] and gathered[0]["repl"] == gathered[1]["repl"]
    assert gathered[0]["uneven"] != gathered[1]["uneven"]
    assert hash(even._spec) == hash(again._spec)


def test_spec_stable_hash_two_ranks():
    run_ranks(_spec_hashes, world=2)

"""Cluster tree, learned field kernels and the GLOBE model (CPU).

Follows the reference's ``test/experimental/models/globe`` strategy: structural invariants of the tree
and of the interaction lists, agreement of the tree-accelerated kernel with the exact sum, and the
physical symmetries the architecture promises (rotation / translation equivariance, invariance to a
uniform rescaling, insensitivity to boundary refinement).
"""
import math

import pytest
import torch

from physicsnemo_b200.experimental.models.globe import GLOBE, BarnesHutKernel, Kernel, MultiscaleKernel
from physicsnemo_b200.mesh.cluster_tree import ClusterTree, ragged_arange
from physicsnemo_b200.mesh.mesh import Mesh


def test_ragged_arange():
    pos, row = ragged_arange(torch.tensor([5, 0, 9]), torch.tensor([2, 0, 3]))
    assert pos.tolist() == [5, 6, 9, 10, 11] and row.tolist() == [0, 0, 2, 2, 2]


@pytest.mark.parametrize("leaf_size", [1, 3, 8])
def test_tree_structure(leaf_size):
    torch.manual_seed(0)
    pts = torch.randn(257, 3)
    tree = ClusterTree.from_points(pts, leaf_size)
    assert sorted(tree.order.tolist()) == list(range(257))
    leaves = tree.left < 0
    assert int(tree.count[leaves].sum()) == 257 and int(tree.count[leaves].max()) <= leaf_size
    inner = (~leaves).nonzero().squeeze(1)
    assert torch.equal(tree.count[inner], tree.count[tree.left[inner]] + tree.count[tree.right[inner]])
    assert torch.equal(tree.start[tree.left[inner]], tree.start[inner])
    assert bool((tree.left[inner] > inner).all())
    for i in (0, 1, int(inner[-1]), tree.n_nodes - 1):
        p = pts[tree.order[tree.start[i]:tree.start[i] + tree.count[i]]]
        assert torch.equal(p.min(0).values, tree.lo[i]) and torch.equal(p.max(0).values, tree.hi[i])
    w = torch.rand(257)
    agg = tree.aggregates(pts, w, {"f": pts[:, :2] * 2})
    i = int(inner[len(inner) // 2])
    ids = tree.order[tree.start[i]:tree.start[i] + tree.count[i]]
    want = (pts[ids] * w[ids, None]).sum(0) / w[ids].sum()
    assert torch.allclose(agg.centroid[i], want, atol=1e-6)
    assert torch.allclose(agg.data["f"][i], 2 * want[:2], atol=1e-6)
    assert ClusterTree.from_points(pts[:0]).n_nodes == 0


@pytest.mark.parametrize("theta", [0.0, 0.6, 2.0])
@pytest.mark.parametrize("leaf_size", [1, 4])
def test_plan_covers_every_pair_once(theta, leaf_size):
    torch.manual_seed(1)
    src, tgt = torch.rand(150, 2), torch.rand(90, 2) + torch.tensor([0.8, 0.0])
    st, tt = ClusterTree.from_points(src, leaf_size), ClusterTree.from_points(tgt, leaf_size)
    plan = st.find_interactions(tt, theta)
    cover = torch.zeros(90, 150)
    cover.index_put_((plan.near_targets, plan.near_sources), torch.ones(plan.n_near), accumulate=True)
    pos, row = ragged_arange(st.start[plan.far_nodes], st.count[plan.far_nodes])
    cover.index_put_((plan.far_targets[row], st.order[pos]), torch.ones(pos.numel()), accumulate=True)
    assert torch.equal(cover, torch.ones_like(cover))
    if theta == 0.0:
        assert plan.n_far == 0
    # self interaction: the same tree on both sides
    plan = st.find_interactions(st, theta)
    assert plan.n_near + sum(int(st.count[n]) for n in plan.far_nodes.tolist()) == 150 * 150


def _kernel_inputs(n_s=50, n_t=35, d=3):
    torch.manual_seed(2)
    data = {"normals": torch.nn.functional.normalize(torch.randn(n_s, d), dim=-1), "physical": {"a": torch.randn(n_s)}}
    glob = {"re": torch.tensor(0.3), "dir": torch.nn.functional.normalize(torch.randn(d), dim=0)}
    return torch.randn(n_s, d), torch.randn(n_t, d), torch.rand(n_s), data, glob


@pytest.mark.parametrize("d", [2, 3])
@pytest.mark.parametrize("network_type", ["pade", "mlp"])
def test_tree_kernel_matches_exact_sum(d, network_type):
    src, tgt, strength, data, glob = _kernel_inputs(d=d)
    k = BarnesHutKernel(n_spatial_dims=d, output_field_ranks={"p": 0, "u": 1}, leaf_size=2,
                        source_data_ranks={"normals": 1, "physical": {"a": 0}}, global_data_ranks={"re": 0, "dir": 1},
                        hidden_layer_sizes=[16, 16], network_type=network_type).eval()
    assert k.network_in_features == 2 + 3 + 3 * 4 and k.network_out_features == 1 + 5
    common = dict(reference_length=torch.tensor(0.7), source_points=src, target_points=tgt, source_strengths=strength,
                  source_data=data, global_data=glob)
    with torch.no_grad():
        exact = Kernel.forward(k, **common)
        chunked = Kernel.forward(k, target_chunk_size=8, **common)
    errs = []
    for theta in (0.0, 0.4, 1.2):
        with torch.no_grad():
            fast = k(theta=theta, chunk_size=500, **common)
        errs.append(max(float((fast[n] - exact[n]).abs().max() / exact[n].abs().max()) for n in exact))
    assert errs[0] < 1e-5 and errs[1] < 0.1 and errs[1] <= errs[2] + 1e-6
    for n in exact:
        assert exact[n].shape == ((35,) if n == "p" else (35, d))
        assert torch.allclose(exact[n], chunked[n], atol=1e-6)
    with pytest.raises(ValueError, match="lacks"):
        k(reference_length=torch.tensor(1.0), source_points=src, target_points=tgt, source_data={}, global_data=glob)


def test_kernel_gradients_with_checkpointing():
    src, tgt, strength, data, glob = _kernel_inputs()
    ranks = dict(n_spatial_dims=3, output_field_ranks={"p": 0, "u": 1}, leaf_size=2,
                 source_data_ranks={"normals": 1, "physical": {"a": 0}}, global_data_ranks={"re": 0, "dir": 1},
                 hidden_layer_sizes=[8])
    grads = []
    for ckpt in (True, False):
        torch.manual_seed(5)
        k = BarnesHutKernel(use_gradient_checkpointing=ckpt, **ranks).train()
        s = strength.clone().requires_grad_(True)
        out = k(reference_length=torch.tensor(0.7), source_points=src, target_points=tgt, source_strengths=s,
                source_data=data, global_data=glob, theta=0.8, chunk_size=300)
        (out["p"].sum() + out["u"].square().sum()).backward()
        grads.append([s.grad] + [p.grad for p in k.parameters()])
    for a, b in zip(*grads):
        assert torch.allclose(a, b, atol=1e-6)


def _ring(n, radius, centre=(0.0, 0.0)):
    a = torch.linspace(0, 2 * math.pi, n + 1)[:-1]
    pts = torch.stack([radius * a.cos() + centre[0], radius * a.sin() + centre[1]], 1)
    cells = torch.stack([torch.arange(n), (torch.arange(n) + 1) % n], 1)
    return pts, cells


def _globe_2d(theta=0.0, **kw):
    torch.manual_seed(3)
    args = dict(n_spatial_dims=2, output_field_ranks={"p": 0, "u": 1},
                boundary_source_data_ranks={"wall": {"temp": 0, "slip": 1}, "far": {}},
                reference_length_names=["chord", "delta"], reference_area=1.0, global_data_ranks={"re": 0, "wind": 1},
                hidden_layer_sizes=[16, 16], n_latent_scalars=3, n_latent_vectors=2, theta=theta,
                n_communication_hyperlayers=1)
    args.update(kw)
    return GLOBE(**args).eval()


def _globe_inputs(n_wall=36, scale=1.0, rot=None, shift=None, reverse_cells=False):
    torch.manual_seed(4)
    rot = torch.eye(2) if rot is None else rot
    shift = torch.zeros(2) if shift is None else shift
    p, c = _ring(n_wall, 1.0)
    angle = torch.atan2(p[c].mean(1)[:, 1], p[c].mean(1)[:, 0])
    slip = torch.stack([angle.cos() * 0.3, (2 * angle).sin()], 1)
    wall = Mesh(scale * (p @ rot.T) + shift, c, cell_data={"temp": (3 * angle).sin(), "slip": slip @ rot.T})
    p2, c2 = _ring(20, 6.0)
    if reverse_cells:       # a reflection reverses orientation; the vertex order restores outward normals
        wall = Mesh(wall.points, c.flip(1), cell_data=wall.cell_data)
        c2 = c2.flip(1)
    far = Mesh(scale * (p2 @ rot.T) + shift, c2)
    q = torch.randn(25, 2) * 2.5
    lengths = {"chord": torch.tensor(1.0 * scale), "delta": torch.tensor(0.05 * scale)}
    glob = {"re": torch.tensor(0.3), "wind": torch.tensor([1.0, 0.2]) @ rot.T}
    return scale * (q @ rot.T) + shift, {"wall": wall, "far": far}, lengths, glob


def test_globe_forward_shapes_backward_and_validation():
    model = _globe_2d(theta=0.7).train()
    q, meshes, lengths, glob = _globe_inputs()
    out = model(q, meshes, lengths, glob, prediction_chunk_size=10)
    assert out.point_data["p"].shape == (25,) and out.point_data["u"].shape == (25, 2)
    assert out.n_cells == 0 and torch.equal(out.points, q)
    sum(v.square().sum() for v in out.point_data.values()).backward()
    assert all(p.grad is not None for p in model.parameters())
    assert len(model.kernel_layers) == 2 and set(model.kernel_layers[0].keys()) == {"wall", "far"}
    assert [lin.bias is not None for lin in model.final_field_transforms] == [True, False]
    # a subset of the boundary types is allowed, unknown types and wrong reference lengths are not
    model(q, {"wall": meshes["wall"]}, lengths, glob)
    with pytest.raises(ValueError, match="instantiated for"):
        model(q, {"inlet": meshes["far"]}, lengths, glob)
    with pytest.raises(ValueError, match="reference lengths"):
        model(q, meshes, {"chord": torch.tensor(1.0)}, glob)
    with pytest.raises(KeyError, match="temp"):
        model(q, {"wall": meshes["far"]}, lengths, glob)
    with pytest.raises(ValueError, match="theta"):
        _globe_2d(theta=-1.0)
    with pytest.raises(ValueError, match="must not contain"):
        _globe_2d(boundary_source_data_ranks={"a.b": {}})


def test_globe_is_equivariant_to_rigid_motions_and_uniform_scaling():
    model = _globe_2d(theta=0.0, latent_compression_scale=2.0)
    with torch.no_grad():
        base = model(*_globe_inputs()).point_data
        a = 0.9
        rot = torch.tensor([[math.cos(a), -math.sin(a)], [math.sin(a), math.cos(a)]])
        moved = model(*_globe_inputs(rot=rot, shift=torch.tensor([3.0, -1.0]))).point_data
        mirrored = model(*_globe_inputs(rot=torch.tensor([[1.0, 0.0], [0.0, -1.0]]), reverse_cells=True)).point_data
    assert torch.allclose(moved["p"], base["p"], atol=2e-5)
    assert torch.allclose(moved["u"], base["u"] @ rot.T, atol=2e-5)
    assert torch.allclose(mirrored["p"], base["p"], atol=2e-5)
    assert torch.allclose(mirrored["u"], base["u"] * torch.tensor([1.0, -1.0]), atol=2e-5)
    # all lengths × 4, so the boundary measure (a length in 2-D) and its reference × 4: the same nondimensional problem
    big = _globe_2d(theta=0.0, latent_compression_scale=2.0, reference_area=4.0)
    big.load_state_dict({k: v for k, v in model.state_dict().items() if k != "reference_area"}, strict=False)
    with torch.no_grad():
        scaled = big(*_globe_inputs(scale=4.0)).point_data
    assert torch.allclose(scaled["p"], base["p"], atol=2e-5) and torch.allclose(scaled["u"], base["u"], atol=2e-5)


def test_globe_is_insensitive_to_boundary_refinement_and_theta():
    model = _globe_2d(theta=0.0)
    with torch.no_grad():
        coarse = model(*_globe_inputs(n_wall=60)).point_data
        fine = model(*_globe_inputs(n_wall=240)).point_data
        model.theta = 0.5
        fast = model(*_globe_inputs(n_wall=60)).point_data
    for k in coarse:
        scale = coarse[k].abs().max()
        assert (fine[k] - coarse[k]).abs().max() < 0.05 * scale
        assert (fast[k] - coarse[k]).abs().max() < 0.1 * scale


def test_globe_checkpoint_roundtrip(tmp_path):
    model = _globe_2d(theta=0.3)
    model.save(str(tmp_path / "globe.mdlus"))
    from physicsnemo_b200.core.module import Module
    again = Module.from_checkpoint(str(tmp_path / "globe.mdlus")).eval()
    assert type(again) is GLOBE and again.theta == 0.3
    with torch.no_grad():
        a, b = model(*_globe_inputs()).point_data, again(*_globe_inputs()).point_data
    assert all(torch.equal(a[k], b[k]) for k in a)

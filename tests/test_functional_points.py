"""Interpolation, neighbour search, kNN and FPS: torch formulations (CPU), CUDA kernels against them (GPU)."""
import pytest
import torch

from physicsnemo_b200.nn.functional.geometry.farthest_point_sampling import farthest_point_sampling
from physicsnemo_b200.nn.functional.interpolation import interpolation, point_to_grid_interpolation
from physicsnemo_b200.nn.functional.neighbors import knn, radius_search

TYPES = ["nearest_neighbor", "linear", "smooth_step_1", "smooth_step_2", "gaussian"]


def test_interpolation_torch_properties():
    grid = [(0.0, 1.0, 11), (0.0, 2.0, 21), (-1.0, 1.0, 9)]
    axes = [torch.linspace(a, b, n) for a, b, n in grid]
    X, Y, Z = torch.meshgrid(*axes, indexing="ij")
    f = torch.stack([2 * X + 3 * Y - Z, torch.ones_like(X)])
    q = torch.rand(64, 3) * torch.tensor([1.0, 2.0, 2.0]) + torch.tensor([0.0, 0.0, -1.0])
    out = interpolation(q, f, grid, interpolation_type="linear")
    assert torch.allclose(out[:, 0], 2 * q[:, 0] + 3 * q[:, 1] - q[:, 2], atol=1e-5)   # trilinear is exact on linear fields
    for t in TYPES[:4]:
        assert torch.allclose(interpolation(q, f, grid, interpolation_type=t)[:, 1], torch.ones(64), atol=1e-5)
    inner = q * 0.5 + torch.tensor([0.25, 0.5, 0.0])                                    # ≥ 2 cells from the boundary
    assert torch.allclose(interpolation(inner, f, grid, interpolation_type="gaussian")[:, 1], torch.ones(64), atol=1e-5)
    v, g = torch.randn(64, 2), torch.randn(2, 11, 21, 9)
    for t in TYPES:                                                                     # <G2P g, v> == <g, P2G v>
        a = (interpolation(q, g, grid, interpolation_type=t) * v).sum()
        b = (point_to_grid_interpolation(q, v, grid, interpolation_type=t) * g).sum()
        assert torch.allclose(a, b, rtol=1e-4)
    g1 = g.clone().requires_grad_(True)
    interpolation(q, g1, grid).sum().backward()
    assert g1.grad.shape == g.shape
    q1 = q.clone().requires_grad_(True)
    interpolation(q1, f, grid, interpolation_type="linear")[:, 0].sum().backward()
    assert torch.allclose(q1.grad, torch.tensor([2.0, 3.0, -1.0]).expand(64, 3), atol=1e-4)
    with pytest.raises(RuntimeError):
        interpolation(q, f, grid, interpolation_type="cubic")


def test_radius_knn_fps_torch():
    torch.manual_seed(0)
    p, q = torch.rand(300, 3), torch.rand(40, 3)
    pairs, d = radius_search(p, q, 0.2, return_dists=True)
    full = torch.cdist(q, p)
    assert pairs.shape[1] == int((full <= 0.2).sum()) and torch.all(d <= 0.2 + 1e-6)
    idx, pts, dist = radius_search(p, q, 0.2, max_points=5, return_dists=True, return_points=True)
    assert idx.shape == (40, 5) and pts.shape == (40, 5, 3) and dist.shape == (40, 5)
    nearest = full.topk(5, largest=False)
    ok = nearest.values <= 0.2
    assert torch.equal(idx, torch.where(ok, nearest.indices, 0))
    i, dd = knn(p, q, k=6)
    assert torch.equal(i, full.topk(6, largest=False).indices) and torch.allclose(dd, full.topk(6, largest=False).values, atol=1e-5)
    i2, _ = knn(p, q, k=6, implementation="torch")
    assert torch.equal(i, i2)
    s = farthest_point_sampling(p, 10)
    assert s.shape == (10,) and s[0] == 0 and len(set(s.tolist())) == 10
    assert s[1] == ((p - p[0]) ** 2).sum(-1).argmax()
    with pytest.raises(ValueError):
        farthest_point_sampling(p, 301)


@pytest.mark.gpu
def test_interpolation_cuda_matches_torch():
    dev = "cuda"
    for grid in ([(0.0, 1.0, 64)], [(0.0, 1.0, 40), (-1.0, 1.0, 33)], [(0.0, 1.0, 20), (0.0, 2.0, 24), (-1.0, 1.0, 17)]):
        dims = len(grid)
        lo = torch.tensor([g[0] for g in grid], device=dev)
        hi = torch.tensor([g[1] for g in grid], device=dev)
        q = torch.rand(5000, dims, device=dev) * (hi - lo) * 1.1 + lo - 0.05 * (hi - lo)   # some points outside
        f = torch.randn(3, *[g[2] for g in grid], device=dev)
        v = torch.randn(5000, 3, device=dev)
        for t in TYPES:
            f1, f2 = f.clone().requires_grad_(True), f.clone().requires_grad_(True)
            a = interpolation(q, f1, grid, interpolation_type=t, implementation="cuda")
            b = interpolation(q, f2, grid, interpolation_type=t, implementation="torch")
            assert (a - b).abs().max() < 2e-4, (dims, t)
            (a * v).sum().backward(); (b * v).sum().backward()
            assert (f1.grad - f2.grad).abs().max() < 1e-3, (dims, t)
            c = point_to_grid_interpolation(q, v, grid, interpolation_type=t, implementation="cuda")
            d = point_to_grid_interpolation(q, v, grid, interpolation_type=t, implementation="torch")
            assert (c - d).abs().max() < 1e-3, (dims, t)


@pytest.mark.gpu
def test_neighbors_cuda_match_torch():
    dev = "cuda"
    torch.manual_seed(1)
    p, q = torch.rand(20000, 3, device=dev), torch.rand(3000, 3, device=dev) * 1.2 - 0.1
    r = 0.05
    a = radius_search(p, q, r, implementation="cuda")
    b = radius_search(p, q, r, implementation="torch")
    key = lambda t: torch.unique(t[0] * 100000 + t[1])  # noqa: E731
    assert a.shape == b.shape and torch.equal(key(a), key(b))
    ia, pa, da = radius_search(p, q, r, max_points=16, return_dists=True, return_points=True, implementation="cuda")
    ib, pb, db = radius_search(p, q, r, max_points=16, return_dists=True, return_points=True, implementation="torch")
    assert torch.allclose(da, db, atol=1e-6) and torch.allclose(pa, pb, atol=1e-6)
    assert (ia != ib).float().mean() < 1e-3                      # identical up to exact distance ties
    pb3, qb3 = torch.rand(2, 5000, 3, device=dev), torch.rand(2, 700, 3, device=dev)
    a3 = radius_search(pb3, qb3, 0.1, implementation="cuda")
    b3 = radius_search(pb3, qb3, 0.1, implementation="torch")
    assert a3.shape == b3.shape
    for k in (1, 5, 16, 33, 64):
        i1, d1 = knn(p, q, k=k, implementation="cuda")
        i2, d2 = knn(p, q, k=k, implementation="torch")
        assert torch.allclose(d1, d2, atol=1e-5) and (i1 != i2).float().mean() < 1e-3
    i1, d1 = knn(p[:, :2].contiguous(), q[:, :2].contiguous(), k=4, implementation="cuda")
    i2, d2 = knn(p[:, :2].contiguous(), q[:, :2].contiguous(), k=4, implementation="torch")
    assert torch.allclose(d1, d2, atol=1e-5)
    cloud = torch.rand(3, 10000, 3, device=dev)
    s1 = farthest_point_sampling(cloud, 256, implementation="cuda")
    s2 = farthest_point_sampling(cloud, 256, implementation="torch")
    assert (s1 != s2).float().mean() < 0.02                       # fp summation order may flip rare near-ties
    assert s1.shape == (3, 256) and all(len(set(r.tolist())) == 256 for r in s1)

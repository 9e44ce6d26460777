"""Derivative functionals: torch formulation against closed forms (CPU), CUDA kernels against it (GPU)."""
import math

import pytest
import torch

from physicsnemo_b200.nn.functional import derivatives as D


def _field(shape, dtype=torch.float64, device="cpu"):
    axes = [torch.arange(n, dtype=dtype, device=device) / n for n in shape]
    g = torch.meshgrid(*axes, indexing="ij")
    f = sum((i + 1) * torch.sin(2 * math.pi * (i + 1) * x) for i, x in enumerate(g))
    return f, g


@pytest.mark.parametrize("shape", [(64,), (32, 48), (16, 20, 24)])
@pytest.mark.parametrize("order", [2, 4])
def test_uniform_gradient_converges_and_transposes(shape, order):
    f, g = _field(shape)
    sp = [1.0 / n for n in shape]
    out = D.uniform_grid_gradient(f, spacing=sp, order=order, derivative_orders=(1, 2), include_mixed=len(shape) > 1)
    nd = len(shape)
    n_mixed = nd * (nd - 1) // 2 if nd > 1 else 0
    assert out.shape == (2 * nd + n_mixed, *shape)
    for i, x in enumerate(g):
        k = 2 * math.pi * (i + 1)
        exact1 = (i + 1) * k * torch.cos(k * x)
        exact2 = -(i + 1) * k * k * torch.sin(k * x)
        tol = 0.15 if order == 2 else 0.02
        assert (out[i] - exact1).abs().max() / exact1.abs().max() < tol
        assert (out[nd + i] - exact2).abs().max() / exact2.abs().max() < tol
    if n_mixed:
        assert out[2 * nd:].abs().max() < 1e-8   # separable field: mixed derivatives vanish
    # transposed program == autograd of an independent roll formulation
    f1 = f.clone().requires_grad_(True)
    w = torch.randn(nd, *shape, dtype=f.dtype)
    (D.uniform_grid_gradient(f1, spacing=sp, order=order) * w).sum().backward()
    f2 = f.clone().requires_grad_(True)
    ref = []
    for ax in range(nd):
        if order == 2:
            ref.append((torch.roll(f2, -1, ax) - torch.roll(f2, 1, ax)) / (2 * sp[ax]))
        else:
            ref.append((-torch.roll(f2, -2, ax) + 8 * torch.roll(f2, -1, ax) - 8 * torch.roll(f2, 1, ax) + torch.roll(f2, 2, ax)) / (12 * sp[ax]))
    (torch.stack(ref) * w).sum().backward()
    assert torch.allclose(f1.grad, f2.grad, atol=1e-9)


def test_div_curl_laplacian_identities():
    shape = (16, 20, 24)
    sp = [1.0 / n for n in shape]
    f, _ = _field(shape)
    grad = D.uniform_grid_gradient(f, spacing=sp, order=4)
    assert D.uniform_grid_curl(grad, spacing=sp, order=4).abs().max() < 1e-8      # curl grad = 0 (discrete operators commute)
    lap = D.uniform_grid_laplacian(f, spacing=sp, order=2)
    second = D.uniform_grid_gradient(f, spacing=sp, order=2, derivative_orders=2)
    assert torch.allclose(lap, second.sum(0), atol=1e-9)
    v = torch.randn(3, *shape, dtype=torch.float64)
    div = D.uniform_grid_divergence(v, spacing=sp, order=2)
    ref = sum((torch.roll(v[a], -1, a) - torch.roll(v[a], 1, a)) / (2 * sp[a]) for a in range(3))
    assert torch.allclose(div, ref, atol=1e-10)
    assert torch.allclose(D.uniform_grid_divergence(D.uniform_grid_curl(v, spacing=sp), spacing=sp),
                          torch.zeros(shape, dtype=torch.float64), atol=1e-8)
    c2 = D.uniform_grid_curl(v[:2, :, :, 0], spacing=sp[:2])
    assert c2.shape == shape[:2]
    with pytest.raises(ValueError):
        D.uniform_grid_gradient(f, order=3)
    with pytest.raises(ValueError):
        D.uniform_grid_gradient(f[0, 0], include_mixed=True, derivative_orders=2)


def test_rectilinear_matches_uniform_and_handles_stretching():
    shape = (24, 30)
    f, _ = _field(shape)
    coords = [torch.arange(n, dtype=torch.float64) / n for n in shape]
    sp = [1.0 / n for n in shape]
    a = D.rectilinear_grid_gradient(f, coords, derivative_orders=(1, 2), include_mixed=True)
    b = D.uniform_grid_gradient(f, spacing=sp, order=2, derivative_orders=(1, 2), include_mixed=True)
    assert torch.allclose(a, b, atol=1e-8)
    v = torch.randn(2, *shape, dtype=torch.float64)
    assert torch.allclose(D.rectilinear_grid_divergence(v, coords), D.uniform_grid_divergence(v, spacing=sp), atol=1e-9)
    assert torch.allclose(D.rectilinear_grid_curl(v, coords), D.uniform_grid_curl(v, spacing=sp), atol=1e-9)
    assert torch.allclose(D.rectilinear_grid_laplacian(f, coords), D.uniform_grid_laplacian(f, spacing=sp), atol=1e-7)
    # stretched grid: exact for quadratics away from the periodic seam
    x = torch.cumsum(torch.rand(40, dtype=torch.float64) + 0.5, 0)
    q = 3 * x ** 2 - x
    g = D.rectilinear_grid_gradient(q, [x], derivative_orders=(1, 2))
    assert torch.allclose(g[0, 1:-1], (6 * x - 1)[1:-1], atol=1e-8)
    assert torch.allclose(g[1, 1:-1], torch.full_like(x, 6.0)[1:-1], atol=1e-8)
    q1 = q.clone().requires_grad_(True)
    D.rectilinear_grid_gradient(q1, [x]).sum().backward()
    assert q1.grad.shape == q.shape
    with pytest.raises(ValueError):
        D.rectilinear_grid_gradient(q, [x.flip(0)])


def test_meshless_and_spectral():
    pts = torch.rand(50, 2, dtype=torch.float64)
    h = 1e-3
    st = D.meshless_fd_stencil_points(pts, spacing=h)
    assert st.shape == (50, 9, 2)
    vals = torch.sin(st[..., 0]) * torch.cos(2 * st[..., 1])
    d1 = D.meshless_fd_derivatives(vals, spacing=h, order=1)
    assert torch.allclose(d1[0], torch.cos(pts[:, 0]) * torch.cos(2 * pts[:, 1]), atol=1e-5)
    d2 = D.meshless_fd_derivatives(vals, spacing=h, order=2, return_mixed_derivs=True)
    assert torch.allclose(d2[2], -2 * torch.cos(pts[:, 0]) * torch.sin(2 * pts[:, 1]), atol=1e-4)
    f, g = _field((32, 32))
    s = D.spectral_grid_gradient(f, lengths=1.0, order=1)
    assert torch.allclose(s[0], 2 * math.pi * torch.cos(2 * math.pi * g[0]), atol=1e-8)
    s2 = D.spectral_grid_gradient(f, lengths=1.0, order=2, return_mixed_derivs=True)
    assert s2.shape[0] == 3 and s2[2].abs().max() < 1e-7


def _ring_neighbours(n, k):
    idx = torch.arange(n)
    nb = torch.stack([(idx + s) % n for s in range(-k, k + 1) if s != 0], 1)
    return torch.arange(0, n * 2 * k + 1, 2 * k), nb.reshape(-1)


def test_mesh_lsq_and_green_gauss_torch():
    torch.manual_seed(0)
    n = 200
    pts = torch.rand(n, 3, dtype=torch.float64)
    d = torch.cdist(pts, pts)
    nb = d.topk(9, largest=False).indices[:, 1:]
    offs = torch.arange(0, n * 8 + 1, 8)
    A = torch.randn(3, 2, dtype=torch.float64)
    vals = pts @ A + 0.5
    g = D.mesh_lsq_gradient(pts, vals, offs, nb.reshape(-1))
    assert g.shape == (n, 3, 2)
    assert torch.allclose(g, A.expand(n, 3, 2), atol=1e-8)         # exact for linear fields
    g0 = D.mesh_lsq_gradient(pts, vals, offs, nb.reshape(-1), min_neighbors=9)
    assert g0.abs().max() == 0
    # Green-Gauss on a two-triangle square: linear field, interior face averaged
    p = torch.tensor([[0.0, 0], [1, 0], [1, 1], [0, 1]], dtype=torch.float64)
    cells = torch.tensor([[0, 1, 2], [0, 2, 3]])
    nbrs = torch.tensor([[-1, 1, -1], [-1, -1, 0]])   # face f is opposite vertex f
    cv = torch.tensor([[1.0], [1.0]], dtype=torch.float64)
    gg = D.mesh_green_gauss_gradient(p, cells, nbrs, cv)
    assert gg.shape == (2, 2, 1) and gg.abs().max() < 1e-12        # constant field: closed surface integral vanishes
    cv2 = torch.tensor([1.0, 3.0], dtype=torch.float64, requires_grad=True)
    D.mesh_green_gauss_gradient(p, cells, nbrs, cv2).sum().backward()
    assert cv2.grad is not None


@pytest.mark.gpu
def test_cuda_kernels_match_torch():
    dev = "cuda"
    for shape, order in [((4096,), 2), ((300, 257), 4), ((40, 33, 65), 2), ((40, 33, 65), 4)]:
        f, _ = _field(shape, torch.float32, dev)
        f = f + 0.1 * torch.randn_like(f)
        sp = [0.01 * (i + 1) for i in range(len(shape))]
        mixed = len(shape) > 1
        kw = dict(spacing=sp, order=order, derivative_orders=(1, 2), include_mixed=mixed)
        f1, f2 = f.clone().requires_grad_(True), f.clone().requires_grad_(True)
        a = D.uniform_grid_gradient(f1, implementation="cuda", **kw)
        b = D.uniform_grid_gradient(f2, implementation="torch", **kw)
        scale = b.abs().max()
        assert (a - b).abs().max() / scale < 1e-5
        w = torch.randn_like(a)
        (a * w).sum().backward(); (b * w).sum().backward()
        assert (f1.grad - f2.grad).abs().max() / f2.grad.abs().max() < 1e-5
    v = torch.randn(3, 30, 41, 52, device=dev)
    coords = [torch.cumsum(torch.rand(n, device=dev) + 0.5, 0) for n in v.shape[1:]]
    for fn, args in [(D.uniform_grid_divergence, (v,)), (D.uniform_grid_curl, (v,)), (D.uniform_grid_laplacian, (v[0],)),
                     (D.rectilinear_grid_divergence, (v, coords)), (D.rectilinear_grid_curl, (v, coords)),
                     (D.rectilinear_grid_laplacian, (v[0], coords)), (D.rectilinear_grid_gradient, (v[0], coords))]:
        a, b = fn(*args, implementation="cuda"), fn(*args, implementation="torch")
        assert (a - b).abs().max() / b.abs().max() < 1e-5, fn.__name__
    n = 5000
    pts = torch.rand(n, 3, device=dev)
    nb = torch.randint(0, n, (n * 12,), device=dev)
    offs = torch.arange(0, n * 12 + 1, 12, device=dev)
    vals1 = torch.randn(n, 4, device=dev, requires_grad=True)
    vals2 = vals1.detach().clone().requires_grad_(True)
    a = D.mesh_lsq_gradient(pts, vals1, offs, nb, implementation="cuda")
    b = D.mesh_lsq_gradient(pts, vals2, offs, nb, implementation="torch")
    assert (a - b).abs().max() / b.abs().max() < 1e-3
    w = torch.randn_like(a)
    (a * w).sum().backward(); (b * w).sum().backward()
    assert (vals1.grad - vals2.grad).abs().max() / vals2.grad.abs().max() < 1e-3
    p = torch.rand(400, 3, device=dev)
    cells = torch.stack([torch.randperm(400, device=dev)[:4] for _ in range(300)])
    nbrs = torch.randint(-1, 300, (300, 4), device=dev)
    cv1 = torch.randn(300, 2, device=dev, requires_grad=True)
    cv2 = cv1.detach().clone().requires_grad_(True)
    a = D.mesh_green_gauss_gradient(p, cells, nbrs, cv1, implementation="cuda")
    b = D.mesh_green_gauss_gradient(p, cells, nbrs, cv2, implementation="torch")
    assert (a - b).abs().max() / b.abs().max() < 1e-4
    w = torch.randn_like(a)
    (a * w).sum().backward(); (b * w).sum().backward()
    assert (cv1.grad - cv2.grad).abs().max() / cv2.grad.abs().max() < 1e-4

"""Symbolic PDE layer: graph scheduling, SymPy compilation, the five gradient methods."""
import math

import pytest
import torch

sympy = pytest.importorskip("sympy")

from physicsnemo_b200.sym import PDE, GradientCalculator, PhysicsInformer, compute_connectivity_tensor  # noqa: E402
from physicsnemo_b200.sym.computation import Computation  # noqa: E402
from physicsnemo_b200.sym.graph import Graph  # noqa: E402


class Burgersish(PDE):
    """u_t + u u_x + v u_y - nu (u_xx + u_yy)  and a divergence."""

    def __init__(self, nu=0.1, dim=2):
        x, y, t = sympy.symbols("x y t")
        u = sympy.Function("u")(x, y, t)
        v = sympy.Function("v")(x, y, t)
        self.dim = dim
        self.equations = {
            "momentum_x": u.diff(t) + u * u.diff(x) + v * u.diff(y) - nu * (u.diff(x, 2) + u.diff(y, 2)),
            "continuity": u.diff(x) + v.diff(y),
            "cross": u.diff(x).diff(y),
        }


def _fields(n=64):
    L = 2 * math.pi
    xs = torch.arange(n, dtype=torch.float64) * (L / n)
    X, Y = torch.meshgrid(xs, xs, indexing="ij")
    u = torch.sin(X) * torch.cos(2 * Y)
    v = torch.cos(X) * torch.sin(Y)
    ut = 0.3 * torch.cos(X + Y)
    exact = {
        "u__x": torch.cos(X) * torch.cos(2 * Y), "u__y": -2 * torch.sin(X) * torch.sin(2 * Y),
        "u__x__x": -u, "u__y__y": -4 * u, "v__y": torch.cos(X) * torch.cos(Y),
        "u__x__y": -2 * torch.cos(X) * torch.sin(2 * Y),
    }
    return L / n, u, v, ut, exact


@pytest.mark.parametrize("method,tol", [("spectral", 1e-9), ("finite_difference", 3e-2)])
def test_physics_informer_grid_methods(method, tol):
    dx, u, v, ut, ex = _fields()
    pi = PhysicsInformer(["momentum_x", "continuity", "cross"], Burgersish(), method, fd_dx=dx,
                         bounds=[2 * math.pi] * 2)
    assert set(pi.required_inputs) == {"u", "v", "u__t"}
    out = pi.forward({"u": u[None, None], "v": v[None, None], "u__t": ut[None, None]})
    want_m = ut + u * ex["u__x"] + v * ex["u__y"] - 0.1 * (ex["u__x__x"] + ex["u__y__y"])
    assert out["momentum_x"].shape == (1, 1, 64, 64)
    assert (out["momentum_x"][0, 0] - want_m).abs().max() < tol
    assert (out["continuity"][0, 0] - (ex["u__x"] + ex["v__y"])).abs().max() < tol
    assert (out["cross"][0, 0] - ex["u__x__y"]).abs().max() < tol


def test_autodiff_and_meshless():
    class Lap(PDE):
        def __init__(self):
            x, y, z = sympy.symbols("x y z")
            u = sympy.Function("u")(x, y, z)
            self.dim = 3
            self.equations = {"lap": u.diff(x, 2) + u.diff(y, 2) + u.diff(z, 2), "gx": u.diff(x)}

    f = lambda p: (p[:, :1] ** 2 * p[:, 1:2] + torch.sin(p[:, 2:3]))  # noqa: E731
    pts = torch.rand(50, 3, dtype=torch.float64, requires_grad=True)
    want_lap = 2 * pts[:, 1:2] - torch.sin(pts[:, 2:3])
    pi = PhysicsInformer(["lap", "gx"], Lap(), "autodiff")
    assert "coordinates" in pi.required_inputs
    out = pi.forward({"u": f(pts), "coordinates": pts})
    assert torch.allclose(out["lap"], want_lap, atol=1e-10) and torch.allclose(out["gx"], 2 * pts[:, :1] * pts[:, 1:2])
    h = 1e-3
    pm = PhysicsInformer(["lap"], Lap(), "meshless_finite_difference", fd_dx=h)
    feed = {"u": f(pts)}
    for a, name in enumerate("xyz"):
        for s in (1, -1):
            e = torch.zeros(3, dtype=torch.float64)
            e[a] = s * h
            feed[f"u>>{name}::{s}"] = f(pts + e)
    assert set(pm.required_inputs) == set(feed)
    assert (pm.forward(feed)["lap"] - want_lap).abs().max() < 1e-4


def test_least_squares_on_graph():
    g = torch.Generator().manual_seed(0)
    n = 12
    xs = torch.linspace(0, 1, n, dtype=torch.float64)
    P = torch.stack(torch.meshgrid(xs, xs, indexing="ij"), -1).reshape(-1, 2)
    P = P + 0.01 * torch.rand(P.shape, generator=g, dtype=torch.float64)
    idx = torch.arange(n * n).reshape(n, n)
    edges = torch.cat([torch.stack([idx[:-1].flatten(), idx[1:].flatten()], 1),
                       torch.stack([idx[:, :-1].flatten(), idx[:, 1:].flatten()], 1),
                       torch.stack([idx[:-1, :-1].flatten(), idx[1:, 1:].flatten()], 1)])
    offs, ind, mat = compute_connectivity_tensor(torch.arange(n * n), edges)
    assert offs[-1] == 2 * len(edges) and mat.shape[0] == n * n and (mat[0] >= 0).sum() == offs[1] - offs[0]

    class Div(PDE):
        def __init__(self):
            x, y = sympy.symbols("x y")
            u, v = sympy.Function("u")(x, y), sympy.Function("v")(x, y)
            self.dim = 2
            self.equations = {"div": u.diff(x) + v.diff(y)}

    pi = PhysicsInformer(["div"], Div(), "least_squares")
    u, v = 3 * P[:, :1] + P[:, 1:], 2 * P[:, 1:] - P[:, :1]
    out = pi.forward({"u": u, "v": v, "coordinates": P, "nodes": torch.arange(n * n), "edges": edges})
    assert torch.allclose(out["div"], torch.full_like(u, 5.0), atol=1e-8)


def test_graph_scheduling_and_errors():
    a = Computation(["p"], ["q"], torch.nn.Identity(), "a")

    class Add(torch.nn.Module):
        def forward(self, d):
            return {"r": d["q"] + d["p__x"]}

    class Dx(torch.nn.Module):
        def forward(self, d):
            return {"p__x": 2 * d["p"]}

    a.evaluate = type("Q", (torch.nn.Module,), {"forward": lambda self, d: {"q": d["p"] + 1}})()
    b = Computation(["q", "p__x"], ["r"], Add(), "b")
    dn = Computation(["p"], ["p__x"], Dx(), "dx")
    g = Graph([b, a], ["p"], ["r"], diff_nodes=[dn])
    assert g.node_names == ["a", "dx", "b"]
    assert float(g({"p": torch.tensor(3.0)})["r"]) == 10.0
    with pytest.raises(RuntimeError):
        Graph([b, a], ["zz"], ["r"], diff_nodes=[dn])
    mod = GradientCalculator().get_gradient_module("finite_difference", "u", dx=0.1, dim=1, order=1)
    x = torch.arange(10.0)[None, None] * 0.1
    assert torch.allclose(mod({"u": 2 * x})["u__x"][0, 0, 1:-1], torch.full((8,), 2.0), atol=1e-5)


def test_sympy_functions_and_freeze():
    from physicsnemo_b200.sym.utils.sympy.torch_printer import SympyToTorch

    a, b = sympy.symbols("a b")
    expr = sympy.sqrt(a) + sympy.Max(a, b, 0.5) * sympy.Heaviside(b) + sympy.Abs(b)
    m = SympyToTorch(expr, "o")
    A, B = torch.tensor([0.0, 4.0]), torch.tensor([-1.0, 9.0])
    got = m({"a": A, "b": B})["o"]
    assert torch.allclose(got, torch.tensor([1e-3 + 0 + 1.0, 2 + 9 + 9.0]), atol=1e-6)
    fz = SympyToTorch(a * a + a * b, "o", freeze_terms=[0])
    A = torch.tensor([2.0], requires_grad=True)
    out = fz({"a": A, "b": torch.tensor([3.0])})["o"]
    out.backward()
    terms = sympy.Add.make_args(a * a + a * b)
    want = 3.0 if str(terms[0]) == "a**2" else 4.0
    assert float(out) == 10.0 and float(A.grad) == want

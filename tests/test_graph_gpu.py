"""Graph kernels and the fused MeshGraphNet path against PyTorch fp32 references."""
import copy

import pytest
import torch

from physicsnemo_b200 import ops
from physicsnemo_b200.models.meshgraphnet import MeshGraphNet
from physicsnemo_b200.nn.module.gnn_layers.graph_types import Graph

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("C", [8, 128, 200])
def test_gather_and_segment(C):
    dev = "cuda"
    N, E = 1000, 7777
    idx = torch.randint(0, N, (E,), device=dev)
    seg = ops.SegmentIndex(idx, N)
    x = torch.randn(N, C, device=dev).to(torch.bfloat16).requires_grad_(True)
    e = torch.randn(E, C, device=dev).to(torch.bfloat16).requires_grad_(True)
    g = ops.gather_rows(x, seg)
    assert torch.equal(g, x[idx])
    for mode in ("sum", "mean"):
        s = ops.segment_reduce(e, seg, mode)
        ref = torch.zeros(N, C, device=dev).index_add_(0, idx, e.detach().float())
        if mode == "mean":
            ref = ref / seg.counts.clamp_min(1).unsqueeze(1)
        assert _rel(s, ref) < 1e-2
        (ge,) = torch.autograd.grad(s, e, torch.ones_like(s))
        gref = torch.ones(E, C, device=dev)
        if mode == "mean":
            gref = gref * seg.inv_count[idx].unsqueeze(1)
        assert _rel(ge, gref) < 1e-2
    (gx,) = torch.autograd.grad(g, x, torch.ones_like(g))
    assert _rel(gx, seg.counts.float().unsqueeze(1).expand(N, C)) < 1e-2


def test_three_source_chain():
    M = 3000
    xs = [torch.randn(M, 128, device="cuda").to(torch.bfloat16).requires_grad_(True) for _ in range(3)]
    ws = [torch.randn(128, 384, device="cuda") * 0.05, torch.randn(128, 128, device="cuda") * 0.08]
    bs = [torch.randn(128, device="cuda") * 0.1, torch.randn(128, device="cuda") * 0.1]
    for t in ws + bs:
        t.requires_grad_(True)
    y = ops.mlp_chain(xs, ws, bs, [ops.ACT_SILU, ops.ACT_NONE])
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = [t.detach().float().requires_grad_(True) for t in xs]
    wr = [t.detach().clone().requires_grad_(True) for t in ws]
    br = [t.detach().clone().requires_grad_(True) for t in bs]
    h = torch.nn.functional.silu(torch.cat(xr, 1) @ wr[0].t() + br[0]) @ wr[1].t() + br[1]
    h.backward(dy.float())
    assert _rel(y, h) < 2e-2
    for a, b in zip([t.grad for t in xs + ws + bs], [t.grad for t in xr + wr + br]):
        assert _rel(a, b) < 4e-2


def test_meshgraphnet_fused_matches_fp32():
    dev = torch.device("cuda")
    model = MeshGraphNet(6, 3, 3, processor_size=3, mlp_activation_fn="silu", hidden_dim_processor=128).to(dev)
    ref = copy.deepcopy(model)
    N, E = 2000, 12000
    g = Graph(torch.randint(0, N, (2, E), device=dev), N)
    nf, ef = torch.randn(N, 6, device=dev), torch.randn(E, 3, device=dev)
    tgt = torch.randn(N, 3, device=dev)
    before = ops.kernel_launches()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = model(nf, ef, g)
    loss = torch.nn.functional.mse_loss(out.float(), tgt)
    loss.backward()
    assert ops.kernel_launches() - before > 30
    out_ref = ref(nf, ef, g)
    torch.nn.functional.mse_loss(out_ref, tgt).backward()
    assert ops.device_error() == 0
    assert _rel(out, out_ref) < 5e-2
    bad = [(n, _rel(p.grad, q.grad)) for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters())
           if _rel(p.grad, q.grad) > 0.25]
    assert not bad, bad

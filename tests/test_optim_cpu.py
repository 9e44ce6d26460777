"""Optimizers against torch.optim / closed forms (model: the reference's ``test/optim``)."""
import pytest
import torch

from physicsnemo_b200.optim import CombinedOptimizer, FusedAdam, FusedAdamW, Muon, grad_global_norm
from physicsnemo_b200.optim.muon import _batched_newton_schulz


def _run(opt_a, opt_b, pa, pb, steps=5):
    for s in range(steps):
        for group, opt in ((pa, opt_a), (pb, opt_b)):
            for i, p in enumerate(group):
                torch.manual_seed(100 * s + i)
                p.grad = torch.randn_like(p)
            opt.step()
    for a, b in zip(pa, pb):
        assert torch.allclose(a, b, atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("wmode", [False, True])
def test_fused_adam_cpu_path_matches_torch(wmode):
    torch.manual_seed(0)
    pa = [torch.randn(7, 5), torch.randn(33)]
    pb = [p.clone() for p in pa]
    ours = FusedAdam(pa, lr=1e-2, weight_decay=0.1, adam_w_mode=wmode)
    ref = (torch.optim.AdamW if wmode else torch.optim.Adam)(pb, lr=1e-2, weight_decay=0.1)
    _run(ours, ref, pa, pb)
    assert isinstance(FusedAdamW(pa), FusedAdam)


def test_newton_schulz_orthogonalises():
    torch.manual_seed(1)
    g = torch.randn(3, 16, 32)
    o = _batched_newton_schulz(g, (3.4445, -4.775, 2.0315), 5, 1e-7).float()
    s = torch.linalg.svdvals(o)
    assert s.min() > 0.3 and s.max() < 1.3
    tall = _batched_newton_schulz(g.transpose(1, 2).contiguous(), (3.4445, -4.775, 2.0315), 5, 1e-7)
    assert tall.shape == (3, 32, 16)
    with pytest.raises(ValueError):
        _batched_newton_schulz(g[0], (1, 2, 3), 5, 1e-7)


def test_muon_matches_torch_muon():
    torch.manual_seed(2)
    pa = [torch.randn(8, 16), torch.randn(8, 16), torch.randn(12, 4)]
    pb = [p.clone() for p in pa]
    ours, ref = Muon(pa, lr=0.02), torch.optim.Muon(pb, lr=0.02)
    for s in range(3):
        for group in (pa, pb):
            for i, p in enumerate(group):
                torch.manual_seed(10 * s + i)
                p.grad = torch.randn_like(p)
        ours.step(), ref.step()
    for a, b in zip(pa, pb):
        assert torch.allclose(a, b, atol=2e-2)   # bf16 Newton-Schulz on both sides, different GEMM grouping
    with pytest.raises(ValueError):
        Muon([torch.randn(3)])


def test_combined_optimizer():
    w, b = torch.nn.Parameter(torch.randn(4, 4)), torch.nn.Parameter(torch.randn(4))
    combo = CombinedOptimizer([Muon([w], lr=0.01), FusedAdam([b], lr=0.01)])
    assert len(combo.param_groups) == 2
    (w.sum() + b.sum()).backward()
    w0, b0 = w.detach().clone(), b.detach().clone()
    combo.step()
    assert not torch.equal(w, w0) and not torch.equal(b, b0)
    sd = combo.state_dict()
    combo.load_state_dict(sd)
    combo.zero_grad()
    assert w.grad is None
    with pytest.raises(ValueError):
        CombinedOptimizer([Muon([w]), FusedAdam([w])])
    with pytest.raises(NotImplementedError):
        combo.add_param_group({"params": [torch.nn.Parameter(torch.randn(2))]})
    sched = torch.optim.lr_scheduler.StepLR(combo, step_size=1, gamma=0.5)
    combo.step(); sched.step()
    assert combo.optimizers[0].param_groups[0]["lr"] == pytest.approx(0.005)


def test_grad_norm_cpu():
    ps = [torch.nn.Parameter(torch.randn(5)), torch.nn.Parameter(torch.randn(2, 3))]
    for p in ps:
        p.grad = torch.randn_like(p)
    ref = torch.sqrt(sum((p.grad ** 2).sum() for p in ps))
    assert torch.allclose(grad_global_norm(ps), ref)

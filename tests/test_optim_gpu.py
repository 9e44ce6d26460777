"""Multi-tensor Adam kernel against torch.optim (fp32 reference of the same update)."""
import pytest
import torch

from physicsnemo_b200.optim import FusedAdam, grad_global_norm

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("wmode", [False, True])
def test_fused_adam_kernel(wmode):
    torch.manual_seed(0)
    shapes = [(256, 256), (1024,), (3, 5, 7), (1,), (8192 * 3 + 17,)]
    pa = [torch.randn(s, device="cuda") for s in shapes]
    pb = [p.clone() for p in pa]
    ours = FusedAdam(pa, lr=1e-2, weight_decay=0.05, adam_w_mode=wmode)
    ref = (torch.optim.AdamW if wmode else torch.optim.Adam)(pb, lr=1e-2, weight_decay=0.05)
    for s in range(4):
        for i, (a, b) in enumerate(zip(pa, pb)):
            torch.manual_seed(100 * s + i)
            g = torch.randn_like(a)
            a.grad, b.grad = g, g.float()
        ours.step(), ref.step()
    assert ours.kernel_launches == 4
    for a, b in zip(pa, pb):
        assert torch.allclose(a, b, atol=1e-5, rtol=1e-4)


def test_grad_norm_kernel():
    ps = [torch.nn.Parameter(torch.randn(n, device="cuda")) for n in (5, 70000, 8192)]
    for i, p in enumerate(ps):
        p.grad = torch.randn_like(p)
    ref = torch.sqrt(sum((p.grad.float() ** 2).sum() for p in ps))
    assert torch.allclose(grad_global_norm(ps), ref, rtol=1e-4)

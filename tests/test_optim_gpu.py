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


def test_fused_adam_alternating_grad_buffers_without_sync():
    """Gradient buffers change from step to step and the host runs ahead of the device (a long kernel is queued before
    every step): each step must still read ITS pointers from the staged table."""
    torch.manual_seed(1)
    shapes = [(512, 512), (4097,), (64, 3)]
    pa = [torch.randn(s, device="cuda") for s in shapes]
    pb = [p.clone() for p in pa]
    ours = FusedAdam(pa, lr=3e-3)
    ref = torch.optim.Adam(pb, lr=3e-3)
    pool = [[torch.randn_like(p) for p in pa] for _ in range(5)]        # five distinct sets of gradient tensors
    big = torch.randn(8192, 8192, device="cuda")
    for s in range(10):
        _ = big @ big                                                   # keeps the device behind the host
        for a, b, g in zip(pa, pb, pool[s % 5]):
            a.grad, b.grad = g, g.clone()
        ours.step()
    torch.cuda.synchronize()
    for s in range(10):
        for b, g in zip(pb, pool[s % 5]):
            b.grad = g.clone()
        ref.step()
    for a, b in zip(pa, pb):
        assert torch.allclose(a, b, atol=1e-5, rtol=1e-4)


def test_fused_adam_capturable_resume_keeps_step_count():
    """A capturable optimizer's step count lives on the device and advances in graph replays; ``state_dict`` must carry
    it, and a fresh optimizer that loads it must continue with the same bias correction as torch.optim.Adam."""
    torch.manual_seed(2)
    p0 = torch.randn(1000, device="cuda")
    grads = [torch.randn(1000, device="cuda") for _ in range(8)]
    a, b = p0.clone(), p0.clone()
    ours = FusedAdam([a], lr=1e-2, capturable=True)
    ref = torch.optim.Adam([b], lr=1e-2)
    static_g = torch.zeros_like(a)
    a.grad = static_g
    static_g.copy_(grads[0])
    ours.step()                                             # warm-up step (eager)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):                           # capture runs nothing: the replays below are steps 2 .. 5
        ours.step()
    for g in grads[1:5]:
        static_g.copy_(g)
        graph.replay()
    torch.cuda.synchronize()
    sd = ours.state_dict()
    assert sd["state"][0]["step"] == 5
    a2 = a.detach().clone()
    resumed = FusedAdam([a2], lr=1e-2, capturable=True)
    resumed.load_state_dict(sd)
    for g in grads[5:]:
        a2.grad = g.clone()
        resumed.step()
    for g in grads:
        b.grad = g.clone()
        ref.step()
    assert torch.allclose(a2, b, atol=1e-5, rtol=1e-4)

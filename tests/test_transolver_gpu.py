"""Fused sm_100a Transolver path against the plain PyTorch fp32 path of the same model."""
import copy

import pytest
import torch

from physicsnemo_b200 import ops
from physicsnemo_b200.models.transolver import Transolver

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def test_fused_block_matches_fp32_reference():
    dev = torch.device("cuda")
    model = Transolver(functional_dim=3, out_dim=4, embedding_dim=3, n_layers=2, n_hidden=256, n_head=8,
                       slice_num=64, mlp_ratio=4, use_te=False).to(dev)
    # move away from the init point so every parameter matters
    with torch.no_grad():
        for p in model.parameters():
            p.add_(torch.randn_like(p) * 0.02)
    ref = copy.deepcopy(model)
    n = 5000
    fx, emb = torch.randn(1, n, 3, device=dev), torch.randn(1, n, 3, device=dev)
    tgt = torch.randn(1, n, 4, device=dev)
    before = ops.kernel_launches()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = model(fx, embedding=emb)
    loss = torch.nn.functional.mse_loss(out.float(), tgt)
    loss.backward()
    assert ops.kernel_launches() - before >= 20, "fused kernels were not used"
    out_ref = ref(fx, embedding=emb)  # fp32, PyTorch ops only
    loss_ref = torch.nn.functional.mse_loss(out_ref, tgt)
    loss_ref.backward()
    assert ops.device_error() == 0
    assert _rel(out, out_ref) < 3e-2, _rel(out, out_ref)
    # every gradient within 2 % of its own norm plus 1 % of the model's total gradient norm (the floor covers tensors
    # whose gradient nearly cancels at this point, e.g. the slice projections: they move by a few % of their own tiny
    # norm between two runs of the same bf16 model)
    total = torch.sqrt(sum(q.grad.float().pow(2).sum() for q in ref.parameters())).item()
    bad = []
    for (name, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        assert p.grad is not None, name
        d = (p.grad.float() - q.grad.float()).norm().item()
        r = d / (q.grad.float().norm().item() + 1e-2 * total)
        if r > 2e-2:
            bad.append((name, r))
    assert not bad, bad


def test_fused_batch_two():
    dev = torch.device("cuda")
    model = Transolver(functional_dim=2, out_dim=1, embedding_dim=3, n_layers=1, n_hidden=128, n_head=4,
                       slice_num=64, use_te=False).to(dev)
    ref = copy.deepcopy(model)
    fx, emb = torch.randn(2, 777, 2, device=dev), torch.randn(2, 777, 3, device=dev)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = model(fx, embedding=emb)
    assert _rel(out, ref(fx, embedding=emb)) < 3e-2

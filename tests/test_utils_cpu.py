"""Checkpoint / resume, static capture (CPU path), loggers and profiler plumbing."""
import os

import pytest
import torch

from physicsnemo_b200.distributed import DistributedManager
from physicsnemo_b200.models.mlp import FullyConnected
from physicsnemo_b200.utils import (LaunchLogger, Profiler, StaticCaptureTraining, load_checkpoint, save_checkpoint)
from physicsnemo_b200.utils.capture import _StaticCapture
from physicsnemo_b200.utils.profiling.timing import _uncovered


@pytest.fixture(autouse=True)
def _manager():
    if not DistributedManager.is_initialized():
        for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
            os.environ.pop(k, None)
        DistributedManager._shared_state["_is_initialized"] = True
    yield


def _train(model, opt, steps, seed):
    g = torch.Generator().manual_seed(seed)
    for _ in range(steps):
        x = torch.randn(16, 4, generator=g)
        loss = (model(x) - x.sum(1, keepdim=True)).pow(2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
    return loss.item()


def test_resume_is_bit_exact_and_falls_back_on_damaged_file(tmp_path):
    torch.manual_seed(0)
    a = FullyConnected(4, 8, 1, num_layers=2)
    opt_a = torch.optim.Adam(a.parameters(), lr=1e-2)
    _train(a, opt_a, 5, seed=1)
    save_checkpoint(str(tmp_path), models=a, optimizer=opt_a, epoch=1, metadata={"note": "first"})
    ref_loss = _train(a, opt_a, 5, seed=2)
    save_checkpoint(str(tmp_path), models=a, optimizer=opt_a, epoch=2)
    # resume from epoch 1 in a fresh process-like state
    b = FullyConnected(4, 8, 1, num_layers=2)
    opt_b = torch.optim.Adam(b.parameters(), lr=1e-2)
    meta = {}
    epoch = load_checkpoint(str(tmp_path), models=b, optimizer=opt_b, epoch=1, metadata_dict=meta)
    assert epoch == 1 and meta["note"] == "first"
    assert _train(b, opt_b, 5, seed=2) == ref_loss
    # damage the newest training-state file: the loader falls back to the previous index
    newest = [p for p in tmp_path.iterdir() if p.name.startswith("checkpoint.0.2")][0]
    newest.write_bytes(newest.read_bytes()[:20])
    c = FullyConnected(4, 8, 1, num_layers=2)
    opt_c = torch.optim.Adam(c.parameters(), lr=1e-2)
    assert load_checkpoint(str(tmp_path), optimizer=opt_c) == 1


def test_static_capture_training_cpu():
    _StaticCapture.reset_state()
    torch.manual_seed(0)
    model = FullyConnected(4, 8, 1, num_layers=2)
    opt = torch.optim.SGD(model.parameters(), lr=1e-2)

    @StaticCaptureTraining(model=model, optim=opt, use_graphs=False, use_amp=False)
    def step(x, y):
        return torch.nn.functional.mse_loss(model(x), y)

    x, y = torch.randn(32, 4), torch.randn(32, 1)
    first = step(x, y).item()
    for _ in range(20):
        last = step(x, y).item()
    assert last < first
    assert "scaler_0" in _StaticCapture.state_dict()


def test_launch_logger_and_profiler(tmp_path, capsys):
    with LaunchLogger("train", epoch=1, num_mini_batch=4, mini_batch_log_freq=2) as log:
        for i in range(4):
            log.log_minibatch({"loss": 1.0 / (i + 1)})
        log.log_epoch({"lr": 0.1})
    Profiler._clear_instance()
    prof = Profiler()
    prof.output_path = tmp_path
    prof.enable("torch")
    with prof:
        torch.randn(64, 64) @ torch.randn(64, 64)
        prof.step()
    prof.finalize()
    assert (tmp_path / "torchprofile" / "cpu_time.txt").exists()
    Profiler._clear_instance()


def test_exposed_interval_arithmetic():
    assert _uncovered([(0, 10)], [(2, 4), (3, 6)]) == pytest.approx(6.0)
    assert _uncovered([(0, 5), (7, 9)], [(4, 8)]) == pytest.approx(5.0)
    assert _uncovered([(1, 2)], []) == pytest.approx(1.0)

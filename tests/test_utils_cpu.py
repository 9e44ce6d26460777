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


# ---- solar geometry ------------------------------------------------------------------------------------------------------
def test_zenith_angle_and_insolation():
    import datetime

    import numpy as np

    from physicsnemo_b200.utils.insolation import insolation
    from physicsnemo_b200.utils.zenith_angle import (cos_zenith_angle, cos_zenith_angle_from_timestamp, irradiance,
                                                     toa_incident_solar_radiation_accumulated, zenith_azimuth_angles)

    noon = datetime.datetime(2021, 6, 21, 12, 0)                       # June solstice, noon UTC: Sun overhead near (23.44 N, 0 E)
    assert float(cos_zenith_angle(noon, np.array(0.0), np.array(23.44))) > 0.999
    assert float(cos_zenith_angle(noon, np.array(180.0), np.array(-23.44))) < -0.999   # antipode: midnight
    lat, lon = np.linspace(-80, 80, 9)[:, None] * np.ones((1, 8)), np.linspace(0, 315, 8)[None, :] * np.ones((9, 1))
    cz = cos_zenith_angle(noon, lon, lat)
    assert cz.shape == (9, 8) and cz.dtype == np.float32
    ts = noon.replace(tzinfo=datetime.timezone.utc).timestamp()
    t_lat, t_lon = torch.tensor(lat, dtype=torch.float32), torch.tensor(lon, dtype=torch.float32)
    assert torch.allclose(cos_zenith_angle_from_timestamp(torch.tensor(ts, dtype=torch.float64), t_lon, t_lat), torch.tensor(cz), atol=1e-6)
    sz, cz2, sa, ca = zenith_azimuth_angles(noon, lon, lat)
    assert np.allclose(sz ** 2 + cz2 ** 2, 1, atol=1e-5) and np.allclose(sa ** 2 + ca ** 2, 1, atol=2e-2)
    assert 1310 < float(irradiance(np.array(ts))) < 1330              # aphelion side of the year
    jan = datetime.datetime(2021, 1, 4, tzinfo=datetime.timezone.utc).timestamp()
    assert float(irradiance(np.array(jan))) > 1400                     # perihelion
    # accumulated TOA radiation over an hour equals the time integral of S max(cos z, 0)
    acc = toa_incident_solar_radiation_accumulated(np.array(ts), lat, lon, interval=3600)
    steps = np.linspace(ts - 3600, ts, 121)
    quad = np.trapezoid(np.stack([np.maximum(cos_zenith_angle_from_timestamp(np.array(s), lon, lat), 0) * float(irradiance(np.array(s))) for s in steps]), steps, axis=0)
    assert np.allclose(acc, quad, rtol=2e-3, atol=50.0)
    dates = np.array(["2020-01-01T06", "2020-07-01T18"], dtype="datetime64[h]")
    sol = insolation(dates, lat, lon)
    assert sol.shape == (2, 9, 8) and sol.min() >= 0 and sol.dtype == np.float32
    assert sol[1, -1].mean() > sol[0, -1].mean()                       # the Arctic is lit in July, dark in January
    with pytest.raises(ValueError):
        insolation(dates, lat, lon[0])


def test_sdf_to_stl_and_memory_module(tmp_path):
    from physicsnemo_b200.mesh.io import read_stl
    from physicsnemo_b200.utils import memory
    from physicsnemo_b200.utils.mesh import sdf_to_stl

    ax = torch.linspace(-1, 1, 17)
    g = torch.stack(torch.meshgrid(ax, ax, ax, indexing="ij"), -1)
    sdf_to_stl((g.norm(dim=-1) - 0.5).numpy(), filename=str(tmp_path / "s.stl"))
    m = read_stl(tmp_path / "s.stl")
    assert m.n_cells > 100
    assert memory.unified_gpu_memory is None or memory.unified_gpu_memory is True      # no rmm here: a no-op
    assert memory.srt2bool("Yes") and not memory.srt2bool("0")
    with pytest.raises(AttributeError):
        memory.nothing_here

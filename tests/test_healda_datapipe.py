"""HealDA data pipeline on synthetic arrays (CPU): indexing over gaps, restartable sampling, prefetching,
observation filtering and featurisation, and the dataset → loader → two-stage transform path."""
import datetime
import math

import numpy as np
import pytest
import torch

from physicsnemo_b200.experimental.datapipes import healda as H
from physicsnemo_b200.experimental.datapipes.healda import time_utils as TU
from physicsnemo_b200.experimental.datapipes.healda.configs import channel_names, concat_tables, empty_table
from physicsnemo_b200.experimental.datapipes.healda.indexing import FrameIndexGenerator, get_flat_indexer, split_array_contiguous
from physicsnemo_b200.experimental.datapipes.healda.transforms import (compute_unified_metadata, compute_unified_metadata_reference,
                                                                      local_solar_time)
from physicsnemo_b200.experimental.datapipes.healda.transforms.obs_filtering import filter_observations
from physicsnemo_b200.nn.module.hpx.tokenizer import healpix_lonlat_to_xy, healpix_xy_lonlat


def test_indexing_respects_gaps_and_model_parallel_time_split():
    t = np.array([0, 6, 12, 18, 36, 42, 48, 54, 60])
    assert [s.tolist() for s in split_array_contiguous(t)] == [[0, 6, 12, 18], [36, 42, 48, 54, 60]]
    assert split_array_contiguous(np.array([])) == [] and len(split_array_contiguous(np.array([5]))) == 1
    g = FrameIndexGenerator(t, time_length=2, frame_step=2, model_rank=0, model_world_size=1)
    assert g.segment_valid_lengths == [2, 3] and g.get_valid_length() == 5
    assert g.generate_frame_indices(range(5)) == [[0, 2], [1, 3], [4, 6], [5, 7], [6, 8]]
    with pytest.raises(IndexError):
        g.generate_frame_indices([5])
    half = FrameIndexGenerator(t, time_length=4, frame_step=1, model_rank=1, model_world_size=2)
    assert half.generate_frame_indices([0, 1]) == [[2, 3], [6, 7]]

    class DS(dict):
        sizes = {"ens": 3}

    index = get_flat_indexer(DS(time=t), ["ens"], "time", 2, 2, 0, 1)
    assert len(index) == 15 and index[7] == {"ens": 1, "time": [4, 6]}


def test_restartable_sampler_resumes_mid_epoch():
    data = list(range(23))
    parts = [H.RestartableDistributedSampler(data, rank=r, num_replicas=4, seed=7) for r in range(4)]
    seen = [list(p) for p in parts]
    assert all(len(s) == 5 for s in seen) and len({i for s in seen for i in s}) == 20
    s = H.RestartableDistributedSampler(data, rank=1, num_replicas=4, seed=7)
    it = iter(s)
    first = [next(it) for _ in range(2)]
    state = s.state_dict()
    rest = list(it)
    assert first + rest == seen[1] and s.epoch == 1
    resumed = H.RestartableDistributedSampler(data, rank=1, num_replicas=4, seed=7)
    resumed.load_state_dict(state)
    assert list(resumed) == rest
    second_epoch = list(resumed)
    assert sorted(second_epoch) != sorted(seen[1]) or second_epoch != seen[1]
    plain = H.RestartableDistributedSampler(data, rank=0, num_replicas=2, shuffle=False)
    assert list(plain) == list(range(0, 22, 2))


def test_prefetch_map_order_errors_and_restart():
    loader = [{"x": torch.full((2,), float(i))} for i in range(5)]
    it = H.prefetch_map(loader, lambda b: {"x": b["x"] * 2}, queue_size=2)
    assert [float(b["x"][0]) for b in it] == [0, 2, 4, 6, 8] and len(it) == 5
    assert [float(b["x"][0]) for b in it] == [0, 2, 4, 6, 8]            # iterable again

    def bad(b):
        if float(b["x"][0]) == 3:
            raise RuntimeError("boom")
        return b

    with pytest.raises(RuntimeError, match="boom"):
        list(H.prefetch_map(loader, bad))
    with pytest.raises(RuntimeError, match="not started"):
        next(H.prefetch_map(loader, bad))


def test_time_encodings_and_batch_info():
    t = datetime.datetime(2021, 3, 1, 6, 30, tzinfo=datetime.timezone.utc)
    assert TU.compute_second_of_day(t) == 6.5 * 3600 and TU.compute_day_of_year(t) == 59 + 6.5 / 24
    assert TU.compute_timestamp(t) == int(t.timestamp()) == int(TU.as_timestamp(np.datetime64("2021-03-01T06:30"))[0])
    c = TU.as_cftime(np.datetime64("2021-03-01T06:30"))
    assert (c.year, c.hour, c.minute) == (2021, 6, 30) and TU.compute_timestamp(c) == int(t.timestamp())
    info = H.BatchInfo(channels=["a", "b", "c"], time_step=6, scales=[1.0, 2.0, 3.0], center=[0.0, 1.0, 2.0])
    again = H.BatchInfo.loads(info.dumps())
    assert again.channels == info.channels and again.time_unit is H.TimeUnit.HOUR
    sub = info.sel_channels(["c", "a"])
    assert sub.scales.tolist() == [3.0, 1.0] and info.get_time_delta(2) == datetime.timedelta(hours=12)
    x = torch.ones(3, 2, 4)
    assert torch.equal(info.denormalize(x)[:, 0, 0], torch.tensor([1.0, 3.0, 5.0]))
    with pytest.raises(ValueError):
        H.BatchInfo(channels=[], time_unit="h")
    assert len(channel_names(H.VARIABLE_CONFIGS["era5"])) == 5 * 13 + 9


def test_split_by_sensor_and_empty_batch():
    lengths = torch.tensor([[[2, 1]], [[0, 3]]])                         # 2 sensors, B = 1, T = 2
    n = int(lengths.sum())
    obs = H.UnifiedObservation(obs=torch.arange(n, dtype=torch.float32), time=torch.arange(n), float_metadata=torch.zeros(n, 28),
                               pix=torch.arange(n), local_channel=torch.zeros(n, dtype=torch.long),
                               local_platform=torch.zeros(n, dtype=torch.long), obs_type=torch.zeros(n, dtype=torch.long),
                               global_channel=torch.arange(n), hpx_level=4, lengths=lengths)
    parts = H.split_by_sensor(obs, [10, 11, 12])
    assert parts[10].obs.tolist() == [0, 1, 2] and parts[11].obs.tolist() == [3, 4, 5] and parts[12].obs.numel() == 0
    assert parts[11].lengths.tolist() == [[[0, 3]]] and parts[12].lengths.shape == (1, 1, 2) and parts[10].global_platform is None
    with pytest.raises(ValueError):
        H.split_by_sensor(obs, [10])
    batch = H.empty_batch(batch_gpu=2, out_channels=5, condition_channels=2, time_length=3, x_size=48, device="cpu")
    assert batch["target"].shape == (2, 5, 3, 48) and batch["unified_obs"].batch_dims == (2, 3)
    assert batch["unified_obs"].to(dtype=torch.float64).pix.dtype == torch.long


def test_metadata_features_match_their_definition():
    n = 7
    target = torch.full((n,), 1_700_000_000)
    time = target * 10 ** 9 + torch.arange(n) * 1800 * 10 ** 9
    lon, lat = torch.linspace(-170, 170, n), torch.linspace(-80, 80, n)
    nan = float("nan")
    height = torch.tensor([100.0, nan, 5e4, 1e5, 0.0, nan, 3.0])
    cols = dict(height=height, pressure=torch.tensor([500.0, nan, 10, 2000, 1100, nan, 850]),
                scan_angle=torch.tensor([nan, 10.0, nan, nan, nan, -40.0, nan]),
                sat_zenith_angle=torch.tensor([nan, 30.0, nan, nan, nan, 60.0, nan]),
                sol_zenith_angle=torch.tensor([nan, 100.0, nan, nan, nan, 20.0, nan]))
    f = compute_unified_metadata(target, time=time, lon=lon, **cols)
    assert f.shape == (n, 28) and not bool(f.isnan().any())
    lst = local_solar_time(lon, time)
    assert bool(((lst >= 0) & (lst < 24)).all())
    assert torch.allclose(f[:, 0], torch.sin(lst / 24 * 2 * math.pi), atol=1e-5) and torch.allclose(f[:, 3], torch.cos(lst / 6 * math.pi), atol=1e-5)
    assert torch.allclose(f[:, 4], torch.arange(n) * 1800 / 86400.0, atol=1e-6) and torch.allclose(f[:, 5], f[:, 4] ** 2)
    assert float(f[1, 6:22].abs().sum()) == 0                             # no height / pressure reported
    assert torch.allclose(f[3, 6:10], torch.zeros(4), atol=1e-5) and torch.allclose(f[3, 10:14], torch.ones(4), atol=1e-5)   # clamped
    assert torch.allclose(f[1, 22:24], torch.tensor([0.2, 0.04])) and torch.allclose(f[5, 24], torch.tensor(0.5), atol=1e-6)
    assert torch.allclose(f[1, 26:28], torch.tensor([math.cos(math.radians(100)), math.sin(math.radians(100))]), atol=1e-6)
    assert float(f[0, 22:].abs().sum()) == 0
    e = compute_unified_metadata(target, time=time, lon=lon, lat=lat, extended=True, **cols)
    assert e.shape == (n, 30) and torch.allclose(e[:, 8], torch.sin(torch.deg2rad(lat)), atol=1e-6)
    assert torch.allclose(e[0, 10], torch.sin(torch.tensor(100 / 6e4 * 2 * math.pi)), atol=1e-6)            # conventional row
    assert torch.allclose(e[1, 10], torch.sin(torch.tensor(10 / 50 * 2 * math.pi)), atol=1e-6)              # satellite row
    assert torch.allclose(e[5, 27:30], torch.cos(torch.tensor([1.0, 2.0, 3.0]) * 20 / 180 * 2 * math.pi), atol=1e-5)
    with pytest.raises(ValueError):
        compute_unified_metadata_reference(target, time=time, lon=lon, extended=True)


@pytest.mark.gpu
def test_metadata_feature_kernel_matches_reference():
    torch.manual_seed(0)
    n = 100_003
    target = torch.randint(1_600_000_000, 1_700_000_000, (n,))
    time = target * 10 ** 9 + torch.randint(-3 * 3600, 3 * 3600, (n,)) * 10 ** 9
    lon, lat = torch.rand(n) * 360 - 180, torch.rand(n) * 180 - 90
    conv = torch.rand(n) < 0.4
    nan = torch.full((n,), float("nan"))
    cols = dict(height=torch.where(conv, torch.rand(n) * 7e4, nan), pressure=torch.where(conv, torch.rand(n) * 1200, nan),
                scan_angle=torch.where(conv, nan, torch.rand(n) * 100 - 50), sat_zenith_angle=torch.where(conv, nan, torch.rand(n) * 70),
                sol_zenith_angle=torch.where(conv, nan, torch.rand(n) * 180))
    for extended in (False, True):
        want = compute_unified_metadata_reference(target, time=time, lon=lon, lat=lat, extended=extended, **cols)
        got = compute_unified_metadata(target.cuda(), time=time.cuda(), lon=lon.cuda(), lat=lat.cuda(), extended=extended,
                                       **{k: v.cuda() for k, v in cols.items()})
        assert got.shape == want.shape and float((got.cpu() - want).abs().max()) < 2e-4


def _registry():
    return H.SensorRegistry([H.SensorConfig("mw", ["sat-a", "sat-b"], channels=3, means=[250.0, 260.0, 270.0], stds=[10.0, 10.0, 20.0]),
                             H.SensorConfig("conv", ["gps", "raob"], channels=4, min_valid=-100.0, max_valid=400.0,
                                            sensor_type="conventional")])


def _window(seed, when, registry, n_mw=30, n_conv=20):
    g = np.random.default_rng(seed)
    nan = np.full(n_mw, np.nan, dtype=np.float32)
    mw = {"Latitude": g.uniform(-90, 90, n_mw), "Longitude": g.uniform(0, 360, n_mw), "Observation": g.uniform(200, 300, n_mw),
          "Global_Channel_ID": registry.global_channel("mw", g.integers(0, 3, n_mw)), "Platform_ID": g.integers(0, 2, n_mw),
          "Observation_Type": np.zeros(n_mw, dtype=np.int64), "Height": nan, "Pressure": nan, "Scan_Angle": g.uniform(-50, 50, n_mw),
          "Sat_Zenith_Angle": g.uniform(0, 60, n_mw), "Sol_Zenith_Angle": g.uniform(0, 180, n_mw), "QC_Flag": g.integers(0, 2, n_mw)}
    nanc = np.full(n_conv, np.nan, dtype=np.float32)
    conv = {"Latitude": g.uniform(-90, 90, n_conv), "Longitude": g.uniform(0, 360, n_conv), "Observation": g.uniform(-50, 50, n_conv),
            "Global_Channel_ID": registry.global_channel("conv", g.integers(0, 4, n_conv)), "Platform_ID": g.integers(2, 4, n_conv),
            "Observation_Type": g.integers(200, 300, n_conv), "Height": g.uniform(-500, 70000, n_conv),
            "Pressure": g.uniform(0, 1200, n_conv), "Scan_Angle": nanc, "Sat_Zenith_Angle": nanc, "Sol_Zenith_Angle": nanc,
            "QC_Flag": np.zeros(n_conv, dtype=np.int64)}
    conv["Observation"][0] = np.nan
    mw["Observation"][0] = 1000.0                                           # outside the sensor's valid range
    table = {k: np.concatenate([mw[k], conv[k]]) for k in mw}
    table["Absolute_Obs_Time"] = when + g.integers(-5400, 5400, n_mw + n_conv).astype("timedelta64[s]")
    return table


def test_observation_filter():
    reg = _registry()
    table = _window(0, np.datetime64("2021-01-01T00", "ns"), reg)
    stats = reg.channel_stats()
    ch = table["Global_Channel_ID"]
    for name in ("sensor_id", "local_channel_id", "min_valid", "max_valid", "is_conv"):
        table[name] = stats[name][ch]
    kept = filter_observations(table)
    assert 0 < len(kept["Observation"]) < 50 and np.isfinite(kept["Observation"]).all() and kept["Observation"].max() <= 400
    conv = kept["is_conv"].astype(bool)
    assert (kept["Height"][conv] >= 0).all() and (kept["Height"][conv] <= 60000).all() and (kept["Pressure"][conv] <= 1100).all()
    gps_like = kept["local_channel_id"][conv] <= 2
    assert (kept["Pressure"][conv][~gps_like] >= 200).all() and (kept["Pressure"][conv][gps_like] >= 0.5).all()
    strict = filter_observations(table, qc_filter=True)
    assert (strict["QC_Flag"][~strict["is_conv"].astype(bool)] == 0).all() and len(strict["Observation"]) < len(kept["Observation"])
    dropped = filter_observations(table, drop_channels=[1, 2])
    assert not np.isin(dropped["local_channel_id"][dropped["is_conv"].astype(bool)], [1, 2]).any()
    assert len(concat_tables([empty_table(), empty_table()])["Observation"]) == 0


def test_dataset_loader_and_two_stage_transform():
    reg = _registry()
    hours = np.concatenate([np.arange(0, 48, 6), np.arange(72, 120, 6)])                 # a one-day gap
    times = np.datetime64("2021-06-01T00", "ns") + hours.astype("timedelta64[h]")
    level, n_ch = 2, 5
    npix = 12 * 4 ** level
    g = np.random.default_rng(1)
    data = g.normal(size=(len(times), n_ch, npix)).astype(np.float32) * 3 + 7
    store = H.ArrayStateStore(data, times, [f"c{i}" for i in range(n_ch)], center=np.full(n_ch, 7.0), scales=np.full(n_ch, 3.0))
    windows = {t + np.timedelta64(h, "h"): _window(int(i * 10 + h), t + np.timedelta64(h, "h"), reg)
               for i, t in enumerate(times) for h in (0, 3)}
    loader = H.TableObsLoader(windows, reg, obs_context_hours=(-3, 3), data_spacing=3)
    assert [int(x) for x in (loader.interval_times(times[0]) - times[0]) / np.timedelta64(1, "h")] == [0, 3]
    static = torch.randn(2, npix)
    tf = H.ERA5ObsTransform(store.batch_info, reg, sensors=["mw", "conv"], hpx_level=4, static_condition=static)
    ds = H.ObsERA5Dataset(store, loader, tf, time_length=2, frame_step=1)
    assert len(ds) == 2 * (8 - 1)
    sampler = H.RestartableDistributedSampler(ds, shuffle=False)
    batches = torch.utils.data.DataLoader(ds, batch_sampler=torch.utils.data.BatchSampler(sampler, 3, drop_last=False),
                                          collate_fn=H.identity_collate)
    out = list(H.prefetch_map(batches, lambda b: tf.device_transform(b, torch.device("cpu"))))
    assert [b["target"].shape[0] for b in out] == [3, 3, 3, 3, 2]
    first = out[0]
    assert first["target"].shape == (3, n_ch, 2, npix) and first["condition"].shape == (3, 2, 2, npix)
    assert torch.allclose(first["target"][1, :, 0], torch.from_numpy((data[1] - 7) / 3), atol=1e-6)
    assert torch.equal(first["condition"][2, :, 1], static) and first["second_of_day"].tolist()[0] == [0.0, 6 * 3600.0]
    assert first["timestamp"][0, 0].item() == int(times[0].astype("datetime64[s]").astype(np.int64))
    obs = first["unified_obs"]
    assert obs.lengths.shape == (2, 3, 2) and int(obs.lengths.sum()) == obs.obs.shape[0] > 0
    assert obs.float_metadata.shape == (obs.obs.shape[0], 28) and obs.pix.max() < 12 * 4 ** 4
    parts = H.split_by_sensor(obs, [0, 1])
    assert bool(parts[0].float_metadata[:, 6:22].abs().sum() == 0) and bool((parts[1].float_metadata[:, 22:] == 0).all())
    assert set(parts[0].local_platform.tolist()) <= {0, 1} and set(parts[1].local_platform.tolist()) <= {0, 1}
    assert set(parts[1].global_platform.tolist()) <= {2, 3}
    # the first (sensor 0, item 0, frame 0) group holds the two windows of the first time, normalised per channel
    n000 = int(obs.lengths[0, 0, 0])
    w = concat_tables([windows[times[0]], windows[times[0] + np.timedelta64(3, "h")]])
    mw_ok = (w["Global_Channel_ID"] < 3) & (w["Observation"] <= 400)
    assert n000 == int(mw_ok.sum())
    ch = w["Global_Channel_ID"][mw_ok]
    want = (w["Observation"][mw_ok] - np.array([250.0, 260.0, 270.0])[ch]) / np.array([10.0, 10.0, 20.0])[ch]
    assert np.allclose(obs.obs[:n000].numpy(), want, atol=1e-5)
    lon, lat = healpix_xy_lonlat(4)
    assert torch.equal(healpix_lonlat_to_xy(lon, lat, 4), torch.arange(12 * 4 ** 4))
    # windows beyond the archive are simply empty; a dataset restricted to other years has no samples
    assert len(H.ObsERA5Dataset(store, loader, tf, split=[1999])) == 0
    assert len(H.ObsERA5Dataset(store, loader, tf, split="train", time_length=4)) == 2 * (8 - 3)

"""Datapipes: readers / transforms / loader on CPU; PDE generators (tensor formulation on CPU, kernels vs it on GPU)."""
import os

import numpy as np
import pytest
import torch

from physicsnemo_b200.datapipes import (BoundingBoxFilter, Compose, ConcatCollator, ConcatFields, DataLoader, Dataset,
                                        FieldSlice, MultiDataset, Normalize, NumpyReader, Purge, Rename, SubsamplePoints,
                                        TensorDict, Translate)
from physicsnemo_b200.datapipes._indexing import _cyclic_block_indices
from physicsnemo_b200.datapipes._rng import derive_seed
from physicsnemo_b200.datapipes.benchmarks import Darcy2D, KelvinHelmholtz2D
from physicsnemo_b200.datapipes.benchmarks.darcy import darcy_multigrid_torch, permeability_from_fourier
from physicsnemo_b200.datapipes.benchmarks.kelvin_helmholtz import kh_simulate_torch


@pytest.fixture()
def npz_dir(tmp_path):
    rng = np.random.default_rng(0)
    for i in range(9):
        np.savez(tmp_path / f"s{i:02d}.npz", coords=rng.random((50, 3), dtype=np.float32), p=rng.random((50, 2), dtype=np.float32),
                 idx=np.full((1,), i, dtype=np.float32))
    return tmp_path


def test_reader_transforms_loader(npz_dir):
    r = NumpyReader(npz_dir)
    assert len(r) == 9 and set(r.field_names) == {"coords", "p", "idx"}
    data, meta = r[-1]
    assert meta["index"] == 8 and meta["source_filename"] == "s08.npz" and isinstance(data, TensorDict)
    norm = Normalize(["p"], means={"p": 0.5}, stds={"p": 0.25}, method="mean_std")
    tf = [norm, Translate(["coords"], torch.tensor([1.0, 0.0, 0.0])), SubsamplePoints(["coords", "p"], 20, algorithm="uniform"),
          ConcatFields(["coords", "p"], "x"), FieldSlice({"x": {"-1": [0, 3]}}), Rename({"idx": "sample_id"})]
    ds = Dataset(r, transforms=tf)
    out, _ = ds[3]
    assert out["x"].shape == (20, 2) and float(out["sample_id"]) == 3.0 and out["coords"][:, 0].min() >= 1.0
    back = norm.inverse(TensorDict({"p": out["p"].clone()}))["p"]
    assert back.min() >= -1e-5 and back.max() <= 1 + 1e-5
    # same seed -> same shuffling and sub-sampling, with and without prefetch threads
    runs = []
    for prefetch in (0, 2):
        dl = DataLoader(Dataset(NumpyReader(npz_dir), transforms=[SubsamplePoints(["coords", "p"], 20, algorithm="uniform")]),
                        batch_size=4, shuffle=True, seed=7, prefetch_factor=prefetch, collate_metadata=True)
        runs.append([(b["coords"].clone(), [m["index"] for m in meta]) for b, meta in dl])
        assert len(dl) == 3
    for (a, ia), (b, ib) in zip(*runs):
        assert ia == ib and torch.equal(a, b)
    cat = next(iter(DataLoader(Dataset(r), batch_size=2, collate_fn=ConcatCollator())))
    assert cat["coords"].shape == (100, 3) and cat["batch_idx"].tolist() == [0] * 50 + [1] * 50
    md = MultiDataset(Dataset(r), Dataset(r))
    assert len(md) == 18 and md[10][1]["dataset_index"] == 1 and md[10][1]["index"] == 1
    kept = Compose([BoundingBoxFilter(["coords"], torch.zeros(3), torch.full((3,), 0.5), dependent_keys=["p"]),
                    Purge(keep_only=["coords", "p"])])(r[0][0])
    assert kept["coords"].shape[0] == kept["p"].shape[0] and kept["coords"].max() <= 0.5 and "idx" not in kept.keys()
    with pytest.raises(KeyError):
        Normalize(["nope"], means=0.0, stds=1.0, method="mean_std")(r[0][0])


def test_rng_and_indexing():
    assert derive_seed(1, 2, 3) == derive_seed(1, 2, 3) != derive_seed(1, 3, 2)
    idx = _cyclic_block_indices(10, 4, start=8)
    assert idx.tolist() == [0, 1, 8, 9]
    g = torch.Generator().manual_seed(0)
    counts = torch.zeros(10)
    for _ in range(2000):
        counts[_cyclic_block_indices(10, 4, generator=g)] += 1
    assert (counts / 2000 - 0.4).abs().max() < 0.05


def test_darcy_torch_solves_the_pde():
    torch.manual_seed(0)
    res = 32
    f = torch.rand(4, 2, 3, 3) * 2 - 1
    k = permeability_from_fourier(f, res, 0.5, 2.0)
    assert set(k.unique().tolist()) <= {0.5, 2.0}
    u = darcy_multigrid_torch(k, res, levels=3, max_iterations=20000, check_every=500, threshold=1e-7)
    dx = 1.0 / (res + 1)
    up = torch.nn.functional.pad(u, (1, 1, 1, 1))
    kp = torch.nn.functional.pad(k, (1, 1, 1, 1), mode="replicate")
    lap = (up[:, 2:, 1:-1] + up[:, :-2, 1:-1] + up[:, 1:-1, 2:] + up[:, 1:-1, :-2] - 4 * u) / dx ** 2
    gx = (kp[:, 2:, 1:-1] - kp[:, :-2, 1:-1]) * (up[:, 2:, 1:-1] - up[:, :-2, 1:-1]) / (2 * dx)
    gy = (kp[:, 1:-1, 2:] - kp[:, 1:-1, :-2]) * (up[:, 1:-1, 2:] - up[:, 1:-1, :-2]) / (2 * dx)
    residual = k * lap + gx + gy + 1.0          # the discrete operator of the scheme (cross terms over 2·dx)
    assert residual.abs().max() < 5e-2 and u.min() > 0
    pipe = Darcy2D(resolution=16, batch_size=2, nr_multigrids=2, max_iterations=500, iterations_per_convergence_check=100, device="cpu")
    it = iter(pipe)
    a = next(it)
    ptr = a["darcy"].data_ptr()
    b = next(it)
    assert b["darcy"].data_ptr() == ptr and b["permeability"].shape == (2, 1, 16, 16)


def test_kelvin_helmholtz_torch_conserves():
    w = torch.rand(2, 3) * 0.2 - 0.1
    N, dx = 32, 1 / 32
    dt = 0.4 * dx / ((5 / 3 * 5.0) ** 0.5 + 2.0)
    r, v, p = kh_simulate_torch(w, N, snapshots=3, steps=10, gamma=5 / 3, dx=dx, dt=dt, sigma=0.05 / 2 ** 0.5)
    assert r.shape == (3, 2, N, N) and v.shape == (3, 2, N, N, 2)
    mass = r.sum((2, 3))
    assert torch.allclose(mass[0], mass[-1], rtol=1e-5)                           # periodic finite volumes conserve mass
    assert (r > 0).all() and (p > 0).all() and not torch.equal(r[0], r[-1])
    pipe = KelvinHelmholtz2D(resolution=16, batch_size=2, seq_length=2, nr_snapshots=4, iteration_per_snapshot=2, device="cpu")
    out = next(iter(pipe))
    assert out["velocity"].shape == (2, 2, 2, 16, 16)


@pytest.mark.gpu
def test_pde_kernels_match_tensor_formulation():
    torch.manual_seed(0)
    d = Darcy2D(resolution=64, batch_size=3, nr_multigrids=3, max_iterations=4000, iterations_per_convergence_check=500,
                convergence_threshold=1e-6, device="cuda")
    d.generate_batch()
    k_ref = permeability_from_fourier(d.rand_fourier, 64, 0.5, 2.0)
    assert (d.permeability != k_ref).float().mean() < 1e-3                       # sign flips only where the field is ~0
    u_ref = darcy_multigrid_torch(d.permeability.clone(), 64, 3, 4000, 500, 1e-6)
    assert (d.darcy0 - u_ref).abs().max() / u_ref.abs().max() < 2e-3
    assert int(d.inf_residual[1]) > 0
    k = KelvinHelmholtz2D(resolution=64, batch_size=2, seq_length=2, nr_snapshots=3, iteration_per_snapshot=8, device="cuda")
    k.generate_batch()
    r, v, p = kh_simulate_torch(k.w, 64, 3, 8, k.gamma, k.dx, k.dt, 0.05 / 2 ** 0.5)
    assert (k.seq_rho - r).abs().max() < 1e-4 and (k.seq_vel - v).abs().max() < 1e-4 and (k.seq_p - p).abs().max() < 2e-4
    out = next(iter(k))
    assert out["density"].shape == (2, 2, 1, 64, 64)

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


# ---- domain datapipes --------------------------------------------------------------------------------------------------
def test_domino_datapipe_feeds_the_model():
    import copy

    from physicsnemo_b200.datapipes.cae import DoMINODataPipe, compute_scaling_factors
    from physicsnemo_b200.mesh import primitives
    from physicsnemo_b200.models.domino import DEFAULT_MODEL_PARAMS, DoMINO

    torch.manual_seed(0)
    s = primitives.icosphere(3)
    V, F = s.points.float() * 0.5, s.cells
    tri = V[F]
    n = torch.linalg.cross(tri[:, 1] - tri[:, 0], tri[:, 2] - tri[:, 0])
    centers, areas, normals = tri.mean(1), 0.5 * n.norm(dim=-1), n / n.norm(dim=-1, keepdim=True)
    vol = torch.rand(3000, 3) * 2 - 1
    sample = dict(stl_coordinates=V, stl_faces=F.reshape(-1), stl_centers=centers, stl_areas=areas, global_params_values=torch.tensor([[30.0], [1.2]]),
                  global_params_reference=torch.tensor([[30.0], [1.2]]), surface_mesh_centers=centers, surface_normals=normals, surface_areas=areas,
                  surface_fields=torch.randn(centers.shape[0], 4) * 3 + 1, volume_mesh_centers=vol, volume_fields=torch.randn(3000, 5))
    factors = compute_scaling_factors([sample])
    assert torch.allclose(factors["surface_fields"]["mean"], sample["surface_fields"].mean(0), atol=1e-4)
    pipe = DoMINODataPipe(model_type="combined", dataset=[sample], device="cpu", bounding_box_dims=[(1, 1, 1), (-1, -1, -1)],
                          bounding_box_dims_surf=[(0.6, 0.6, 0.6), (-0.6, -0.6, -0.6)], grid_resolution=(8, 8, 8), sampling=True,
                          surface_points_sample=64, volume_points_sample=80, geom_points_sample=300, num_surface_neighbors=5,
                          normalize_coordinates=False, deterministic=True, scaling_type="mean_std_scaling",
                          surface_factors=torch.stack([factors["surface_fields"]["mean"], factors["surface_fields"]["std"]]),
                          volume_factors=torch.stack([factors["volume_fields"]["mean"], factors["volume_fields"]["std"]]))
    out = pipe[0]
    assert out["surface_mesh_neighbors"].shape == (1, 64, 4, 3) and out["sdf_grid"].shape == (1, 8, 8, 8)
    r = out["volume_mesh_centers"][0].norm(dim=-1)
    assert (out["sdf_nodes"][0, :, 0] - (r - 0.5)).abs().max() < 5e-3                       # signed distance to the sphere
    assert torch.allclose(out["pos_volume_closest"][0].norm(dim=-1), out["sdf_nodes"][0, :, 0].abs(), atol=1e-4)
    _, back = pipe.unscale_model_outputs(surface_fields=out["surface_fields"])
    assert float(back.std()) == pytest.approx(3.0, rel=0.2)
    p = copy.deepcopy(DEFAULT_MODEL_PARAMS)
    p.interp_res = [8, 8, 8]
    gc, gl = p.geometry_rep.geo_conv, p.geometry_local
    gc.volume_radii, gc.volume_neighbors_in_radius, gc.surface_radii, gc.surface_neighbors_in_radius = [0.5], [4], [0.5], [4]
    gl.volume_radii, gl.volume_neighbors_in_radius, gl.surface_radii, gl.surface_neighbors_in_radius = [0.6], [4], [0.6], [4]
    p.nn_basis_functions.base_layer = p.aggregation_model.base_layer = p.position_encoder.base_neurons = 8
    p.num_neighbors_volume, p.num_neighbors_surface = 2, 5
    model = DoMINO(input_features=3, output_features_vol=5, output_features_surf=4, model_parameters=p)
    vol_pred, surf_pred = model(out)
    assert vol_pred.shape == out["volume_fields"].shape and surf_pred.shape == out["surface_fields"].shape
    with pytest.raises(ValueError):
        pipe.process_data({"stl_coordinates": V})


def test_climate_datapipes(tmp_path):
    from physicsnemo_b200.datapipes.climate import ERA5Datapipe, SyntheticWeatherDataLoader

    loader = SyntheticWeatherDataLoader(channels=[0, 1, 2], num_samples_per_year=12, num_steps=2, device="cpu", grid_size=(8, 16),
                                        batch_size=4, seed=1)
    batch = next(iter(loader))[0]
    assert batch["invar"].shape == (4, 3, 8, 16) and batch["outvar"].shape == (4, 2, 3, 8, 16)
    assert float(batch["invar"][:, 0].mean()) > float(batch["invar"][:, 2].mean())          # lapse rate: higher channels are colder
    rng = np.random.default_rng(0)
    for year in (2000, 2001):
        np.save(tmp_path / f"{year}.npy", rng.normal(5.0, 2.0, size=(10, 4, 9, 12)).astype(np.float32))
    stats = tmp_path / "stats"
    stats.mkdir()
    np.save(stats / "global_means.npy", np.full((1, 4, 1, 1), 5.0, np.float32))
    np.save(stats / "global_stds.npy", np.full((1, 4, 1, 1), 2.0, np.float32))
    pipe = ERA5Datapipe(str(tmp_path), str(stats), channels=[0, 2], batch_size=3, num_steps=2, stride=2, num_history=1, patch_size=4,
                        shuffle=False, device="cpu")
    items = list(pipe)
    assert len(items) == len(pipe) == (2 * (10 - 2 - 4)) // 3
    b = items[0][0]
    assert b["invar"].shape == (3, 2, 2, 8, 12) and b["outvar"].shape == (3, 2, 2, 8, 12)
    raw = np.load(tmp_path / "2000.npy")
    assert torch.allclose(b["invar"][0, 1], torch.from_numpy((raw[2][[0, 2]][:, :8] - 5.0) / 2.0), atol=1e-6)   # first window starts at t = 2
    assert torch.allclose(b["invar"][0, 0], torch.from_numpy((raw[0][[0, 2]][:, :8] - 5.0) / 2.0), atol=1e-6)   # history is one stride back
    assert torch.allclose(b["outvar"][0, 1], torch.from_numpy((raw[6][[0, 2]][:, :8] - 5.0) / 2.0), atol=1e-6)
    halves = [ERA5Datapipe(str(tmp_path), None, batch_size=1, shuffle=True, seed=3, device="cpu", process_rank=r, world_size=2) for r in (0, 1)]
    seen = [torch.stack([it[0]["invar"] for it in h]).sum().item() for h in halves]
    assert len(halves[0]) == len(halves[1]) and seen[0] != seen[1]                           # ranks read disjoint halves


def test_mesh_graph_time_series_dataset(tmp_path):
    from physicsnemo_b200.datapipes.gnn import VortexSheddingDataset, cells_to_edges, load_json, save_json

    rng = np.random.default_rng(0)
    pos = rng.random((6, 2)).astype(np.float32)
    cells = np.array([[0, 1, 2], [1, 2, 3], [2, 3, 4], [3, 4, 5]])
    traj = dict(mesh_pos=pos, cells=cells, node_type=np.array([0, 0, 4, 6, 0, 5]), velocity=rng.normal(size=(5, 6, 2)).astype(np.float32),
                pressure=rng.normal(size=(5, 6, 1)).astype(np.float32))
    ei = cells_to_edges(torch.as_tensor(cells))
    assert ei.shape == (2, 18)                                        # 9 unique edges, both directions
    np.savez(tmp_path / "traj0.npz", **traj)
    ds = VortexSheddingDataset.from_npz_dir(tmp_path, split="train", noise_std=0.0)
    assert len(ds) == 4
    s = ds[1]
    assert s["x"].shape == (6, 2 + 7) and s["edge_attr"].shape == (18, 3) and s["y"].shape == (6, 3)
    dv, p = ds.denormalize(s["y"])
    assert torch.allclose(dv, torch.as_tensor(traj["velocity"][2] - traj["velocity"][1]), atol=1e-5)
    assert torch.allclose(p, torch.as_tensor(traj["pressure"][2]), atol=1e-5)
    save_json(ds.node_stats, tmp_path / "node_stats.json")
    stats = load_json(tmp_path / "node_stats.json")
    val = VortexSheddingDataset([traj], split="valid", node_stats=stats, edge_stats=ds.edge_stats)
    assert torch.allclose(val[1]["y"], s["y"], atol=1e-5)
    noisy = VortexSheddingDataset([traj], split="train", noise_std=0.1)[0]
    clean = VortexSheddingDataset([traj], split="train", noise_std=0.0)[0]
    moved = (noisy["x"][:, :2] - clean["x"][:, :2]).abs().sum(-1) > 0
    assert moved.tolist() == [True, True, False, False, True, False]  # only normal nodes are perturbed
    with pytest.raises(ValueError):
        VortexSheddingDataset([traj], split="test")


def test_mesh_transforms_and_dataset(tmp_path):
    import math

    from physicsnemo_b200.datapipes.mesh_dataset import MeshDataset, MeshReader, save_mesh_npz
    from physicsnemo_b200.datapipes.transforms.mesh import (CenterMesh, ComputeCellCentroids, ComputeSurfaceNormals, DropMeshFields,
                                                           MeshToTensorDict, NormalizeMeshFields, RandomRotateMesh, RandomScaleMesh,
                                                           RenameMeshFields, RestructureTensorDict, RotateMesh, ScaleMesh, SetGlobalField,
                                                           SubsampleMesh, TranslateMesh)
    from physicsnemo_b200.mesh import Mesh, primitives

    torch.manual_seed(0)
    base = primitives.icosphere(2)
    mesh = Mesh(base.points.float() + torch.tensor([1.0, 2.0, 3.0]), base.cells, point_data={"p": torch.randn(base.points.shape[0], 1), "u": torch.randn(base.points.shape[0], 3)})
    centred = CenterMesh()(mesh.clone())
    assert centred.points.mean(0).abs().max() < 1e-2
    rot = RotateMesh(math.pi / 2, axis="z", transform_point_data=True)(centred.clone())
    assert torch.allclose(rot.points[:, 0], -centred.points[:, 1], atol=1e-6) and torch.allclose(rot.point_data["u"][:, 1], centred.point_data["u"][:, 0], atol=1e-6)
    assert torch.allclose(rot.point_data["p"], centred.point_data["p"])                  # scalars do not rotate
    moved = TranslateMesh([1.0, 0, 0])(ScaleMesh(2.0)(centred.clone()))
    assert torch.allclose(moved.points, centred.points * 2 + torch.tensor([1.0, 0, 0]), atol=1e-6)
    sub = SubsampleMesh(n_cells=40)(centred.clone())
    assert sub.n_cells == 40 and int(sub.cells.max()) == sub.n_points - 1 and sub.point_data["p"].shape[0] == sub.n_points
    out = ComputeCellCentroids()(ComputeSurfaceNormals()(centred.clone()))
    assert (out.cell_data["normals"] * out.cell_data["centroids"]).sum(-1).min() > 0      # outward on a sphere
    norm = NormalizeMeshFields("point_data", {"p": {"mean": [0.5], "std": [2.0]}})
    scaled = norm(centred.clone())
    assert torch.allclose(norm.inverse(scaled).point_data["p"], centred.point_data["p"], atol=1e-5)
    tidy = SetGlobalField({"mach": [0.3]})(RenameMeshFields(point_data={"u": "velocity"})(DropMeshFields(point_data=["p"])(centred.clone())))
    assert set(tidy.point_data) == {"velocity"} and float(tidy.global_data["mach"]) == pytest.approx(0.3)
    td = RestructureTensorDict({"inputs": {"pos": "points"}, "targets": {"vel": "point_data.velocity"}})(MeshToTensorDict()(tidy))
    assert td["inputs"]["pos"].shape == (tidy.n_points, 3) and td["targets"]["vel"].shape == (tidy.n_points, 3)
    r = RandomRotateMesh(seed=3)
    a, b = r(centred.clone()), r(centred.clone())
    assert not torch.allclose(a.points, b.points) and torch.allclose(a.points.norm(dim=-1), centred.points.norm(dim=-1), atol=1e-5)
    for i in range(3):
        save_mesh_npz(mesh, tmp_path / f"m{i}.npz")
    ds = MeshDataset(MeshReader(tmp_path, subsample_n_cells=100), transforms=[CenterMesh(), RandomScaleMesh(seed=1)])
    assert len(ds) == 3 and ds[0].n_cells == 100 and "p" in ds[0].point_data
    ds.set_epoch(0)
    first = ds[1].points.clone()
    ds.set_epoch(0)
    assert torch.equal(ds[1].points, first)                                               # same epoch, same augmentation
    ds.set_epoch(1)
    assert not torch.equal(ds[1].points, first)


def test_transolver_datapipe_feeds_the_model():
    from physicsnemo_b200.datapipes.cae import TransolverDataPipe
    from physicsnemo_b200.mesh import primitives
    from physicsnemo_b200.models.transolver import Transolver

    torch.manual_seed(0)
    s = primitives.icosphere(3)
    V, F = s.points.float() * 0.5 + torch.tensor([2.0, 0, 0]), s.cells
    tri = V[F]
    n = torch.linalg.cross(tri[:, 1] - tri[:, 0], tri[:, 2] - tri[:, 0])
    centers, areas = tri.mean(1), 0.5 * n.norm(dim=-1)
    sample = dict(stl_coordinates=V, stl_faces=F.reshape(-1), stl_centers=centers, surface_mesh_centers=centers, surface_normals=n,
                  surface_areas=areas, surface_fields=torch.randn(centers.shape[0], 4) * 2 + 5, air_density=torch.tensor(1.2),
                  stream_velocity=torch.tensor(30.0), volume_mesh_centers=torch.rand(5000, 3) * 4, volume_fields=torch.randn(5000, 5))
    factors = {"mean": sample["surface_fields"].mean(0), "std": sample["surface_fields"].std(0)}
    pipe = TransolverDataPipe(model_type="surface", dataset=[sample], resolution=400, scaling_type="mean_std_scaling", surface_factors=factors,
                              translational_invariance=True, include_geometry=True, geometry_sampling=100)
    out = pipe[0]
    assert out["embeddings"].shape == (1, 400, 6) and out["fx"].shape == (1, 400, 2) and out["fields"].shape == (1, 400, 4)
    assert out["geometry"].shape == (1, 100, 3) and out["surface_areas_sub"].shape == (1, 400)
    assert torch.allclose(out["embeddings"][0, :, 3:].norm(dim=-1), torch.ones(400), atol=1e-5)          # unit normals
    assert out["embeddings"][0, :, :3].norm(dim=-1).max() < 0.51                                         # centred on the body
    back = pipe.unscale_model_targets(out["fields"][0])
    assert float(back.mean()) == pytest.approx(5.0, abs=0.5)
    model = Transolver(functional_dim=2, out_dim=4, embedding_dim=6, n_layers=2, n_hidden=32, n_head=4, slice_num=8, use_te=False)
    pred = model(out["fx"], out["embeddings"])
    assert pred.shape == out["fields"].shape
    vol = TransolverDataPipe(model_type="volume", dataset=[sample], resolution=300, include_sdf=True)[0]
    assert vol["embeddings"].shape == (1, 300, 7)                                                        # xyz, sdf, direction to the surface
    r = (vol["embeddings"][0, :, :3] - torch.tensor([2.0, 0, 0])).norm(dim=-1)
    assert (vol["embeddings"][0, :, 3] - (r - 0.5)).abs().max() < 5e-3
    both = TransolverDataPipe(model_type="combined", dataset=[sample], resolution=200)[0]
    assert [e.shape[1] for e in both["embeddings"]] == [200, 200]
    with pytest.raises(ValueError):
        TransolverDataPipe(model_type="surface").process_data({"stl_centers": centers})


# -------------------------------------------------------------------------------------------------- CAE dataset
def _write_cae_samples(root, layout, n=4, nvol=200, nsurf=50):
    import numpy as np

    rng = np.random.default_rng(0)
    samples = []
    for i in range(n):
        s = {"volume_mesh_centers": rng.normal(size=(nvol, 3)).astype(np.float32), "volume_fields": rng.normal(size=(nvol, 2)).astype(np.float32) + i,
             "surface_fields": rng.normal(size=(nsurf, 4)).astype(np.float32), "stl_faces": rng.integers(0, 10, size=(30,)).astype(np.int64)}
        samples.append(s)
        if layout == "npy":
            np.save(root / f"s{i}.npy", s, allow_pickle=True)
        elif layout == "npz":
            np.savez(root / f"s{i}.npz", **s)
        else:
            d = root / f"s{i}"
            d.mkdir()
            for k, v in s.items():
                np.save(d / f"{k}.npy", v)
    return samples


@pytest.mark.parametrize("layout", ["npy", "npz", "npydir"])
def test_cae_dataset_layouts_and_readahead(tmp_path, layout):
    import numpy as np

    from physicsnemo_b200.datapipes.cae import CAEDataset, compute_mean_std_min_max

    samples = _write_cae_samples(tmp_path, layout)
    keys = ["volume_mesh_centers", "volume_fields", "surface_fields", "stl_faces"]
    ds = CAEDataset(tmp_path, keys, {"air_density": torch.tensor([1.2])}, torch.device("cpu"), preload_depth=2)
    assert len(ds) == 4
    got = list(ds)                                            # iteration with read-ahead
    assert len(got) == 4
    for g, s in zip(got, samples):
        assert torch.equal(g["volume_fields"], torch.from_numpy(s["volume_fields"])) and g["stl_faces"].dtype == torch.int32
        assert torch.equal(g["air_density"], torch.tensor([1.2]))
    ds.set_indices([3, 1])
    assert [float(d["volume_fields"][0, 0]) for d in ds] == [float(samples[3]["volume_fields"][0, 0]), float(samples[1]["volume_fields"][0, 0])]
    ds.preload(2)
    assert torch.equal(ds[2]["surface_fields"], torch.from_numpy(samples[2]["surface_fields"]))
    with pytest.raises(IndexError):
        ds[7]
    if layout == "npy":
        with pytest.raises(NotImplementedError):
            ds.set_volume_sampling_size(10)
    else:
        np.random.seed(0)
        ds.set_volume_sampling_size(64)
        sub = ds[0]
        assert sub["volume_fields"].shape == (64, 2) and sub["volume_mesh_centers"].shape == (64, 3) and sub["surface_fields"].shape == (50, 4)
        # the same rows of all volume arrays, as one cyclic block of the file
        full_f, full_c = samples[0]["volume_fields"], samples[0]["volume_mesh_centers"]
        start = int(np.where((full_f == sub["volume_fields"][0].numpy()).all(1))[0][0])
        rows = (start + np.arange(64)) % 200
        assert np.array_equal(sub["volume_fields"].numpy(), full_f[rows]) and np.array_equal(sub["volume_mesh_centers"].numpy(), full_c[rows])
        ds.set_volume_sampling_size(None)
    ds2 = CAEDataset(tmp_path, ["volume_fields"], None, torch.device("cpu"))
    mean, std, lo, hi = compute_mean_std_min_max(ds2, ["volume_fields"], max_samples=4)
    allv = np.concatenate([s["volume_fields"] for s in samples]).astype(np.float64)
    assert np.allclose(mean["volume_fields"].numpy(), allv.mean(0), atol=1e-6) and np.allclose(std["volume_fields"].numpy(), allv.std(0, ddof=1), atol=1e-6)
    assert np.allclose(lo["volume_fields"].numpy(), allv.min(0), atol=1e-6) and np.allclose(hi["volume_fields"].numpy(), allv.max(0), atol=1e-6)
    ds.close(); ds2.close()
    with pytest.raises(ValueError):
        CAEDataset(tmp_path, ["not_there"], None, torch.device("cpu"))[0]
    with pytest.raises(FileNotFoundError):
        CAEDataset(tmp_path / "missing", keys, None, torch.device("cpu"))


def _surface_sample(rng, n):
    import numpy as np

    pos = rng.random((n, 3)).astype(np.float32)
    cells = np.array([[i, (i + 1) % n, (i + 2) % n] for i in range(n)])
    return dict(pos=pos, cells=cells, p=rng.random((n, 1)), wallShearStress=rng.random((n, 3)), velocity=30.0 + n,
                reynolds_number=1e6 + n, length=1000.0 + n, width=300.0, height=280.0 + n, ground_clearance=50.0 + n, slant_angle=25.0 + n,
                fillet_radius=10.0 + n)


def test_static_graph_datasets(tmp_path):
    import numpy as np

    from physicsnemo_b200.datapipes.gnn import AhmedBodyDataset, DrivAerNetDataset, StokesDataset

    rng = np.random.default_rng(0)
    train = AhmedBodyDataset(samples=[_surface_sample(rng, 20), _surface_sample(rng, 24)], stats_dir=tmp_path, compute_drag=True)
    g, case, normals, areas, coeff = train[1]
    assert g.x.shape == (24, 11) and g.y.shape == (24, 4) and g.edge_attr.shape[1] == 4
    assert float(g.y.min()) >= -1 - 1e-6 and float(g.y.max()) <= 1 + 1e-6               # min-max bounds
    assert normals.shape == (24, 3) and areas.shape == (24,) and coeff > 0
    pred, gt = train.denormalize(g.y, g.y)
    raw = torch.cat([train._raw_nodes[1]["p"], train._raw_nodes[1]["wallShearStress"]], 1)
    assert torch.allclose(pred, raw, atol=1e-5)
    valid = AhmedBodyDataset(samples=[_surface_sample(rng, 20)], split="validation", stats_dir=tmp_path)      # reuses the statistics
    assert valid[0].x.shape == (20, 11)
    with pytest.raises(IOError):
        AhmedBodyDataset(samples=[_surface_sample(rng, 20)], split="test", stats_dir=tmp_path / "nowhere")
    car = DrivAerNetDataset(samples=[dict(_surface_sample(rng, 16), c_d=0.31)])
    assert car[0].x.shape == (16, 3) and abs(float(car[0].c_d) - 0.31) < 1e-6
    flow = StokesDataset(samples=[dict(pos=rng.random((15, 2)), cells=np.array([[i, (i + 1) % 15, (i + 2) % 15] for i in range(15)]),
                                       marker=rng.integers(0, 5, 15), u=rng.random(15), v=rng.random(15), p=rng.random(15))])
    assert flow[0].x.shape == (15, 2 + 5) and flow[0].y.shape == (15, 3)


def test_lagrangian_and_hydrograph_datasets(tmp_path):
    import numpy as np

    from physicsnemo_b200.datapipes.gnn import HydroGraphDataset, LagrangianDataset

    rng = np.random.default_rng(1)
    meta = dict(dim=2, sequence_length=11, dt=0.0025, default_connectivity_radius=0.15, bounds=[[0.1, 0.9], [0.1, 0.9]],
                vel_mean=[0, 0], vel_std=[0.01, 0.01], acc_mean=[0, 0], acc_std=[0.001, 0.001])
    traj = [dict(position=(0.5 + 0.3 * rng.random((12, 30, 2))).astype(np.float32), particle_type=np.array([5] * 25 + [3] * 5))
            for _ in range(2)]
    ds = LagrangianDataset(trajectories=traj, metadata=meta, num_history=5, split="valid")
    assert len(ds) == 2 * (12 - 5 - 1)
    g = ds[3]
    assert g.x.shape == (30, 2 + 5 * 2 + 4 + 6) and g.y.shape == (30, 6) and g.edge_attr.shape[1] == 3
    pos, vel, kinds = ds.unpack_inputs(g)
    assert vel.shape == (5, 30, 2) and torch.equal(kinds.argmax(1), torch.tensor([5] * 25 + [3] * 5))
    seq = traj[0]["position"]
    want_v = (torch.as_tensor(seq[8] - seq[7]) - ds.vel_mean) / ds.vel_std               # sample 3: t = 8 is the current step
    assert torch.allclose(vel[-1], want_v, atol=1e-5) and torch.allclose(pos, torch.as_tensor(seq[8]))
    assert int(g.mask.sum()) == 25
    # hydrographs
    n, T = 40, 16
    static = dict(xy_coords=rng.random((n, 2)), **{k: rng.random(n) for k in
                                                   ("area", "elevation", "slope", "aspect", "curvature", "manning", "flow_accum", "infiltration")})
    events = [dict(water_depth=rng.random((T, n)), volume=rng.random((T, n)), precipitation=rng.random(T), inflow_hydrograph=rng.random(T))
              for _ in range(3)]
    tr = HydroGraphDataset(static=static, hydrographs=events, n_time_steps=4, k=3, stats_dir=tmp_path, return_physics=True)
    assert len(tr) == 3 * (T - 4)
    g, phys = tr[5]
    assert g.x.shape == (n, 2 + 8 + 2 + 4 + 4) and g.y.shape == (n, 2) and g.edge_attr.shape[1] == 3
    assert set(phys) >= {"flow_future", "precip_future", "past_volume", "future_volume"}
    te = HydroGraphDataset(static=static, hydrographs=events[:1], n_time_steps=4, k=3, stats_dir=tmp_path, split="test", rollout_length=6)
    g, roll = te[0]
    assert roll["water_depth"].shape == (6, n) and g.x.shape[0] == n


def test_bistride_multilayer_graph(tmp_path):
    from physicsnemo_b200.datapipes.gnn import BistrideMultiLayerGraph, BistrideMultiLayerGraphDataset, cells_to_edges
    from physicsnemo_b200.nn.module.gnn_layers.graph_types import Graph

    n = 9
    xs = torch.linspace(0, 1, n)
    X, Y = torch.meshgrid(xs, xs, indexing="ij")
    pos = torch.stack([X.reshape(-1), Y.reshape(-1)], 1)
    cells = []
    for i in range(n - 1):
        for j in range(n - 1):
            a, b, c, d = i * n + j, (i + 1) * n + j, (i + 1) * n + j + 1, i * n + j + 1
            cells += [[a, b, c], [a, c, d]]
    g = Graph(cells_to_edges(torch.tensor(cells)), num_nodes=n * n, pos=pos)
    ms = BistrideMultiLayerGraph(g, 2)
    sizes = [n * n] + [ids.numel() for ids in ms.m_ids]
    assert sizes[1] < 0.7 * sizes[0] and sizes[2] < 0.7 * sizes[1] and sizes[2] >= 4
    for level, (edges, count) in enumerate(zip(ms.m_flat_es[1:], sizes[1:])):
        assert int(edges.max()) < count and (edges[0] != edges[1]).all()
    # every node that was dropped has a surviving neighbour one hop away (the strides alternate)
    kept = torch.zeros(n * n, dtype=torch.bool)
    kept[ms.m_ids[0]] = True
    e0 = ms.m_flat_es[0]
    covered = kept.clone()
    covered[e0[0][kept[e0[1]]]] = True
    assert bool(covered.all())

    class One(torch.utils.data.Dataset):
        split = "train"

        def __len__(self):
            return 1

        def __getitem__(self, i):
            return g

    wrapped = BistrideMultiLayerGraphDataset(One(), 2, cache_dir=tmp_path)
    first, again = wrapped[0], wrapped[0]
    assert len(first["ms_edges"]) == 3 and len(first["ms_ids"]) == 2
    assert all(torch.equal(a, b) for a, b in zip(first["ms_ids"], again["ms_ids"]))


def _healpix_store(T=40, C=3, F=12, H=4):
    import numpy as np

    rng = np.random.default_rng(0)
    t0 = np.datetime64("2020-01-01T00:00:00")
    time = t0 + np.arange(T) * np.timedelta64(3, "h")
    data = rng.random((T, C, F, H, H)).astype(np.float32)
    data[:, 0] += np.arange(T, dtype=np.float32)[:, None, None, None]           # channel 0 encodes its time index
    lat = rng.uniform(-80, 80, (F, H, H)).astype(np.float32)
    lon = rng.uniform(0, 360, (F, H, H)).astype(np.float32)
    return dict(inputs=data, targets=data.copy(), time=time, lat=lat, lon=lon, constants=rng.random((2, F, H, H)).astype(np.float32),
                channel_in=np.array(["z500", "t2m", "sst"]), channel_out=np.array(["z500", "t2m", "sst"]))


def test_healpix_timeseries_dataset_shapes_and_indices():
    import numpy as np

    from physicsnemo_b200.datapipes.healpix import TimeSeriesDataset

    store = _healpix_store()
    scaling = {k: {"mean": 0.0, "std": 1.0} for k in ("z500", "t2m", "sst")}
    ds = TimeSeriesDataset(store, scaling, input_time_dim=2, output_time_dim=2, data_time_step="3h", time_step="6h", batch_size=4,
                           add_insolation=True)
    window = 2 * 1 + 1 + 2 + 2                                                   # (T_in-1)*2 + 1 + gap 2 + (T_out-1)*2
    assert ds._window_length == window and len(ds) == int(np.ceil((40 - window + 1) / 4))
    (x, sol, const), y = ds[1]
    assert x.shape == (4, 12, 2, 3, 4, 4) and y.shape == (4, 12, 2, 3, 4, 4)
    assert sol.shape == (4, 12, 4, 1, 4, 4) and const.shape == (12, 2, 4, 4)
    t_in = np.round(x[:, 0, :, 0, 0, 0] - store["inputs"][0, 0, 0, 0, 0] % 1).astype(int)
    first = np.floor(x[:, 0, :, 0, 0, 0]).astype(int)
    assert (first == np.array([[4, 6], [5, 7], [6, 8], [7, 9]])).all()           # batch 1 starts at time index 4, stride 2
    assert (np.floor(y[:, 0, :, 0, 0, 0]).astype(int) == np.array([[8, 10], [9, 11], [10, 12], [11, 13]])).all()
    last_inputs, _ = ds[len(ds) - 1]
    assert 1 <= last_inputs[0].shape[0] <= 4                                     # ragged last batch unless drop_last
    fc = TimeSeriesDataset(store, scaling, input_time_dim=2, output_time_dim=2, batch_size=4,
                           forecast_init_times=[store["time"][10], store["time"][20]])
    assert len(fc) == 2 and fc[0][0].shape == (1, 12, 2, 3, 4, 4)
    assert np.floor(fc[1][0][0, 0, :, 0, 0, 0]).astype(int).tolist() == [18, 20]  # history ends at the initial time
    del t_in


def test_healpix_coupled_dataset_and_couplers():
    import numpy as np

    from physicsnemo_b200.datapipes.healpix import ConstantCoupler, CoupledTimeSeriesDataset, TrailingAverageCoupler

    store = _healpix_store()
    scaling = {k: {"mean": 0.0, "std": 1.0} for k in ("z500", "t2m", "sst")}
    coupler = TrailingAverageCoupler(store, batch_size=3, variables=["z500"], input_time_dim=2, output_time_dim=2,
                                     input_times=["6h", "12h"], averaging_window="6h")
    ds = CoupledTimeSeriesDataset(store, ["t2m", "sst"], ["t2m"], scaling, input_time_dim=2, output_time_dim=2, batch_size=3,
                                  couplings=[coupler])
    (x, const, coupled), y = ds[0]
    assert x.shape == (3, 12, 2, 2, 4, 4) and y.shape == (3, 12, 2, 1, 4, 4)
    assert coupled.shape == (1, 3, 2, 12, 4, 4)                                  # [integration steps, B, var x lead, F, H, W]
    # z500 carries its time index: offsets are b + (T_in * i + 1) * interval + lead / dt
    assert np.floor(coupled[0, :, :, 0, 0, 0]).astype(int).tolist() == [[4, 6], [5, 7], [6, 8]]

    class Ocean:
        output_variables = ["z500", "other"]
        time_step = "6h"

    coupler.setup_coupling(Ocean())
    fields = torch.arange(4.0).reshape(1, 1, 4, 1, 1, 1).expand(1, 12, 4, 2, 4, 4)      # time index as value
    coupler.set_coupled_fields(fields)
    preset = coupler.construct_integrated_couplings()
    assert preset.shape == (1, 1, 2, 12, 4, 4)
    assert preset[0, 0, :, 0, 0, 0].tolist() == [0.0, 1.0]                        # windows [0:1] and [1:2] of the other model's steps
    const_c = ConstantCoupler(store, batch_size=3, variables=["sst"], input_time_dim=2, output_time_dim=2, input_times=["6h"])
    const_c.compute_coupled_indices(2, "3h")
    got = const_c.construct_integrated_couplings({"time": slice(5, 20)}, 2)
    assert got.shape == (1, 2, 1, 12, 4, 4)
    assert np.allclose(got[0, 0, 0], store["inputs"][5 + 2, 2])


def test_healpix_data_modules(tmp_path):
    import numpy as np

    from physicsnemo_b200.datapipes.healpix import (ArrayStore, CoupledTimeSeriesDataModule, TimeSeriesDataModule,
                                                    create_time_series_dataset_classic,
                                                    open_time_series_dataset_classic_prebuilt)

    src, dst = tmp_path / "src", tmp_path / "dst"
    src.mkdir()
    n_t = 60
    time = np.datetime64("2020-01-01T00") + np.arange(n_t) * np.timedelta64(3, "h")
    rng = np.random.default_rng(0)
    fields = {v: (rng.normal(size=(n_t, 12, 4, 4)) + i).astype(np.float32) for i, v in enumerate(("z500", "t2m", "sst"))}
    for v, a in fields.items():
        np.save(src / f"era5_{v}.npy", a)
    np.save(src / "era5_lsm.npy", rng.random((12, 4, 4)).astype(np.float32))
    np.savez(src / "era5_coords.npz", time=time, lat=rng.random((12, 4, 4)), lon=rng.random((12, 4, 4)))
    scaling = {v: {"mean": float(i), "std": 2.0} for i, v in enumerate(("z500", "t2m", "sst"))}
    path = create_time_series_dataset_classic(str(src), str(dst), "ds", ["z500", "t2m", "sst"], ["t2m"], {"lsm": "land_sea_mask"},
                                              prefix="era5_", scaling=scaling)
    store = open_time_series_dataset_classic_prebuilt(str(dst), "ds", constants=True)
    assert store.inputs.shape == (n_t, 3, 12, 4, 4) and store.targets.shape == (n_t, 1, 12, 4, 4) and store.channel_c == ["land_sea_mask"]
    sub = store.sel(channel_in=["sst", "z500"], time=slice("2020-01-02", "2020-01-03T21"))
    assert sub.inputs.shape == (16, 2, 12, 4, 4) and sub.time[0] == np.datetime64("2020-01-02T00") and sub.channel_in == ["sst", "z500"]
    assert np.array_equal(sub.inputs[2:4], np.stack([fields["sst"], fields["z500"]], 1)[10:12])
    with pytest.raises(KeyError):
        store.sel(channel_in=["u10"])
    with pytest.raises(FileNotFoundError):
        open_time_series_dataset_classic_prebuilt(str(dst), "missing")
    splits = dict(train_date_start="2020-01-01", train_date_end="2020-01-04T21", val_date_start="2020-01-05",
                  val_date_end="2020-01-06T21", test_date_start="2020-01-07", test_date_end="2020-01-08T09")
    dm = TimeSeriesDataModule(str(src), str(dst), "ds", prefix="era5_", batch_size=4, input_variables=["t2m", "z500"],
                              output_variables=["t2m"], constants={"lsm": "land_sea_mask"}, scaling=scaling, splits=splits,
                              input_time_dim=2, output_time_dim=2, num_workers=0, shuffle=False)
    assert os.path.samefile(path, dst / "ds")
    assert len(dm.train_dataset.ds.time) == 32 and len(dm.val_dataset.ds.time) == 16 and len(dm.test_dataset.ds.time) == 12
    loader, sampler = dm.train_dataloader()
    (x, *_), y = next(iter(loader))
    assert sampler is None and tuple(x.shape[:4]) == (4, 12, 2, 2) and tuple(y.shape[:4]) == (4, 12, 2, 1)
    want = (fields["t2m"][0] - 1.0) / 2.0                                       # first sample, first input step, scaled
    assert np.allclose(np.asarray(x)[0, :, 0, 0], want, atol=1e-6)
    assert dm.get_constants().shape == (12, 1, 4, 4)
    sharded, s2 = dm.val_dataloader(num_shards=2, shard_id=1)
    assert s2 is not None and len(list(sharded)) == len(s2)
    forecast = TimeSeriesDataModule(dataset=store, input_variables=["z500"], output_variables=["t2m"], scaling=scaling, batch_size=2,
                                    input_time_dim=1, output_time_dim=1, num_workers=0,
                                    forecast_init_times=[np.datetime64("2020-01-02T00"), np.datetime64("2020-01-03T12")])
    assert forecast.train_dataset is None and len(forecast.test_dataset) == 2
    coupled = CoupledTimeSeriesDataModule(dataset=ArrayStore({"inputs": np.stack(list(fields.values()), 1), "time": time,
                                                              "lat": np.zeros((12, 4, 4)), "lon": np.zeros((12, 4, 4)),
                                                              "channel_in": np.asarray(["z500", "t2m", "sst"])}),
                                          input_variables=["t2m"], output_variables=["t2m"], scaling=scaling, splits=splits,
                                          batch_size=3, input_time_dim=2, output_time_dim=2, num_workers=0,
                                          couplings=[{"coupler": "ConstantCoupler",
                                                      "params": {"batch_size": 3, "variables": ["sst"], "input_times": ["6h"]}}])
    assert coupled._archive_variables() == ["t2m", "sst"] and len(coupled.train_dataset) > 0
    with pytest.raises(ValueError):
        TimeSeriesDataModule(dataset=store, data_format="zarr")

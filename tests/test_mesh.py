"""Mesh geometry / topology / calculus / generators / IO (CPU) and the BVH kernels against all-pairs search (GPU)."""
import math

import pytest
import torch

from physicsnemo_b200.mesh import DomainMesh, Mesh, io, operations as O, primitives as P, spatial as S
from physicsnemo_b200.mesh import primitives
from physicsnemo_b200.nn.functional.geometry import ray_mesh_intersect, signed_distance_field


def test_geometry_and_topology():
    s = P.icosphere(3)
    assert s.n_manifold_dims == 2 and s.codimension == 1
    assert abs(float(s.cell_areas.sum()) - 4 * math.pi) < 0.1
    assert (s.cell_normals * s.cell_centroids).sum(-1).min() > 0.9               # outward
    assert (s.point_normals * s.points).sum(-1).min() > 0.99
    rep = O.validate(s)
    assert rep["is_watertight"] and rep["euler_characteristic"] == 2 and rep["n_boundary_facets"] == 0
    assert O.validate(P.torus())["euler_characteristic"] == 0
    assert abs(float(O.enclosed_volume(s)) - 4 / 3 * math.pi) < 0.05
    assert abs(float(O.enclosed_volume(P.cube_surface(3))) - 1.0) < 1e-5
    g = P.unit_square(4)
    assert g.get_boundary_mesh().n_cells == 16 and g.to_edge_graph().n_cells == 16 * 2 + 16 + 8
    nb = g.facet_neighbors()
    assert (nb >= 0).sum() == 2 * (g.to_edge_graph().n_cells - 16)
    c2c = g.get_cell_to_cells_adjacency()
    assert int(c2c.counts().max()) == 3 and c2c.n_sources == g.n_cells
    p2p = g.get_point_to_points_adjacency()
    assert int(p2p.counts().min()) >= 2
    assert g.to_dual_graph().n_points == g.n_cells
    b = P.box_volume(2, 3, 2)
    assert abs(float(b.cell_areas.sum()) - 1.0) < 1e-6 and (torch.linalg.det(b.points[b.cells[:, 1:]] - b.points[b.cells[:, :1]]) > 0).all()
    assert O.validate(b.get_boundary_mesh())["is_watertight"]
    with pytest.raises(ValueError):
        b.cell_normals
    with pytest.raises(ValueError):
        Mesh(torch.zeros(3, 2), torch.tensor([[0, 1, 5]]))


def test_data_and_editing():
    g = P.unit_square(6)
    g = g.with_data(point_data={"f": g.points[:, 0] ** 2 + 3 * g.points[:, 1], "v": g.points.clone()}, cell_data={"c": g.cell_centroids[:, 0]})
    grad = g.gradient("f")
    interior = ((g.points > 0.01) & (g.points < 0.99)).all(-1)
    assert torch.allclose(grad[interior, 0], 2 * g.points[interior, 0], atol=1e-4) and torch.allclose(grad[interior, 1], torch.full_like(grad[interior, 1], 3.0), atol=1e-4)
    assert torch.allclose(g.laplacian("f")[interior], torch.full((int(interior.sum()),), 2.0), atol=1e-3)
    assert torch.allclose(g.divergence("v")[interior], torch.full((int(interior.sum()),), 2.0), atol=1e-4)
    assert g.curl("v")[interior].abs().max() < 1e-4
    assert torch.allclose(g.point_data_to_cell_data().cell_data["f"], g.point_data["f"][g.cells].mean(1))
    p = g.cell_data_to_point_data().point_data["c"]
    assert p.shape == (g.n_points,) and 0 <= p.min() and p.max() <= 1
    half = g.slice_points(torch.nonzero(g.points[:, 0] <= 0.5).squeeze(1))
    assert half.n_points == 4 * 7 and half.n_cells == 3 * 6 * 2 and half.point_data["f"].shape[0] == half.n_points
    merged = Mesh.merge([g, g.translate([1.0, 0.0])])
    assert merged.n_points == 2 * g.n_points
    welded = merged.clean(tolerance=1e-6)
    assert welded.n_points == 2 * g.n_points - 7 and welded.n_cells == merged.n_cells
    sub = g.subdivide(1)
    assert sub.n_cells == 4 * g.n_cells and abs(float(sub.cell_areas.sum()) - 1.0) < 1e-6 and "f" in sub.point_data
    assert P.single_tetrahedron().subdivide(2).n_cells == 64
    pts, cell = g.sample_points(500, generator=torch.Generator().manual_seed(0))
    assert pts.shape == (500, 2) and pts.min() >= 0 and pts.max() <= 1
    smooth = O.laplacian_smooth(P.perturb(g, 0.02, generator=torch.Generator().manual_seed(0)), iterations=20)
    assert smooth.quality_metrics["shape_quality"].min() > P.perturb(g, 0.02, generator=torch.Generator().manual_seed(0)).quality_metrics["shape_quality"].min()
    r = g.rotate(math.pi / 2)
    assert torch.allclose(r.points[:, 0], -g.points[:, 1], atol=1e-6)
    assert g.pad_to_next_power(2.0).n_points == 64
    dec = O.cluster_decimate(P.icosphere(3), 0.5)
    assert 0 < dec.n_points < 642
    flipped = Mesh(g.points, torch.cat([g.cells[:10].flip(1), g.cells[10:]]))
    fixed = O.orient_consistently(flipped)
    n = torch.linalg.det(fixed.points[fixed.cells[:, 1:]] - fixed.points[fixed.cells[:, :1]])
    assert (n > 0).all() or (n < 0).all()


def test_curvature_and_domain(tmp_path):
    s = P.icosphere(3, radius=2.0)
    K, H = s.gaussian_curvature_vertices, s.mean_curvature_vertices
    assert abs(float(K.mean()) - 0.25) < 0.01 and abs(float(H.mean()) - 0.5) < 0.01
    assert abs(float((K * O.vertex_areas(s)).sum()) - 4 * math.pi) < 1e-3          # Gauss-Bonnet
    d = DomainMesh.from_interior(P.box_volume(2, 2, 2))
    d2 = d.split_boundary("boundary", lambda c: c[:, 0] < 1e-6, ("inlet", "walls"))
    assert set(d2.boundary_names) == {"inlet", "walls"} and d2.boundaries["inlet"].n_cells == 8
    for name, writer, reader in (("m.obj", io.write_obj, io.read_obj), ("m.stl", io.write_stl, io.read_stl)):
        writer(s, tmp_path / name)
        back = reader(tmp_path / name)
        assert back.n_cells == s.n_cells and abs(float(back.cell_areas.sum() - s.cell_areas.sum())) < 1e-3
    s.save(tmp_path / "m.pt")
    assert Mesh.load(tmp_path / "m.pt").n_points == s.n_points


def test_sdf_and_rays_torch():
    s = P.icosphere(3)
    q = torch.randn(200, 3) * 0.8
    for wn in (False, True):
        sdf, cp, face = signed_distance_field(s.points, s.cells, q, use_sign_winding_number=wn)
        assert (sdf - (q.norm(dim=-1) - 1)).abs().max() < 0.02 and face.min() >= 0
        assert ((cp - q).norm(dim=-1) - sdf.abs()).abs().max() < 1e-5
    far = signed_distance_field(s.points, s.cells, torch.tensor([[10.0, 0, 0]]), max_dist=1.0)
    assert torch.isnan(far[0]).all() and int(far[2]) == -1
    o = torch.tensor([[0.0, 0, -3], [3.0, 0, -3], [0.2, 0.1, -3]])
    d = torch.tensor([[0.0, 0, 2], [0, 0, 1.0], [0, 0, 1.0]])
    hit, t, pt, face, n = ray_mesh_intersect(s.points, s.cells, o, d)
    assert hit.tolist() == [True, False, True] and abs(float(t[0]) - 2.0) < 0.01 and torch.isinf(t[1]) and int(face[1]) == -1
    assert (n[0] * torch.tensor([0.0, 0, -1])).sum() > 0.99 and pt[1].abs().sum() == 0
    bvh = S.BVH(s.points, s.cells)
    assert bvh.n_leaves == 2048 and bvh.bounds.shape == (4095, 2, 3)
    assert torch.allclose(bvh.bounds[0, 0], s.points.amin(0)) and torch.allclose(bvh.bounds[0, 1], s.points.amax(0))


@pytest.mark.gpu
def test_bvh_kernels_match_all_pairs():
    dev = "cuda"
    m = P.lumpy_sphere(4, generator=torch.Generator().manual_seed(0)).to(dev)
    q = (torch.rand(20000, 3, device=dev) - 0.5) * 3
    for wn in (False, True):
        a = signed_distance_field(m.points, m.cells, q, use_sign_winding_number=wn, implementation="cuda")
        b = signed_distance_field(m.points, m.cells, q, use_sign_winding_number=wn, implementation="torch")
        assert (a[0] - b[0]).abs().max() < 1e-4 and (a[1] - b[1]).abs().max() < 1e-3
        # closest points on shared edges / vertices belong to several faces: check the reported face holds the point
        tri = m.points[m.cells[a[2]]]
        nrm = torch.linalg.cross(tri[:, 1] - tri[:, 0], tri[:, 2] - tri[:, 0])
        nrm = nrm / nrm.norm(dim=-1, keepdim=True)
        assert ((a[1] - tri[:, 0]) * nrm).sum(-1).abs().max() < 1e-4
        lo, hi = tri.amin(1) - 1e-4, tri.amax(1) + 1e-4
        assert ((a[1] >= lo) & (a[1] <= hi)).all()
    near = signed_distance_field(m.points, m.cells, q, max_dist=0.05, implementation="cuda")
    assert torch.isnan(near[0]).any() and (near[0][~torch.isnan(near[0])].abs() <= 0.05 + 1e-6).all()
    o = torch.cat([(torch.rand(5000, 2, device=dev) - 0.5) * 3, torch.full((5000, 1), -3.0, device=dev)], 1)
    d = torch.tensor([0.0, 0, 1], device=dev).expand(5000, 3) + 0.1 * torch.randn(5000, 3, device=dev)
    ha = ray_mesh_intersect(m.points, m.cells, o, d, implementation="cuda")
    hb = ray_mesh_intersect(m.points, m.cells, o, d, implementation="torch")
    agree = ha[0] == hb[0]
    assert agree.float().mean() > 0.999
    both = ha[0] & hb[0]
    assert (ha[1][both] - hb[1][both]).abs().max() < 1e-3 and (ha[2][both] - hb[2][both]).abs().max() < 1e-3
    out = ray_mesh_intersect(m.points, m.cells, o, d, return_bvh=True)
    again = ray_mesh_intersect(m.points, m.cells, o, d, bvh=out[-1])
    assert torch.equal(out[3], again[3])


# ---- generation, repair, tessellation ------------------------------------------------------------------------------------
def test_marching_cubes_sphere_is_watertight_and_outward():
    import math

    from physicsnemo_b200.mesh.generate import marching_cubes, project_to_zero_set, sdf_box, sdf_difference, sdf_sphere

    ax = torch.linspace(-1, 1, 33)
    grid = torch.stack(torch.meshgrid(ax, ax, ax, indexing="ij"), -1)
    phi = sdf_sphere([0.1, 0.0, -0.1], 0.6)
    m = marching_cubes(phi(grid), 0.0, (ax, ax, ax))
    e = torch.cat([m.cells[:, [0, 1]], m.cells[:, [1, 2]], m.cells[:, [2, 0]]])
    _, cnt = torch.unique(e.sort(1).values, dim=0, return_counts=True)
    assert cnt.unique().tolist() == [2] and torch.unique(e, dim=0).shape[0] == e.shape[0]      # closed, consistently oriented
    assert m.n_points - cnt.shape[0] + m.n_cells == 2                                             # sphere topology
    assert (phi(m.points).abs().max()) < 5e-3
    p = m.points - torch.tensor([0.1, 0.0, -0.1])
    vol = float((p[m.cells[:, 0]] * torch.linalg.cross(p[m.cells[:, 1]], p[m.cells[:, 2]])).sum() / 6)
    assert vol == pytest.approx(4 / 3 * math.pi * 0.6 ** 3, rel=0.02)                             # positive: normals point outward
    on = project_to_zero_set(phi, m.points + 0.05 * torch.randn_like(m.points))
    assert phi(on).abs().max() < 1e-5
    shell = sdf_difference(sdf_box([-0.5] * 3, [0.5] * 3), sdf_sphere([0, 0, 0], 0.3))
    assert float(shell(torch.zeros(1, 3))) > 0 and float(shell(torch.tensor([[0.4, 0.4, 0.4]]))) < 0
    idx = marching_cubes(phi(grid))                                                               # index space without coords
    assert float(idx.points.max()) <= 32
    assert marching_cubes(torch.ones(4, 4, 4)).n_cells == 0


def test_fill_holes_and_degenerate_removal():
    from physicsnemo_b200.mesh import primitives
    from physicsnemo_b200.mesh.repair import fill_holes, remove_degenerate_cells

    s = primitives.icosphere(2)
    keep = torch.ones(s.n_cells, dtype=torch.bool)
    keep[[3, 100]] = False                                        # two separate triangular holes
    holed = s.slice_cells(keep.nonzero().squeeze(1))
    filled, stats = fill_holes(holed)
    assert stats["n_holes_detected"] == 2 and stats["n_holes_filled"] == 2 and stats["n_faces_added"] == 6
    e = torch.cat([filled.cells[:, [0, 1]], filled.cells[:, [1, 2]], filled.cells[:, [2, 0]]])
    assert torch.unique(e.sort(1).values, dim=0, return_counts=True)[1].unique().tolist() == [2]
    assert torch.unique(e, dim=0).shape[0] == e.shape[0]          # orientation of the patches matches the surface
    _, skipped = fill_holes(holed, max_hole_edges=2)
    assert skipped["n_holes_skipped"] == 2
    bad = torch.cat([s.cells, torch.tensor([[0, 0, 1]])])
    cleaned, info = remove_degenerate_cells(type(s)(s.points, bad))
    assert info["n_cells_removed"] == 1 and cleaned.n_cells == s.n_cells


def test_tessellation_polygons_and_delaunay():
    from physicsnemo_b200.mesh.tessellation import delaunay_mesh_2d, ear_clip, fill_interior, triangulate

    L = torch.tensor([[0.0, 0], [2, 0], [2, 1], [1, 1], [1, 2], [0, 2]])          # non-convex L shape, area 3
    tris = ear_clip(L.numpy())
    area = sum(0.5 * abs(float((L[b] - L[a])[0] * (L[c] - L[a])[1] - (L[b] - L[a])[1] * (L[c] - L[a])[0])) for a, b, c in tris)
    assert len(tris) == 4 and area == pytest.approx(3.0)
    m = triangulate(torch.cat([L, torch.zeros(6, 1)], 1), [[0, 1, 2, 3, 4, 5]])
    assert m.n_cells == 4 and float(m.cell_areas.sum()) == pytest.approx(3.0)
    torch.manual_seed(0)
    d = delaunay_mesh_2d(torch.rand(40, 2))
    assert d.n_cells > 40 and float(d.cell_areas.min()) > 0
    filled = fill_interior(L, [[0, 1, 2, 3, 4, 5]], spacing=0.25)
    assert float(filled.cell_areas.sum()) == pytest.approx(3.0, rel=1e-6) and filled.n_points > 20


def _grid_mesh(n=6):
    from physicsnemo_b200.mesh.mesh import Mesh

    xs = torch.linspace(0, 1, n)
    X, Y = torch.meshgrid(xs, xs, indexing="ij")
    pts = torch.stack([X.reshape(-1), Y.reshape(-1)], 1)
    cells = []
    for i in range(n - 1):
        for j in range(n - 1):
            a, b, c, d = i * n + j, (i + 1) * n + j, (i + 1) * n + j + 1, i * n + j + 1
            cells += [[a, b, c], [a, c, d]]
    return Mesh(pts, torch.tensor(cells))


def test_mesh_calculus_is_exact_for_linear_fields():
    from physicsnemo_b200.mesh import calculus as K

    m = _grid_mesh()
    p = m.points
    g = K.gradient(m, 2 * p[:, 0] + 3 * p[:, 1])
    assert torch.allclose(g, torch.tensor([2.0, 3.0]).expand_as(g), atol=1e-5)
    assert torch.allclose(K.divergence(m, p), torch.full((m.n_points,), 2.0), atol=1e-5)
    assert torch.allclose(K.curl(m, torch.stack([-p[:, 1], p[:, 0]], 1)), torch.full((m.n_points,), 2.0), atol=1e-5)
    assert abs(float(K.integrate(m, torch.ones(m.n_points))) - 1.0) < 1e-6
    assert abs(float(K.integrate(m, p[:, 0])) - 0.5) < 1e-5                      # ∫ x over the unit square
    # a surface in 3-D: the gradient of z on a tilted plane lies in the plane
    from physicsnemo_b200.mesh.mesh import Mesh

    tilt = torch.stack([p[:, 0], p[:, 1], 0.5 * p[:, 0]], 1)
    s = Mesh(tilt, m.cells)
    gz = K.gradient(s, tilt[:, 2], at="cells")
    normal = torch.tensor([-0.5, 0.0, 1.0]) / (1.25 ** 0.5)
    assert float((gz @ normal).abs().max()) < 1e-5 and torch.allclose(gz.norm(dim=1), torch.full((s.n_cells,), 0.5 / 1.25 ** 0.5), atol=1e-5)


def test_mesh_subdivision_linear_and_loop():
    from physicsnemo_b200.mesh import subdivide_linear, subdivide_loop
    from physicsnemo_b200.mesh.mesh import Mesh
    from physicsnemo_b200.mesh.operations import validate

    m = _grid_mesh(4)
    m.point_data["f"] = m.points[:, 0].clone()
    m.cell_data["id"] = torch.arange(m.n_cells)
    fine = subdivide_linear(m, 2)
    assert fine.n_cells == 16 * m.n_cells and abs(float(fine.cell_areas.sum()) - 1.0) < 1e-5
    assert torch.allclose(fine.point_data["f"], fine.points[:, 0], atol=1e-6)      # linear data stays linear
    assert torch.equal(fine.cell_data["id"][::16], m.cell_data["id"])
    octa = Mesh(torch.tensor([[1.0, 0, 0], [-1, 0, 0], [0, 1, 0], [0, -1, 0], [0, 0, 1], [0, 0, -1]]),
                torch.tensor([[0, 2, 4], [2, 1, 4], [1, 3, 4], [3, 0, 4], [2, 0, 5], [1, 2, 5], [3, 1, 5], [0, 3, 5]]))
    smooth = subdivide_loop(octa, 3)
    report = validate(smooth)
    assert report["is_watertight"] and report["is_manifold"] and report["euler_characteristic"] == 2
    radii = smooth.points.norm(dim=1)
    assert float(radii.max() - radii.min()) < 0.1                                   # the octahedron rounds to a near-sphere
    flat = subdivide_loop(_grid_mesh(4), 1)                                         # boundary rule keeps a square a square
    assert abs(float(flat.cell_areas.sum()) - 1.0) < 0.05 and float(flat.points.min()) >= -1e-6


def test_boundary_detection_and_topology_checks():
    from physicsnemo_b200.mesh import boundaries as B

    sq = primitives.unit_square(4)
    assert int(B.get_boundary_vertices(sq).sum()) == 16 and B.get_boundary_edges(sq).shape == (16, 2)
    assert int(B.get_boundary_cells(sq).sum()) == 14            # two corner triangles own two boundary edges each
    assert int(B.get_boundary_cells(sq, boundary_codimension=2).sum()) == 2      # the two corners with a single triangle
    assert not B.is_watertight(sq) and B.is_manifold(sq)
    sphere = primitives.icosphere(1)
    assert B.is_watertight(sphere) and B.is_manifold(sphere) and B.get_boundary_edges(sphere).shape == (0, 2)
    assert not bool(B.get_boundary_vertices(sphere).any())
    box = primitives.box_volume(2, 2, 2)
    assert int(B.get_boundary_vertices(box).sum()) == 26 and B.is_manifold(box)
    edges = B.get_boundary_edges(box)                            # edges of the 48 boundary triangles: V - E + F = 2
    assert 26 - edges.shape[0] + 48 == 2
    bow_tie = Mesh(torch.tensor([[0.0, 0], [1, 0], [0, 1], [-1, 0], [0, -1]]), torch.tensor([[0, 1, 2], [0, 3, 4]]))
    assert B.is_manifold(bow_tie, "facets") and not B.is_manifold(bow_tie)
    fin = Mesh(torch.tensor([[0.0, 0, 0], [1, 0, 0], [0, 1, 0], [0, -1, 0], [0, 0, 1]]),
               torch.tensor([[0, 1, 2], [0, 1, 3], [0, 1, 4]]))         # three triangles on one edge
    assert not B.is_manifold(fin, "facets")
    with pytest.raises(ValueError):
        B.get_boundary_cells(sq, boundary_codimension=3)


def test_embed_project_extrude():
    from physicsnemo_b200.mesh import boundaries as B
    from physicsnemo_b200.mesh.projections import embed, extrude, project

    sq = primitives.unit_square(3).with_data(point_data={"v": torch.rand(16, 2), "s": torch.rand(16)},
                                             cell_data={"c": torch.arange(18.0)})
    up = embed(sq, 3)
    assert up.n_spatial_dims == 3 and float(up.points[:, 2].abs().max()) == 0 and embed(sq, 2) is sq
    mid = embed(sq, 3, insert_at=1)
    assert torch.equal(mid.points[:, [0, 2]], sq.points) and float(mid.points[:, 1].abs().max()) == 0
    back = project(up, 2)
    assert torch.equal(back.points, sq.points) and project(up, keep_dims=[0, 1, 2]) is up
    lifted = up.with_data(point_data={"w": torch.rand(16, 3)})
    flat = project(lifted, keep_dims=[2, 0], transform_point_data=True)
    assert flat.n_spatial_dims == 2 and torch.equal(flat.point_data["w"], lifted.point_data["w"][:, [2, 0]])
    with pytest.raises(ValueError):
        project(up, 1)                                            # below the manifold dimension
    with pytest.raises(ValueError):
        embed(up, 2)
    with pytest.raises(ValueError):
        project(up, 2, keep_dims=[0, 1])
    slab = extrude(sq, [0.0, 0.0, 0.5], allow_new_spatial_dims=True)
    assert slab.n_manifold_dims == 3 and slab.n_cells == 3 * sq.n_cells and slab.n_points == 2 * sq.n_points
    assert abs(float(slab.cell_areas.sum()) - 0.5) < 1e-6 and B.is_manifold(slab)
    rel = slab.points[slab.cells[:, 1:]] - slab.points[slab.cells[:, :1]]
    assert bool((torch.det(rel) > 0).all())
    assert torch.equal(slab.cell_data["c"], sq.cell_data["c"].repeat(3)) and slab.point_data["s"].shape == (32,)
    band = extrude(embed(primitives.circle(24), 3))       # closed curve → open tube of height 1
    assert band.n_manifold_dims == 2 and band.n_spatial_dims == 3 and B.get_boundary_edges(band).shape[0] == 48
    with pytest.raises(ValueError):
        extrude(sq)
    with pytest.raises(NotImplementedError):
        extrude(sq, capping=True)


def test_further_primitives():
    from physicsnemo_b200.mesh import boundaries as B

    closed = {"tetrahedron_surface": 8 / math.sqrt(3), "octahedron_surface": 4 * math.sqrt(3), "icosahedron_surface": None,
              "cone": None}
    for name, area in closed.items():
        m = getattr(primitives, name)()
        assert B.is_watertight(m) and B.is_manifold(m), name
        assert float(m.cell_normals.mul(m.cell_centroids - m.points.mean(0)).sum(1).min()) > 0, name   # outward faces
        if area is not None:
            assert abs(float(m.cell_areas.sum()) - area) < 1e-4
    assert abs(float(primitives.cone(64, 8).cell_areas.sum()) - math.pi * (math.sqrt(5) + 1)) < 0.05
    assert abs(float(primitives.hemisphere(16, 64).cell_areas.sum()) - 2 * math.pi) < 0.05
    assert abs(float(primitives.annulus().cell_areas.sum()) - math.pi * 0.75) < 0.03
    assert abs(float(primitives.circular_arc(64).cell_areas.sum()) - math.pi / 2) < 1e-3
    assert abs(float(primitives.cylinder_volume(4, 32, 4).cell_areas.sum()) - 2 * math.pi) < 0.1
    strip = primitives.mobius_strip()
    assert B.is_manifold(strip) and not B.is_watertight(strip)
    loops = B.get_boundary_edges(strip)                          # one boundary loop of twice the circumference count
    assert loops.shape[0] == 2 * 64 and orient_consistently_fails(strip)
    grid = primitives.perturbed_grid(8, 8, 0.3, generator=torch.Generator().manual_seed(0))
    assert abs(float(grid.cell_areas.sum()) - 1.0) < 1e-5
    for name in ("three_points", "three_edges", "line_segments_1d", "spline", "equilateral_triangle", "sphere_volume",
                 "tetrahedron_volume", "lumpy_ball", "cylinder_open"):
        m = getattr(primitives, name)()
        assert m.n_cells > 0 and B.is_manifold(m), name
    ring = primitives.spline(torch.tensor([[1.0, 0, 0], [0, 1, 0], [-1, 0, 0], [0, -1, 0]]), 40, closed=True)
    assert ring.n_cells == 40 and not bool(B.get_boundary_vertices(ring).any())
    bumpy = primitives.noisy_mesh(primitives.icosphere(2), amplitude=0.1)
    radii = bumpy.points.norm(dim=1)
    assert float(radii.std()) > 1e-3 and float((radii - 1).abs().max()) <= 0.1 + 1e-6


def orient_consistently_fails(mesh) -> bool:
    """A one-sided surface admits no consistent orientation: some neighbouring pair keeps traversing a shared edge the same way."""
    from physicsnemo_b200.mesh.operations import orient_consistently

    c = orient_consistently(mesh).cells
    directed = torch.cat([c[:, [0, 1]], c[:, [1, 2]], c[:, [2, 0]]])
    key = directed[:, 0] * mesh.n_points + directed[:, 1]
    return bool((torch.unique(key, return_counts=True)[1] > 1).any())


def test_angles_dual_volumes_and_cotangent_weights():
    from physicsnemo_b200.mesh import geometry as G

    a = torch.tensor([[1.0, 0, 0], [1.0, 1e-9, 0], [-1.0, 1e-9, 0]])
    b = torch.tensor([[0.0, 2, 0], [1.0, 0, 0], [1.0, 0, 0]])
    ang = G.stable_angle_between_vectors(a.double(), b.double())
    assert torch.allclose(ang, torch.tensor([math.pi / 2, 1e-9, math.pi - 1e-9], dtype=torch.float64), atol=1e-12)
    grid = primitives.perturbed_grid(6, 6, 0.3, generator=torch.Generator().manual_seed(1))
    sums = G.compute_vertex_angle_sums(grid)
    from physicsnemo_b200.mesh.boundaries import get_boundary_vertices
    inner = ~get_boundary_vertices(grid)
    assert torch.allclose(sums[inner], torch.full_like(sums[inner], 2 * math.pi), atol=1e-5)
    assert abs(float(sums.sum()) - math.pi * grid.n_cells) < 1e-3
    # dual volumes tile the mesh, with obtuse triangles included
    sliver = Mesh(torch.tensor([[0.0, 0], [4, 0], [2, 0.3], [2, -3]]), torch.tensor([[0, 1, 2], [0, 3, 1]]))
    for m in (grid, sliver, primitives.icosphere(2), primitives.box_volume(2, 2, 2), primitives.circle(12)):
        assert abs(float(G.compute_dual_volumes_0(m).sum() - m.cell_areas.sum())) < 1e-4 * float(m.cell_areas.sum())
    assert torch.allclose(G.compute_dual_volumes_0(sliver)[2], sliver.cell_areas[0] / 2)       # the obtuse corner
    right = Mesh(torch.tensor([[0.0, 0], [2, 0], [0, 2]]), torch.tensor([[0, 1, 2]]))
    assert torch.allclose(G.compute_dual_volumes_0(right), torch.tensor([1.0, 0.5, 0.5]))      # circumcentric shares
    cc = G.compute_circumcenters(right.points[right.cells])
    assert torch.allclose(cc, torch.tensor([[1.0, 1.0]]))
    tet = primitives.single_tetrahedron()
    centre = G.compute_circumcenters(tet.points[tet.cells])[0]
    assert float((tet.points - centre).norm(dim=1).std()) < 1e-6
    flat3d = G.compute_circumcenters(torch.tensor([[[0.0, 0, 1], [2, 0, 1], [0, 2, 1]]]))
    assert torch.allclose(flat3d, torch.tensor([[1.0, 1.0, 1.0]]))
    # cotangent weights: equilateral triangles give cot(60°)/2 per incident triangle; curves give 1 / length
    w, edges = G.compute_cotan_weights_fem(primitives.equilateral_triangle())
    assert edges.shape == (3, 2) and torch.allclose(w, torch.full((3,), 0.5 / math.sqrt(3)), atol=1e-6)
    w, _ = G.compute_cotan_weights_fem(primitives.line_segments_1d(4))
    assert torch.allclose(w, torch.full((4,), 4.0), atol=1e-5)
    # the weights reproduce the Laplacian of a linear field (zero) and of x² (−2 · dual area) at interior vertices
    w, edges = G.compute_cotan_weights_fem(grid)
    x = grid.points[:, 0]
    lap = torch.zeros(grid.n_points)
    for f in (x, x ** 2):
        lap = torch.zeros(grid.n_points).index_add_(0, edges[:, 0], w * (f[edges[:, 1]] - f[edges[:, 0]])) \
                                         .index_add_(0, edges[:, 1], w * (f[edges[:, 0]] - f[edges[:, 1]]))
        if f is x:
            assert float(lap[inner].abs().max()) < 1e-5
    dual = G.compute_dual_volumes_0(grid)
    assert abs(float(lap[inner].sum()) - 2 * float(dual[inner].sum())) < 0.35 * float(dual[inner].sum())
    grads = G.compute_barycentric_gradients(grid)
    assert float(grads.sum(dim=1).abs().max()) < 1e-5
    lin = (grid.points[grid.cells] @ torch.tensor([2.0, -1.0]))[:, :, None]
    assert torch.allclose((grads * lin).sum(dim=1), torch.tensor([2.0, -1.0]).expand(grid.n_cells, 2), atol=1e-4)
    vol, e1 = G.compute_dual_volumes_1(grid)
    assert vol.shape[0] == e1.shape[0]


def test_point_location_and_data_sampling():
    from physicsnemo_b200.mesh import sampling as SM

    grid = primitives.perturbed_grid(5, 5, 0.25, generator=torch.Generator().manual_seed(2))
    grid = grid.with_data(point_data={"lin": grid.points @ torch.tensor([3.0, -2.0]) + 1, "vec": grid.points * 2,
                                      "id": torch.arange(grid.n_points)},
                          cell_data={"cid": torch.arange(grid.n_cells), "val": torch.arange(grid.n_cells, dtype=torch.float32)})
    pts, cell = grid.sample_points(200, generator=torch.Generator().manual_seed(3))
    found, bary = SM.find_containing_cells(grid, pts)
    assert torch.equal(found, cell) and torch.allclose(bary.sum(1), torch.ones(200), atol=1e-5) and float(bary.min()) > -1e-6
    assert torch.allclose((bary[:, :, None] * grid.points[grid.cells[found]]).sum(1), pts, atol=1e-5)
    outside = torch.tensor([[1.5, 0.5], [-0.1, 0.2]])
    miss, nb = SM.find_containing_cells(grid, outside)
    assert miss.tolist() == [-1, -1] and bool(nb.isnan().all())
    got = SM.sample_data_at_points(grid, torch.cat([pts, outside]), data_source="points")
    assert torch.allclose(got["lin"][:200], pts @ torch.tensor([3.0, -2.0]) + 1, atol=1e-4) and bool(got["lin"][200:].isnan().all())
    assert torch.allclose(got["vec"][:200], pts * 2, atol=1e-5) and got["id"].dtype == torch.float64
    cells = SM.sample_data_at_points(grid, torch.cat([pts, outside]))
    assert torch.equal(cells["val"][:200], cell.float()) and cells["cid"].dtype == torch.float64 and bool(cells["val"][200:].isnan().all())
    # a vertex of the grid lies in several cells: mean of their values, or NaN on request
    v = grid.points[12:13]
    owners = (grid.cells == 12).any(1).nonzero().squeeze(1)
    qi, ci, _ = SM.find_all_containing_cells(grid, v)
    assert sorted(ci.tolist()) == sorted(owners.tolist()) and set(qi.tolist()) == {0}
    assert torch.allclose(SM.sample_data_at_points(grid, v)["val"], owners.float().mean()[None])
    assert bool(SM.sample_data_at_points(grid, v, multiple_cells_strategy="nan")["val"].isnan().all())
    # surfaces: off-manifold queries miss unless projected onto the nearest cell
    sphere = primitives.icosphere(2).with_data(cell_data={"k": torch.arange(320, dtype=torch.float32)})
    q = sphere.cell_centroids[:5] * 1.2
    assert bool(SM.sample_data_at_points(sphere, q)["k"].isnan().all())
    assert SM.sample_data_at_points(sphere, q, project_onto_nearest_cell=True)["k"].tolist() == [0, 1, 2, 3, 4]
    assert torch.equal(SM.find_nearest_cells(sphere, q), torch.arange(5))
    assert SM.match_points(grid.points[[3, 7]] + 1e-8, grid.points).tolist() == [3, 7]
    assert SM.match_points(torch.tensor([[9.0, 9.0]]), grid.points).tolist() == [-1]
    assert SM.compute_barycentric_coordinates(pts[:4], grid.points[grid.cells[:6]]).shape == (4, 6, 3)
    with pytest.raises(ValueError):
        SM.sample_data_at_points(grid, pts, data_source="edges")

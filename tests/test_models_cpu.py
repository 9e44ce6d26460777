"""CPU checks of the model zoo: parameter counts of the five headline configurations,
checkpoint round trips, and agreement of structure with the published layouts."""
import warnings

import pytest
import torch

import physicsnemo_b200 as pn
from physicsnemo_b200.models.afno import AFNO
from physicsnemo_b200.models.diffusion_unets import SongUNet
from physicsnemo_b200.models.fno import FNO
from physicsnemo_b200.models.meshgraphnet import MeshGraphNet
from physicsnemo_b200.models.transolver import Transolver
from physicsnemo_b200.nn.module.gnn_layers.graph_types import Graph


def test_headline_parameter_counts():
    fno = FNO(in_channels=1, out_channels=1, decoder_layers=1, decoder_layer_size=128, dimension=2,
              latent_channels=32, num_fno_layers=4, num_fno_modes=12, padding=8, activation_fn="gelu")
    assert (fno.num_parameters(), len(fno.state_dict())) == (2_368_481, 24)
    mgn = MeshGraphNet(6, 3, 3, processor_size=15, mlp_activation_fn="silu", hidden_dim_processor=128)
    assert (mgn.num_parameters(), len(mgn.state_dict())) == (2_332_419, 262)
    tr = Transolver(functional_dim=3, out_dim=4, embedding_dim=3, n_layers=8, n_hidden=256, n_head=8, slice_num=64,
                    mlp_ratio=4, use_te=False)
    assert (tr.num_parameters(), len(tr.state_dict())) == (5_969_732, 152)
    with torch.device("meta"):
        unet = SongUNet(img_resolution=1024, in_channels=16, out_channels=4, model_channels=128,
                        channel_mult=[1, 2, 2, 4], num_blocks=2, attn_resolutions=[64])
        afno = AFNO(inp_shape=[720, 1440], in_channels=73, out_channels=73, patch_size=[8, 8], embed_dim=768,
                    depth=12, num_blocks=8, sparsity_threshold=0.01)
    assert (sum(p.numel() for p in unet.parameters()), len(unet.state_dict())) == (73_761_156, 349)
    assert (sum(p.numel() for p in afno.parameters()), len(afno.state_dict())) == (79_900_416, 148)


@pytest.mark.parametrize("legacy", [False, True])
def test_checkpoint_round_trip(tmp_path, legacy):
    model = FNO(in_channels=2, out_channels=1, dimension=2, latent_channels=8, num_fno_layers=2, num_fno_modes=3,
                padding=2, decoder_layer_size=8)
    path = tmp_path / "fno.mdlus"
    model.save(str(path), legacy_format=legacy)
    loaded = pn.Module.from_checkpoint(str(path))
    assert type(loaded) is FNO
    x = torch.randn(2, 2, 12, 12)
    assert torch.equal(model(x), loaded(x))
    other = FNO(in_channels=2, out_channels=1, dimension=2, latent_channels=8, num_fno_layers=2, num_fno_modes=3,
                padding=2, decoder_layer_size=8)
    other.load(str(path))
    assert torch.equal(model(x), other(x))


def test_checkpoint_fallback_keeps_model_and_state_on_one_index(tmp_path):
    """A damaged newest training-state file makes load_checkpoint fall back one index; the model weights must then be
    the ones of that same index, not the newest model file."""
    import glob

    from physicsnemo_b200.utils.checkpoint import load_checkpoint, save_checkpoint

    lin = torch.nn.Linear(3, 2)
    opt = torch.optim.SGD(lin.parameters(), lr=0.1, momentum=0.9)
    weights = {}
    for epoch in (1, 2):
        lin(torch.randn(4, 3)).sum().backward()
        opt.step()
        weights[epoch] = lin.weight.detach().clone()
        save_checkpoint(str(tmp_path), models=lin, optimizer=opt, epoch=epoch)
    newest = glob.glob(str(tmp_path / "checkpoint.0.2.pt"))
    assert len(newest) == 1
    with open(newest[0], "wb") as f:
        f.write(b"truncated")
    other = torch.nn.Linear(3, 2)
    opt2 = torch.optim.SGD(other.parameters(), lr=0.1, momentum=0.9)
    assert load_checkpoint(str(tmp_path), models=other, optimizer=opt2) == 1
    assert torch.equal(other.weight, weights[1])


def test_nested_modules_and_overrides(tmp_path):
    class Inner(pn.Module):
        _overridable_args = {"scale"}

        def __init__(self, width, scale=1.0):
            super().__init__(meta=pn.ModelMetaData())
            self.lin = torch.nn.Linear(width, width)
            self.scale = scale

    class Outer(pn.Module):
        def __init__(self, inner, depth=1):
            super().__init__()
            self.inner, self.depth = inner, depth

    import sys
    mod = sys.modules[__name__]
    mod.Inner, mod.Outer = Inner, Outer
    Inner.__qualname__, Outer.__qualname__ = "Inner", "Outer"
    m = Outer(Inner(4, scale=2.0), depth=3)
    p = tmp_path / "o.mdlus"
    m.save(str(p))
    r = pn.Module.from_checkpoint(str(p), override_args={"inner.scale": 5.0})
    assert r.depth == 3 and r.inner.scale == 5.0 and torch.equal(r.inner.lin.weight, m.inner.lin.weight)
    with pytest.raises(ValueError):
        pn.Module.from_checkpoint(str(p), override_args={"depth": 2})


def test_from_torch_and_registry():
    from physicsnemo_b200.core import ModelRegistry

    class Net(torch.nn.Module):
        def __init__(self, n):
            super().__init__()
            self.l = torch.nn.Linear(n, n)

        def forward(self, x):
            return self.l(x)

    Wrapped = pn.Module.from_torch(Net, meta=pn.ModelMetaData(), name="WrappedNetForTest", register=True)
    m = Wrapped(3)
    assert isinstance(m, pn.Module) and m(torch.randn(2, 3)).shape == (2, 3)
    assert ModelRegistry().factory("WrappedNetForTest") is Wrapped


def test_small_forward_backward_all_models():
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        g = Graph(torch.randint(0, 30, (2, 90)), 30)
        MeshGraphNet(4, 3, 2, processor_size=2)(torch.randn(30, 4), torch.randn(90, 3), g).sum().backward()
        AFNO([16, 16], 2, 2, patch_size=[4, 4], embed_dim=16, depth=1, num_blocks=4)(torch.randn(1, 2, 16, 16)).sum().backward()
        SongUNet(16, 3, 2, model_channels=8, channel_mult=[1, 2], num_blocks=1, attn_resolutions=[8])(
            torch.randn(1, 3, 16, 16), torch.rand(1)).sum().backward()
        Transolver(2, 1, structured_shape=(8, 8), unified_pos=True, n_hidden=16, n_head=2, slice_num=4, use_te=False)(
            torch.randn(1, 8, 8, 2)).sum().backward()


def test_graphcast_small():
    import numpy as np

    from physicsnemo_b200.models.graphcast import GraphCastNet
    from physicsnemo_b200.models.graphcast.utils.icosahedral_mesh import (get_hierarchy_of_triangular_meshes_for_sphere,
                                                                         merge_meshes)

    meshes = get_hierarchy_of_triangular_meshes_for_sphere(3)
    assert [(m.vertices.shape[0], m.faces.shape[0]) for m in meshes] == [(12, 20), (42, 80), (162, 320), (642, 1280)]
    assert np.abs(np.linalg.norm(meshes[-1].vertices, axis=1) - 1).max() < 1e-6
    assert merge_meshes(meshes).faces.shape[0] == 1700
    f = meshes[1].faces
    v = meshes[1].vertices
    assert (np.einsum("fi,fi->f", np.cross(v[f[:, 1]] - v[f[:, 0]], v[f[:, 2]] - v[f[:, 0]]), v[f].mean(1)) > 0).all()
    kw = dict(mesh_level=2, input_res=(19, 36), input_dim_grid_nodes=5, output_dim_grid_nodes=3, processor_layers=3, hidden_dim=16)
    net = GraphCastNet(**kw)
    assert net.mesh_graph.num_nodes == 162 and net.m2g_graph.num_edges == 3 * 19 * 36
    assert torch.bincount(net.m2g_graph.edge_index[1]).unique().tolist() == [3]
    x = torch.randn(1, 5, 19, 36)
    y = net(x)
    assert y.shape == (1, 3, 19, 36)
    y.sum().backward()
    assert all(p.grad is not None for p in net.parameters())
    net.set_checkpoint_processor(1)
    assert torch.allclose(net(x), y, atol=1e-5)
    trick = GraphCastNet(**kw, do_concat_trick=True, processor_type="GraphTransformer", khop_neighbors=2)
    assert trick(x).shape == (1, 3, 19, 36)
    with pytest.raises(ValueError):
        net(torch.randn(2, 5, 19, 36))


def test_meshgraphnet_variants():
    from physicsnemo_b200.models.meshgraphnet import BiStrideMeshGraphNet, HybridMeshGraphNet, MeshGraphKAN
    from physicsnemo_b200.nn.module.gnn_layers.graph_types import Graph

    torch.manual_seed(0)
    N, E = 30, 90
    ei = torch.randint(0, N, (2, E))
    g = Graph(ei, num_nodes=N)
    g.pos = torch.randn(N, 3)
    x, e = torch.randn(N, 4), torch.randn(E, 3)
    small = dict(processor_size=2, hidden_dim_processor=16, hidden_dim_node_encoder=16, hidden_dim_edge_encoder=16,
                 hidden_dim_node_decoder=16)
    assert MeshGraphKAN(4, 3, 2, **small)(x, e, g).shape == (N, 2)
    hyb = HybridMeshGraphNet(4, 3, 2, **small)
    assert not hasattr(hyb, "edge_encoder") and hyb(x, e[:60], e[60:], g).shape == (N, 2)
    with pytest.raises(NotImplementedError):
        HybridMeshGraphNet(4, 3, 2, do_concat_trick=True)
    bi = BiStrideMeshGraphNet(4, 3, 2, num_mesh_levels=2, **small)
    ids = [torch.arange(0, N, 2), torch.arange(0, 15, 2)]
    edges = [ei, torch.randint(0, 15, (2, 40)), torch.randint(0, 8, (2, 20))]
    out = bi(x, e, g, ms_edges=edges, ms_ids=ids)
    assert out.shape == (N, 2)
    out.sum().backward()
    assert bi.bistride_processor.bottom_gmp.mlp_edge.model[0].weight.grad is not None


def test_dpot_mesh_reduced_vfgn():
    from types import SimpleNamespace as NS

    from physicsnemo_b200.models.dpot import DPOTNet, DPOTNet3D
    from physicsnemo_b200.models.mesh_reduced import Mesh_Reduced, Sequence_Model
    from physicsnemo_b200.models.vfgn import VFGNLearnedSimulator
    from physicsnemo_b200.nn.module.gnn_layers.graph_types import Graph

    torch.manual_seed(0)
    net = DPOTNet(inp_shape=16, patch_size=4, in_channels=2, out_channels=2, in_timesteps=3, out_timesteps=2, num_blocks=2,
                  embed_dim=16, out_layer_dim=8, depth=2, modes=3, normalize=True)
    assert net(torch.randn(2, 16, 16, 3, 2)).shape == (2, 16, 16, 2, 2)
    net3 = DPOTNet3D(inp_shape=8, patch_size=4, in_channels=1, out_channels=2, in_timesteps=2, num_blocks=2, embed_dim=8,
                     out_layer_dim=4, depth=1, modes=2, temporal_modes=2)
    assert net3(torch.randn(1, 8, 8, 8, 2, 1)).shape == (1, 8, 8, 8, 1, 2)

    N, E, P = 40, 120, 8
    pos, piv = torch.rand(N, 2), torch.rand(P, 2)
    ei = torch.randint(0, N, (2, E))
    g = Graph(torch.cat([ei, ei + N], 1), num_nodes=2 * N)
    g.batch = torch.arange(2).repeat_interleave(N)
    small = dict(processor_size=2, hidden_dim_processor=16, hidden_dim_node_encoder=16, hidden_dim_edge_encoder=16,
                 hidden_dim_node_decoder=16)
    mr = Mesh_Reduced(3, 2, 3, output_encode_dim=4, **small)
    x, e = torch.randn(2 * N, 3), torch.randn(2 * E, 2)
    z = mr.encode(x, e, g, pos, piv)
    assert z.shape == (2 * P, 4) and mr.decode(z, e, g, pos, piv).shape == (2 * N, 3)
    # interpolating a constant field returns the constant
    const, *_ = mr.knn_interpolate(torch.full((N, 1), 2.5), pos, piv, k=3)
    assert torch.allclose(const, torch.full((P, 1), 2.5), atol=1e-5)
    seq = Sequence_Model(4 * P, 3, None, num_heads=4)
    zz = z.reshape(2, 1, -1)
    assert seq.sample(zz, 3, torch.randn(2, 1, 3)).shape == (2, 4, 4 * P)

    stats = {k: NS(mean=torch.zeros(3), std=torch.ones(3)) for k in ("velocity", "acceleration")}
    sim = VFGNLearnedSimulator(num_dimensions=3, num_seq=5, boundaries=torch.zeros(3, 2), normalization_stats=stats)
    n, m = 12, 30
    seqp = torch.randn(2 * n, 5, 3)
    pred, tgt = sim(torch.randn(2 * n, 3), sim.get_random_walk_noise_for_position_sequence(seqp, 1e-3), seqp,
                    torch.tensor([n, n]), torch.tensor([m, m]), torch.randint(0, n, (2 * m,)), torch.randint(0, n, (2 * m,)),
                    1, None, torch.randint(0, 3, (2 * n,)))
    assert pred.shape == tgt.shape == (2 * n, 3)
    assert "lin_s.weight" in dict(sim._graph_network._decoder_network.mlp.named_parameters())


def test_geotransolver_streams_and_context():
    from physicsnemo_b200.models.geotransolver import GeoTransolver

    torch.manual_seed(0)
    net = GeoTransolver(functional_dim=(3, 2), out_dim=(2, 1), geometry_dim=3, global_dim=4, n_layers=2, n_hidden=32, n_head=4,
                        slice_num=8)
    a, b = net((torch.randn(2, 50, 3), torch.randn(2, 30, 2)), None, torch.randn(2, 3, 4), torch.randn(2, 40, 3))
    assert a.shape == (2, 50, 2) and b.shape == (2, 30, 1)
    (a + 0).sum().backward()
    grid = GeoTransolver(functional_dim=3, out_dim=2, geometry_dim=2, n_layers=1, n_hidden=32, n_head=4, slice_num=8,
                         structured_shape=(6, 5), attention_type="GALE")
    out, states = grid(torch.randn(2, 6, 5, 3), geometry=torch.randn(2, 6, 5, 2), return_embedding_states=True)
    assert out.shape == (2, 6, 5, 2) and states.shape == (2, 4, 8, 8)
    with pytest.raises(ValueError):
        GeoTransolver(functional_dim=3, out_dim=2, structured_shape=(4, 4), include_local_features=True)


def test_healpix_padding_table():
    from physicsnemo_b200.nn.module.hpx import HEALPixAvgPool, HEALPixLayer, HEALPixPadding, padding_index_table

    n, p = 8, 2
    idx = padding_index_table(n, p)
    assert idx.shape == (2, 12, n + 2 * p, n + 2 * p) and int(idx.min()) >= 0 and int(idx.max()) < 12 * n * n
    # the centre of every padded face is the face itself
    own = torch.arange(12 * n * n).reshape(12, n, n)
    assert torch.equal(idx[0, :, p:-p, p:-p], own) and torch.equal(idx[1, :, p:-p, p:-p], own)
    # only the equatorial faces' free corners average two sources
    differs = (idx[0] != idx[1]).flatten(1).any(1)
    assert differs.tolist() == [False] * 4 + [True] * 4 + [False] * 4
    x = torch.randn(24, 3, n, n, requires_grad=True)
    y = HEALPixPadding(p)(x)
    assert y.shape == (24, 3, n + 2 * p, n + 2 * p) and torch.equal(y[:, :, p:-p, p:-p], x)
    # a constant field stays constant under padding (all weights sum to one)
    assert torch.allclose(HEALPixPadding(3)(torch.full((12, 1, n, n), 2.5)), torch.full((12, 1, n + 6, n + 6), 2.5))
    y.sum().backward()
    assert x.grad.min() >= 1.0                                   # every pixel is used at least by its own centre copy
    conv = HEALPixLayer(torch.nn.Conv2d, in_channels=3, out_channels=5, kernel_size=3)
    assert conv(x.detach()).shape == (24, 5, n, n)
    assert HEALPixAvgPool(pooling=2)(x.detach()).shape == (24, 3, n // 2, n // 2)


# ---- DLWP-HEALPix U-Nets ---------------------------------------------------------------------------------------------
def _hpx_configs(recurrent: bool, cln: bool = False):
    P = "physicsnemo.models.dlwp_healpix.layers"
    act = {"_target_": "torch.nn.LeakyReLU", "negative_slope": 0.1}
    block = "SymmetricConvNeXtBlock" if cln else "ConvNeXtBlock"
    conv = {"_target_": f"{P}.healpix_blocks.{block}", "in_channels": 3, "out_channels": 1, "activation": act, "kernel_size": 3,
            "dilation": 1, "upscale_factor": 2, "_recursive_": True}
    if cln:
        conv["conditional_layer_norm"] = {"_target_": f"{P}.normalization.ConditionalLayerNorm", "_partial_": True, "condition_shape": 5,
                                          "mlp_hidden_dims": [8]}
    enc = {"_target_": f"{P}.healpix_encoder.UNetEncoder", "conv_block": conv,
           "down_sampling_block": {"_target_": "physicsnemo.models.dlwp_healpix_layers.healpix_blocks.AvgPool", "pooling": 2},
           "n_channels": [8, 16], "n_layers": [1, 1], "dilations": [1, 2], "_recursive_": False}
    dec = {"_target_": f"{P}.UNetDecoder", "conv_block": conv,
           "up_sampling_block": {"_target_": f"{P}.TransposedConvUpsample", "activation": act, "upsampling": 2},
           "output_layer": {"_target_": f"{P}.BasicConvBlock", "kernel_size": 1, "dilation": 1, "n_layers": 1},
           "n_channels": [16, 8], "n_layers": [1, 1], "dilations": [2, 1], "_recursive_": False}
    if recurrent:
        dec["recurrent_block"] = {"_target_": f"{P}.ConvGRUBlock", "kernel_size": 1}
    return enc, dec


def test_healpix_unets_forward_backward_and_rollout_shapes():
    from physicsnemo_b200.models.dlwp_healpix import HEALPixRecUNet, HEALPixUNet
    from physicsnemo_b200.models.dlwp_healpix.layers import ConvGRUBlock, build

    torch.manual_seed(0)
    B, F, H = 2, 12, 8
    enc, dec = _hpx_configs(recurrent=True)
    rec = HEALPixRecUNet(enc, dec, input_channels=3, output_channels=4, n_constants=2, decoder_input_channels=1, input_time_dim=2,
                         output_time_dim=4, delta_time="6h", reset_cycle="24h", presteps=1)
    x = [torch.randn(B, F, 4, 3, H, H), torch.randn(B, F, 6, 1, H, H), torch.randn(F, 2, H, H)]
    y = rec(x)
    assert y.shape == (B, F, 4, 4, H, H)                       # 2 integration steps x 2 time levels, 3 prognostic + 1 diagnostic
    assert rec(x, output_only_last=True).shape == (B, F, 2, 4, H, H)
    y.square().mean().backward()
    assert all(p.grad is not None for p in rec.parameters())
    assert any(isinstance(m, ConvGRUBlock) for m in rec.modules())
    assert torch.allclose(rec(x), rec(x))                      # hidden state is reset at the start of every call
    enc, dec = _hpx_configs(recurrent=False)
    net = HEALPixUNet(enc, dec, input_channels=3, output_channels=3, n_constants=2, decoder_input_channels=1, input_time_dim=2,
                      output_time_dim=2, residual_prediction=True)
    xin = [x[0][:, :, :2], x[1][:, :, :2], x[2]]
    out = net(xin)
    assert out.shape == (B, F, 2, 3, H, H)
    with torch.no_grad():                                      # zero network output -> residual prediction returns its input
        for p in net.decoder.output_layer.parameters():
            p.zero_()
    assert torch.allclose(net(xin), xin[0], atol=1e-6)
    with pytest.raises(ValueError):
        HEALPixUNet(enc, dec, 3, 3, 2, 1, input_time_dim=2, output_time_dim=3)
    assert isinstance(build({"_target_": "torch.nn.Linear", "in_features": 3}, out_features=2), torch.nn.Linear)


def test_healpix_unet_conditional_layer_norm_and_constraints():
    from physicsnemo_b200.models.dlwp_healpix import HEALPixUNet
    from physicsnemo_b200.models.dlwp_healpix.layers import ConditionalLayerNorm, NonnegativeConstraint

    torch.manual_seed(0)
    B, F, H = 2, 12, 8
    enc, dec = _hpx_configs(recurrent=False, cln=True)
    enc["per_level_cln"] = [True, False]
    net = HEALPixUNet(enc, dec, input_channels=2, output_channels=2, n_constants=1, decoder_input_channels=1, input_time_dim=1,
                      output_time_dim=1, residual_prediction=False,
                      constraints={"nonneg": {"_target_": "physicsnemo.models.dlwp_healpix.layers.healpix_constraints.NonnegativeConstraint",
                                              "variables": ["q"], "channels": ["t", "q"], "scaling": {"q": {"mean": 1.0, "std": 2.0}}}})
    n_cln_enc = sum(isinstance(m, ConditionalLayerNorm) for m in net.encoder.modules())
    assert n_cln_enc == 3                                      # only the first encoder level keeps its three CLN layers
    x = [torch.randn(B, F, 1, 2, H, H), torch.randn(B, F, 1, 1, H, H), torch.randn(F, 1, H, H)]
    cond = [torch.randn(B, 5)]
    y = net(x, conditions_cln=cond)
    assert y.shape == (B, F, 1, 2, H, H)
    assert float(y[:, :, :, 1].min()) >= -0.5 - 1e-6           # q >= (0 - mean) / std
    with pytest.raises(ValueError):
        net(x)                                                 # conditions are required once CLN is enabled
    assert isinstance(net.constraints[0], NonnegativeConstraint)


# ---- DoMINO ----------------------------------------------------------------------------------------------------------
def _domino_small_params(**over):
    import copy

    from physicsnemo_b200.models.domino import DEFAULT_MODEL_PARAMS

    p = copy.deepcopy(DEFAULT_MODEL_PARAMS)
    p.interp_res = [8, 8, 8]
    gc, gl = p.geometry_rep.geo_conv, p.geometry_local
    gc.volume_radii, gc.volume_neighbors_in_radius = [0.5, 1.5], [4, 8]
    gc.surface_radii, gc.surface_neighbors_in_radius = [0.5, 1.0], [4, 6]
    gl.volume_radii, gl.volume_neighbors_in_radius = [0.6, 1.2], [4, 8]
    gl.surface_radii, gl.surface_neighbors_in_radius = [0.6], [5]
    p.nn_basis_functions.base_layer = p.aggregation_model.base_layer = p.position_encoder.base_neurons = 16
    p.parameter_model.base_layer = 8
    p.num_neighbors_volume, p.num_neighbors_surface = 3, 4
    for k, v in over.items():
        if k == "processor_type":
            p.geometry_rep.geo_processor.processor_type = v
        else:
            p[k] = v
    return p


def _domino_batch(B=2, N=30, G=8):
    torch.manual_seed(3)
    lin = torch.linspace(-1, 1, G)
    grid = torch.stack(torch.meshgrid(lin, lin, lin, indexing="ij"), -1).unsqueeze(0).expand(B, -1, -1, -1, -1).contiguous()
    u = lambda *s: torch.rand(*s) * 1.6 - 0.8  # noqa: E731
    return dict(geometry_coordinates=u(B, 200, 3), surf_grid=grid, sdf_surf_grid=torch.randn(B, G, G, G), grid=grid,
                sdf_grid=torch.randn(B, G, G, G), global_params_values=torch.rand(B, 2, 1) + 0.5, global_params_reference=torch.ones(B, 2, 1),
                sdf_nodes=torch.randn(B, N, 1), pos_volume_closest=torch.randn(B, N, 3), pos_volume_center_of_mass=torch.randn(B, N, 3),
                volume_mesh_centers=u(B, N, 3), pos_surface_center_of_mass=torch.randn(B, N, 3), surface_mesh_centers=u(B, N, 3),
                surface_mesh_neighbors=u(B, N, 3, 3), surface_normals=torch.randn(B, N, 3), surface_neighbors_normals=torch.randn(B, N, 3, 3),
                surface_areas=torch.rand(B, N) + 0.1, surface_neighbors_areas=torch.rand(B, N, 3) + 0.1)


@pytest.mark.parametrize("over", [dict(), dict(processor_type="conv", encode_parameters=True), dict(combine_volume_surface=True)])
def test_domino_forward_backward(over):
    from physicsnemo_b200.models.domino import DoMINO

    torch.manual_seed(0)
    model = DoMINO(input_features=3, output_features_vol=2, output_features_surf=3, global_features=2, model_parameters=_domino_small_params(**over))
    data = _domino_batch()
    vol, surf = model(data)
    assert vol.shape == (2, 30, 2) and surf.shape == (2, 30, 3)
    assert torch.isfinite(vol).all() and torch.isfinite(surf).all()
    (vol.square().mean() + surf.square().mean()).backward()
    touched = [n for n, p in model.named_parameters() if p.grad is not None and float(p.grad.abs().sum()) > 0]
    assert any(n.startswith("geo_rep_volume") for n in touched) and any(n.startswith("agg_model_surf") for n in touched)


def test_domino_single_branch_and_validation():
    from physicsnemo_b200.models.domino import Config, DoMINO

    surf_only = DoMINO(input_features=3, output_features_surf=2, model_parameters=dict(_domino_small_params()))   # plain dict accepted
    data = _domino_batch()
    vol, surf = surf_only(data)
    assert vol is None and surf.shape == (2, 30, 2)
    with pytest.raises(ValueError):
        surf_only({k: v for k, v in data.items() if k != "surface_normals"})
    with pytest.raises(ValueError):
        DoMINO(input_features=3)
    cfg = Config({"a": {"b": 1}})
    cfg.c = {"d": 2}
    assert cfg.a.b == 1 and cfg.c.d == 2 and isinstance(cfg.c, Config)


# ---- FIGConvUNet -----------------------------------------------------------------------------------------------------
def test_figconvunet_forward_backward_variants():
    from physicsnemo_b200.models.figconvnet import FIGConvUNet

    torch.manual_seed(0)
    pairs = [("b_xc_y_z", (2, 12, 12)), ("b_yc_x_z", (12, 2, 12)), ("b_zc_x_y", (12, 12, 2))]
    net = FIGConvUNet(in_channels=4, out_channels=3, kernel_size=3, hidden_channels=[8, 16, 16], num_levels=2, mlp_channels=[32, 32],
                      aabb_max=(1, 1, 1), aabb_min=(-1, -1, -1), resolution_memory_format_pairs=pairs, pos_encode_dim=8,
                      communication_types=["sum", "mul"])
    v = torch.rand(2, 300, 3) * 2 - 1
    y, drag = net(v)
    assert y.shape == (2, 300, 3) and drag.shape == (2, 1)
    (y.square().mean() + drag.square().mean()).backward()
    assert all(p.grad is not None for p in net.parameters())
    perm = torch.randperm(300)
    y2, drag2 = net(v[:, perm])
    assert torch.allclose(y2, y[:, perm], atol=1e-4) and torch.allclose(drag2, drag, atol=1e-4)     # point order does not matter
    net2 = FIGConvUNet(in_channels=4, out_channels=1, kernel_size=3, hidden_channels=[8, 16], num_levels=1, aabb_max=(1, 1, 1),
                       aabb_min=(-1, -1, -1), resolution_memory_format_pairs=[("b_xc_y_z", (3, 10, 8)), ("b_zc_x_y", (10, 8, 3))],
                       pos_encode_dim=8, has_input_features=True, to_point_sample_method="interp", neighbor_search_type="knn", knn_k=4,
                       use_scalar_output=False, reductions=["mean", "max"], pooling_type="attention")
    y, drag = net2(v, torch.randn(2, 300, 4))
    assert y.shape == (2, 300, 1) and drag is None
    with pytest.raises(ValueError):
        net2(v, torch.randn(2, 300, 5))
    with pytest.raises(ValueError):
        net2(v)


def test_figconv_factor_grid_helpers():
    from physicsnemo_b200.models.figconvnet.figconvunet import _fold, _node_positions, _unfold, segment_reduce

    x = torch.randn(2, 3, 4, 5, 6)
    for axis, depth in ((0, 4), (1, 5), (2, 6)):
        folded = _fold(x, axis)
        assert folded.shape[1] == 3 * depth and torch.equal(_unfold(folded, axis, depth), x)
    pos = _node_positions((4, 5, 6), x.device, x.dtype).unsqueeze(0).expand(2, -1, -1, -1, -1)
    assert torch.allclose(torch.nn.functional.grid_sample(x, pos, align_corners=True), x, atol=1e-5)   # a grid sampled at its own nodes
    vals, seg = torch.tensor([[1.0], [3.0], [5.0], [2.0]]), torch.tensor([0, 0, 2, 2])
    assert segment_reduce(vals, seg, 3, "mean").flatten().tolist() == [2.0, 0.0, 3.5]
    assert segment_reduce(vals, seg, 3, "max").flatten().tolist() == [3.0, 0.0, 5.0]
    assert segment_reduce(vals, seg, 3, "var").flatten().tolist() == [1.0, 0.0, 2.25]


# ---- point transformer attention -------------------------------------------------------------------------------------
def test_local_point_transformer_blocks():
    from physicsnemo_b200.nn.module.point_transformer_attention import (AdaLNResidualMLP, LocalPointTransformerBlock,
                                                                         LocalTokenCrossAttentionBlock)

    torch.manual_seed(0)
    blk = LocalPointTransformerBlock(dim=16, num_heads=4, neighbor_k=6, dilation=2, mlp_ratio=2, dropout=0.0, conditioning_dim=5)
    f, c, cond = torch.randn(40, 16), torch.rand(40, 3), torch.randn(5)
    for p in blk.parameters():
        torch.nn.init.normal_(p, std=0.2)
    ids = torch.arange(40) // 20
    out = blk(f, c, cond=cond, batch_ids=ids)
    assert out.shape == (40, 16)
    f2 = f.clone()
    f2[20:] = torch.randn(20, 16)                                  # other batch element changes ...
    assert torch.allclose(blk(f2, c, cond=cond, batch_ids=ids)[:20], out[:20], atol=1e-5)   # ... this one does not see it
    perm = torch.randperm(40)
    assert torch.allclose(blk(f[perm], c[perm], cond=cond, batch_ids=ids[perm]), out[perm], atol=1e-5)
    out.sum().backward()
    assert all(p.grad is not None for p in blk.parameters())
    cross = LocalTokenCrossAttentionBlock(dim=16, num_heads=4, neighbor_k=5, mlp_ratio=2, dropout=0.0)
    q = cross(torch.randn(30, 16), torch.rand(30, 3), torch.randn(12, 16), torch.rand(12, 3))
    assert q.shape == (30, 16)
    assert cross(torch.randn(0, 16), torch.rand(0, 3), torch.randn(12, 16), torch.rand(12, 3)).shape == (0, 16)
    mlp = AdaLNResidualMLP(16, 2, 0.0, conditioning_dim=5)
    x = torch.randn(7, 16)
    assert torch.allclose(mlp(x, torch.randn(5)), x + mlp.net(mlp.norm(x)), atol=1e-6)      # zero-initialised modulation
    with pytest.raises(ValueError):
        mlp(x)


def test_healpix_pixel_centres_and_patch_tokenizer():
    """Own HEALPix geometry (equal-area centres, face-local origin at the northern corner) and the GEMM-form patch
    tokenizer / detokenizer against their strided-convolution definitions."""
    import math

    from physicsnemo_b200.nn.module.hpx import HEALPixPatchDetokenizer, HEALPixPatchTokenizer, healpix_xy_lonlat

    lon, lat = healpix_xy_lonlat(3)
    npix = 12 * 4 ** 3
    assert lon.shape == (npix,) and len({(round(float(a), 6), round(float(b), 6)) for a, b in zip(lon, lat)}) == npix
    v = torch.stack([torch.cos(torch.deg2rad(lat)) * torch.cos(torch.deg2rad(lon)),
                     torch.cos(torch.deg2rad(lat)) * torch.sin(torch.deg2rad(lon)), torch.sin(torch.deg2rad(lat))], -1)
    assert float(v.mean(0).abs().max()) < 1e-12                       # equal-area centres balance
    z = torch.sin(torch.deg2rad(lat))
    assert abs(float((z ** 2).mean()) - 1.0 / 3.0) < 2e-3             # <z^2> of a uniform sphere
    per_face = lat.view(12, -1)
    assert all(int(per_face[f].argmax()) == 0 for f in range(12))      # pixel 0 of a face is its northern corner
    assert float(per_face[:4].min()) > 0 and float(per_face[8:].max()) < 0
    # nearest-neighbour spacing is close to the pixel size everywhere
    d = torch.cdist(v, v) + 10 * torch.eye(npix, dtype=v.dtype)
    assert 0.5 < float(d.min(1).values.min()) / math.sqrt(4 * math.pi / npix) < 1.2

    torch.manual_seed(0)
    tk = HEALPixPatchTokenizer(in_channels=3, hidden_size=16, level_fine=2, level_coarse=1, separate_time_axis=True)
    x = torch.randn(2, 3, 2, 12 * 16)
    sod, doy = torch.rand(2, 2) * 86400, torch.rand(2, 2) * 365
    faces = x.view(2, 3, 2, 12, 4, 4).permute(0, 2, 3, 1, 4, 5).reshape(48, 3, 4, 4)
    conv = tk.conv(faces).view(2, 2, 12, 16, 2, 2).permute(0, 1, 2, 4, 5, 3).reshape(2, 2, 48, 16)
    cal = tk.calendar_embed(second_of_day=sod, day_of_year=doy).permute(0, 2, 3, 1)
    assert torch.allclose(tk(x, sod, doy), conv + cal + tk.pos_embed, atol=1e-5)
    dt = HEALPixPatchDetokenizer(hidden_size=16, out_channels=5, level_coarse=1, level_fine=2, time_length=2, condition_dim=7)
    dt.initialize_weights()
    tok, c = torch.randn(2, 2 * 48, 16), torch.randn(2, 7)
    normed = dt.norm_out(tok.view(2, 2, 48, 16))
    ref = dt.conv_t(normed.view(2, 2, 12, 2, 2, 16).permute(0, 1, 2, 5, 3, 4).reshape(48, 16, 2, 2)).view(2, 2, 12, 5, 4, 4)
    assert torch.allclose(dt(tok, c), ref.permute(0, 3, 1, 2, 4, 5).reshape(2, 5, 2, 192), atol=1e-5)


def test_healda_v1_forward_backward():
    import warnings

    from physicsnemo_b200.experimental.models.healda import HealDA

    torch.manual_seed(0)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        net = HealDA(in_channels=3, out_channels=2, nchannel_per_sensor=[2, 1], nplatform_per_sensor=[1, 1], hidden_size=32, num_layers=2,
                     num_heads=4, level_in=2, level_model=1, time_length=1, embed_dim=8, meta_dim=3, fusion_dim=8)
    B, T, npix = 2, 1, 12 * 16
    offsets = torch.randint(1, 9, (2, B, T)).flatten().cumsum(0).view(2, B, T)
    n = int(offsets[-1, -1, -1])
    y = net(torch.randn(B, 3, T, npix), torch.rand(B), torch.randn(n), torch.randn(n, 3), torch.randint(0, npix, (n,)),
            torch.zeros(n, dtype=torch.long), torch.zeros(n, dtype=torch.long), torch.randint(0, 5, (n,)), offsets,
            torch.rand(B, T) * 86400, torch.rand(B, T) * 365)
    assert y.shape == (B, 2, T, npix)
    y.square().sum().backward()
    assert sum(p.grad is not None for p in net.parameters()) > 10


def test_video_healda_is_causal_in_time_and_reads_observations():
    from physicsnemo_b200.experimental.models import VideoHealDA
    from physicsnemo_b200.experimental.models.healda import prepare_obs_context

    torch.manual_seed(0)
    net = VideoHealDA(in_channels=2, out_channels=3, hidden_size=32, num_layers=2, num_heads=4, level_in=2, level_model=1, time_length=3,
                      condition_embed_dim=16, noise_channels=16, obs_token_dim=8, obs_meta_dim=5, obs_film_hidden_dim=16,
                      pixel_attn_n_q_heads=16, pixel_attn_n_kv_heads=1, pixel_attn_head_dim=8, drop_path=0.0).eval()
    with torch.no_grad():
        for p in net.parameters():
            p.add_(0.05 * torch.randn_like(p))                      # leave the zero-initialised gates
    B, T, npix_c = 2, 3, 48
    P, n = B * T * npix_c, 400
    ids = torch.randint(0, 5, (n,))
    flat = torch.randint(0, P, (n,))
    obs, meta = torch.randn(n), torch.randn(n, 5)
    ctx = prepare_obs_context(obs, meta, ids, ids, ids, flat, P)
    x, t = torch.randn(B, 2, T, 192), torch.rand(B)
    sod, doy = torch.rand(B, T) * 86400, torch.rand(B, T) * 365
    with torch.no_grad():
        y = net(x, t, sod, doy, ctx)
        assert y.shape == (B, 3, T, 192)
        x2 = x.clone()
        x2[:, :, 2] += 1.0                                            # perturb the last frame only
        d = (net(x2, t, sod, doy, ctx) - y).abs().amax(dim=(0, 1, 3))
        assert float(d[:2].max()) < 1e-5 and float(d[2]) > 1e-4
        # observations matter, and only through the site they belong to and later frames of the same sample
        obs2 = obs.clone()
        target = int(flat[0])
        obs2[flat == target] += 3.0
        ctx2 = prepare_obs_context(obs2, meta, ids, ids, ids, flat, P)
        dy = (net(x, t, sod, doy, ctx2) - y).abs().amax(dim=(1, 3))    # [B, T]
        b0, t0 = target // (T * npix_c), (target // npix_c) % T
        assert float(dy[b0, t0]) > 1e-5 and float(dy[1 - b0].max()) < 1e-6 and float(dy[b0, :t0].max() if t0 else 0.0) < 1e-6
    with pytest.raises(ValueError):
        net(x[:, :, :2], t, sod[:, :2], doy[:, :2], ctx)
    with pytest.raises(ValueError):
        net(x, t, sod, doy, ctx, class_labels=torch.zeros(B, 2))


def test_model_registry_lists_and_loads_every_entry_point():
    from physicsnemo_b200.core.module import Module
    from physicsnemo_b200.core.registry import ModelRegistry

    reg = ModelRegistry()
    names = reg.list_models()
    for expected in ("FNO", "AFNO", "ModAFNO", "DistributedAFNO", "MeshGraphNet", "Transolver", "SongUNet", "GraphCastNet"):
        assert expected in names
    assert len(names) >= 35
    for name in names:
        assert issubclass(reg.factory(name), Module), name


def test_modafno_forward_backward_and_key_scheme():
    from physicsnemo_b200.models.afno import ModAFNO

    for mode in ("complex", "real"):
        m = ModAFNO([16, 32], in_channels=3, out_channels=2, patch_size=[2, 2], embed_dim=32, mod_dim=16, depth=2,
                    num_blocks=4, scale_shift_mode=mode, embed_model=dict(dim=16))
        y = m(torch.randn(2, 3, 16, 32), torch.rand(2))
        assert y.shape == (2, 2, 16, 32)
        y.square().mean().backward()
        keys = set(m.state_dict())
        for k in ("pos_embed", "mod_additive_proj.weight", "mod_embed_net.sinusoid_embed.freqs", "mod_embed_net.mlp.0.weight",
                  "blocks.0.filter.scale_shift.net.layers.0.weight", "blocks.1.mlp.scale_shift.net.layers.2.bias",
                  "blocks.0.filter.w1", "head.weight"):
            assert k in keys, k
        assert all(p.grad is not None for p in m.parameters())
    plain = ModAFNO([16, 32], in_channels=3, out_channels=2, patch_size=[2, 2], embed_dim=32, mod_dim=16, depth=1, num_blocks=4,
                    modulate_filter=False, modulate_mlp=False)
    assert plain(torch.randn(1, 3, 16, 32), torch.rand(1, 16)).shape == (1, 2, 16, 32)


def test_topodiff_layout_and_forward():
    """Key scheme of the constraint-conditioned U-Net and of its encoder head; forward shapes; input checks."""
    from physicsnemo_b200.models.topodiff import TopoDiff, UNetEncoder

    torch.manual_seed(0)
    net = TopoDiff(img_resolution=16, in_channels=4, out_channels=1, model_channels=32, channel_mult=[1, 2, 2], num_blocks=1,
                   attn_resolutions=[8])
    assert list(net.enc.keys()) == ["16x16_conv", "16x16_block0", "8x8_down", "8x8_block0", "4x4_down", "4x4_block0"]
    assert list(net.dec.keys()) == ["4x4_in0", "4x4_in1", "4x4_block0", "4x4_block1", "8x8_up", "8x8_block0", "8x8_block1",
                                    "16x16_up", "16x16_block0", "16x16_block1"]
    assert net.dec["8x8_block0"].in_channels == 64 + 64 and net.dec["16x16_block1"].in_channels == 32 + 32
    with torch.no_grad():
        net.out_conv.weight.normal_(std=0.1)
    x, cons, t = torch.randn(2, 1, 16, 16), torch.randn(2, 3, 16, 16), torch.tensor([1.0, 5.0])
    y = net(x, cons, t)
    assert y.shape == (2, 1, 16, 16) and torch.isfinite(y).all() and float(y.abs().max()) > 0
    with pytest.raises(ValueError):
        net(x, cons[:1], t)
    with pytest.raises(ValueError):
        net(x, cons, t[:1])
    enc = UNetEncoder(in_channels=3, out_channels=2, model_channels=32, num_res_blocks=2, channel_mult=(1, 2),
                      attention_resolutions=(2,), output_prob=True)
    assert len(enc.encoder) == 4 and isinstance(enc.out[-1], torch.nn.Sigmoid)
    p = enc(torch.randn(2, 3, 16, 16), t)
    assert p.shape == (2, 2) and float(p.min()) >= 0 and float(p.max()) <= 1


def test_mdlus_files_cross_load_with_the_reference():
    """FNO, AFNO, Transolver, SongUNet (outputs), MeshGraphNet and FIGConvUNet (tensors): ``.mdlus`` files written by the reference load
    here and the other way round.  Runs in a child process; skipped when the reference is not installed beside the repo."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if not os.path.isdir(os.path.join(root, "baseline", "_ref", "physicsnemo")):
        pytest.skip("the reference package is not installed under baseline/_ref")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    proc = subprocess.run([sys.executable, os.path.join(root, "tests", "helpers", "crossload_worker.py")], capture_output=True,
                          text=True, timeout=900, env=env)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert proc.stdout.count(": ok") == 6, proc.stdout


def test_domino_utils():
    import math

    from physicsnemo_b200.mesh import primitives
    from physicsnemo_b200.models.domino import utils as U

    torch.manual_seed(0)
    x = torch.randn(50, 3) * 4 + 1
    n = U.normalize(x)
    assert torch.allclose(n.amin(0), -torch.ones(3)) and torch.allclose(n.amax(0), torch.ones(3))
    assert torch.allclose(U.unnormalize(n, x.amax(0, keepdim=True), x.amin(0, keepdim=True)), x, atol=1e-5)
    s = U.standardize(x)
    assert torch.allclose(s.mean(0), torch.zeros(3), atol=1e-5) and torch.allclose(U.unstandardize(s, x.mean(0), x.std(0)), x, atol=1e-5)
    enc = U.calculate_pos_encoding(torch.tensor([0.0, 1.0]), d=4)
    assert len(enc) == 4 and torch.allclose(enc[1], torch.tensor([1.0, math.cos(1.0)])) and torch.allclose(enc[2][1], torch.sin(torch.tensor(0.01)))
    assert U.calculate_normal_positional_encoding(x, x + 1, (0.5, 0.5, 0.5)).shape == (50, 12)
    assert U.pad(x, 60, -1.0).shape == (60, 3) and float(U.pad(x, 60, -1.0)[55, 0]) == -1.0 and U.pad(x, 10) is x
    assert U.pad_inp(torch.ones(2, 3, 3), 4).shape == (4, 3, 3)
    grid = U.create_grid(torch.tensor([1.0, 1, 1]), torch.tensor([0.0, 0, 0]), [3, 4, 5])
    assert grid.shape == (3, 4, 5, 3)
    field = x[:, :1] * 2
    assert torch.allclose(U.nd_interpolator(x, field, x, k=1), field)
    assert U.combine_dict({"a": 1, "b": 2.0}, {"a": 2, "b": 0.5}) == {"a": 3, "b": 2.5}
    out = U.mean_std_sampling(torch.tensor([[0.0, 0], [10, 0], [0, -9]]), torch.zeros(2), torch.ones(2), 3.0)
    assert sorted(int(i) for i in out) == [1, 2]
    moved = U.dict_to_device({"x": x, "filename": "f"}, "cpu")
    assert list(moved) == ["x"]
    picked, idx = U.area_weighted_shuffle_array(x, 10, torch.rand(50) + 0.1, 2.0)
    assert picked.shape == (10, 3) and torch.equal(picked, x[idx]) and len(set(idx.tolist())) == 10
    assert U.solution_weighted_shuffle_array(x, 80, torch.rand(50) + 0.1)[0].shape[0] == 50
    sphere = primitives.icosphere(2)
    pts, face, area, normal = U.sample_points_on_mesh(sphere.points, sphere.cells, 2000)
    assert pts.shape == (2000, 3) and float((pts.norm(dim=1) - 1).abs().max()) < 0.03          # on the faces of the unit sphere
    assert torch.allclose(area, sphere.cell_areas[face], atol=1e-6) and float((normal * pts).sum(1).min()) > 0.9
    assert abs(float(pts.mean(0).norm())) < 0.08                                               # area-uniform

"""Point-cloud helpers, tokenizer and the AeroJEPA components (CPU).

Mirrors ``test/experimental/nn/test_point_*`` and ``test/experimental/models/aerojepa`` of the
reference: shape / mask contracts of the helpers, every tokenizer strategy, agreement of the batched
and the single-cloud paths of each component, decoder options, and a checkpoint round trip.
"""
import pytest
import torch

from physicsnemo_b200.core.module import Module
from physicsnemo_b200.experimental.models.aerojepa import (AeroJEPA, AeroJEPATrunk, ContextTransformer, PrototypeTokenJEPAHead,
                                                           QueryTokenDecoder, TargetTransformer, TokenSet, build_geometry_features,
                                                           pad_token_sets, trim_batched_tokens)
from physicsnemo_b200.experimental.models.aerojepa.prototype_anchors import (build_target_prototype_anchors,
                                                                             ensure_target_prototype_anchors, kmeans_centres)
from physicsnemo_b200.experimental.models.aerojepa.tokens import FlatTokens, reshape_token_features_for_sigreg
from physicsnemo_b200.experimental.nn import point_utils as pu
from physicsnemo_b200.experimental.nn.point_tokenizer import PointCloudTokenizer, voxel_mean_positions
from physicsnemo_b200.nn.module.embedding_layers import FourierPositionalEmbedding


def test_point_utils_roundtrip_and_masks():
    counts = torch.tensor([3, 0, 2])
    mask = pu.counts_to_mask(counts, 4)
    assert mask.tolist() == [[True, True, True, False], [False] * 4, [True, True, False, False]]
    x = torch.arange(3 * 4 * 2.0).reshape(3, 4, 2)
    flat = pu.flatten_padded_batch(x, mask)
    assert flat.shape == (5, 2)
    back = pu.unflatten_to_padded(flat, mask)
    assert torch.equal(back[mask], x[mask]) and float(back[~mask].abs().sum()) == 0
    assert pu.gather_rows(x[0], torch.tensor([[0, 3], [1, 1]])).shape == (2, 2, 2)
    mean = pu.masked_mean(x, mask)
    assert mean.shape == (3, 1, 2) and torch.allclose(mean[0, 0], x[0, :3].mean(0)) and float(mean[1].abs().sum()) == 0
    assert torch.allclose(pu.masked_mean(x[0], None), x[0].mean(0, keepdim=True))
    with pytest.raises(ValueError):
        pu.unflatten_to_padded(flat[:-1], mask)


def test_batch_offsets_keep_items_apart():
    torch.manual_seed(0)
    coords = torch.rand(3, 20, 3) * 5
    mask = pu.counts_to_mask(torch.tensor([20, 11, 7]), 20)
    step = pu.compute_batch_offset_step(coords, mask)
    assert step >= 4 * 5 * 0.5
    flat, shifted, batch = pu.flatten_batched_coords(coords, mask, offset_step=step)
    assert flat.shape == (38, 3) and torch.equal(shifted[:, 1:], flat[:, 1:])
    idx = pu.chunked_knn_indices(query_coords=shifted, key_coords=shifted, k=5, chunk_size=16)
    assert torch.equal(batch[idx], batch[:, None].expand(-1, 5))
    dil = pu.chunked_knn_indices(query_coords=shifted, key_coords=shifted, k=3, chunk_size=16, dilation=2)
    wide = pu.chunked_knn_indices(query_coords=shifted, key_coords=shifted, k=6, chunk_size=16)
    assert torch.equal(dil, wide[:, ::2])
    assert pu.compute_batch_offset_step(coords[:, :0]) == 1.0


def test_fourier_positional_embedding_layout():
    emb = FourierPositionalEmbedding(in_dim=3, num_bands=4)
    assert emb.out_dim == 27 and emb(torch.zeros(5, 3)).shape == (5, 27)
    x = torch.tensor([[0.25, -0.5]])
    e = FourierPositionalEmbedding(in_dim=2, num_bands=2, include_input=False, base_freq=1.0)(x)
    want = torch.tensor([0.25, 0.5]).sin().tolist() + torch.tensor([0.25, 0.5]).cos().tolist()
    assert torch.allclose(e[0, :4], torch.tensor(want))
    assert "freqs" in emb.state_dict()
    with pytest.raises(ValueError):
        FourierPositionalEmbedding(freqs=torch.ones(2, 2))


@pytest.mark.parametrize("strategy", ["identity", "random", "fps", "random_cluster", "fps_cluster", "voxel_fps_cluster",
                                      "data_prototype_cluster"])
def test_tokenizer_strategies(strategy):
    torch.manual_seed(1)
    pos, feat = torch.rand(150, 3), torch.randn(150, 4)
    tok = PointCloudTokenizer(max_point_tokens=25, strategy=strategy, cluster_size=6, voxel_size=0.25,
                              prototype_coords=torch.rand(9, 3)).eval()
    p, f, members = tok.tokenize_with_clusters(point_positions=pos, point_features=feat)
    want = {"identity": 150, "data_prototype_cluster": 9}.get(strategy, 25)
    assert p.shape == (want, 3) and f.shape == (want, 4)
    assert (members is not None) == tok.uses_cluster_pooling
    if members is not None:
        assert torch.allclose(f, feat[members].mean(1))
        d = (pos[None] - p[:, None]).norm(dim=-1)
        assert torch.equal(members.sort(1).values, d.topk(members.shape[1], largest=False).indices.sort(1).values)
    p2, _ = tok(point_positions=pos, point_features=feat)
    assert torch.equal(p, p2)                         # eval mode is deterministic
    small = tok(point_positions=pos[:10], point_features=feat[:10])[0]
    assert small.shape[0] == (9 if strategy == "data_prototype_cluster" else 10)
    bp, bf, bm, bc = tok.forward_batched(point_positions=torch.stack([pos, pos]), point_features=torch.stack([feat, feat]),
                                         point_counts=torch.tensor([150, 10]))
    assert bc.tolist() == [want, 9 if strategy == "data_prototype_cluster" else 10] and bm.sum(1).tolist() == bc.tolist()


def test_tokenizer_validation_and_voxels():
    with pytest.raises(ValueError, match="cluster_size"):
        PointCloudTokenizer(max_point_tokens=4, strategy="fps_cluster")
    with pytest.raises(ValueError, match="prototype_coords"):
        PointCloudTokenizer(strategy="data_prototype_cluster")
    with pytest.raises(ValueError, match="must be one of"):
        PointCloudTokenizer(strategy="octree")
    pts = torch.tensor([[0.0, 0, 0], [0.1, 0, 0], [1.0, 1, 1]])
    vox = voxel_mean_positions(pts, 0.5)
    assert vox.shape == (2, 3) and torch.allclose(vox.sort(0).values[0], torch.tensor([0.05, 0, 0]))
    empty = PointCloudTokenizer(strategy="data_prototype_cluster", prototype_coords=torch.rand(4, 3))
    p, f, m = empty.tokenize_with_clusters(point_positions=torch.zeros(0, 3), point_features=torch.zeros(0, 2))
    assert p.shape == (4, 3) and f.shape == (4, 2) and m.shape == (4, 0)


def test_geometry_features_and_token_sets():
    pos, feat = torch.rand(6, 3), torch.rand(6, 3 + 5)
    assert build_geometry_features(context_pos=pos, context_feat=feat) is pos
    g = build_geometry_features(context_pos=pos, context_feat=feat, use_sdf=True, use_solid_n_dot_uinf=True)
    assert torch.equal(g[:, 3:], feat[:, -2:])
    g = build_geometry_features(context_pos=pos, context_feat=feat, use_sdf=True, use_solid_normals=True, use_solid_n_dot_uinf=True)
    assert torch.equal(g[:, 3:], feat[:, -5:])
    with pytest.raises(ValueError):
        build_geometry_features(context_pos=pos, context_feat=feat[:, :4], use_solid_normals=True)
    a = TokenSet(torch.randn(4, 8), torch.rand(4, 3))
    b = TokenSet(torch.randn(2, 8), torch.rand(2, 3), global_token=torch.ones(1, 8))
    both = pad_token_sets([a, b])
    assert both.is_batched and both.mask.sum(1).tolist() == [4, 2] and both.token_dim == 8
    assert torch.allclose(both.global_token[0], a.features.mean(0)) and torch.equal(both.global_token[1], torch.ones(8))
    one = trim_batched_tokens(both, 1, 2)
    assert torch.equal(one.features, b.features) and one.global_token.shape == (1, 8)
    assert reshape_token_features_for_sigreg(both.features, both.mask).shape == (1, 6, 8)
    assert a.with_updates(coords=b.coords[:0]).coords.shape[0] == 0
    flat = FlatTokens.from_padded(both.coords, both.mask)
    assert torch.equal(flat.scatter(flat.gather(both.features))[both.mask], both.features[both.mask])


_ENC = dict(token_dim=32, max_point_tokens=20, tokenizer_strategy="fps_cluster", tokenizer_cluster_size=5, num_heads=4,
            num_layers=2, neighbor_k=6, dilation_schedule=[1, 2])


def _model(**decoder_kw):
    torch.manual_seed(0)
    ctx = ContextTransformer(point_input_dim=4, use_sdf=True, tokenizer_cluster_pooling="graph", **_ENC)
    tgt = TargetTransformer(point_input_dim=7, **_ENC)
    kw = dict(token_dim=32, hidden_dim=48, num_layers=2, out_dim=4, use_sdf=True, cond_dim=2 + 32, pe_num_bands=4,
              cross_attention_heads=4, cross_attention_layers=2, cross_attention_k=8, query_chunk_size=50)
    kw.update(decoder_kw)
    trunk = AeroJEPATrunk(context_encoder=ctx, target_encoder=tgt, decoder=QueryTokenDecoder(**kw), mask_prediction_enabled=True)
    head = PrototypeTokenJEPAHead(token_dim=32, cond_dim=2, depth=2, num_heads=4, neighbor_k=6)
    return AeroJEPA(trunk=trunk, predictor=head).eval()


def _case(seed=0):
    g = torch.Generator().manual_seed(seed)
    pos = torch.rand(120, 3, generator=g)
    return dict(pos=pos, feat=torch.cat([pos, torch.randn(120, 1, generator=g)], 1), gen=torch.tensor([0.3, 2.0]),
                q=torch.rand(130, 3, generator=g), sdf=torch.rand(130, 1, generator=g) - 0.2,
                s_pos=torch.rand(60, 3, generator=g), s_feat=torch.randn(60, 7, generator=g),
                v_pos=torch.rand(80, 3, generator=g), v_feat=torch.randn(80, 7, generator=g))


def _pad2(t, n):
    """Batch of two: the full tensor and its first ``n`` rows, zero padded."""
    return torch.stack([t, torch.cat([t[:n], torch.zeros_like(t[n:])])])


def test_aerojepa_forward_backward_and_training_pieces():
    model, c = _model(), _case()
    out = model(context_pos=c["pos"], context_feat=c["feat"], gen_params=c["gen"], query_pos=c["q"], query_sdf=c["sdf"])
    assert out.shape == (130, 4)
    out.square().mean().backward()
    used = [n for n, p in model.named_parameters() if p.grad is not None]
    assert any(n.startswith("predictor.") for n in used) and any(n.startswith("trunk.context_encoder.") for n in used)
    assert any("graph_pool" in n for n in used) and not any(n.startswith("trunk.target_encoder.encoder.blocks") for n in used)
    # the training route: encode both views, predict target tokens from the context, decode either token set
    views = model.encode_geometry_and_flow(context_pos=c["pos"], context_feat=c["feat"], target_surface_pos=c["s_pos"],
                                           target_surface_main_feat=c["s_feat"], target_volume_pos=c["v_pos"],
                                           target_volume_feat=c["v_feat"], gen_params=c["gen"])
    tgt = views["target_tokens"]
    assert tgt.features.shape == (20, 32) and views["cond_global"].shape == (1, 34)
    predicted = model.predict_field_tokens(context_tokens=views["context_tokens"], target_positions=tgt.coords, conditions=c["gen"])
    assert predicted.shape == tgt.features.shape
    pred, logits = model.decode_field(target_tokens=tgt.with_updates(features=predicted), cond_global=views["cond_global"],
                                      query_pos=c["q"], query_sdf=c["sdf"], return_mask_logits=True)
    assert pred.shape == (130, 4) and logits.shape == (130, 1)
    chunked = model.decode_field_chunked(target_tokens=tgt, cond_global=views["cond_global"], query_pos=c["q"], query_sdf=c["sdf"],
                                         chunk_size=37)
    with torch.no_grad():
        whole = model.decode_field(target_tokens=tgt, cond_global=views["cond_global"], query_pos=c["q"], query_sdf=c["sdf"])
    assert torch.allclose(chunked, whole, atol=1e-5)
    with pytest.raises(ValueError, match="query_sdf"):
        model(context_pos=c["pos"], context_feat=c["feat"], gen_params=c["gen"], query_pos=c["q"])
    with pytest.raises(ValueError, match="point count"):
        model(context_pos=c["pos"], context_feat=c["feat"][:5], gen_params=c["gen"], query_pos=c["q"], query_sdf=c["sdf"])


def test_batched_paths_match_the_single_cloud_paths():
    model, c = _model(), _case()
    trunk = model.trunk
    with torch.no_grad():
        single, single_logits = trunk.forward_single(
            context_pos=c["pos"], context_feat=c["feat"], target_surface_pos=c["s_pos"], target_surface_main_feat=c["s_feat"],
            target_volume_pos=c["v_pos"], target_volume_feat=c["v_feat"], query_pos=c["q"], query_sdf=c["sdf"], gen_params=c["gen"],
            return_mask_logits=True)
        batch, batch_logits = trunk.forward_batch(
            context_pos=_pad2(c["pos"], 100), context_feat=_pad2(c["feat"], 100), context_pos_n=torch.tensor([120, 100]),
            target_surface_pos=_pad2(c["s_pos"], 50), target_surface_main_feat=_pad2(c["s_feat"], 50),
            target_surface_pos_n=torch.tensor([60, 50]), target_volume_pos=_pad2(c["v_pos"], 70),
            target_volume_feat=_pad2(c["v_feat"], 70), target_volume_pos_n=torch.tensor([80, 70]), query_pos=_pad2(c["q"], 90),
            query_sdf=_pad2(c["sdf"], 90), query_pos_n=torch.tensor([130, 90]), gen_params=torch.stack([c["gen"]] * 2),
            return_mask_logits=True)
        short = trunk.forward_single(
            context_pos=c["pos"][:100], context_feat=c["feat"][:100], target_surface_pos=c["s_pos"][:50],
            target_surface_main_feat=c["s_feat"][:50], target_volume_pos=c["v_pos"][:70], target_volume_feat=c["v_feat"][:70],
            query_pos=c["q"][:90], query_sdf=c["sdf"][:90], gen_params=c["gen"])
    assert torch.allclose(batch[0], single, atol=1e-5) and torch.allclose(batch_logits[0], single_logits, atol=1e-5)
    assert torch.allclose(batch[1, :90], short, atol=1e-5) and float(batch[1, 90:].abs().max()) == 0
    # predictor: a batch of two context sets against shared target positions
    ctx = model.context_encoder.forward_batched(context_pos=_pad2(c["pos"], 100), context_feat=_pad2(c["feat"], 100),
                                                context_pos_n=torch.tensor([120, 100])).tokens
    tgt_pos = torch.rand(15, 3)
    with torch.no_grad():
        both = model.predictor(context_tokens=ctx, target_positions=tgt_pos, cond=c["gen"])
        first = model.predictor(context_tokens=trim_batched_tokens(ctx, 0, int(ctx.mask[0].sum())), target_positions=tgt_pos,
                                cond=c["gen"])
    assert both.shape == (2, 15, 32) and torch.allclose(both[0], first, atol=1e-5)
    with pytest.raises(ValueError, match="does not match"):
        model.predictor(context_tokens=ctx, target_positions=tgt_pos, cond=torch.zeros(3, 2))


@pytest.mark.parametrize("options", [
    dict(pressure_split_head_enabled=True, pressure_head_style="siren", final_refinement_style="siren"),
    dict(pressure_split_head_enabled=True, wall_velocity_gate_enabled=True, extra_sdf_features_enabled=True),
    dict(use_sdf=False, cond_dim=0, out_dim=6)])
def test_decoder_options(options):
    torch.manual_seed(0)
    kw = dict(token_dim=16, hidden_dim=24, num_layers=2, use_sdf=True, cond_dim=3, pe_num_bands=3, cross_attention_heads=2,
              cross_attention_layers=1, cross_attention_k=4, query_chunk_size=7)
    kw.update(options)
    dec = QueryTokenDecoder(**kw).eval()
    tokens = TokenSet(torch.randn(12, 16), torch.rand(12, 3), mask=torch.arange(12) < 9)
    q, sdf = torch.rand(20, 3), torch.linspace(-1, 1, 20)[:, None]
    cond = torch.randn(20, 3) if kw["cond_dim"] else None
    pred, emb = dec(query_pos=q, query_sdf=sdf if kw["use_sdf"] else None, target_tokens=tokens, cond=cond)
    assert pred.shape == (20, kw.get("out_dim", 4) if not kw.get("pressure_split_head_enabled") else 4) and emb.shape == (20, 16)
    if options.get("wall_velocity_gate_enabled"):
        dec.wall_velocity_gate_enabled = False
        raw = dec(query_pos=q, query_sdf=sdf, target_tokens=tokens, cond=cond)[0]
        gate = torch.sigmoid(20.0 * sdf)
        assert torch.allclose(pred[:, :3], raw[:, :3] * gate, atol=1e-6) and torch.allclose(pred[:, 3:], raw[:, 3:])
    with pytest.raises(ValueError, match="at least one valid token"):
        dec(query_pos=q, query_sdf=sdf, target_tokens=tokens.with_updates(mask=torch.zeros(12, dtype=torch.bool)), cond=cond)
    with pytest.raises(ValueError, match="pressure_head_style"):
        QueryTokenDecoder(token_dim=8, pressure_head_style="kan")


def test_prototype_anchors_and_checkpoint(tmp_path):
    torch.manual_seed(0)
    blobs = torch.cat([torch.randn(80, 3) * 0.05 + c for c in torch.tensor([[0.0, 0, 0], [1, 0, 0], [0, 1, 0], [0, 0, 1]])])
    centres = kmeans_centres(blobs, num_clusters=4, num_iters=8, seed=3)
    assert (torch.cdist(centres, torch.tensor([[0.0, 0, 0], [1, 0, 0], [0, 1, 0], [0, 0, 1]])).min(0).values < 0.05).all()
    data = [{"surface_pos": torch.rand(40, 3), "surface_main_feat": torch.randn(40, 2), "volume_pos": torch.rand(60, 3),
             "volume_feat": torch.randn(60, 2)} for _ in range(3)]
    cfg = dict(prototype_anchor_count=8, prototype_source_strategy="fps", prototype_source_max_point_tokens=16,
               prototype_anchor_path=str(tmp_path / "anchors" / "target.npz"))
    anchors = build_target_prototype_anchors(train_dataset=data, target_cfg=cfg, output_path=cfg["prototype_anchor_path"], seed=1)
    assert anchors.shape == (8, 3) and bool((anchors[1:, 0] >= anchors[:-1, 0]).all())
    assert torch.equal(ensure_target_prototype_anchors(train_dataset=[], target_cfg=cfg), anchors)      # loaded, not rebuilt
    enc = dict(_ENC, tokenizer_strategy="data_prototype_cluster", tokenizer_prototype_coords=anchors)
    tgt = TargetTransformer(point_input_dim=2, **enc).eval()
    out = tgt(surface_pos=data[0]["surface_pos"], surface_main_feat=data[0]["surface_main_feat"], volume_pos=data[0]["volume_pos"],
              volume_feat=data[0]["volume_feat"])
    assert out.tokens.features.shape == (8, 32) and torch.allclose(out.tokens.coords, anchors)
    tgt.save(str(tmp_path / "tgt.mdlus"))
    again = Module.from_checkpoint(str(tmp_path / "tgt.mdlus")).eval()
    assert torch.allclose(again.encoder.tokenizer.prototype_coords, anchors)
    model, c = _model(), _case()
    model.save(str(tmp_path / "aerojepa.mdlus"))
    clone = Module.from_checkpoint(str(tmp_path / "aerojepa.mdlus")).eval()
    args = dict(context_pos=c["pos"], context_feat=c["feat"], gen_params=c["gen"], query_pos=c["q"], query_sdf=c["sdf"])
    assert type(clone) is AeroJEPA and torch.equal(clone.predict(**args), model.predict(**args))

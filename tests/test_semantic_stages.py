"""Semantic routing stages, the vision tower, objective graphs and gradient-free training, on CPU.

Oracles are small direct restatements of each stage's definition (loops over rows / windows), not the
vectorised code under test."""
import math

import pytest
import torch
import torch.nn.functional as F

from neuralfn_b200 import presets
from neuralfn_b200.tensor import evolution as evo
from neuralfn_b200.tensor import stages_semantic as S
from neuralfn_b200.tensor import stages_vision as V
from neuralfn_b200.torch_backend import CompiledTorchGraph, TorchTrainConfig, TorchTrainer, build_module
from neuralfn_b200.torch_templates import build_gpt_root_graph

SMALL = dict(vocab_size=64, num_layers=2, model_dim=32, num_heads=4)
DIMS, VEC = S.semantic_geometry("")


def test_geometry_and_registry():
    assert VEC == DIMS + 1 and DIMS >= 2
    for name in ("semantic_projector", "semantic_chunk_projector", "semantic_hasher", "semantic_chunk_hasher", "semantic_moe_router",
                 "semantic_hash_router", "causal_chunk_state", "semantic_moe_jepa_evo_router", "broadcast_chunk_routes",
                 "route_balance_loss", "route_selection_loss", "route_distillation_loss", "routed_attention_experts",
                 "attentionless_decoder", "semantic_alignment_loss", "muse_glimmer_vision_tower", "muse_glimmer_perception_norm",
                 "muse_glimmer_media_scatter"):
        from neuralfn_b200.tensor.ports import MODULE_PORTS
        assert name in MODULE_PORTS, name


def test_projector_shapes_and_chunk_consistency():
    torch.manual_seed(0)
    pooled = build_module("semantic_projector", {"input_dim": 16, "residual_dim": 8, "n_sig_buckets": 32})
    chunked = build_module("semantic_chunk_projector", {"input_dim": 16, "residual_dim": 8, "n_sig_buckets": 32})
    chunked.load_state_dict(pooled.state_dict())
    x = torch.randn(3, 5, 16)
    sem, res, topic = pooled(x)
    assert sem.shape == (3, VEC) and res.shape == (3, 5, 8) and topic.shape == (3, DIMS, pooled.max_terms)
    assert sem[:, :DIMS].abs().max() <= 1 and 0 <= sem[:, DIMS].min() and sem[:, DIMS].max() <= 1
    # the chunk projector applied to the mean-pooled state (one chunk) is the pooled projector
    sem_c, _res_c, topic_c = chunked(x.mean(dim=1, keepdim=True))
    torch.testing.assert_close(sem_c[:, 0], sem)
    torch.testing.assert_close(topic_c[:, 0], topic)
    # first coordinate: argmax of the first head mapped onto [-1, 1]
    lg = pooled.topic_heads[0](x.mean(1))
    n = pooled.term_counts[0]
    torch.testing.assert_close(sem[:, 0], 2.0 * lg.argmax(-1).float() / (n - 1) - 1.0)


def test_hasher_matches_bitwise_definition():
    h = build_module("semantic_hasher", {"dim": VEC, "tables": 3, "planes": 5, "seed": 7})
    v = torch.randn(4, VEC)
    out = h(v)
    for b in range(4):
        for t in range(3):
            bits = [(h.proj[t, p] @ v[b] > 0).item() for p in range(5)]
            assert out[b, t].item() == sum(int(bit) << p for p, bit in enumerate(bits))
    hc = build_module("semantic_chunk_hasher", {"dim": VEC, "tables": 3, "planes": 5, "seed": 7})
    torch.testing.assert_close(hc(v.view(2, 2, VEC)).view(4, 3), out)


def test_causal_chunk_state_modes():
    x = torch.randn(2, 10, 4)
    prefix = build_module("causal_chunk_state", {"chunk_size": 4, "mode": "prefix"})(x)
    mean = build_module("causal_chunk_state", {"chunk_size": 4, "mode": "mean"})(x)
    assert prefix.shape == mean.shape == (2, 3, 4)
    torch.testing.assert_close(prefix[:, 0], x[:, 0])                       # nothing before the first chunk but token 0
    torch.testing.assert_close(prefix[:, 1], x[:, :4].mean(1))               # tokens before position 4
    torch.testing.assert_close(prefix[:, 2], x[:, :8].mean(1))
    torch.testing.assert_close(mean[:, 2], x[:, 8:10].mean(1))               # ragged last chunk
    # causality: chunk c's prefix state ignores tokens of chunk c and later
    y = x.clone()
    y[:, 4:] += 100.0
    torch.testing.assert_close(build_module("causal_chunk_state", {"chunk_size": 4})(y)[:, 1], prefix[:, 1])


def test_hash_router_forces_target_dimensions():
    torch.manual_seed(1)
    r = build_module("semantic_hash_router", {"n_experts": DIMS, "semantic_dim": VEC, "top_k": 2, "tables": 2, "n_buckets": 16})
    topic = torch.randn(3, DIMS, 10)
    tgt = torch.full((3, VEC), -100)
    tgt[0, 2] = 1                        # one forced dimension -> one live slot
    tgt[1, 1], tgt[1, 4], tgt[1, 5] = 0, 0, 0    # three forced, top_k = 2 of them by score
    w, idx = r(torch.zeros(3, VEC), torch.randint(0, 16, (3, 2)), topic, tgt)
    assert idx[0, 0].item() == 2 and w[0, 0].item() == pytest.approx(1.0) and w[0, 1].item() == 0.0
    assert set(idx[1].tolist()) <= {1, 4, 5} and w[1].sum().item() == pytest.approx(1.0)
    conf = torch.stack([F.softmax(topic[2, i, :r.term_counts[i]], -1).max() for i in range(DIMS)])
    assert set(idx[2].tolist()) == set(conf.topk(2).indices.tolist())        # unforced row: plain top-k of confidences
    with pytest.raises(ValueError):
        build_module("semantic_hash_router", {"n_experts": DIMS + 1})


def test_chunk_router_layout_and_losses():
    torch.manual_seed(2)
    shared, free, k = 2, 3, 2
    r = build_module("semantic_moe_jepa_evo_router", {"semantic_dim": VEC, "top_k": k, "shared_experts": shared, "free_experts": free,
                                                      "tables": 2, "n_buckets": 16})
    b, c = 2, 3
    sem, topic = torch.randn(b, c, VEC), torch.randn(b, c, DIMS, 10)
    tgt = torch.full((b, VEC), -100)
    tgt[0, 3] = 2
    w, idx, logits = r(sem, torch.randint(0, 16, (b, c, 2)), topic, tgt)
    total = shared + DIMS + free
    assert w.shape == idx.shape == (b, c, shared + k) and logits.shape == (b, c, total)
    assert (idx[..., :shared] == torch.arange(shared)).all()                # shared experts always first
    assert (idx[0, :, shared] == shared + 3).all()                          # forced semantic expert of row 0
    assert ((idx[..., shared:] >= shared) & (idx[..., shared:] < total)).all()
    torch.testing.assert_close(w.sum(-1), torch.ones(b, c))
    assert len(r.route_evo_parameters()) == 6
    bal = build_module("route_balance_loss", {})(logits)
    dens = F.softmax(logits.reshape(-1, total), -1).mean(0)
    torch.testing.assert_close(bal, total * (dens ** 2).sum())
    sel = build_module("route_selection_loss", {"shared_experts": shared, "free_experts": free})(logits, tgt)
    expect = F.binary_cross_entropy_with_logits(logits[0, :, shared + 3], torch.ones(c))
    torch.testing.assert_close(sel, expect)
    assert build_module("route_selection_loss", {"shared_experts": shared, "free_experts": free})(logits, torch.full((b, VEC), -100)) == 0
    dist = build_module("route_distillation_loss", {"shared_experts": shared, "free_experts": free})(logits, topic)
    assert dist.ndim == 0 and dist >= 0
    bw, bi = build_module("broadcast_chunk_routes", {"chunk_size": 4})(torch.zeros(b, 10, 8), w, idx)
    assert bw.shape == (b, 10, shared + k) and (bi[:, 5] == idx[:, 1]).all() and (bi[:, 9] == idx[:, 2]).all()


def test_alignment_loss_matches_per_dimension_mean():
    torch.manual_seed(3)
    loss = build_module("semantic_alignment_loss", {})
    logits = torch.randn(4, DIMS, 10, requires_grad=True)
    tgt = torch.full((4, VEC), -100)
    tgt[0, 0], tgt[1, 0], tgt[2, 1] = 1, 3, 0
    tgt[3, 1] = 99                       # out of range: ignored
    counts = S._term_counts(S._vocab(""))
    d0 = F.cross_entropy(logits[:2, 0, :counts[0]], tgt[:2, 0])
    d1 = F.cross_entropy(logits[2:3, 1, :counts[1]], tgt[2:3, 1])
    got = loss(logits, tgt)
    torch.testing.assert_close(got, (d0 + d1) / DIMS)    # dimensions without a target contribute zero
    got.backward()
    assert logits.grad[3].abs().sum() == 0


def test_routed_attention_experts_against_loop():
    torch.manual_seed(4)
    m = build_module("routed_attention_experts", {"model_dim": 16, "num_heads": 4, "num_kv_heads": 2, "experts": 3, "top_k": 2})
    x = torch.randn(3, 6, 16)
    w = torch.tensor([[0.7, 0.3], [1.0, 0.0], [0.5, 0.5]])
    idx = torch.tensor([[0, 2], [1, 1], [2, 0]])
    out = m(x, w.unsqueeze(1), idx.unsqueeze(1))
    ref = torch.zeros_like(x)
    for b in range(3):
        for s in range(2):
            ref[b] += w[b, s] * m._expert(x[b:b + 1], int(idx[b, s]))[0]
    torch.testing.assert_close(out, ref, atol=1e-5, rtol=1e-5)
    # causal: the first position's output does not depend on later tokens
    y = x.clone()
    y[:, 1:] += 1.0
    torch.testing.assert_close(m(y, w, idx)[:, 0], out[:, 0], atol=1e-5, rtol=1e-5)


def test_semantic_targets_from_tokens_majority():
    st = S.SemanticTargetsFromTokensStage(64, period=1)
    tok = torch.tensor([[0, 0, DIMS, 5, 5, 5]])
    out = st(tok)
    assert out.shape == (1, VEC)
    col0 = st.table[tok[0], 0]
    vals = col0[col0 >= 0]
    assert out[0, 0].item() == vals.mode().values.item()


# ------------------------------------------------------------------------------ vision --
def _naive_tower(t: V.MuseGlimmerVisionTowerStage, pixels, grid):
    """Per-medium, per-window loops with explicit bilinear corners."""
    side = t.window_patches
    table = t.position_embedding.weight
    pos = []
    for tt, h, w in grid.tolist():
        rows = torch.zeros(h * w, table.shape[1])
        for i in range(h):
            for j in range(w):
                y, x = (i + 0.5) * side / h - 0.5, (j + 0.5) * side / w - 0.5
                y0, x0 = math.floor(y), math.floor(x)
                for yy, wy in ((y0, 1 - (y - y0)), (y0 + 1, y - y0)):
                    for xx, wx in ((x0, 1 - (x - x0)), (x0 + 1, x - x0)):
                        if 0 <= yy < side and 0 <= xx < side:
                            rows[i * w + j] += wy * wx * table[yy * side + xx]
        pos.append(rows.repeat(tt, 1))
    h_all = t.pre_norm(t.patch_embedding(pixels) + torch.cat(pos))
    outs, off = [], 0
    last = len(t.layers) - 1
    for tt, h, w in grid.tolist():
        n = tt * h * w
        x = h_all[off:off + n]
        off += n
        coords = [(f, i, j) for f in range(tt) for i in range(h) for j in range(w)]
        xy = torch.tensor([[j + 1, i + 1] for _f, i, j in coords])
        for li, layer in enumerate(t.layers):
            full = (li + 1) % 4 == 0 or li == last
            groups = {}
            for p, (f, i, j) in enumerate(coords):
                key = 0 if full else (f, i // side, j // side)
                groups.setdefault(key, []).append(p)
            a = layer.attn
            hn = layer.norm1(x)
            cos, sin = a.rope_tables(xy, x.dtype)
            q = a._rotate(a.q_proj(hn).view(n, a.num_heads, a.head_dim), cos, sin)
            k = a._rotate(a.k_proj(hn).view(n, a.num_heads, a.head_dim), cos, sin)
            v = a.v_proj(hn).view(n, a.num_heads, a.head_dim)
            o = torch.zeros_like(q)
            for members in groups.values():
                ids = torch.tensor(members)
                o[ids] = F.scaled_dot_product_attention(q[ids].transpose(0, 1), k[ids].transpose(0, 1), v[ids].transpose(0, 1)).transpose(0, 1)
            x = x + a.proj(o.reshape(n, -1))
            x = x + layer.fc2(F.gelu(layer.fc1(layer.norm2(x))))
        x = t.post_norm(x)
        m = t.merge_size
        merged = []
        for f in range(tt):
            for bi in range(h // m):
                for bj in range(w // m):
                    cell = [x[f * h * w + (bi * m + di) * w + bj * m + dj] for di in range(m) for dj in range(m)]
                    merged.append(torch.stack(cell, dim=-1).reshape(-1))
        outs.append(torch.stack(merged))
    return torch.cat(outs)


def test_vision_tower_matches_windowed_loops():
    torch.manual_seed(5)
    tower = build_module("muse_glimmer_vision_tower", {"hidden_size": 32, "intermediate_size": 48, "num_heads": 4, "num_layers": 5,
                                                       "patch_size": 2, "patch_temporal": 1, "merge_size": 2, "pos_emb_height": 4,
                                                       "pos_emb_width": 4})
    grid = torch.tensor([[1, 6, 4], [2, 4, 8]])            # windows of 4x4 patches: ragged tiles on the first image
    pixels = torch.randn(int(grid.prod(-1).sum()), 12)
    out = tower(pixels, grid)
    assert out.shape == (int(grid.prod(-1).sum()) // 4, 32 * 4)
    torch.testing.assert_close(out, _naive_tower(tower, pixels, grid), atol=2e-5, rtol=1e-4)
    out.sum().backward()
    assert tower.position_embedding.weight.grad.abs().sum() > 0
    with pytest.raises(ValueError):
        tower(pixels, torch.tensor([[1, 5, 4]]))


def test_perception_norm_and_media_scatter():
    x = torch.randn(5, 16) * 3
    y = build_module("muse_glimmer_perception_norm", {"eps": 1e-5})(x)
    torch.testing.assert_close(y, x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5))
    sc = build_module("muse_glimmer_media_scatter", {"token_id": 7})
    emb = torch.randn(2, 4, 3, requires_grad=True)
    ids = torch.tensor([[1, 7, 7, 2], [7, 3, 4, 5]])
    feats = torch.randn(3, 3, requires_grad=True)
    out = sc(emb, ids, feats)
    torch.testing.assert_close(out[0, 1], feats[0])
    torch.testing.assert_close(out[0, 2], feats[1])
    torch.testing.assert_close(out[1, 0], feats[2])
    torch.testing.assert_close(out[1, 1], emb[1, 1])
    out.sum().backward()
    assert emb.grad[0, 1].abs().sum() == 0 and feats.grad.abs().sum() > 0
    with pytest.raises(ValueError):
        sc(emb, ids, feats[:2])


# -------------------------------------------------------------------- objectives / EMA --
def _data(n=16, t=16):
    d = torch.randint(0, 64, (n, t + 1), generator=torch.Generator().manual_seed(0))
    return d[:, :-1], d[:, 1:]


def test_semantic_presets_contain_semantic_modules():
    want = {"semantic_router_moe": {"semantic_projector", "semantic_hasher", "semantic_hash_router", "broadcast_expert_routes",
                                    "semantic_alignment_loss", "expert_dispatch"},
            "semantic_moe_jepa_evo": {"causal_chunk_state", "semantic_chunk_projector", "semantic_chunk_hasher", "semantic_moe_jepa_evo_router",
                                      "broadcast_chunk_routes", "route_balance_loss", "route_selection_loss", "route_distillation_loss",
                                      "jepa_mask", "latent_mse_loss"},
            "jepa_semantic_hybrid": {"routed_attention_experts", "semantic_hash_router", "jepa_predictor"},
            "llm_jepa": {"jepa_mask", "latent_pool", "jepa_projector", "jepa_predictor", "latent_mse_loss"},
            "diffusion": {"random_timesteps", "mask_scheduler", "denoise_head"}}

    def types(g, acc):
        for node in g.nodes.values():
            nd = node.neuron_def
            if nd.kind == "module":
                acc.add(nd.module_type)
            elif nd.subgraph is not None:
                types(nd.subgraph, acc)
        return acc

    for name, need in want.items():
        g = build_gpt_root_graph(presets.build_preset(name, **SMALL))
        have = types(g, set())
        assert need <= have, (name, need - have)


def test_jepa_target_encoder_is_frozen_copy_and_tracks_ema():
    torch.manual_seed(0)
    spec = presets.build_preset("semantic_moe_jepa_evo", **SMALL)
    spec.ema_decay = 0.5
    spec.route_evo_enabled = False
    graph = build_gpt_root_graph(spec)
    x, y = _data()
    tr = TorchTrainer(graph, TorchTrainConfig(learning_rate=1e-2, epochs=1, batch_size=8, device="cpu", seed=0, max_steps=1))
    infos = []
    tr.train(x, y, on_step=infos.append)          # sem_targets derived from the tokens
    stage = tr.compiled
    online, target = stage.node_modules["online_encoder"], stage.node_modules["target_encoder"]
    assert all(not p.requires_grad for p in target.parameters())
    assert all(p.grad is None for p in target.parameters())
    moved = 0
    for (k, t), (_k2, o) in zip(target.named_parameters(), online.named_parameters()):
        moved += int(not torch.equal(t, o))
    assert moved > 0                               # after one step: target = 0.5 * start + 0.5 * online, not online itself
    assert infos and math.isfinite(infos[0]["loss"])


def test_ar_jepa_target_pairs_with_trunk():
    spec = presets.build_preset("llm_jepa", **SMALL)
    model = CompiledTorchGraph(build_gpt_root_graph(spec))
    tr = TorchTrainer(model.graph, TorchTrainConfig(device="cpu"))
    tr._prepare_ema_targets(model)
    (tp, op, _bufs, target), = tr._ema
    assert len(tp) == len(list(target.parameters())) and len(tp) == len(op)
    for t, o in zip(tp, op):
        assert torch.equal(t, o) and t is not o


def test_route_and_layer_evolution_report_and_keep_best():
    torch.manual_seed(0)
    spec = presets.build_preset("semantic_moe_jepa_evo", **SMALL)
    spec.route_evo_fraction, spec.route_evo_population, spec.route_evo_seed = 1.0, 3, 5
    spec.layer_evo_enabled, spec.layer_evo_fraction, spec.layer_evo_population, spec.layer_evo_index, spec.layer_evo_seed = True, 0.5, 2, 1, 9
    x, y = _data()
    tr = TorchTrainer(build_gpt_root_graph(spec), TorchTrainConfig(learning_rate=1e-3, epochs=1, batch_size=8, device="cpu", seed=0, max_steps=2))
    infos = []
    tr.train(x, y, on_step=infos.append)
    assert len(infos) == 2
    assert all("route_evo" in i and i["route_evo"]["candidate_count"] == 3 for i in infos)
    assert "layer_evo" not in infos[0] and infos[1]["layer_evo"]["layer_index"] == 1
    frozen = evo.layer_evo_parameters(tr.compiled, 1)
    assert frozen and all(not p.requires_grad for p in frozen)


def test_evolutionary_training_improves_and_is_reproducible():
    spec = presets.build_preset("gpt2", vocab_size=16, num_layers=1, model_dim=16, num_heads=2)
    d = torch.randint(0, 16, (8, 9), generator=torch.Generator().manual_seed(1))
    x, y = d[:, :-1], d[:, 1:]

    def run():
        torch.manual_seed(0)
        cfg = TorchTrainConfig(epochs=12, batch_size=8, device="cpu", seed=0, evolutionary=True, evo_population_size=12,
                               evo_mutation_rate=0.2, evo_mutation_scale=0.05, evo_elite_count=2, evo_seed=3)
        tr = TorchTrainer(build_gpt_root_graph(spec), cfg)
        steps = []
        hist = tr.train(x, y, on_step=steps.append)
        return hist, steps, tr

    hist, steps, tr = run()
    assert steps[0]["optimization_method"] == "evolutionary" and steps[0]["learning_rates"] == []
    assert hist[-1] < hist[0]                          # elitism: the best loss never gets worse on a fixed batch
    assert all(b <= a + 1e-6 for a, b in zip(hist, hist[1:]))
    assert tr.graph.torch_config["evolutionary"]["population_size"] == 12
    hist2, _s, _t = run()
    assert hist == hist2
    with pytest.raises(ValueError):
        TorchTrainer(build_gpt_root_graph(spec), TorchTrainConfig(device="cpu", evolutionary=True, evo_elite_count=99)).train(x, y)


def test_population_operators():
    s = evo.EvolutionSettings(population_size=6, mutation_rate=0.0, mutation_scale=0.1, crossover_rate=0.5, tournament_size=2,
                              elite_count=2, seed=1)
    pop = evo.Population(torch.zeros(10), s)
    assert torch.equal(pop.members[0], torch.zeros(10))
    assert ((pop.members[1:] != 0).sum(1) >= 1).all()       # forced mutation even at rate 0
    before = pop.members.clone()
    scores = torch.tensor([5.0, 1.0, float("nan"), 3.0, 2.0, 4.0])
    pop.next_generation(scores)
    assert torch.equal(pop.members[0], before[1]) and torch.equal(pop.members[1], before[4])     # elites in score order
    # children with mutation rate 0 are pure crossovers: every coordinate comes from some parent
    for child in pop.members[2:]:
        assert all((child[j] == before[:, j]).any() for j in range(10))


def test_activation_checkpointing_same_gradients():
    spec = presets.build_preset("llama", **SMALL)
    g = build_gpt_root_graph(spec)
    a, b = CompiledTorchGraph(g), CompiledTorchGraph(g)
    b.load_state_dict(a.state_dict())
    assert b.enable_activation_checkpointing() == 2
    x, y = _data(4)
    la, lb = a(x, y)[0], b(x, y)[0]
    la.backward()
    lb.backward()
    torch.testing.assert_close(la, lb)
    for pa, pb in zip(a.parameters(), b.parameters()):
        torch.testing.assert_close(pa.grad, pb.grad)

"""Template builders, part 3: model-stage graphs of the non-autoregressive and semantic objectives.

Each ``build_*_stage`` returns a graph whose inputs are the objective's data tensors and whose one
output is the scalar loss:

=========================  ==========================================  ==============================
objective                  inputs                                      loss
=========================  ==========================================  ==============================
``seq2seq``                enc_tokens, dec_tokens, target_ids          CE of the decoder
``diffusion``              tokens                                      CE of the denoised tokens
``jepa``                   tokens                                      latent MSE (online vs EMA target)
``ar_jepa``                tokens, target_ids                          a*CE + j*latent MSE
``jepa_semantic``          tokens, target_ids, sem_targets             a*CE + j*MSE + s*alignment
``semantic_router``        tokens, target_ids, sem_targets             CE + s*alignment
``semantic_router_jepa``   tokens, target_ids, sem_targets             a*CE + j*MSE + s*alignment
``semantic_dense_jepa_evo``tokens, target_ids, sem_targets             a*CE + j*MSE + s*alignment
``semantic_moe_jepa_evo``  tokens, target_ids, sem_targets             the above + r*(balance+selection+distillation)
=========================  ==========================================  ==============================

Node ids ``online_encoder`` / ``target_encoder`` mark the pair that the trainer keeps in EMA lock-step
(target initialised from online, frozen, updated after every optimizer step). Topologies follow the
reference's stage builders (``neuralfn/torch_templates.py:1759-2026`` seq2seq / diffusion / JEPA,
``:2026-2280`` AR+JEPA, ``:2280-3600`` the semantic family), written with ``GraphBuilder``.
"""
from __future__ import annotations

import copy

from .config import ModelSpec
from .graph import NeuronGraph
from .torch_templates import GraphBuilder, Ref, _norm, build_decoder_block_graph
from .torch_templates_roots import BLOCK_FAMILY, _head, _sum_aux

SEMANTIC_OBJECTIVES = ("jepa_semantic", "semantic_router", "semantic_router_jepa", "semantic_dense_jepa_evo",
                       "semantic_moe_jepa_evo")


# --------------------------------------------------------------------------- pieces --
def _embed(b: GraphBuilder, spec: ModelSpec, tokens: Ref, prefix: str = "") -> tuple[Ref, Ref]:
    bs, d = spec.block_spec, spec.model_dim
    emb = b.node("token_embedding", {"vocab_size": spec.vocab_size, "model_dim": d}, [tokens], f"{prefix}token_embedding")
    h: Ref = (emb, 0)
    if bs.pos_encoding == "absolute":
        h = (b.node("absolute_position_embedding", {"max_seq_len": spec.max_position_embeddings, "model_dim": d},
                    [h], f"{prefix}position_embedding"), 0)
    if bs.embedding_norm_kind == "weightless_rms":
        h = (b.node("rms_norm", {"eps": bs.embedding_norm_eps, "force_float32": True}, [h], f"{prefix}embedding_norm"), 0)
    return h, (emb, 1)


def _stack(b: GraphBuilder, spec: ModelSpec, h: Ref, *, prefix: str = "", family: str | None = None,
           context: Ref | None = None, routes: tuple[Ref, Ref] | None = None, routed_experts: int = 0) -> tuple[Ref, list[Ref]]:
    """``num_layers`` decoder blocks bound to one variant-library family; returns (hidden, aux refs)."""
    bs = spec.block_spec
    fam = family or BLOCK_FAMILY.get(bs.family, "transformer_block")
    proto = build_decoder_block_graph(spec, 0, cross=context is not None, routed_experts=routed_experts)
    b.graph.variant_library.setdefault(fam, {})["v0"] = proto
    moe = bs.mlp_type == "moe" and not routed_experts
    auxes: list[Ref] = []
    ins_alias = ["x"] + (["context"] if context is not None else []) + (["routing_weights", "routing_indices"] if routes else [])
    for layer in range(spec.num_layers):
        g = NeuronGraph.from_dict_raw(proto.to_dict())
        ins = [h] + ([context] if context is not None else []) + (list(routes) if routes else [])
        nid = b.subgraph(g, f"{prefix}block_{layer}", ins, f"{prefix}block_{layer}", ins_alias,
                         ["y", "aux_loss"] if moe else ["y"], {"family": fam, "version": "v0"})
        h = (nid, 0)
        if moe:
            auxes.append((nid, 1))
    return h, auxes


def _dense_spec(spec: ModelSpec, *, causal: bool | None = None) -> ModelSpec:
    """A copy whose blocks use a dense MLP (encoders and the JEPA towers never route)."""
    s = copy.copy(spec)
    s.block_spec = copy.copy(spec.block_spec)
    if s.block_spec.mlp_type == "moe":
        s.block_spec.mlp_type = "swiglu"
    if causal is not None:
        s.block_spec.is_causal = causal
    return s


def _mask_cfg(spec: ModelSpec) -> dict:
    return {"mask_ratio": spec.jepa_mask_ratio, "mask_token_id": 0, "mask_strategy": spec.jepa_mask_strategy,
            "num_blocks": spec.jepa_num_blocks, "min_block_ratio": spec.jepa_min_block_ratio,
            "max_block_ratio": spec.jepa_max_block_ratio}


def _weighted_sum(b: GraphBuilder, terms: list[tuple[Ref, float, str]]) -> Ref:
    total: Ref | None = None
    for ref, coef, name in terms:
        scaled: Ref = (b.node("loss_scale", {"coef": float(coef)}, [ref], f"{name}_scaled"), 0)
        total = scaled if total is None else (b.node("aux_loss_add", {"coef": 1.0}, [total, scaled]), 0)
    assert total is not None
    return total


def _semantic_cfg(spec: ModelSpec) -> dict:
    return {"input_dim": spec.model_dim, "semantic_dim": spec.semantic_dim, "residual_dim": spec.semantic_residual_dim,
            "n_sig_buckets": 2 ** min(spec.semantic_n_lsh_planes, 12), "semantic_vocab_ref": spec.semantic_vocab_ref}


def _sem_geometry(spec: ModelSpec) -> tuple[int, int]:
    from .tensor.stages_semantic import semantic_geometry
    return semantic_geometry(spec.semantic_vocab_ref)


# ------------------------------------------------------------------------- encoders --
def build_hidden_backbone_graph(spec: ModelSpec) -> NeuronGraph:
    """tokens -> final-normed hidden states of a dense copy of the trunk."""
    s = _dense_spec(spec)
    b = GraphBuilder("hidden_backbone")
    tokens = b.input("tokens", "tokens")
    h, _w = _embed(b, s, tokens)
    h, _aux = _stack(b, s, h, family="encoder_block")
    return b.outputs(_norm(b, h, s, node_id="final_norm"))


def build_jepa_encoder_graph(spec: ModelSpec) -> NeuronGraph:
    """(tokens, mask) -> latent: backbone, masked mean pool, projector."""
    b = GraphBuilder("jepa_encoder")
    tokens, mask = b.input("tokens", "tokens"), b.input("mask")
    hidden = (b.subgraph(build_hidden_backbone_graph(spec), "backbone", [tokens], "backbone", ["tokens"], ["hidden"]), 0)
    pooled = (b.node("latent_pool", {}, [hidden, mask], "pool"), 0)
    z = b.node("jepa_projector", {"input_dim": spec.model_dim, "latent_dim": spec.jepa_latent_dim}, [pooled], "projector")
    return b.outputs((z, 0))


def build_jepa_semantic_encoder_graph(spec: ModelSpec) -> NeuronGraph:
    """(tokens, mask) -> (semantic vector of the pooled sequence, hidden states, topic logits)."""
    b = GraphBuilder("jepa_semantic_encoder")
    tokens, mask = b.input("tokens", "tokens"), b.input("mask")
    hidden = (b.subgraph(build_hidden_backbone_graph(spec), "backbone", [tokens], "backbone", ["tokens"], ["hidden"]), 0)
    pooled = (b.node("latent_pool", {}, [hidden, mask], "pool"), 0)
    proj = b.node("semantic_projector", _semantic_cfg(spec), [pooled], "sem_proj")
    return b.outputs((proj, 0), hidden, (proj, 2))


def _encoder_pair(b: GraphBuilder, enc: NeuronGraph, tokens: Ref, mask_node: str, outs: list[str]) -> tuple[str, str]:
    online = b.subgraph(NeuronGraph.from_dict_raw(enc.to_dict()), "online_encoder", [(mask_node, 0), (mask_node, 1)],
                        "online_encoder", ["tokens", "mask"], outs)
    target = b.subgraph(NeuronGraph.from_dict_raw(enc.to_dict()), "target_encoder", [tokens, (mask_node, 1)],
                        "target_encoder", ["tokens", "mask"], outs)
    return online, target


# --------------------------------------------------------------------------- stages --
def build_seq2seq_stage(spec: ModelSpec) -> NeuronGraph:
    """Encoder (bidirectional, dense MLP) + decoder (causal self-attention, cross-attention, the
    spec's own MLP incl. MoE) with separate embeddings and an untied head."""
    b = GraphBuilder("model_stage")
    enc_tokens, dec_tokens = b.input("enc_tokens", "tokens"), b.input("dec_tokens", "tokens")
    targets = b.input("target_ids", "tokens")
    enc_spec = _dense_spec(spec, causal=False)
    e, _ = _embed(b, enc_spec, enc_tokens, "enc_")
    e, _ = _stack(b, enc_spec, e, prefix="enc_", family="enc_block")
    d, _ = _embed(b, spec, dec_tokens, "dec_")
    d, auxes = _stack(b, spec, d, prefix="dec_", family="dec_block", context=e)
    d = _norm(b, d, spec, node_id="final_norm")
    logits = (b.node("lm_head", {"model_dim": spec.model_dim, "vocab_size": spec.vocab_size}, [d], "lm_head"), 0)
    loss: Ref = (b.node("token_cross_entropy", {"z_loss_coef": spec.z_loss_coef}, [logits, targets], "loss"), 0)
    return b.outputs(_sum_aux(b, loss, auxes))


def build_diffusion_stage(spec: ModelSpec) -> NeuronGraph:
    """Masked-token diffusion: sample a time step per sequence, replace that share of tokens by the
    mask token, denoise with a bidirectional trunk, score against the clean tokens."""
    s = copy.copy(spec)
    s.block_spec = copy.copy(spec.block_spec)
    s.block_spec.is_causal = False
    b = GraphBuilder("model_stage")
    tokens = b.input("tokens", "tokens")
    t = (b.node("random_timesteps", {}, [tokens], "timesteps"), 0)
    sched = b.node("mask_scheduler", {"vocab_size": spec.vocab_size, "mask_token_id": 0}, [tokens, t], "mask_sched")
    h, _w = _embed(b, s, (sched, 0))
    h, auxes = _stack(b, s, h)
    h = _norm(b, h, s, node_id="final_norm")
    logits = (b.node("denoise_head", {"model_dim": spec.model_dim, "vocab_size": spec.vocab_size}, [h], "denoise_head"), 0)
    loss: Ref = (b.node("token_cross_entropy", {"z_loss_coef": spec.z_loss_coef}, [logits, tokens], "loss"), 0)
    return b.outputs(_sum_aux(b, loss, auxes))


def build_jepa_stage(spec: ModelSpec) -> NeuronGraph:
    b = GraphBuilder("model_stage")
    tokens = b.input("tokens", "tokens")
    mask = b.node("jepa_mask", _mask_cfg(spec), [tokens], "mask")
    online, target = _encoder_pair(b, build_jepa_encoder_graph(spec), tokens, mask, ["latent"])
    pred = (b.node("jepa_predictor", {"latent_dim": spec.jepa_latent_dim}, [(online, 0)], "predictor"), 0)
    return b.outputs((b.node("latent_mse_loss", {}, [pred, (target, 0)], "loss"), 0))


def build_ar_jepa_stage(spec: ModelSpec) -> NeuronGraph:
    """The trunk reads the masked tokens and serves both heads: next-token CE, and a pooled latent
    that predicts the EMA target encoder's latent of the clean tokens."""
    b = GraphBuilder("model_stage")
    tokens, targets = b.input("tokens", "tokens"), b.input("target_ids", "tokens")
    mask = b.node("jepa_mask", _mask_cfg(spec), [tokens], "mask")
    target = b.subgraph(build_jepa_encoder_graph(spec), "target_encoder", [tokens, (mask, 1)], "target_encoder",
                        ["tokens", "mask"], ["latent"])
    h, weight = _embed(b, spec, (mask, 0))
    h, auxes = _stack(b, spec, h)
    h = _norm(b, h, spec, node_id="final_norm")
    pooled = (b.node("latent_pool", {}, [h, (mask, 1)], "online_pool"), 0)
    z = (b.node("jepa_projector", {"input_dim": spec.model_dim, "latent_dim": spec.jepa_latent_dim}, [pooled], "online_projector"), 0)
    pred = (b.node("jepa_predictor", {"latent_dim": spec.jepa_latent_dim}, [z], "predictor"), 0)
    jepa: Ref = (b.node("latent_mse_loss", {}, [pred, (target, 0)], "jepa_loss"), 0)
    ar: Ref = (b.node("token_cross_entropy", {"z_loss_coef": spec.z_loss_coef}, [_head(b, spec, h, weight), targets], "ar_loss"), 0)
    total = _weighted_sum(b, [(ar, spec.ar_loss_coef, "ar_loss"), (jepa, spec.jepa_loss_coef, "jepa_loss")])
    return b.outputs(_sum_aux(b, total, auxes))


def build_jepa_semantic_stage(spec: ModelSpec) -> NeuronGraph:
    """JEPA on semantic vectors, plus hash routing of the online encoder's hidden states into
    sequence-level attention experts that feed the language-model head."""
    bs = spec.block_spec
    vocab_dims, vec_dim = _sem_geometry(spec)
    use_vecs = bool(spec.experimental_semantic_router_vecs)
    b = GraphBuilder("model_stage")
    tokens, targets = b.input("tokens", "tokens"), b.input("target_ids", "tokens")
    sem_targets = b.input("sem_targets", "tokens")
    router_vecs = b.input("semantic_router_vecs") if use_vecs else None
    mask = b.node("jepa_mask", _mask_cfg(spec), [tokens], "mask")
    online, target = _encoder_pair(b, build_jepa_semantic_encoder_graph(spec), tokens, mask,
                                   ["semantic_vec", "hidden", "topic_logits"])
    pred = (b.node("jepa_predictor", {"latent_dim": vec_dim}, [(online, 0)], "predictor"), 0)
    jepa: Ref = (b.node("latent_mse_loss", {}, [pred, (target, 0)], "jepa_loss"), 0)
    buckets = (b.node("semantic_hasher", {"dim": vec_dim, "tables": spec.semantic_n_lsh_tables,
                                          "planes": spec.semantic_n_lsh_planes}, [(online, 0)], "hasher"), 0)
    top_k = min(int(bs.top_k or 2), vocab_dims)
    router = b.node("semantic_hash_router", {
        "n_experts": vocab_dims, "semantic_dim": vec_dim, "top_k": top_k, "tables": spec.semantic_n_lsh_tables,
        "n_buckets": 2 ** min(spec.semantic_n_lsh_planes, 12), "semantic_vocab_ref": spec.semantic_vocab_ref,
        "routing_source": "semantic_vec" if use_vecs else "topic_logits"},
        [router_vecs if router_vecs is not None else (online, 0), buckets, (online, 2), sem_targets], "hash_router")
    experts = b.node("routed_attention_experts", {
        "model_dim": spec.model_dim, "num_heads": bs.num_heads, "num_kv_heads": bs.num_kv_heads or bs.num_heads,
        "rope_base": bs.rope_theta, "qk_gain_init": bs.qk_gain_init, "experts": vocab_dims, "top_k": top_k,
        "is_causal": True}, [(online, 1), (router, 0), (router, 1)], "routed_experts")
    h: Ref = (b.node("residual_add", {"dim": spec.model_dim, "init_scale": 1.0}, [(online, 1), (experts, 0)], "expert_residual"), 0)
    h = _norm(b, h, spec, node_id="final_norm")
    ar: Ref = (b.node("token_cross_entropy", {"z_loss_coef": spec.z_loss_coef}, [_head(b, spec, h, None), targets], "ar_loss"), 0)
    align: Ref = (b.node("semantic_alignment_loss", {"semantic_vocab_ref": spec.semantic_vocab_ref},
                         [(online, 2), sem_targets], "sem_align_loss"), 0)
    return b.outputs(_weighted_sum(b, [(ar, spec.ar_loss_coef, "ar_loss"), (jepa, spec.jepa_loss_coef, "jepa_loss"),
                                       (align, spec.semantic_align_loss_coef, "sem_align_loss")]))


def build_semantic_router_stage(spec: ModelSpec, *, with_jepa: bool = False) -> NeuronGraph:
    """AR MoE trunk whose blocks all reuse one sequence-level semantic route: embedding -> semantic
    projector -> LSH -> hash router -> routes broadcast over positions -> routed blocks. With
    ``with_jepa`` the projector's semantic vector also predicts an EMA target encoder's."""
    bs = spec.block_spec
    vocab_dims, vec_dim = _sem_geometry(spec)
    use_vecs = bool(spec.experimental_semantic_router_vecs)
    b = GraphBuilder("model_stage")
    tokens, targets = b.input("tokens", "tokens"), b.input("target_ids", "tokens")
    sem_targets = b.input("sem_targets", "tokens")
    router_vecs = b.input("semantic_router_vecs") if use_vecs else None
    h, weight = _embed(b, spec, tokens)
    proj = b.node("semantic_projector", _semantic_cfg(spec), [h], "semantic_projector")
    buckets = (b.node("semantic_hasher", {"dim": vec_dim, "tables": spec.semantic_n_lsh_tables,
                                          "planes": spec.semantic_n_lsh_planes}, [(proj, 0)], "semantic_hasher"), 0)
    router = b.node("semantic_hash_router", {
        "n_experts": vocab_dims, "semantic_dim": vec_dim, "top_k": min(int(bs.top_k or 2), vocab_dims),
        "tables": spec.semantic_n_lsh_tables, "n_buckets": 2 ** min(spec.semantic_n_lsh_planes, 12),
        "semantic_vocab_ref": spec.semantic_vocab_ref, "routing_source": "semantic_vec" if use_vecs else "topic_logits"},
        [router_vecs if router_vecs is not None else (proj, 0), buckets, (proj, 2), sem_targets], "semantic_hash_router")
    routes = b.node("broadcast_expert_routes", {}, [h, (router, 0), (router, 1)], "broadcast_routes")
    h, _aux = _stack(b, spec, h, family="semantic_router_block", routes=((routes, 0), (routes, 1)), routed_experts=vocab_dims)
    h = _norm(b, h, spec, node_id="final_norm")
    ar: Ref = (b.node("token_cross_entropy", {"z_loss_coef": spec.z_loss_coef}, [_head(b, spec, h, weight), targets], "ar_loss"), 0)
    align: Ref = (b.node("semantic_alignment_loss", {"semantic_vocab_ref": spec.semantic_vocab_ref},
                         [(proj, 2), sem_targets], "sem_align_loss"), 0)
    terms = [(ar, spec.ar_loss_coef if with_jepa else 1.0, "ar_loss")]
    if with_jepa:
        mask = b.node("jepa_mask", _mask_cfg(spec), [tokens], "mask")
        target = b.subgraph(build_jepa_semantic_encoder_graph(spec), "target_encoder", [tokens, (mask, 1)], "target_encoder",
                            ["tokens", "mask"], ["semantic_vec", "hidden", "topic_logits"])
        pred = (b.node("jepa_predictor", {"latent_dim": vec_dim}, [(proj, 0)], "predictor"), 0)
        terms.append(((b.node("latent_mse_loss", {}, [pred, (target, 0)], "jepa_loss"), 0), spec.jepa_loss_coef, "jepa_loss"))
    terms.append((align, spec.semantic_align_loss_coef, "sem_align_loss"))
    return b.outputs(_weighted_sum(b, terms))


def build_semantic_jepa_evo_stage(spec: ModelSpec, *, moe: bool) -> NeuronGraph:
    """Chunk-level semantic planning. An online / EMA-target encoder pair reads masked / clean tokens;
    causal chunk states of both go through chunk projectors; the online semantic chunk vectors
    predict the target's (JEPA) and are aligned with the semantic targets. ``moe``: the online chunk
    vectors also drive the chunk router ([shared | semantic | free] experts) whose routes, broadcast
    to positions, steer every block's expert MLP, with balance / selection / distillation route
    losses. Otherwise the decoder is a plain dense control."""
    bs = spec.block_spec
    vocab_dims, vec_dim = _sem_geometry(spec)
    chunk = int(spec.route_chunk_size)
    shared, free = int(spec.semantic_shared_experts), int(spec.semantic_free_experts)
    b = GraphBuilder("model_stage")
    tokens, targets = b.input("tokens", "tokens"), b.input("target_ids", "tokens")
    sem_targets = b.input("sem_targets", "tokens")
    mask = b.node("jepa_mask", _mask_cfg(spec), [tokens], "mask")
    online, target = _encoder_pair(b, build_jepa_semantic_encoder_graph(spec), tokens, mask,
                                   ["semantic_vec", "hidden", "topic_logits"])
    o_state = (b.node("causal_chunk_state", {"chunk_size": chunk, "mode": "prefix"}, [(online, 1)], "online_chunk_state"), 0)
    o_proj = b.node("semantic_chunk_projector", _semantic_cfg(spec), [o_state], "online_chunk_projector")
    t_state = (b.node("causal_chunk_state", {"chunk_size": chunk, "mode": "prefix"}, [(target, 1)], "target_chunk_state"), 0)
    t_proj = b.node("semantic_chunk_projector", _semantic_cfg(spec), [t_state], "target_chunk_projector")
    h, weight = _embed(b, spec, tokens)
    terms: list[tuple[Ref, float, str]] = []
    router = None
    if moe:
        buckets = (b.node("semantic_chunk_hasher", {"dim": vec_dim, "tables": spec.semantic_n_lsh_tables,
                                                    "planes": spec.semantic_n_lsh_planes}, [(o_proj, 0)], "online_chunk_hasher"), 0)
        router = b.node("semantic_moe_jepa_evo_router", {
            "semantic_dim": vec_dim, "top_k": int(bs.top_k or 2), "shared_experts": shared, "free_experts": free,
            "tables": spec.semantic_n_lsh_tables, "n_buckets": 2 ** min(spec.semantic_n_lsh_planes, 12),
            "semantic_vocab_ref": spec.semantic_vocab_ref}, [(o_proj, 0), buckets, (o_proj, 2), sem_targets], "semantic_moe_router")
        routes = b.node("broadcast_chunk_routes", {"chunk_size": chunk}, [h, (router, 0), (router, 1)], "broadcast_chunk_routes")
        h, _aux = _stack(b, spec, h, family="semantic_moe_jepa_evo_block", routes=((routes, 0), (routes, 1)),
                         routed_experts=shared + vocab_dims + free)
    else:
        h, _aux = _stack(b, _dense_spec(spec), h, family="semantic_dense_jepa_evo_block")
    h = _norm(b, h, spec, node_id="final_norm")
    ar: Ref = (b.node("token_cross_entropy", {"z_loss_coef": spec.z_loss_coef}, [_head(b, spec, h, weight), targets], "ar_loss"), 0)
    pred = (b.node("jepa_predictor", {"latent_dim": vec_dim}, [(o_proj, 0)], "route_predictor"), 0)
    jepa: Ref = (b.node("latent_mse_loss", {}, [pred, (t_proj, 0)], "jepa_loss"), 0)
    align: Ref = (b.node("semantic_alignment_loss", {"semantic_vocab_ref": spec.semantic_vocab_ref},
                         [(o_proj, 2), sem_targets], "sem_align_loss"), 0)
    terms += [(ar, spec.ar_loss_coef, "ar_loss"), (jepa, spec.jepa_loss_coef, "jepa_loss"),
              (align, spec.semantic_align_loss_coef, "sem_align_loss")]
    if router is not None:
        r = float(bs.router_aux_loss_coef)
        cfg = {"semantic_vocab_ref": spec.semantic_vocab_ref, "shared_experts": shared, "free_experts": free}
        terms += [((b.node("route_balance_loss", {}, [(router, 2)], "route_balance_loss"), 0), r, "route_balance_loss"),
                  ((b.node("route_selection_loss", cfg, [(router, 2), sem_targets], "route_selection_loss"), 0), r, "route_selection_loss"),
                  ((b.node("route_distillation_loss", cfg, [(router, 2), (t_proj, 2)], "route_distill_loss"), 0), r, "route_distill_loss")]
    return b.outputs(_weighted_sum(b, terms))


def build_objective_stage(spec: ModelSpec) -> NeuronGraph | None:
    """Stage graph of the template's objective, or ``None`` for plain next-token training."""
    obj = spec.template.objective
    if obj == "seq2seq":
        return build_seq2seq_stage(spec)
    if obj == "diffusion":
        return build_diffusion_stage(spec)
    if obj == "jepa":
        return build_jepa_stage(spec)
    if obj == "ar_jepa":
        return build_ar_jepa_stage(spec)
    if obj == "jepa_semantic":
        return build_jepa_semantic_stage(spec)
    if obj == "semantic_router":
        return build_semantic_router_stage(spec)
    if obj == "semantic_router_jepa":
        return build_semantic_router_stage(spec, with_jepa=True)
    if obj == "semantic_dense_jepa_evo":
        return build_semantic_jepa_evo_stage(spec, moe=False)
    if obj == "semantic_moe_jepa_evo":
        return build_semantic_jepa_evo_stage(spec, moe=True)
    return None

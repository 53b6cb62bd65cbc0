"""Template builders, part 2: model-stage graphs and root graphs per objective
(pre-training, SFT, DPO, reward model, PPO). See ``torch_templates`` for the block level."""
from __future__ import annotations

import copy
from dataclasses import asdict
from typing import Any

from .config import ModelSpec, spec_from_dict
from .graph import NeuronGraph
from .torch_templates import GraphBuilder, Ref, _norm, build_decoder_block_graph

BLOCK_FAMILY = {"gpt2": "gpt2", "nanogpt": "nanogpt", "llama": "llama", "mixllama": "mixllama",
                "muse_glimmer": "muse_glimmer"}


def _block_versions(spec: ModelSpec) -> list[tuple[int, NeuronGraph]]:
    """Distinct block graphs: layers whose attention schedule / family behaviour differs get
    their own library version (hybrid local/global stacks, Jamba's alternating layers)."""
    bs = spec.block_spec
    period = len(bs.layer_attention_pattern) or (2 if bs.family == "jamba" else 1)
    return [(i, build_decoder_block_graph(spec, i)) for i in range(min(period, max(spec.num_layers, 1)))]


def _trunk(b: GraphBuilder, spec: ModelSpec, tokens: Ref) -> tuple[Ref, Ref, list[Ref]]:
    """tokens -> (final hidden, embedding weight ref, aux loss refs)."""
    bs = spec.block_spec
    d = spec.model_dim
    if bs.family == "hnet" or spec.template.tokenization == "byte_hnet":
        emb = b.node("byte_patch_embed", {"model_dim": d, "patch_size": bs.byte_patch_size,
                                          "stride": bs.byte_patch_stride, "vocab_size": spec.vocab_size},
                     [tokens], "byte_patch_embed")
        h: Ref = (emb, 0)
        weight: Ref | None = None
    else:
        emb = b.node("token_embedding", {"vocab_size": spec.vocab_size, "model_dim": d}, [tokens], "token_embedding")
        h, weight = (emb, 0), (emb, 1)
    if bs.pos_encoding == "absolute":
        h = (b.node("absolute_position_embedding", {"max_seq_len": spec.max_position_embeddings, "model_dim": d},
                    [h], "position_embedding"), 0)
    if bs.embedding_norm_kind == "weightless_rms":
        h = (b.node("rms_norm", {"eps": bs.embedding_norm_eps, "force_float32": True}, [h], "embedding_norm"), 0)
    family = BLOCK_FAMILY.get(bs.family, "transformer_block")
    versions = _block_versions(spec)
    library = {f"v{idx}": g for idx, g in versions}
    b.graph.variant_library[family] = library
    period = len(versions)
    auxes: list[Ref] = []
    is_moe = bs.mlp_type == "moe"
    if bs.family == "universal":
        h = (b.node("universal_transformer", {"model_dim": d, "num_heads": bs.num_heads,
                                              "mlp_mult": bs.mlp_multiplier, "max_steps": spec.max_recurrence_steps,
                                              "halt_epsilon": spec.halt_epsilon}, [h], "universal_block"), 0)
    else:
        for layer in range(spec.num_layers):
            idx, _g = versions[layer % period]
            block_graph = NeuronGraph.from_dict_raw(library[f"v{idx}"].to_dict())
            out_aliases = ["y", "aux_loss"] if is_moe else ["y"]
            nid = b.subgraph(block_graph, f"block_{layer}", [h], f"block_{layer}", ["x"], out_aliases,
                             {"family": family, "version": f"v{idx}"})
            h = (nid, 0)
            if is_moe:
                auxes.append((nid, 1))
    if bs.family == "hnet" or spec.template.tokenization == "byte_hnet":
        h = (b.node("byte_patch_merge", {"patch_size": bs.byte_patch_size, "stride": bs.byte_patch_stride},
                    [h, tokens], "byte_patch_merge"), 0)
    final_spec = spec
    if bs.family == "muse_glimmer":
        final_spec = copy.copy(spec)
        final_spec.block_spec = copy.copy(bs)
        final_spec.block_spec.centered_rms_norm = False
    h = _norm(b, h, final_spec, node_id="final_norm")
    return h, weight, auxes  # type: ignore[return-value]


def _head(b: GraphBuilder, spec: ModelSpec, hidden: Ref, weight: Ref | None) -> Ref:
    if spec.tie_embeddings and weight is not None:
        logits: Ref = (b.node("tied_lm_head", {}, [hidden, weight], "lm_head"), 0)
    else:
        logits = (b.node("lm_head", {"model_dim": spec.model_dim, "vocab_size": spec.vocab_size}, [hidden], "lm_head"), 0)
    if spec.output_multiplier != 1.0:
        logits = (b.node("tensor_scale", {"scale": spec.output_multiplier}, [logits], "output_multiplier"), 0)
    if spec.logit_softcap > 0:
        logits = (b.node("logit_softcap", {"softcap": spec.logit_softcap}, [logits], "logit_softcap"), 0)
    return logits


def _sum_aux(b: GraphBuilder, loss: Ref, auxes: list[Ref]) -> Ref:
    for a in auxes:
        loss = (b.node("aux_loss_add", {"coef": 1.0}, [loss, a]), 0)
    return loss


def _torch_config(spec: ModelSpec, extra: dict[str, Any] | None = None) -> dict[str, Any]:
    cfg = {"template_spec": spec.to_dict(), "amp_dtype": "bfloat16"}
    if spec.finetune is not None:
        cfg["finetune_spec"] = asdict(spec.finetune)
    cfg.update(extra or {})
    return cfg


def build_model_stage_graph(spec: ModelSpec, *, with_loss: bool = True) -> NeuronGraph:
    """(tokens[, target_ids]) -> loss, or tokens -> logits when ``with_loss`` is False."""
    b = GraphBuilder("model_stage")
    tokens = b.input("tokens", "tokens")
    targets = b.input("target_ids", "tokens") if with_loss else None
    hidden, weight, auxes = _trunk(b, spec, tokens)
    logits = _head(b, spec, hidden, weight)
    if not with_loss:
        return b.outputs(logits)
    loss: Ref = (b.node("token_cross_entropy", {"z_loss_coef": spec.z_loss_coef}, [logits, targets], "loss"), 0)
    return b.outputs(_sum_aux(b, loss, auxes))


def build_gpt_root_graph(model_spec: ModelSpec | None = None, **kwargs: Any) -> NeuronGraph:
    """Root training graph for a preset. Dispatches on the fine-tune objective when present."""
    spec = model_spec or ModelSpec(**kwargs)
    objective = spec.finetune.objective if spec.finetune is not None else "pretrain"
    if objective == "sft":
        return build_sft_root_graph(spec)
    if objective == "dpo":
        return build_dpo_root_graph(spec)
    if objective == "reward_model":
        return build_reward_model_root_graph(spec)
    if objective == "ppo":
        return build_ppo_root_graph(spec)
    if objective == "pretrain" and spec.template.objective in ("sft", "dpo", "reward_model", "ppo"):
        return {"sft": build_sft_root_graph, "dpo": build_dpo_root_graph, "reward_model": build_reward_model_root_graph,
                "ppo": build_ppo_root_graph}[spec.template.objective](spec)
    from .torch_templates_objectives import build_objective_stage
    g = build_objective_stage(spec) or build_model_stage_graph(spec)
    g.name = f"{spec.template.backbone}_root"
    g.torch_config = _torch_config(spec)
    g.validate()
    return g


def build_gpt_template_payload(model_spec: ModelSpec | None = None, **kwargs: Any) -> dict[str, Any]:
    """JSON payload of the root graph plus the spec it was built from (editor / REST format)."""
    spec = model_spec or ModelSpec(**kwargs)
    graph = build_gpt_root_graph(spec)
    return {"graph": graph.to_dict(), "model_spec": spec.to_dict(), "template": asdict(spec.template)}


def build_model_spec_from_config(torch_config: dict[str, Any]) -> ModelSpec:
    """Recover the ``ModelSpec`` stored in a graph's ``torch_config['template_spec']``."""
    raw = (torch_config or {}).get("template_spec")
    if not raw:
        raise ValueError("graph torch_config has no template_spec")
    return spec_from_dict(raw)


# ------------------------------------------------------------------ post-training roots --
def build_sft_root_graph(spec: ModelSpec) -> NeuronGraph:
    """(tokens, target_ids, loss_mask) -> response-only masked cross-entropy."""
    b = GraphBuilder("sft_root")
    tokens, targets, mask = b.input("tokens", "tokens"), b.input("target_ids", "tokens"), b.input("loss_mask")
    hidden, weight, auxes = _trunk(b, spec, tokens)
    logits = _head(b, spec, hidden, weight)
    loss: Ref = (b.node("masked_token_cross_entropy", {"ignore_index": -100}, [logits, targets, mask], "loss"), 0)
    g = b.outputs(_sum_aux(b, loss, auxes))
    g.torch_config = _torch_config(spec, {"objective": "sft"})
    g.validate()
    return g


def build_dpo_root_graph(spec: ModelSpec) -> NeuronGraph:
    """Chosen/rejected batches are concatenated, run once through the policy (and the frozen
    reference), split, reduced to sequence log-probs and fed to the pairwise loss."""
    ft = spec.finetune
    b = GraphBuilder("dpo_root")
    names = ("chosen_tokens", "chosen_targets", "chosen_mask", "rejected_tokens", "rejected_targets", "rejected_mask")
    ct, cy, cm, rt, ry, rm = (b.input(n, "tokens" if "mask" not in n else "tensor") for n in names)
    toks = (b.node("pair_batch_concat", {}, [ct, rt], "concat_tokens"), 0)
    tgts = (b.node("pair_batch_concat", {}, [cy, ry], "concat_targets"), 0)
    msks = (b.node("pair_batch_concat", {}, [cm, rm], "concat_masks"), 0)
    hidden, weight, auxes = _trunk(b, spec, toks)
    logits = _head(b, spec, hidden, weight)
    pol = (b.node("sequence_logp", {}, [logits, tgts, msks], "policy_logp"), 0)
    ref_logits = (b.node("reference_forward", {"ref_graph_path": ft.ref_graph_path if ft else "",
                                               "ref_weights_path": ft.ref_checkpoint if ft else "",
                                               "vocab_size": spec.vocab_size, "model_dim": spec.model_dim},
                         [toks], "reference"), 0)
    ref = (b.node("sequence_logp", {}, [ref_logits, tgts, msks], "reference_logp"), 0)
    ps = b.node("pair_batch_split", {}, [pol], "split_policy")
    rs = b.node("pair_batch_split", {}, [ref], "split_reference")
    loss = b.node("dpo_pairwise_loss", {"beta": ft.beta if ft else 0.1,
                                        "label_smoothing": ft.dpo_label_smoothing if ft else 0.0,
                                        "loss_type": ft.dpo_loss_type if ft else "sigmoid"},
                  [(ps, 0), (ps, 1), (rs, 0), (rs, 1)], "dpo_loss")
    g = b.outputs(_sum_aux(b, (loss, 0), auxes))
    g.torch_config = _torch_config(spec, {"objective": "dpo"})
    g.validate()
    return g


def build_reward_model_root_graph(spec: ModelSpec) -> NeuronGraph:
    """Bradley-Terry reward model: masked last-token scalar head on chosen vs rejected."""
    b = GraphBuilder("reward_model_root")
    ct, cm, rt, rm = (b.input(n, "tokens" if "tokens" in n else "tensor")
                      for n in ("chosen_tokens", "chosen_mask", "rejected_tokens", "rejected_mask"))
    toks = (b.node("pair_batch_concat", {}, [ct, rt], "concat_tokens"), 0)
    msks = (b.node("pair_batch_concat", {}, [cm, rm], "concat_masks"), 0)
    hidden, _w, auxes = _trunk(b, spec, toks)
    reward = (b.node("masked_reward_head", {"model_dim": spec.model_dim}, [hidden, msks], "reward_head"), 0)
    sp = b.node("pair_batch_split", {}, [reward], "split_reward")
    loss = b.node("preference_bce_loss", {}, [(sp, 0), (sp, 1)], "loss")
    g = b.outputs(_sum_aux(b, (loss, 0), auxes))
    g.torch_config = _torch_config(spec, {"objective": "reward_model"})
    g.validate()
    return g


def build_reward_scoring_graph(spec: ModelSpec) -> NeuronGraph:
    """(tokens, mask) -> one reward per row: the trunk and head of the reward-model root without the pair loss
    (same node ids, so the trained weights load unchanged)."""
    b = GraphBuilder("reward_scoring")
    toks, msks = b.input("tokens", "tokens"), b.input("mask")
    hidden, _w, _auxes = _trunk(b, spec, toks)
    reward = (b.node("masked_reward_head", {"model_dim": spec.model_dim}, [hidden, msks], "reward_head"), 0)
    g = b.outputs(reward)
    g.validate()
    return g


def build_ppo_root_graph(spec: ModelSpec) -> NeuronGraph:
    """PPO update graph over a stored rollout: (tokens, targets, loss_mask, logp_old, value_old,
    advantages, returns) -> clipped policy/value loss with entropy bonus."""
    ft = spec.finetune
    b = GraphBuilder("ppo_root")
    tokens = b.input("tokens", "tokens")
    targets = b.input("targets", "tokens")
    mask, logp_old, value_old, adv, ret = (b.input(n) for n in ("loss_mask", "logp_old", "value_old",
                                                                "advantages", "returns"))
    hidden, _w, auxes = _trunk(b, spec, tokens)
    pv = b.node("policy_logits_value", {"model_dim": spec.model_dim, "vocab_size": spec.vocab_size,
                                        "output_multiplier": spec.output_multiplier,
                                        "logit_softcap": spec.logit_softcap}, [hidden], "policy_value")
    le = b.node("token_logp_entropy", {}, [(pv, 0), targets, mask], "logp_entropy")
    loss = b.node("masked_ppo_clipped_loss", {"clip_range": ft.ppo_clip if ft else 0.2,
                                              "vf_coef": ft.ppo_vf_coef if ft else 0.5,
                                              "ent_coef": ft.ppo_ent_coef if ft else 0.0},
                  [(le, 0), logp_old, adv, (pv, 1), value_old, ret, mask, (le, 1)], "ppo_loss")
    g = b.outputs(_sum_aux(b, (loss, 3), auxes))
    g.torch_config = _torch_config(spec, {"objective": "ppo"})
    g.validate()
    return g

"""Port signatures of every tensor stage: ``module_type -> (input names, output names)``.

Used to build ``module`` neuron definitions (catalogue, template builders) and by the
compiler's arity checks. Port dtypes: names starting with ``tok``/ending ``_ids``/``indices``
are token-typed, everything else is a tensor.
"""
from __future__ import annotations

from ..neuron import NeuronDef, module_neuron
from ..port import Port

MODULE_PORTS: dict[str, tuple[tuple[str, ...], tuple[str, ...]]] = {
    # embeddings / heads
    "token_embedding": (("tokens",), ("hidden", "weight")),
    "absolute_position_embedding": (("hidden",), ("hidden",)),
    "tied_lm_head": (("hidden", "weight"), ("logits",)),
    "lm_head": (("hidden",), ("logits",)),
    "logit_softcap": (("logits",), ("logits",)),
    "tensor_scale": (("x",), ("y",)),
    "loss_scale": (("loss",), ("loss",)),
    # norms / residuals
    "rms_norm": (("x",), ("y",)), "layer_norm": (("x",), ("y",)), "dyt": (("x",), ("y",)),
    "group_norm": (("x",), ("y",)), "qk_norm": (("q", "k"), ("q", "k")),
    "residual_add": (("x", "delta"), ("y",)), "residual_mix": (("x", "skip"), ("y",)),
    "manifold_hyper_connection": (("x", "delta"), ("y",)),
    # linears / MLPs
    "linear": (("x",), ("y",)), "bitlinear_ternary": (("x",), ("y",)), "fp8_linear": (("x",), ("y",)),
    "mx_linear": (("x",), ("y",)), "lora_linear": (("x",), ("y",)), "nf4_linear": (("x",), ("y",)),
    "randmap_adapter": (("x",), ("y",)), "gelu": (("x",), ("y",)), "sigmoid": (("x",), ("y",)),
    "silu": (("x",), ("y",)), "multiply": (("a", "b"), ("y",)), "dropout": (("x",), ("y",)),
    "swiglu": (("x",), ("y",)), "geglu": (("x",), ("y",)), "reglu": (("x",), ("y",)), "solu": (("x",), ("y",)),
    "mlp_relu2": (("x",), ("y",)),
    # attention pieces
    "reshape_heads": (("x",), ("heads",)), "merge_heads": (("heads",), ("x",)), "repeat_kv": (("x",), ("x",)),
    "rotary_embedding": (("q", "k"), ("q", "k")), "qk_gain": (("q",), ("q",)),
    "scaled_dot_product_attention": (("q", "k", "v"), ("attn",)),
    "sliding_window_attention": (("q", "k", "v"), ("attn",)),
    "block_sparse_attention": (("q", "k", "v"), ("attn",)),
    "streaming_attention_sinks": (("q", "k", "v"), ("attn",)),
    "native_sparse_attention": (("q", "k", "v"), ("attn",)),
    "differential_attention": (("q", "k", "v"), ("attn",)),
    "causal_self_attention": (("x",), ("y",)), "fused_causal_attention": (("x",), ("y",)),
    "multi_latent_attention": (("x",), ("y",)),
    "dflash_attention": (("block_hidden", "context_hidden", "block_positions", "context_positions",
                          "attention_mask"), ("y",)),
    "kv_cache_read": (("new", "cache"), ("full",)), "kv_cache_write": (("full",), ("cache",)),
    "kv_pca_encode": (("x",), ("z",)), "kv_pca_decode": (("z",), ("x",)),
    "kv_quant_pack": (("x",), ("codes", "scale")), "kv_quant_unpack": (("codes", "scale"), ("x",)),
    # MoE
    "router_logits": (("x",), ("logits",)), "auxfree_load_balancing": (("logits",), ("logits",)),
    "topk_route": (("logits",), ("weights", "indices")),
    "expert_dispatch": (("x", "weights", "indices"), ("y",)), "expert_combine": (("x",), ("y",)),
    "broadcast_expert_routes": (("hidden", "weights", "indices"), ("weights", "indices")),
    "load_balance_loss": (("logits", "weights", "indices"), ("aux_loss", "logits")),
    "router_z_loss": (("logits",), ("z_loss",)), "aux_loss_add": (("loss", "aux_loss"), ("loss",)),
    # losses / post-training
    "token_cross_entropy": (("logits", "target_ids"), ("loss",)),
    "masked_token_cross_entropy": (("logits", "target_ids", "loss_mask"), ("loss",)),
    "sequence_logp": (("logits", "targets", "loss_mask"), ("logp",)),
    "token_logp_entropy": (("logits", "targets", "loss_mask"), ("logp", "entropy")),
    "dpo_pairwise_loss": (("policy_logp_chosen", "policy_logp_rejected", "ref_logp_chosen",
                           "ref_logp_rejected"), ("loss", "chosen_reward", "rejected_reward")),
    "preference_bce_loss": (("reward_chosen", "reward_rejected"), ("loss",)),
    "ppo_clipped_loss": (("logp_new", "logp_old", "advantages", "value_new", "value_old", "returns"),
                         ("policy_loss", "value_loss", "loss")),
    "masked_ppo_clipped_loss": (("logp_new", "logp_old", "advantages", "value_new", "value_old", "returns",
                                 "loss_mask", "entropy"), ("policy_loss", "value_loss", "entropy", "loss")),
    "kl_penalty": (("logp_policy", "logp_ref", "rewards"), ("rewards",)),
    "gae_compute": (("rewards", "values"), ("advantages", "returns")),
    "reward_head": (("hidden",), ("reward",)), "masked_reward_head": (("hidden", "sequence_mask"), ("reward",)),
    "value_head": (("hidden",), ("value",)), "policy_logits_value": (("hidden",), ("logits", "value")),
    "pair_batch_concat": (("chosen", "rejected"), ("paired",)),
    "pair_batch_split": (("paired",), ("chosen", "rejected")),
    "latent_mse_loss": (("predicted", "target"), ("loss",)),
    "softmax_distillation_loss": (("student_logits", "teacher_logits"), ("loss",)),
    "reference_forward": (("tokens",), ("logits",)), "reward_forward": (("tokens",), ("reward",)),
    # sources
    "dataset_source": ((), ("tokens", "target_ids")),
    "sft_dataset_source": ((), ("tokens", "target_ids", "loss_mask")),
    "dpo_dataset_source": ((), ("chosen_tokens", "chosen_targets", "chosen_mask", "rejected_tokens",
                                "rejected_targets", "rejected_mask")),
    "ppo_rollout_source": ((), ("tokens", "targets", "loss_mask", "logp_old", "value_old", "rewards")),
    "semantic_data_source": ((), ("semantic_targets",)),
    # sequence-model variants / JEPA / diffusion / bytes
    "mamba": (("x",), ("y",)), "ttt_linear": (("x",), ("y",)), "universal_transformer": (("x",), ("y",)),
    "act_halt_gate": (("x",), ("p",)), "act_weighted_sum": (("states", "weights"), ("y",)),
    "running_mean_decoder": (("x",), ("y",)),
    "jepa_mask": (("tokens",), ("context_tokens", "mask")), "latent_pool": (("hidden", "mask"), ("latent",)),
    "jepa_projector": (("x",), ("z",)), "jepa_predictor": (("z",), ("z",)),
    "random_timesteps": (("tokens",), ("timesteps",)),
    "mask_scheduler": (("tokens", "timesteps"), ("noisy_tokens", "mask")),
    "denoise_head": (("hidden",), ("logits",)),
    "byte_patch_embed": (("tokens",), ("patches",)), "byte_patch_merge": (("patches", "like"), ("hidden",)),
    # semantic routing
    "semantic_projector": (("hidden",), ("semantic_vec", "residual", "topic_logits")),
    "semantic_chunk_projector": (("chunk_state",), ("semantic_vec", "residual", "topic_logits")),
    "semantic_alignment_loss": (("pred_logits", "target"), ("loss",)),
    "semantic_hasher": (("semantic_vec",), ("bucket_indices",)),
    "semantic_chunk_hasher": (("semantic_vec",), ("bucket_indices",)),
    "semantic_moe_router": (("semantic_vec",), ("expert_weights", "expert_indices")),
    "semantic_hash_router": (("semantic_vec", "bucket_indices", "topic_logits", "sem_targets"),
                             ("expert_weights", "expert_indices")),
    "causal_chunk_state": (("hidden",), ("chunk_state",)),
    "semantic_moe_jepa_evo_router": (("semantic_vec", "bucket_indices", "topic_logits", "sem_targets"),
                                     ("expert_weights", "expert_indices", "route_logits")),
    "broadcast_chunk_routes": (("hidden", "expert_weights", "expert_indices"), ("routing_weights", "routing_indices")),
    "route_balance_loss": (("route_logits",), ("loss",)),
    "route_selection_loss": (("route_logits", "sem_targets"), ("loss",)),
    "route_distillation_loss": (("student_route_logits", "target_topic_logits"), ("loss",)),
    "routed_attention_experts": (("hidden", "expert_weights", "expert_indices"), ("hidden_out",)),
    "attentionless_decoder": (("bucket_indices", "expert_output"), ("logits",)),
    "semantic_unforced_targets": (("hidden",), ("sem_targets",)),
    "semantic_targets_from_tokens": (("tokens",), ("sem_targets",)),
    # vision
    "muse_glimmer_vision_tower": (("pixel_values", "grid_thw"), ("merged_patches",)),
    "muse_glimmer_perception_norm": (("features",), ("normalized",)),
    "muse_glimmer_media_scatter": (("embeddings", "token_ids", "features"), ("fused_embeddings",)),
}

_TOKEN_PORTS = {"tokens", "target_ids", "targets", "indices", "context_tokens", "noisy_tokens",
                "chosen_tokens", "rejected_tokens", "chosen_targets", "rejected_targets",
                "block_positions", "context_positions", "token_ids", "sem_targets", "target"}


def _port(name: str) -> Port:
    return Port(name, dtype="tokens" if name in _TOKEN_PORTS else "tensor")


def module_ports(module_type: str) -> tuple[list[Port], list[Port]]:
    try:
        ins, outs = MODULE_PORTS[module_type]
    except KeyError:
        raise KeyError(f"no port signature registered for module type {module_type!r}") from None
    return [_port(n) for n in ins], [_port(n) for n in outs]


def make_module_neuron(module_type: str, config: dict | None = None, *, name: str | None = None,
                       neuron_id: str | None = None) -> NeuronDef:
    ins, outs = module_ports(module_type)
    return module_neuron(name=name or module_type, module_type=module_type, input_ports=ins,
                         output_ports=outs, module_config=dict(config or {}), neuron_id=neuron_id)

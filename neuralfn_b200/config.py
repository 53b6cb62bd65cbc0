"""Model specification dataclasses (template / block / fine-tune / model).

Field names and defaults follow the reference's public spec objects
(``neuralfn/config.py:53-492``) so that graph payloads, CLI flags and saved
``torch_config`` dictionaries interchange. Preset builders live in
``neuralfn_b200.presets`` and are re-exported here under their reference names
(``build_gpt2_spec`` ... ``build_muse_glimmer_spec``).
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass, field, fields
from typing import Any

NUM_SEMANTIC_DIMS = 86
NUM_VOCAB_DIMS = 86
DEFAULT_SEMANTIC_VOCAB_REF = "vocab_86d"

OBJECTIVES = ("ar", "diffusion", "jepa", "ar_jepa", "jepa_semantic", "semantic_router",
              "semantic_router_jepa", "semantic_dense_jepa_evo", "semantic_moe_jepa_evo", "seq2seq",
              "sft", "dpo", "ppo", "reward_model")
BACKBONES = ("gpt2", "nanogpt", "llama", "mixllama", "jamba", "universal", "ttt", "hnet", "muse_glimmer")
COMPRESSIONS = ("none", "ternary_b158", "binary_1bit", "kv_pca", "fp8_e4m3", "fp8_e5m2", "mxfp4", "mxfp8")
ADAPTERS = ("none", "lora", "qlora", "randmap")
RUNTIMES = ("eager", "compile", "sdpa", "megakernel")

_HEX = set("0123456789abcdef")


def _check_sha256(value: str, name: str) -> str:
    digest = str(value).strip().lower()
    if digest and (len(digest) != 64 or any(ch not in _HEX for ch in digest)):
        raise ValueError(f"{name} must be an empty string or a 64-character SHA-256 digest")
    return digest


@dataclass
class TemplateSpec:
    objective: str = "ar"
    backbone: str = "gpt2"
    tokenization: str = "sp"
    sparsity: str = "dense"
    router_mode: str = "none"
    compression: str = "none"
    adapter: str = "none"
    runtime: str = "eager"
    backend_capabilities: dict[str, bool] = field(default_factory=lambda: {
        "compile": True, "sdpa": True, "cache": True, "quantized_export": True, "megakernel": False})


def resolve_backend_capabilities(spec: TemplateSpec) -> dict[str, bool]:
    """Capability map implied by the runtime choice of a template."""
    return {"compile": spec.runtime in ("compile", "megakernel"), "sdpa": True, "cache": True,
            "quantized_export": True, "megakernel": spec.runtime == "megakernel"}


@dataclass
class LayerAttentionSpec:
    """One entry of a decoder's repeating per-layer attention schedule (hybrid
    local/global stacks): ``kind`` full|local, window, positional encoding none|rope."""
    kind: str = "full"
    window_size: int | None = None
    pos_encoding: str = "none"
    rope_theta: float = 10_000.0


@dataclass
class BlockSpec:
    family: str
    norm_type: str = "layernorm"       # layernorm | rmsnorm | dyt | group_norm
    mlp_type: str = "gelu"             # gelu | swiglu | moe | geglu | reglu | solu
    pos_encoding: str = "absolute"     # absolute | rope
    attention_backend: str = "sdpa"    # sdpa | flex | math
    num_heads: int = 4
    num_kv_heads: int | None = None
    head_dim: int | None = None
    attention_inner_dim: int | None = None
    intermediate_size: int | None = None
    layer_attention_pattern: tuple[LayerAttentionSpec, ...] = ()
    is_causal: bool = True
    linear_bias: bool = True
    dropout_p: float = 0.0
    rope_theta: float = 10000.0
    rope_scaling: dict[str, Any] | None = None
    mlp_multiplier: float = 4.0
    multiple_of: int | None = None
    experts: int | None = None
    top_k: int | None = None
    shared_experts: int = 0
    router_aux_loss_coef: float = 0.0
    router_z_loss_coef: float = 0.0    # extension: coef * mean(logsumexp(router_logits)^2)
    compression: str = "none"
    adapter_dim: int = 0
    adapter_type: str = "none"
    lora_rank: int = 8
    lora_alpha: float = 16.0
    lora_dropout: float = 0.0
    lora_targets: tuple[str, ...] = ("q_proj", "v_proj")
    lora_bias: bool = False
    qlora_group_size: int = 64
    qlora_compute_dtype: str = "bf16"
    ttt_hidden_dim: int = 16
    byte_patch_size: int = 4
    byte_patch_stride: int = 4
    qk_gain_init: float = 1.0
    attention_variant: str = "dense"   # dense | differential | sliding_window | block_sparse | nsa | streaming | mla
    use_qk_norm: bool = False
    qk_norm_kind: str = "none"
    qk_norm_eps: float = 1e-6
    q_scale_factor: float = 1.0
    attention_gate: str = "none"       # none | sigmoid
    attention_gate_dim: int | None = None
    norm_layout: str = "pre"           # pre | sandwich
    centered_rms_norm: bool = False
    norm_eps: float = 1e-6
    post_norm_eps: float = 1e-6
    embedding_norm_kind: str = "none"
    embedding_norm_eps: float = 1e-6
    dyt_alpha_init: float = 1.0
    group_norm_groups: int = 1
    diff_lambda_init: float = 0.8
    moe_balance_mode: str = "aux_loss"  # aux_loss | auxfree
    auxfree_bias_lr: float = 0.001
    router_score_fn: str = "softmax"    # softmax | sigmoid | sqrt_softplus
    residual_type: str = "add"          # add | mhc
    window_size: int | None = None
    sparse_block_size: int = 64
    num_sinks: int = 0
    nsa_compress_stride: int = 16
    mx_block_size: int = 32
    fp8_amax_history_len: int = 16
    fp8_use_stochastic_rounding: bool = True
    activation_mode: str = "single"     # single | moa
    moa_activations: tuple[str, ...] = ("gelu", "relu", "silu", "relu2")
    moa_interval: int = 50

    def layer_attention(self, layer_index: int) -> LayerAttentionSpec | None:
        pat = self.layer_attention_pattern
        return pat[layer_index % len(pat)] if pat else None


@dataclass
class FineTuneSpec:
    """Fine-tuning run: objective, base/reference/reward checkpoints (with optional SHA-256
    pins), DPO and PPO hyper-parameters. Validated on construction."""
    objective: str = "pretrain"
    base_checkpoint: str = ""
    base_checkpoint_sha256: str = ""
    base_weight_precision: str = "bf16"
    tokenizer_sha256: str = ""
    chat_template_sha256: str = ""
    ref_graph_path: str = ""
    ref_checkpoint: str = ""
    ref_checkpoint_sha256: str = ""
    reward_graph_path: str = ""
    reward_checkpoint: str = ""
    reward_checkpoint_sha256: str = ""
    resume_checkpoint: str = ""
    adapter_only_save: bool = False
    beta: float = 0.1
    dpo_loss_type: str = "sigmoid"
    dpo_label_smoothing: float = 0.0
    kl_coef: float = 0.1
    ppo_clip: float = 0.2
    ppo_vf_coef: float = 0.5
    ppo_ent_coef: float = 0.0
    rollout_length: int = 64
    ppo_epochs_per_rollout: int = 4
    ppo_minibatch_size: int = 4
    gae_gamma: float = 1.0
    gae_lambda: float = 0.95

    def __post_init__(self) -> None:
        self.objective = str(self.objective).strip().lower()
        allowed = {"pretrain", "sft", "dpo", "ppo", "reward_model"}
        if self.objective not in allowed:
            raise ValueError(f"Unsupported fine-tuning objective {self.objective!r}; expected one of {sorted(allowed)}")
        self.base_weight_precision = str(self.base_weight_precision).strip().lower()
        if self.base_weight_precision not in {"bf16", "k-quant-17gb", "k-quant-dynamic"}:
            raise ValueError("FineTuneSpec.base_weight_precision must be 'bf16', 'k-quant-17gb', or 'k-quant-dynamic'")
        for name in ("base_checkpoint_sha256", "ref_checkpoint_sha256", "reward_checkpoint_sha256",
                     "tokenizer_sha256", "chat_template_sha256"):
            setattr(self, name, _check_sha256(getattr(self, name), name))
        if self.beta <= 0.0:
            raise ValueError("FineTuneSpec.beta must be positive")
        if self.dpo_loss_type not in {"sigmoid", "hinge", "ipo"}:
            raise ValueError("FineTuneSpec.dpo_loss_type must be 'sigmoid', 'hinge', or 'ipo'")
        if not 0.0 <= self.dpo_label_smoothing < 0.5:
            raise ValueError("FineTuneSpec.dpo_label_smoothing must be in [0, 0.5)")
        if self.kl_coef < 0.0:
            raise ValueError("FineTuneSpec.kl_coef must be non-negative")
        if not 0.0 < self.ppo_clip < 1.0:
            raise ValueError("FineTuneSpec.ppo_clip must be in (0, 1)")
        if self.ppo_vf_coef < 0.0 or self.ppo_ent_coef < 0.0:
            raise ValueError("PPO value and entropy coefficients must be non-negative")
        if min(self.rollout_length, self.ppo_epochs_per_rollout, self.ppo_minibatch_size) <= 0:
            raise ValueError("PPO rollout length, epochs, and minibatch size must be positive")
        if not (0.0 <= self.gae_gamma <= 1.0 and 0.0 <= self.gae_lambda <= 1.0):
            raise ValueError("GAE gamma and lambda must be in [0, 1]")


@dataclass
class MuseGlimmerVisionSpec:
    """Vision tower / projector geometry of the Muse-Glimmer family (non-causal,
    biased, window attention with every 4th layer full)."""
    num_hidden_layers: int = 50
    hidden_size: int = 1_536
    intermediate_size: int = 8_960
    num_attention_heads: int = 16
    patch_size: int = 14
    patch_temporal: int = 2
    merge_size: int = 2
    pos_emb_height: int = 32
    pos_emb_width: int = 32
    rope_theta: float = 10_000.0
    layer_norm_eps: float = 1.0e-5
    projector_hidden_size: int = 4_096
    image_token_id: int = 200_092
    video_token_id: int = 200_091

    def __post_init__(self) -> None:
        dims = (self.num_hidden_layers, self.hidden_size, self.intermediate_size, self.num_attention_heads,
                self.patch_size, self.patch_temporal, self.merge_size, self.pos_emb_height,
                self.pos_emb_width, self.projector_hidden_size)
        if any(int(v) <= 0 for v in dims):
            raise ValueError("Muse Glimmer vision dimensions must be positive")
        if self.hidden_size % self.num_attention_heads:
            raise ValueError("Muse Glimmer vision heads must divide hidden_size")
        if self.pos_emb_height != self.pos_emb_width:
            raise ValueError("Muse Glimmer v1 requires a square learned position table")
        if self.rope_theta <= 0.0 or self.layer_norm_eps <= 0.0:
            raise ValueError("Muse Glimmer vision RoPE/norm values must be positive")
        if self.image_token_id < 0 or self.video_token_id < 0:
            raise ValueError("Muse Glimmer media token IDs must be non-negative")

    def layer_type(self, index: int) -> str:
        if not 0 <= index < self.num_hidden_layers:
            raise IndexError(index)
        full = (index + 1) % 4 == 0 or index == self.num_hidden_layers - 1
        return "full_attention" if full else "window_attention"


@dataclass
class MuseGlimmerDFlashSpec:
    """Shape contract of the DFlash block-drafting assistant bound to a target model."""
    num_hidden_layers: int = 5
    hidden_size: int = 6_656
    intermediate_size: int = 19_968
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    block_size: int = 16
    mask_token_id: int = 201_818
    sliding_window: int = 2_048
    rope_theta: float = 500_000.0
    target_layer_ids: tuple[int, ...] = (1, 13, 25, 37, 49)

    def __post_init__(self) -> None:
        bad = (min(self.num_hidden_layers, self.hidden_size, self.intermediate_size,
                   self.num_attention_heads, self.num_key_value_heads, self.head_dim,
                   self.sliding_window) <= 0
               or self.num_attention_heads % self.num_key_value_heads != 0 or self.head_dim % 2 != 0
               or self.block_size < 2 or self.mask_token_id < 0 or self.rope_theta <= 0.0)
        if bad:
            raise ValueError("invalid Muse Glimmer DFlash contract")
        ids = tuple(int(v) for v in self.target_layer_ids)
        if not ids or ids != tuple(sorted(set(ids))):
            raise ValueError("DFlash target_layer_ids must be sorted and unique")
        self.target_layer_ids = ids


@dataclass
class MuseGlimmerDFlashDistillationSpec:
    """Versioned recipe for training a target-bound DFlash assistant (random anchors,
    self-logit distillation, D-PACE or exponential-decay position weights)."""
    recipe: str = "neuralfn.muse_glimmer_dflash_distill.v1"
    recipe_revision: str = "686da8d893536688e86adae41aa628aa740a1a35"
    target_checkpoint_sha256: str = ""
    target_config_sha256: str = ""
    tokenizer_sha256: str = ""
    chat_template_sha256: str = ""
    num_anchors: int = 512
    loss_objective: str = "dpace"
    dpace_alpha: float = 0.5
    loss_decay_factor: float = 7.0
    self_logit_distillation: bool = True
    seed: int = 20_260_813

    def __post_init__(self) -> None:
        if self.recipe != "neuralfn.muse_glimmer_dflash_distill.v1":
            raise ValueError("Unsupported Muse Glimmer DFlash distillation recipe")
        if len(self.recipe_revision) != 40 or any(c not in _HEX for c in self.recipe_revision):
            raise ValueError("DFlash recipe_revision must be a lowercase Git SHA")
        for name in ("target_checkpoint_sha256", "target_config_sha256", "tokenizer_sha256",
                     "chat_template_sha256"):
            setattr(self, name, _check_sha256(getattr(self, name), name))
        self.loss_objective = str(self.loss_objective).strip().lower()
        if self.loss_objective not in {"dpace", "decay"}:
            raise ValueError("DFlash loss_objective must be 'dpace' or 'decay'")
        if self.num_anchors <= 0:
            raise ValueError("DFlash num_anchors must be positive")
        if not 0.0 < self.dpace_alpha <= 1.0:
            raise ValueError("DFlash dpace_alpha must be in (0, 1]")
        if not math.isfinite(self.loss_decay_factor) or self.loss_decay_factor < 0.0:
            raise ValueError("DFlash loss_decay_factor must be finite and non-negative")
        if self.seed < 0:
            raise ValueError("DFlash seed must be non-negative")


@dataclass
class ModelSpec:
    model_dim: int = 128
    num_layers: int = 4
    vocab_size: int = 256
    tie_embeddings: bool = True
    max_position_embeddings: int = 1024
    output_multiplier: float = 1.0
    logit_softcap: float = 0.0
    z_loss_coef: float = 0.0
    block_spec: BlockSpec = field(default_factory=lambda: BlockSpec(family="gpt2"))
    template: TemplateSpec = field(default_factory=TemplateSpec)
    jepa_latent_dim: int = 128
    jepa_mask_ratio: float = 0.5
    jepa_mask_strategy: str = "random"
    jepa_num_blocks: int = 4
    jepa_min_block_ratio: float = 0.1
    jepa_max_block_ratio: float = 0.25
    ema_decay: float = 0.99
    max_recurrence_steps: int = 4
    halt_epsilon: float = 0.01
    semantic_dim: int = NUM_SEMANTIC_DIMS
    semantic_residual_dim: int = 64
    semantic_n_lsh_tables: int = 8
    semantic_n_lsh_planes: int = 12
    semantic_table_path: str = ""
    semantic_vocab_ref: str = DEFAULT_SEMANTIC_VOCAB_REF
    experimental_semantic_router_vecs: bool = False
    route_chunk_size: int = 32
    semantic_shared_experts: int = 2
    semantic_free_experts: int = 8
    route_evo_enabled: bool = True
    route_evo_fraction: float = 0.10
    route_evo_population: int = 8
    route_evo_mutation_scale: float = 0.05
    route_evo_seed: int | None = None
    layer_evo_enabled: bool = False
    layer_evo_index: int | None = None
    layer_evo_fraction: float = 0.10
    layer_evo_population: int = 8
    layer_evo_mutation_scale: float = 0.02
    layer_evo_seed: int | None = None
    ar_loss_coef: float = 1.0
    jepa_loss_coef: float = 0.25
    semantic_align_loss_coef: float = 0.5
    finetune: FineTuneSpec | None = None
    vision: MuseGlimmerVisionSpec | None = None
    dflash: MuseGlimmerDFlashSpec | None = None
    dflash_distillation: MuseGlimmerDFlashDistillationSpec | None = None

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)

    @property
    def head_dim(self) -> int:
        b = self.block_spec
        return b.head_dim if b.head_dim is not None else self.model_dim // b.num_heads

    @property
    def num_kv_heads(self) -> int:
        b = self.block_spec
        return b.num_kv_heads if b.num_kv_heads is not None else b.num_heads


def spec_from_dict(payload: dict[str, Any]) -> ModelSpec:
    """Rebuild a ``ModelSpec`` from ``ModelSpec.to_dict()`` output (nested dataclasses restored)."""
    data = dict(payload)

    def build(cls, raw):
        if raw is None or isinstance(raw, cls):
            return raw
        names = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in raw.items() if k in names})

    block_raw = dict(data.get("block_spec") or {"family": "gpt2"})
    pattern = block_raw.get("layer_attention_pattern") or ()
    block_raw["layer_attention_pattern"] = tuple(build(LayerAttentionSpec, p) for p in pattern)
    for key in ("lora_targets", "moa_activations"):
        if key in block_raw and block_raw[key] is not None:
            block_raw[key] = tuple(block_raw[key])
    data["block_spec"] = build(BlockSpec, block_raw)
    data["template"] = build(TemplateSpec, data.get("template") or {})
    data["finetune"] = build(FineTuneSpec, data.get("finetune"))
    data["vision"] = build(MuseGlimmerVisionSpec, data.get("vision"))
    dflash_raw = data.get("dflash")
    if isinstance(dflash_raw, dict) and "target_layer_ids" in dflash_raw:
        dflash_raw = {**dflash_raw, "target_layer_ids": tuple(dflash_raw["target_layer_ids"])}
    data["dflash"] = build(MuseGlimmerDFlashSpec, dflash_raw)
    data["dflash_distillation"] = build(MuseGlimmerDFlashDistillationSpec, data.get("dflash_distillation"))
    names = {f.name for f in fields(ModelSpec)}
    return ModelSpec(**{k: v for k, v in data.items() if k in names})


def __getattr__(name: str):
    # preset builders (build_*_spec, PRESET_BUILDERS, ...) are defined in presets.py
    if name.startswith("build_") or name in {"PRESET_BUILDERS", "MODERN_BASE_PRESETS", "preset_names",
                                             "build_preset"}:
        from . import presets
        return getattr(presets, name)
    raise AttributeError(name)

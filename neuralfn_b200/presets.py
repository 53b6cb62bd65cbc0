"""Model presets: every shipped template name maps to a ``ModelSpec`` builder.

The catalogue is declared as data (``_PRESETS``): a preset is a backbone family, a
template override, a block override and model-level defaults; caller keyword
arguments override any of them (``model_dim``/``n_embd``, ``num_layers``/``n_layer``,
``num_heads`` ... exactly the keyword surface of the reference builders,
``neuralfn/config.py:495-560,852-2060``). ``<name>_modern`` variants overlay the
RMSNorm/GeGLU/RoPE+YaRN/QK-norm/aux-free-MoE profile (``:642-667``).
"""
from __future__ import annotations

from typing import Any, Callable

from .config import (BlockSpec, FineTuneSpec, LayerAttentionSpec, ModelSpec, MuseGlimmerDFlashSpec,
                     MuseGlimmerVisionSpec, TemplateSpec, resolve_backend_capabilities,
                     NUM_SEMANTIC_DIMS, DEFAULT_SEMANTIC_VOCAB_REF)

__all__ = ["PRESET_BUILDERS", "MODERN_BASE_PRESETS", "SHIPPED_GPT_TEMPLATE_BASE_PRESETS",
           "SHIPPED_GPT_TEMPLATE_PRESETS", "build_preset", "preset_names", "build_composed_lm_spec"]

_MODEL_KEYS = {
    "vocab_size", "tie_embeddings", "max_position_embeddings", "output_multiplier", "logit_softcap",
    "z_loss_coef", "jepa_latent_dim", "jepa_mask_ratio", "jepa_mask_strategy", "jepa_num_blocks",
    "jepa_min_block_ratio", "jepa_max_block_ratio", "ema_decay", "max_recurrence_steps", "halt_epsilon",
    "semantic_dim", "semantic_residual_dim", "semantic_n_lsh_tables", "semantic_n_lsh_planes",
    "semantic_table_path", "semantic_vocab_ref", "experimental_semantic_router_vecs", "route_chunk_size",
    "semantic_shared_experts", "semantic_free_experts", "route_evo_enabled", "route_evo_fraction",
    "route_evo_population", "route_evo_mutation_scale", "route_evo_seed", "layer_evo_enabled",
    "layer_evo_index", "layer_evo_fraction", "layer_evo_population", "layer_evo_mutation_scale",
    "layer_evo_seed", "ar_loss_coef", "jepa_loss_coef", "semantic_align_loss_coef",
}
_BLOCK_KEYS = {f for f in BlockSpec.__dataclass_fields__ if f != "family"}
_BLOCK_ALIASES = {"rope_base": "rope_theta", "mlp_mult": "mlp_multiplier", "bias": "linear_bias"}


def _base_model_spec(kwargs: dict[str, Any], template: TemplateSpec, block: BlockSpec,
                     default_tie: bool, model_defaults: dict[str, Any] | None = None) -> ModelSpec:
    kw = dict(kwargs)
    template.backend_capabilities = resolve_backend_capabilities(template)
    model_dim = int(kw.get("model_dim", kw.get("n_embd", (model_defaults or {}).get("model_dim", 128))))
    num_layers = int(kw.get("num_layers", kw.get("n_layer", (model_defaults or {}).get("num_layers", 4))))
    for alias, real in _BLOCK_ALIASES.items():
        if alias in kw and real not in kw:
            kw[real] = kw[alias]
    if "n_head" in kw and "num_heads" not in kw:
        kw["num_heads"] = kw["n_head"]
    for key in _BLOCK_KEYS:
        if key in kw and kw[key] is not None:
            value = kw[key]
            if key in ("lora_targets", "moa_activations", "layer_attention_pattern") and not isinstance(value, tuple):
                value = tuple(value)
            setattr(block, key, value)
    finetune = kw.get("finetune")
    if isinstance(finetune, dict):
        finetune = FineTuneSpec(**finetune)
    elif finetune is not None and not isinstance(finetune, FineTuneSpec):
        raise TypeError("finetune must be FineTuneSpec, a mapping, or None")
    fields: dict[str, Any] = {"tie_embeddings": default_tie, "jepa_latent_dim": model_dim}
    fields.update({k: v for k, v in (model_defaults or {}).items() if k in _MODEL_KEYS})
    fields.update({k: kw[k] for k in _MODEL_KEYS if k in kw})
    return ModelSpec(model_dim=model_dim, num_layers=num_layers, block_spec=block, template=template,
                     finetune=finetune, **fields)


def _llama_block(**over: Any) -> dict[str, Any]:
    base = dict(family="llama", norm_type="rmsnorm", mlp_type="swiglu", pos_encoding="rope",
                linear_bias=False, dropout_p=0.0, mlp_multiplier=8.0 / 3.0, multiple_of=256,
                num_heads=4, num_kv_heads=2)
    base.update(over)
    return base


def _moe_block(**over: Any) -> dict[str, Any]:
    base = _llama_block(family="mixllama", mlp_type="moe", multiple_of=None, experts=8, top_k=2,
                        router_aux_loss_coef=0.01)
    base.update(over)
    return base


_GPT2 = dict(family="gpt2", norm_type="layernorm", mlp_type="gelu", pos_encoding="absolute",
             linear_bias=True, num_heads=4)
_NANO = dict(family="nanogpt", norm_type="layernorm", mlp_type="gelu", pos_encoding="absolute",
             linear_bias=False, dropout_p=0.1, num_heads=4)

# name -> (template overrides, block fields, default tie_embeddings, model-level defaults)
_PRESETS: dict[str, tuple[dict, dict, bool, dict]] = {
    "nanogpt": (dict(backbone="nanogpt"), _NANO, True, {}),
    "nanogpt_megakernel": (dict(backbone="nanogpt", runtime="megakernel"), _NANO, True, {}),
    "gpt2": (dict(backbone="gpt2"), _GPT2, True, {}),
    "gpt2_megakernel": (dict(backbone="gpt2", runtime="megakernel"), _GPT2, True, {}),
    "gpt2_zloss": (dict(backbone="gpt2"), _GPT2, True, dict(z_loss_coef=1e-4)),
    "gpt2_softcap": (dict(backbone="gpt2"), _GPT2, True, dict(logit_softcap=30.0)),
    "gpt2_qknorm": (dict(backbone="gpt2"), {**_GPT2, "use_qk_norm": True}, True, {}),
    "gpt2_diff": (dict(backbone="gpt2"), {**_GPT2, "attention_variant": "differential",
                                          "diff_lambda_init": 0.8}, True, {}),
    "gpt2_stable": (dict(backbone="gpt2"), {**_GPT2, "use_qk_norm": True}, True, dict(z_loss_coef=1e-4)),
    "gpt2_evo": (dict(backbone="gpt2"), _GPT2, True,
                 dict(num_layers=10, layer_evo_enabled=True, layer_evo_fraction=0.10,
                      layer_evo_population=8, layer_evo_mutation_scale=0.02)),
    "gpt2_moa": (dict(backbone="gpt2"), {**_GPT2, "activation_mode": "moa"}, True, {}),
    "llama": (dict(backbone="llama"), _llama_block(), False, {}),
    "llama_fast": (dict(backbone="llama", runtime="compile"), _llama_block(), False, {}),
    "llama_fast_megakernel": (dict(backbone="llama", runtime="megakernel"), _llama_block(), False, {}),
    "llama_megakernel": (dict(backbone="llama", runtime="megakernel"), _llama_block(), False, {}),
    "modern_norms_llama": (dict(backbone="llama"),
                           _llama_block(norm_type="dyt", mlp_type="geglu", use_qk_norm=True), False, {}),
    "mixllama": (dict(backbone="mixllama", sparsity="moe"), _moe_block(), False, {}),
    "moe": (dict(backbone="mixllama", sparsity="moe"), _moe_block(), False, {}),
    "mixllama_fast": (dict(backbone="mixllama", sparsity="moe", runtime="compile"), _moe_block(), False, {}),
    "mixllama_fast_megakernel": (dict(backbone="mixllama", sparsity="moe", runtime="megakernel"),
                                 _moe_block(), False, {}),
    "jamba": (dict(backbone="jamba", sparsity="moe", runtime="compile"),
              _moe_block(family="jamba", mlp_multiplier=4.0, router_aux_loss_coef=0.0), False, {}),
    "ternary_b158": (dict(backbone="llama", compression="ternary_b158", runtime="compile"),
                     _llama_block(compression="ternary_b158", mlp_multiplier=4.0, multiple_of=None), False, {}),
    "fp8_llama": (dict(backbone="llama", compression="fp8_e4m3"),
                  _llama_block(compression="fp8_e4m3", use_qk_norm=True), False, {}),
    "mxfp4_llama": (dict(backbone="llama", compression="mxfp4"),
                    _llama_block(compression="mxfp4", use_qk_norm=True), False, {}),
    "gemma3": (dict(backbone="llama"),
               _llama_block(mlp_type="geglu", attention_variant="sliding_window", window_size=256,
                            use_qk_norm=True), False, dict(logit_softcap=30.0)),
    "diff_transformer": (dict(backbone="llama"),
                         _llama_block(attention_variant="differential", diff_lambda_init=0.8), False, {}),
    "longctx_sparse_llama": (dict(backbone="llama"),
                             _llama_block(attention_variant="nsa", window_size=128, sparse_block_size=64,
                                          num_sinks=4, nsa_compress_stride=16, use_qk_norm=True), False, {}),
    "qwen3_longctx": (dict(backbone="llama"),
                      _llama_block(use_qk_norm=True, rope_theta=1_000_000.0,
                                   rope_scaling={"type": "yarn", "factor": 4.0,
                                                 "original_max_position": 32768}), False, {}),
    "deepseek_v3": (dict(backbone="mixllama", sparsity="moe"),
                    _moe_block(attention_variant="mla", shared_experts=1, moe_balance_mode="auxfree",
                               router_aux_loss_coef=0.0, router_score_fn="sigmoid", use_qk_norm=True),
                    False, {}),
    "deepseek_v4": (dict(backbone="mixllama", sparsity="moe"),
                    _moe_block(attention_variant="nsa", shared_experts=1, moe_balance_mode="auxfree",
                               router_aux_loss_coef=0.0, router_score_fn="sqrt_softplus",
                               residual_type="mhc", use_qk_norm=True, window_size=128, num_sinks=4),
                    False, {}),
    "decoder2encoder_moe": (dict(backbone="mixllama", sparsity="moe", objective="seq2seq"),
                            _moe_block(is_causal=False), False, {}),
    "kv_pca_llama": (dict(backbone="llama", compression="kv_pca"), _llama_block(compression="kv_pca"),
                     False, {}),
    "seq2seq": (dict(backbone="llama", objective="seq2seq"), _llama_block(), False, {}),
    "diffusion": (dict(backbone="llama", objective="diffusion"), _llama_block(is_causal=False), False, {}),
    "diffllama": (dict(backbone="llama", objective="diffusion"), _llama_block(is_causal=False), False, {}),
    "ttt_llama": (dict(backbone="ttt"), _llama_block(family="ttt", ttt_hidden_dim=16), False, {}),
    "llm_jepa": (dict(backbone="llama", objective="ar_jepa"), _llama_block(), False, {}),
    "dense_jepa_evo": (dict(backbone="llama", objective="ar_jepa"), _llama_block(), False,
                       dict(route_evo_enabled=True)),
    "moe_jepa_evo": (dict(backbone="mixllama", sparsity="moe", objective="ar_jepa"), _moe_block(), False,
                     dict(route_evo_enabled=True)),
    "auxfree_moe_jepa_evo": (dict(backbone="mixllama", sparsity="moe", objective="ar_jepa"),
                             _moe_block(moe_balance_mode="auxfree", router_aux_loss_coef=0.0), False,
                             dict(route_evo_enabled=True)),
    "hnet_lm": (dict(backbone="hnet", tokenization="byte_hnet"),
                _llama_block(family="hnet", byte_patch_size=4, byte_patch_stride=4), False,
                dict(vocab_size=256)),
    "universal_llama": (dict(backbone="universal"), _llama_block(family="universal"), False,
                        dict(max_recurrence_steps=4, halt_epsilon=0.01)),
    "jepa_semantic_hybrid": (dict(backbone="llama", objective="jepa_semantic", runtime="compile"),
                             _llama_block(), False, {}),
    "jepa_semantic_hybrid_megakernel": (dict(backbone="llama", objective="jepa_semantic",
                                             runtime="megakernel"), _llama_block(), False, {}),
    "semantic_router_moe": (dict(backbone="mixllama", sparsity="moe", router_mode="semantic",
                                 objective="semantic_router", runtime="compile"), _moe_block(), False, {}),
    "semantic_router_moe_megakernel": (dict(backbone="mixllama", sparsity="moe", router_mode="semantic",
                                            objective="semantic_router", runtime="megakernel"),
                                       _moe_block(), False, {}),
    "semantic_dense_jepa_evo": (dict(backbone="llama", objective="semantic_dense_jepa_evo"),
                                _llama_block(), False, {}),
    "semantic_moe_jepa_evo": (dict(backbone="mixllama", sparsity="moe", router_mode="semantic",
                                   objective="semantic_moe_jepa_evo"), _moe_block(), False, {}),
    "diff_semantic_moe_jepa_evo": (dict(backbone="mixllama", sparsity="moe", router_mode="semantic",
                                        objective="semantic_moe_jepa_evo"),
                                   _moe_block(attention_variant="differential"), False, {}),
    "dyt_geglu_semantic_dense_jepa_evo": (dict(backbone="llama", objective="semantic_dense_jepa_evo"),
                                          _llama_block(norm_type="dyt", mlp_type="geglu"), False, {}),
}

MODERN_BASE_PRESETS: tuple[str, ...] = (
    "nanogpt", "gpt2", "llama", "moe", "jamba", "ternary_b158", "seq2seq", "diffusion", "ttt_llama",
    "llm_jepa", "dense_jepa_evo", "moe_jepa_evo", "hnet_lm", "universal_llama", "kv_pca_llama",
    "jepa_semantic_hybrid", "semantic_router_moe", "semantic_dense_jepa_evo", "semantic_moe_jepa_evo")

SHIPPED_GPT_TEMPLATE_BASE_PRESETS: tuple[str, ...] = (
    "nanogpt", "nanogpt_megakernel", "gpt2", "gpt2_megakernel", "gpt2_moa", "gpt2_zloss", "gpt2_softcap",
    "gpt2_qknorm", "gpt2_diff", "gpt2_stable", "llama", "muse_glimmer", "modern_norms_llama", "mixllama",
    "moe", "llama_fast", "llama_fast_megakernel", "mixllama_fast", "mixllama_fast_megakernel", "jamba",
    "ternary_b158", "fp8_llama", "mxfp4_llama", "deepseek_v3", "deepseek_v4", "gemma3", "diff_transformer",
    "longctx_sparse_llama", "qwen3_longctx", "auxfree_moe_jepa_evo", "diff_semantic_moe_jepa_evo",
    "dyt_geglu_semantic_dense_jepa_evo", "llama_megakernel", "kv_pca_llama", "seq2seq", "diffusion",
    "ttt_llama", "llm_jepa", "dense_jepa_evo", "moe_jepa_evo", "jepa_semantic_hybrid",
    "jepa_semantic_hybrid_megakernel", "semantic_router_moe", "semantic_router_moe_megakernel",
    "semantic_moe_jepa_evo", "semantic_dense_jepa_evo", "hnet_lm", "universal_llama")
SHIPPED_GPT_TEMPLATE_PRESETS: tuple[str, ...] = (
    *SHIPPED_GPT_TEMPLATE_BASE_PRESETS, *(f"{p}_modern" for p in MODERN_BASE_PRESETS))


def _apply_modern_profile(spec: ModelSpec) -> ModelSpec:
    """RMSNorm, GeGLU, RoPE + YaRN, QK-norm, aux-loss-free MoE balancing - in place."""
    bs = spec.block_spec
    if bs.norm_type == "layernorm":
        bs.norm_type = "rmsnorm"
    if bs.mlp_type == "gelu":
        bs.mlp_type = "geglu"
    if bs.pos_encoding == "absolute":
        bs.pos_encoding = "rope"
    bs.use_qk_norm = True
    if bs.pos_encoding == "rope" and not bs.rope_scaling:
        bs.rope_scaling = {"type": "yarn", "factor": 2.0, "original_max_position": 2048}
    if bs.mlp_type in ("moe", "mixllama"):
        bs.moe_balance_mode = "auxfree"
        bs.router_aux_loss_coef = 0.0
    return spec


def _table_builder(name: str) -> Callable[..., ModelSpec]:
    tmpl_over, block_fields, tie, model_defaults = _PRESETS[name]

    def build(**kwargs: Any) -> ModelSpec:
        tmpl_kw = dict(tmpl_over)
        if "runtime" in kwargs and name in ("gpt2_zloss", "gpt2_softcap", "gpt2_qknorm", "gpt2_diff",
                                            "gpt2_stable", "gpt2_moa"):
            tmpl_kw["runtime"] = str(kwargs["runtime"])
        if name == "fp8_llama" and str(kwargs.get("fp8_format", "e4m3")).lower() == "e5m2":
            tmpl_kw["compression"] = "fp8_e5m2"
            kwargs = {**kwargs, "compression": "fp8_e5m2"}
        if name == "mxfp4_llama" and str(kwargs.get("mx_format", "mxfp4")).lower() == "mxfp8":
            tmpl_kw["compression"] = "mxfp8"
            kwargs = {**kwargs, "compression": "mxfp8"}
        block = BlockSpec(**{k: (dict(v) if isinstance(v, dict) else v) for k, v in block_fields.items()})
        return _base_model_spec(kwargs, TemplateSpec(**tmpl_kw), block, tie, model_defaults)

    build.__name__ = f"build_{name}_spec"
    build.__doc__ = f"ModelSpec of the '{name}' preset; keyword arguments override its defaults."
    return build


def _modern_builder(base: str) -> Callable[..., ModelSpec]:
    def build(**kwargs: Any) -> ModelSpec:
        return _apply_modern_profile(PRESET_BUILDERS[base](**kwargs))
    build.__name__ = f"build_{base}_modern_spec"
    return build


def _glimmer(**kwargs: Any) -> ModelSpec:
    from .presets_glimmer import build_muse_glimmer_spec
    return build_muse_glimmer_spec(**kwargs)


PRESET_BUILDERS: dict[str, Callable[..., ModelSpec]] = {name: _table_builder(name) for name in _PRESETS}
PRESET_BUILDERS["muse_glimmer"] = _glimmer
# historical aliases of builder function names
_ALIASES = {"jamba_hybrid": "jamba"}
for _base in MODERN_BASE_PRESETS:
    PRESET_BUILDERS[f"{_base}_modern"] = _modern_builder(_base)


def preset_names() -> list[str]:
    return sorted(PRESET_BUILDERS)


def build_preset(name: str, **kwargs: Any) -> ModelSpec:
    key = _ALIASES.get(name, name)
    if key not in PRESET_BUILDERS:
        raise KeyError(f"unknown preset {name!r}; known: {', '.join(preset_names())}")
    return PRESET_BUILDERS[key](**kwargs)


def build_composed_lm_spec(*, base_model: str = "llama", moe: bool = False, router_mode: str = "none",
                           use_jepa: bool = False, runtime: str | None = None, compression: str = "none",
                           adapter: str = "none", **kwargs: Any) -> ModelSpec:
    """Compose a language-model spec from orthogonal choices (dense/MoE, standard/semantic
    router, optional JEPA objective, runtime, compression, adapter), as the recipe
    questionnaire of the legacy CLI does (reference ``build_composed_lm_spec``)."""
    base = str(base_model).strip().lower()
    if base not in {"gpt2", "nanogpt", "llama"}:
        raise ValueError(f"Unsupported composed base model {base_model!r}")
    rt = str(runtime or "default").strip().lower()
    if rt == "default":
        rt = "compile" if base == "llama" else "eager"
    if rt not in {"eager", "compile", "megakernel"}:
        raise ValueError(f"Unsupported composed runtime {runtime!r}")
    if router_mode == "semantic":
        objective = "semantic_router_jepa" if use_jepa else "semantic_router"
    else:
        objective = "ar_jepa" if use_jepa else "ar"
    sparse = moe or router_mode != "none"
    name = {"gpt2": "gpt2", "nanogpt": "nanogpt", "llama": "mixllama" if sparse else "llama"}[base]
    spec = build_preset(name, **kwargs)
    spec.template.objective = objective
    spec.template.runtime = rt
    spec.template.router_mode = router_mode if sparse else "none"
    spec.template.sparsity = "moe" if sparse else "dense"
    spec.template.compression = compression
    spec.template.adapter = adapter
    spec.block_spec.compression = compression
    spec.block_spec.adapter_type = adapter
    if sparse and spec.block_spec.mlp_type != "moe":
        spec.block_spec.mlp_type = "moe"
        spec.block_spec.experts = int(kwargs.get("experts", 8))
        spec.block_spec.top_k = int(kwargs.get("top_k", 2))
    spec.template.backend_capabilities = resolve_backend_capabilities(spec.template)
    return spec


def __getattr__(attr: str):
    # build_<preset>_spec functions, resolved from the table
    if attr.startswith("build_") and attr.endswith("_spec"):
        key = attr[len("build_"):-len("_spec")]
        key = _ALIASES.get(key, key)
        if key in PRESET_BUILDERS:
            return PRESET_BUILDERS[key]
    raise AttributeError(attr)

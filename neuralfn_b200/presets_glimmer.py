"""Muse-Glimmer text-decoder preset (hybrid local/global attention, gated attention,
sandwich RMSNorms) and the DFlash / vision companion specs.

Defaults are the 52-layer 6656-wide production geometry of the reference builder
(``neuralfn/config.py:1027-1210``); small caller-supplied dimensions keep the
defining non-square residual/attention geometry for previews and parity fixtures.
"""
from __future__ import annotations

from typing import Any

from .config import (BlockSpec, LayerAttentionSpec, ModelSpec, MuseGlimmerDFlashSpec,
                     MuseGlimmerVisionSpec, TemplateSpec)

GLIMMER_LORA_TARGETS = ("q_proj", "k_proj", "v_proj", "o_proj", "attn_gate_proj", "gate_proj",
                        "up_proj", "down_proj")


def build_muse_glimmer_spec(**kwargs: Any) -> ModelSpec:
    from .presets import _base_model_spec

    model_dim = int(kwargs.get("model_dim", kwargs.get("n_embd", 6_656)))
    adapter_type = str(kwargs.get("adapter_type", "none")).strip().lower()
    if adapter_type not in {"none", "lora", "qlora"}:
        raise ValueError("Muse Glimmer adapter_type must be 'none', 'lora', or 'qlora'")
    raw_targets = kwargs.get("lora_targets", GLIMMER_LORA_TARGETS)
    if isinstance(raw_targets, str):
        raw_targets = raw_targets.split(",")
    lora_targets = tuple(str(t).strip() for t in raw_targets if str(t).strip())
    unknown = sorted(set(lora_targets) - set(GLIMMER_LORA_TARGETS))
    if unknown:
        raise ValueError(f"Unsupported Muse Glimmer LoRA targets: {unknown}")
    if adapter_type != "none" and not lora_targets:
        raise ValueError("Muse Glimmer LoRA/QLoRA requires at least one projection target")
    if int(kwargs.get("lora_rank", 8)) <= 0 or float(kwargs.get("lora_alpha", 16.0)) <= 0.0:
        raise ValueError("Muse Glimmer lora_rank and lora_alpha must be positive")
    if not 0.0 <= float(kwargs.get("lora_dropout", 0.0)) < 1.0:
        raise ValueError("Muse Glimmer lora_dropout must be in [0, 1)")
    if int(kwargs.get("qlora_group_size", 64)) <= 0:
        raise ValueError("Muse Glimmer qlora_group_size must be positive")
    num_heads = int(kwargs.get("num_heads", kwargs.get("n_head", 32)))
    if num_heads <= 0:
        raise ValueError("Muse Glimmer num_heads must be positive")
    production = model_dim == 6_656 and num_heads == 32
    head_dim = int(kwargs.get("head_dim", 128 if production else max(2, model_dim // (2 * num_heads))))
    inner = int(kwargs.get("attention_inner_dim", num_heads * head_dim))
    if inner != num_heads * head_dim:
        raise ValueError(f"Muse Glimmer attention_inner_dim must equal num_heads * head_dim "
                         f"({num_heads * head_dim}), got {inner}")
    if head_dim % 2:
        raise ValueError("Muse Glimmer head_dim must be even for RoPE")
    num_kv = int(kwargs.get("num_kv_heads", 2 if production else max(1, num_heads // 2)))
    if num_kv <= 0 or num_heads % num_kv:
        raise ValueError("Muse Glimmer num_kv_heads must be positive and divide num_heads")
    window = int(kwargs.get("window_size", 2_048))
    theta = float(kwargs.get("rope_theta", kwargs.get("rope_base", 500_000.0)))
    inter = int(kwargs.get("intermediate_size", 19_968 if model_dim == 6_656 else 3 * model_dim))
    local = LayerAttentionSpec("local", window, "rope", theta)
    pattern = (local, local, local, LayerAttentionSpec("full", None, "none", theta))
    norm_eps = float(kwargs.get("norm_eps", 1e-5))
    block = BlockSpec(
        family="muse_glimmer", norm_type="rmsnorm", mlp_type="swiglu", pos_encoding="none",
        linear_bias=False, dropout_p=0.0, num_heads=num_heads, num_kv_heads=num_kv, head_dim=head_dim,
        attention_inner_dim=inner, intermediate_size=inter, layer_attention_pattern=pattern,
        rope_theta=theta, window_size=window, use_qk_norm=True, qk_norm_kind="weightless_rms",
        qk_norm_eps=float(kwargs.get("qk_norm_eps", norm_eps)),
        q_scale_factor=float(kwargs.get("q_scale_factor", 3.87)), attention_gate="sigmoid",
        attention_gate_dim=inner, norm_layout="sandwich", centered_rms_norm=True, norm_eps=norm_eps,
        post_norm_eps=float(kwargs.get("post_norm_eps", 1e-8)), embedding_norm_kind="weightless_rms",
        embedding_norm_eps=float(kwargs.get("embedding_norm_eps", norm_eps)), adapter_type=adapter_type,
        adapter_dim=int(kwargs.get("adapter_dim", 0)), lora_rank=int(kwargs.get("lora_rank", 8)),
        lora_alpha=float(kwargs.get("lora_alpha", 16.0)), lora_dropout=float(kwargs.get("lora_dropout", 0.0)),
        lora_targets=lora_targets, lora_bias=bool(kwargs.get("lora_bias", False)),
        qlora_group_size=int(kwargs.get("qlora_group_size", 64)),
        qlora_compute_dtype=str(kwargs.get("qlora_compute_dtype", "bf16")))
    passthrough = {k: v for k, v in kwargs.items()
                   if k not in BlockSpec.__dataclass_fields__ and k not in ("rope_base", "n_head")}
    passthrough.setdefault("model_dim", model_dim)
    defaults = dict(num_layers=52, vocab_size=202_048, tie_embeddings=False,
                    max_position_embeddings=131_072, output_multiplier=0.19611613513818404,
                    logit_softcap=20.0)
    adapter = adapter_type if adapter_type in ("lora", "qlora") else "none"
    spec = _base_model_spec(passthrough, TemplateSpec(backbone="muse_glimmer", runtime="eager", adapter=adapter),
                            block, False, defaults)
    if kwargs.get("with_vision") or isinstance(kwargs.get("vision"), (dict, MuseGlimmerVisionSpec)):
        v = kwargs.get("vision")
        spec.vision = v if isinstance(v, MuseGlimmerVisionSpec) else MuseGlimmerVisionSpec(**(v or {}))
    if kwargs.get("with_dflash") or isinstance(kwargs.get("dflash"), (dict, MuseGlimmerDFlashSpec)):
        d = kwargs.get("dflash")
        spec.dflash = d if isinstance(d, MuseGlimmerDFlashSpec) else MuseGlimmerDFlashSpec(**(d or {}))
    return spec


def glimmer_benchmark_shape(**over: Any) -> ModelSpec:
    """The ~29B decoder shape used for TP=8 inference measurements: 48 layers, residual
    6656, 32 q / 2 kv heads x 128, three sliding-window-4096 RoPE layers then one global NoPE
    layer, SwiGLU 24576, untied head over 202048 tokens, output soft-cap 30."""
    args = dict(num_layers=48, window_size=4096, intermediate_size=24_576, logit_softcap=30.0)
    args.update(over)
    return build_muse_glimmer_spec(**args)

"""Which model families this framework can train and serve natively, and how.

Every capability is an explicit record that either proves itself or says why not (fail
closed): a family name or alias resolves to a ``NativeTrainerSpec``; ``classify_native_model``
maps a preset / template / family string to one; ``capability_proof_for`` returns what the
native path can do for it (training engine, inference engine, parallel modes, checkpoint
formats) together with the reason for anything it cannot.

Execution routes in this framework:
  * ``native-gpt``    - ``models/gpt2.py`` + ``trainers/dense_gpt.py`` (explicit forward/backward
                        on the tcgen05 kernel library, one CUDA graph per step, DP/TP)
  * ``native-llama``  - ``models/llama.py`` (same trainer; DP, PP stages)
  * ``tensor-runtime``- the graph compiler + ``TorchTrainer`` (every preset runs here; the hot
                        stages call the kernel library)
The reference ships one native binary per family (``nfn_<family>_native_train``); the family
names, aliases and shipped presets below follow its registry
(``neuralfn/native_registry.py:33-94``, ``cli/nfn.py:217-277``).
"""
from __future__ import annotations

from dataclasses import dataclass, field

__all__ = ["shipped_preset_header", "NativeTrainerSpec", "NativeCapabilityProof", "NATIVE_FAMILIES", "resolve_family", "classify_native_model", "capability_proof_for",
           "native_families_report"]


@dataclass(frozen=True)
class NativeTrainerSpec:
    family: str
    aliases: tuple[str, ...]
    reference_binary: str
    presets: tuple[str, ...]
    route: str                      # native-gpt | native-llama | native-moe | tensor-runtime
    resident_inference: bool = False
    parallel: tuple[str, ...] = ()
    checkpoint_formats: tuple[str, ...] = ()


@dataclass(frozen=True)
class NativeCapabilityProof:
    family: str
    preset: str | None
    native_training: bool
    native_inference: bool
    route: str
    parallel: tuple[str, ...]
    checkpoint_formats: tuple[str, ...]
    reasons: tuple[str, ...] = field(default_factory=tuple)

    def require(self, capability: str) -> None:
        if not getattr(self, capability):
            raise ValueError(f"{self.family}: {capability} is not available ({'; '.join(self.reasons) or 'no proof'})")


def _spec(family, aliases, presets, route="tensor-runtime", **kw) -> NativeTrainerSpec:
    return NativeTrainerSpec(family, tuple(aliases), f"nfn_{family.replace('-', '_')}_native_train", tuple(presets), route, **kw)


_GPT_PRESETS = ("gpt2", "gpt2_diff", "gpt2_megakernel", "gpt2_moa", "gpt2_modern", "gpt2_qknorm", "gpt2_softcap", "gpt2_stable", "gpt2_zloss",
                "nanogpt", "nanogpt_fast")
_LLAMA_PRESETS = ("llama", "llama_fast", "llama_fast_1b", "llama_megakernel", "llama_modern", "modern_norms_llama", "gemma3", "diff_transformer",
                  "longctx_sparse_llama", "qwen3_longctx", "fp8_llama", "mxfp4_llama", "ternary_b158", "kv_pca_llama")

NATIVE_FAMILIES: dict[str, NativeTrainerSpec] = {s.family: s for s in (
    _spec("gpt", ("gpt2", "gpt3", "nanogpt"), _GPT_PRESETS, "native-gpt", resident_inference=True, parallel=("dp", "tp"),
          checkpoint_formats=("dense-v5", "named-tensors")),
    _spec("gpt2-evo", (), ("gpt2_evo",)),
    _spec("llama", (), _LLAMA_PRESETS, "native-llama", resident_inference=True, parallel=("dp", "pp", "tp"),
          checkpoint_formats=("named-tensors", "family-llama-f32", "gguf", "parallel-safetensors", "hf-llama-directory")),
    _spec("mixllama", ("moe",), ("mixllama", "mixllama_fast", "moe", "moe_modern", "deepseek_v3"), "native-moe", parallel=("dp", "ep"),
          checkpoint_formats=("parallel-safetensors",)),
    _spec("muse-glimmer", ("glimmer",), ("muse_glimmer",), resident_inference=True, checkpoint_formats=("named-tensors", "gguf")),
    _spec("deepseek-v4", (), ("deepseek_v4",)), _spec("jepa", (), ("jepa",)), _spec("semantic-dense-jepa", (), ("semantic_dense_jepa",)),
    _spec("moe-jepa-evo", (), ("moe_jepa_evo",)), _spec("semantic-router-moe", (), ("semantic_router_moe",)), _spec("jamba", (), ("jamba",)),
    _spec("seq2seq", (), ("seq2seq",)), _spec("diffusion", (), ("diffusion",)), _spec("ttt-llama", (), ("ttt_llama",)),
    _spec("hnet-lm", (), ("hnet_lm",)), _spec("universal-llama", (), ("universal_llama",)),
)}

# presets whose block differs from what the explicit native engines implement: they train through the tensor runtime
_NATIVE_GPT_OK = {"gpt2", "gpt2_qknorm", "gpt2_softcap", "gpt2_stable", "gpt2_zloss", "nanogpt"}
_NATIVE_LLAMA_OK = {"llama", "llama_fast", "llama_fast_1b", "llama_modern"}
# the expert-parallel MoE Llama (parallel/moe_llama.py) covers the plain routed-SwiGLU block: softmax / sigmoid /
# sqrt-softplus top-k routing, density balance loss, router z-loss; shared experts and aux-free biasing go through the tensor runtime
_NATIVE_MOE_OK = {"moe", "mixllama", "mixllama_fast"}


def _norm(name: str) -> str:
    return str(name).strip().lower().replace("_", "-")


def resolve_family(name: str) -> NativeTrainerSpec:
    key = _norm(name)
    for spec in NATIVE_FAMILIES.values():
        if key == spec.family or key in (_norm(a) for a in spec.aliases):
            return spec
    raise KeyError(f"unknown model family {name!r}; known: {', '.join(sorted(NATIVE_FAMILIES))}")


def classify_native_model(name: str) -> tuple[NativeTrainerSpec, str | None]:
    """Family, alias or preset name -> (spec, preset or None). Unknown names raise."""
    try:
        return resolve_family(name), None
    except KeyError:
        pass
    key = str(name).strip().lower().replace("-", "_")
    for spec in NATIVE_FAMILIES.values():
        if key in spec.presets:
            return spec, key
    raise KeyError(f"{name!r} is neither a model family nor a shipped preset")


def capability_proof_for(name: str) -> NativeCapabilityProof:
    spec, preset = classify_native_model(name)
    reasons: list[str] = []
    route = spec.route
    if route == "native-gpt" and preset is not None and preset not in _NATIVE_GPT_OK:
        route = "tensor-runtime"
        reasons.append(f"preset {preset} uses blocks outside the explicit GPT engine (qk-norm / softcap / z-loss / stable variants are inside)")
    if route == "native-llama" and preset is not None and preset not in _NATIVE_LLAMA_OK:
        route = "tensor-runtime"
        reasons.append(f"preset {preset} uses blocks outside the explicit Llama engine")
    if route == "native-moe" and preset is not None and preset not in _NATIVE_MOE_OK:
        route = "tensor-runtime"
        reasons.append(f"preset {preset} uses blocks outside the expert-parallel MoE Llama (shared experts, aux-free balancing, MLA)")
    native_training = route in ("native-gpt", "native-llama", "native-moe")
    if not native_training and not reasons:
        reasons.append("the family trains through the graph compiler and TorchTrainer; its hot stages call the kernel library")
    if not spec.resident_inference:
        reasons.append("no resident-engine block layout for this family; inference runs through the tensor runtime")
    return NativeCapabilityProof(spec.family, preset, native_training, spec.resident_inference, route,
                                 spec.parallel if native_training else (), spec.checkpoint_formats, tuple(reasons))


def native_families_report() -> list[dict]:
    return [{"family": s.family, "aliases": list(s.aliases), "reference_binary": s.reference_binary, "route": s.route, "presets": list(s.presets),
             "resident_inference": s.resident_inference, "parallel": list(s.parallel), "checkpoint_formats": list(s.checkpoint_formats)}
            for s in NATIVE_FAMILIES.values()]


def shipped_preset_header() -> str:
    """C header with the shipped preset names and the family each one trains under, compiled into
    the host runtime (``nfn_rt_preset_family``) so native tools can validate a template name
    without Python. ``csrc/runtime/shipped_presets.h`` is this text; a test keeps the two equal.
    Reference counterpart: ``csrc/native_train/shipped_gpt_template_presets.h`` and its generator."""
    from .presets import SHIPPED_GPT_TEMPLATE_PRESETS
    rows = []
    for name in SHIPPED_GPT_TEMPLATE_PRESETS:
        try:
            family = classify_native_model(name)[0].family
        except KeyError:
            family = "tensor-runtime"
        rows.append(f'    {{"{name}", "{family}"}},')
    body = "\n".join(rows)
    return ("// Generated by neuralfn_b200.native_registry.shipped_preset_header(); do not edit by hand.\n"
            "#pragma once\n\nnamespace nfn_rt {\n\nstruct ShippedPreset {\n  const char* name;\n  const char* family;\n};\n\n"
            f"constexpr int kShippedPresetCount = {len(rows)};\n"
            "constexpr ShippedPreset kShippedPresets[kShippedPresetCount] = {\n" + body + "\n};\n\n}  // namespace nfn_rt\n")

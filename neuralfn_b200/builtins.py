"""Catalogue of ready-made neurons: the 27 scalar functions and one ``module`` neuron per
tensor stage. ``BUILTIN_MAP[name]`` gives a template ``NeuronDef``; use
``BuiltinNeurons.make(name)`` for a fresh copy (new id) to place in a graph.
Reference: ``neuralfn/builtins.py:1934-2108``."""
from __future__ import annotations

import copy

from .neuron import NeuronDef, new_id
from .scalar_builtins import SPECS, make_builtin
from .tensor.ports import MODULE_PORTS, make_module_neuron

__all__ = ["BuiltinNeurons", "BUILTIN_NEURONS", "BUILTIN_MAP", "default_gpt_config"]


def default_gpt_config() -> dict:
    return {"vocab_size": 256, "num_layers": 4, "model_dim": 128, "num_heads": 4, "num_kv_heads": 2,
            "mlp_mult": 2, "tie_embeddings": True, "logit_softcap": 30.0, "rope_base": 10000.0,
            "qk_gain_init": 1.0}


def _default_config(module_type: str) -> dict:
    g = default_gpt_config()
    d, h, kv = g["model_dim"], g["num_heads"], g["num_kv_heads"]
    hd = d // h
    table = {
        "token_embedding": {"vocab_size": g["vocab_size"], "model_dim": d},
        "absolute_position_embedding": {"max_seq_len": 1024, "model_dim": d},
        "lm_head": {"model_dim": d, "vocab_size": g["vocab_size"]},
        "logit_softcap": {"softcap": g["logit_softcap"]}, "rms_norm": {"eps": 1e-6},
        "layer_norm": {"model_dim": d}, "dyt": {"model_dim": d}, "group_norm": {"model_dim": d},
        "residual_add": {"dim": d, "init_scale": 1.0}, "residual_mix": {"dim": d},
        "manifold_hyper_connection": {"dim": d},
        "linear": {"input_dim": d, "output_dim": d, "bias": False},
        "bitlinear_ternary": {"input_dim": d, "output_dim": d}, "fp8_linear": {"input_dim": d, "output_dim": d},
        "mx_linear": {"input_dim": d, "output_dim": d}, "lora_linear": {"input_dim": d, "output_dim": d},
        "nf4_linear": {"input_dim": d, "output_dim": d}, "randmap_adapter": {"model_dim": d, "adapter_dim": 16},
        "swiglu": {"model_dim": d, "mlp_mult": g["mlp_mult"]}, "geglu": {"model_dim": d}, "reglu": {"model_dim": d},
        "solu": {"model_dim": d}, "mlp_relu2": {"model_dim": d, "mlp_mult": g["mlp_mult"]},
        "reshape_heads": {"num_heads": h}, "repeat_kv": {"num_heads": h, "num_kv_heads": kv},
        "rotary_embedding": {"head_dim": hd, "rope_base": g["rope_base"], "convention": "legacy"},
        "qk_gain": {"num_heads": h, "qk_gain_init": 1.0},
        "scaled_dot_product_attention": {"is_causal": True},
        "causal_self_attention": {"model_dim": d, "num_heads": h, "num_kv_heads": kv, "rope_base": g["rope_base"],
                                  "qk_gain_init": 1.0},
        "fused_causal_attention": {"model_dim": d, "num_heads": h, "num_kv_heads": h},
        "multi_latent_attention": {"model_dim": d, "num_heads": h},
        "dflash_attention": {"model_dim": d, "num_heads": h, "num_kv_heads": kv, "head_dim": hd, "window_size": 256},
        "kv_pca_encode": {"head_dim": 64, "compressed_dim": 16}, "kv_pca_decode": {"head_dim": 64, "compressed_dim": 16},
        "kv_quant_unpack": {"head_dim": 64},
        "router_logits": {"model_dim": d, "experts": 8}, "auxfree_load_balancing": {"experts": 8, "top_k": 2},
        "topk_route": {"top_k": 2, "experts": 8}, "expert_dispatch": {"model_dim": d, "experts": 8, "mlp_mult": 2.0},
        "load_balance_loss": {"experts": 8}, "aux_loss_add": {"coef": 0.01}, "loss_scale": {"coef": 1.0},
        "tensor_scale": {"scale": 1.0}, "mamba": {"model_dim": d}, "ttt_linear": {"input_dim": d, "output_dim": d},
        "universal_transformer": {"model_dim": d, "num_heads": h}, "act_halt_gate": {"model_dim": d},
        "running_mean_decoder": {"model_dim": d}, "attentionless_decoder": {"vocab_size": g["vocab_size"]}, "jepa_projector": {"input_dim": d, "latent_dim": d},
        "jepa_predictor": {"latent_dim": d}, "mask_scheduler": {"vocab_size": g["vocab_size"], "mask_token_id": 0},
        "denoise_head": {"model_dim": d, "vocab_size": g["vocab_size"]}, "byte_patch_embed": {"model_dim": d},
        "reward_head": {"model_dim": d}, "masked_reward_head": {"model_dim": d}, "value_head": {"model_dim": d},
        "policy_logits_value": {"model_dim": d, "vocab_size": g["vocab_size"]},
    }
    return dict(table.get(module_type, {}))


class BuiltinNeurons:
    @staticmethod
    def scalar_names() -> list[str]:
        return [s.name for s in SPECS]

    @staticmethod
    def module_names() -> list[str]:
        return sorted(MODULE_PORTS)

    @staticmethod
    def make(name: str, config: dict | None = None) -> NeuronDef:
        if name in MODULE_PORTS:
            cfg = _default_config(name)
            cfg.update(config or {})
            return make_module_neuron(name, cfg)
        return make_builtin(name)

    @classmethod
    def all(cls) -> list[NeuronDef]:
        return [cls.make(n) for n in cls.scalar_names()] + [cls.make(n) for n in cls.module_names()]


BUILTIN_NEURONS: list[NeuronDef] = BuiltinNeurons.all()
BUILTIN_MAP: dict[str, NeuronDef] = {n.name: n for n in BUILTIN_NEURONS}

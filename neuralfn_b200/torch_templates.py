"""Template builders: ``ModelSpec`` -> graph of tensor-stage neurons.

``build_gpt_root_graph(spec)`` returns a ``NeuronGraph`` (runtime ``torch``) with inputs
``tokens`` and ``target_ids`` and the scalar loss as output:

    embed [+abs-pos] [+embedding norm] -> N x decoder block (subgraph nodes bound to a
    ``variant_library`` entry) -> final norm -> (tied) head [x multiplier] [soft-cap]
    -> cross-entropy (z-loss) [+ coef * sum(aux losses)]

Blocks are pre-norm residual (or sandwich-norm for Muse-Glimmer) around an attention
subgraph (q/k/v linear -> heads -> [qk-norm] -> [rope] -> [repeat-kv] -> attention variant
-> merge -> out-proj) and an MLP subgraph (GELU / gated / MoE with router, top-k, dispatch,
load-balance loss). SFT, DPO, reward-model and PPO roots wrap the same model stage.
Reference: ``neuralfn/torch_templates.py:223-490,1328-1540,4140-5168``.
"""
from __future__ import annotations

from dataclasses import asdict
from typing import Any

from .config import BlockSpec, LayerAttentionSpec, ModelSpec
from .graph import Edge, NeuronGraph, NeuronInstance
from .neuron import NeuronDef, subgraph_neuron
from .tensor.ports import make_module_neuron, module_ports

__all__ = ["GraphBuilder", "build_dense_attention_graph", "build_dense_mlp_graph", "build_moe_mlp_graph",
           "build_decoder_block_graph", "build_model_stage_graph", "build_gpt_root_graph",
           "build_gpt_template_payload", "build_sft_root_graph", "build_dpo_root_graph",
           "build_reward_model_root_graph", "build_ppo_root_graph", "build_model_spec_from_config"]

Ref = tuple[str, int]  # (node id, output port)


class GraphBuilder:
    """Small helper: add module/subgraph nodes wired from ``(node, port)`` references."""

    def __init__(self, name: str, **graph_kw: Any) -> None:
        self.graph = NeuronGraph(name=name, runtime="torch", training_method="torch", **graph_kw)
        self._n = 0
        self._col = 0

    def _add(self, ndef: NeuronDef, node_id: str | None, inputs: list[Ref]) -> str:
        nid = node_id or f"{ndef.name}_{self._n}"
        self._n += 1
        self._col += 1
        self.graph.add_node(NeuronInstance(ndef, instance_id=nid, position=(220.0 * self._col, 80.0 * (self._n % 5))))
        for port, (src, sport) in enumerate(inputs):
            self.graph.add_edge(Edge(id=f"{src}.{sport}->{nid}.{port}", src_node=src, src_port=sport,
                                     dst_node=nid, dst_port=port))
        return nid

    def input(self, name: str, dtype: str = "tensor") -> Ref:
        from .port import Port
        from .neuron import module_neuron
        nd = module_neuron(name=name, module_type="input", input_ports=[], output_ports=[Port(name, dtype=dtype)])
        nid = self._add(nd, name, [])
        self.graph.input_node_ids.append(nid)
        return (nid, 0)

    def node(self, module_type: str, config: dict | None = None, inputs: list[Ref] | None = None,
             node_id: str | None = None) -> str:
        return self._add(make_module_neuron(module_type, config), node_id, inputs or [])

    def subgraph(self, graph: NeuronGraph, name: str, inputs: list[Ref], node_id: str | None = None,
                 in_aliases: list[str] | None = None, out_aliases: list[str] | None = None,
                 variant_ref: dict[str, str] | None = None) -> str:
        if graph.variant_library:
            # variant references resolve against the outermost graph: hoist a nested library
            for fam, versions in graph.variant_library.items():
                self.graph.variant_library.setdefault(fam, {}).update(versions)
            graph.variant_library = {}
        nd = subgraph_neuron(graph, name=name, input_aliases=in_aliases, output_aliases=out_aliases,
                             variant_ref=variant_ref)
        return self._add(nd, node_id, inputs)

    def outputs(self, *refs: Ref) -> NeuronGraph:
        """Mark output nodes. A reference to a non-zero port is routed through a ``tensor_scale(1)``."""
        for nid, port in refs:
            if port != 0 or len(self.graph.nodes[nid].neuron_def.output_ports) != 1:
                nid = self.node("tensor_scale", {"scale": 1.0}, [(nid, port)])
            self.graph.output_node_ids.append(nid)
        return self.graph


def _linear(b: GraphBuilder, x: Ref, din: int, dout: int, bias: bool, bs: BlockSpec, target: str,
            node_id: str | None = None) -> Ref:
    """A projection honouring compression and adapter settings of the block."""
    cfg = {"input_dim": din, "output_dim": dout, "bias": bias}
    adapter = bs.adapter_type
    if adapter in ("lora", "qlora") and target in bs.lora_targets:
        kind = "nf4_linear" if adapter == "qlora" else "lora_linear"
        cfg.update({"rank": bs.lora_rank, "alpha": bs.lora_alpha, "dropout": bs.lora_dropout})
        if kind == "nf4_linear":
            cfg.update({"group_size": bs.qlora_group_size, "compute_dtype": bs.qlora_compute_dtype})
        return (b.node(kind, cfg, [x], node_id), 0)
    comp = bs.compression
    if comp == "ternary_b158":
        return (b.node("bitlinear_ternary", {"input_dim": din, "output_dim": dout}, [x], node_id), 0)
    if comp in ("fp8_e4m3", "fp8_e5m2"):
        cfg.update({"fp8_format": comp.split("_")[1], "amax_history_len": bs.fp8_amax_history_len,
                    "use_stochastic_rounding": bs.fp8_use_stochastic_rounding})
        return (b.node("fp8_linear", cfg, [x], node_id), 0)
    if comp in ("mxfp4", "mxfp8"):
        cfg.update({"mx_format": comp, "mx_block_size": bs.mx_block_size})
        return (b.node("mx_linear", cfg, [x], node_id), 0)
    return (b.node("linear", cfg, [x], node_id), 0)


def _geometry(spec: ModelSpec) -> tuple[int, int, int, int]:
    bs = spec.block_spec
    heads = bs.num_heads
    kv = bs.num_kv_heads or heads
    hd = bs.head_dim or spec.model_dim // heads
    inner = bs.attention_inner_dim or heads * hd
    return heads, kv, hd, inner


def build_dense_attention_graph(spec: ModelSpec, layer_index: int = 0, *, cross: bool = False) -> NeuronGraph:
    """hidden -> attention output (residual not included). ``cross``: a second input ``context``
    supplies keys and values (encoder-decoder attention: bidirectional, no rotary embedding)."""
    bs = spec.block_spec
    d = spec.model_dim
    heads, kv, hd, inner = _geometry(spec)
    b = GraphBuilder(f"cross_attention_{layer_index}" if cross else f"attention_{layer_index}")
    x = b.input("x")
    if cross:
        ctx = b.input("context")
        q = _linear(b, x, d, inner, bs.linear_bias, bs, "q_proj", "q_proj")
        k = _linear(b, ctx, d, kv * hd, bs.linear_bias, bs, "k_proj", "k_proj")
        v = _linear(b, ctx, d, kv * hd, bs.linear_bias, bs, "v_proj", "v_proj")
        qh = (b.node("reshape_heads", {"num_heads": heads}, [q]), 0)
        kh = (b.node("reshape_heads", {"num_heads": kv}, [k]), 0)
        vh = (b.node("reshape_heads", {"num_heads": kv}, [v]), 0)
        if bs.use_qk_norm:
            n = b.node("qk_norm", {"eps": bs.qk_norm_eps}, [qh, kh])
            qh, kh = (n, 0), (n, 1)
        a = b.node("scaled_dot_product_attention", {"is_causal": False, "dropout_p": bs.dropout_p}, [qh, kh, vh])
        merged_c: Ref = (b.node("merge_heads", {}, [(a, 0)]), 0)
        return b.outputs(_linear(b, merged_c, inner, d, bs.linear_bias, bs, "o_proj", "o_proj"))
    if spec.template.runtime == "megakernel" and bs.pos_encoding == "rope" and bs.attention_variant == "dense" \
            and bs.attention_gate == "none" and not bs.layer_attention_pattern:
        y = b.node("fused_causal_attention", {"model_dim": d, "num_heads": heads, "num_kv_heads": kv,
                                              "rope_base": bs.rope_theta, "dropout_p": bs.dropout_p}, [x])
        return b.outputs((y, 0))
    if bs.attention_variant == "mla":
        y = b.node("multi_latent_attention", {"model_dim": d, "num_heads": heads, "rope_base": bs.rope_theta,
                                              "dropout_p": bs.dropout_p}, [x])
        return b.outputs((y, 0))
    layer_attn: LayerAttentionSpec | None = bs.layer_attention(layer_index)
    q = _linear(b, x, d, inner, bs.linear_bias, bs, "q_proj", "q_proj")
    k = _linear(b, x, d, kv * hd, bs.linear_bias, bs, "k_proj", "k_proj")
    v = _linear(b, x, d, kv * hd, bs.linear_bias, bs, "v_proj", "v_proj")
    qh = (b.node("reshape_heads", {"num_heads": heads}, [q]), 0)
    kh = (b.node("reshape_heads", {"num_heads": kv}, [k]), 0)
    vh = (b.node("reshape_heads", {"num_heads": kv}, [v]), 0)
    if bs.use_qk_norm:
        n = b.node("qk_norm", {"eps": bs.qk_norm_eps, "force_float32": bs.family == "muse_glimmer"}, [qh, kh])
        qh, kh = (n, 0), (n, 1)
    if bs.q_scale_factor != 1.0:
        qh = (b.node("tensor_scale", {"scale": bs.q_scale_factor}, [qh]), 0)
    use_rope = bs.pos_encoding == "rope"
    theta = bs.rope_theta
    convention = "hf" if bs.family == "muse_glimmer" else "legacy"
    if layer_attn is not None:
        use_rope = layer_attn.pos_encoding == "rope"
        theta = layer_attn.rope_theta
    if use_rope:
        r = b.node("rotary_embedding", {"head_dim": hd, "rope_base": theta, "rope_scaling": bs.rope_scaling,
                                        "convention": convention}, [qh, kh])
        qh, kh = (r, 0), (r, 1)
    if bs.family in ("nanogpt",) or bs.qk_gain_init != 1.0:
        qh = (b.node("qk_gain", {"num_heads": heads, "qk_gain_init": bs.qk_gain_init}, [qh]), 0)
    if bs.compression == "kv_pca":
        comp_dim = max(2, hd // 4)
        enc_k = (b.node("kv_pca_encode", {"head_dim": hd, "compressed_dim": comp_dim}, [kh]), 0)
        enc_v = (b.node("kv_pca_encode", {"head_dim": hd, "compressed_dim": comp_dim}, [vh]), 0)
        kh = (b.node("kv_pca_decode", {"head_dim": hd, "compressed_dim": comp_dim}, [enc_k]), 0)
        vh = (b.node("kv_pca_decode", {"head_dim": hd, "compressed_dim": comp_dim}, [enc_v]), 0)
    variant = bs.attention_variant
    window = bs.window_size
    if layer_attn is not None:
        variant = "sliding_window" if layer_attn.kind == "local" else "dense"
        window = layer_attn.window_size
    common = {"is_causal": bs.is_causal, "dropout_p": bs.dropout_p}
    if variant == "sliding_window":
        a = b.node("sliding_window_attention", {"window_size": window or 256, **common}, [qh, kh, vh])
    elif variant == "block_sparse":
        a = b.node("block_sparse_attention", {"sparse_block_size": bs.sparse_block_size,
                                              "num_sinks": bs.num_sinks, **common}, [qh, kh, vh])
    elif variant == "streaming":
        a = b.node("streaming_attention_sinks", {"window_size": window or 256, "num_sinks": bs.num_sinks or 4,
                                                 **common}, [qh, kh, vh])
    elif variant == "nsa":
        a = b.node("native_sparse_attention", {"window_size": window or 128, "sparse_block_size": bs.sparse_block_size,
                                               "num_sinks": bs.num_sinks, "compress_stride": bs.nsa_compress_stride,
                                               **common}, [qh, kh, vh])
    elif variant == "differential":
        a = b.node("differential_attention", {"lambda_init": bs.diff_lambda_init, **common}, [qh, kh, vh])
    else:
        a = b.node("scaled_dot_product_attention", {"backend": bs.attention_backend, **common}, [qh, kh, vh])
    merged: Ref = (b.node("merge_heads", {}, [(a, 0)]), 0)
    if bs.attention_gate == "sigmoid":
        g = _linear(b, x, d, bs.attention_gate_dim or inner, False, bs, "attn_gate_proj", "attn_gate_proj")
        gs = (b.node("sigmoid", {}, [g]), 0)
        merged = (b.node("multiply", {}, [merged, gs]), 0)
    out = _linear(b, merged, inner, d, bs.linear_bias, bs, "o_proj", "o_proj")
    if bs.dropout_p > 0:
        out = (b.node("dropout", {"p": bs.dropout_p}, [out]), 0)
    return b.outputs(out)


def build_dense_mlp_graph(spec: ModelSpec) -> NeuronGraph:
    bs = spec.block_spec
    d = spec.model_dim
    b = GraphBuilder("mlp")
    x = b.input("x")
    kind = bs.mlp_type
    if kind == "swiglu":
        if bs.adapter_type in ("lora", "qlora") or bs.compression not in ("none", "kv_pca") or bs.intermediate_size:
            from .tensor.stages_linear import swiglu_hidden
            hidden = bs.intermediate_size or swiglu_hidden(d, bs.mlp_multiplier, bs.multiple_of)
            g = _linear(b, x, d, hidden, False, bs, "gate_proj", "gate_proj")
            u = _linear(b, x, d, hidden, False, bs, "up_proj", "up_proj")
            act = (b.node("silu", {}, [g]), 0)
            h = (b.node("multiply", {}, [act, u]), 0)
            y = _linear(b, h, hidden, d, False, bs, "down_proj", "down_proj")
        else:
            y = (b.node("swiglu", {"model_dim": d, "mlp_mult": bs.mlp_multiplier, "multiple_of": bs.multiple_of}, [x]), 0)
    elif kind in ("geglu", "reglu", "solu"):
        y = (b.node(kind, {"model_dim": d, "mlp_mult": int(bs.mlp_multiplier), "multiple_of": bs.multiple_of}, [x]), 0)
    else:
        hidden = bs.intermediate_size or int(d * bs.mlp_multiplier)
        h = _linear(b, x, d, hidden, bs.linear_bias, bs, "c_fc", "c_fc")
        h = (b.node("gelu", {}, [h]), 0)
        y = _linear(b, h, hidden, d, bs.linear_bias, bs, "c_proj", "c_proj")
    if bs.dropout_p > 0:
        y = (b.node("dropout", {"p": bs.dropout_p}, [y]), 0)
    return b.outputs(y)


def build_moe_mlp_graph(spec: ModelSpec) -> NeuronGraph:
    """hidden -> (expert output, aux loss). Aux = load-balance density loss (+ router z-loss)."""
    bs = spec.block_spec
    d, experts, top_k = spec.model_dim, int(bs.experts or 8), int(bs.top_k or 2)
    b = GraphBuilder("moe_mlp")
    x = b.input("x")
    logits: Ref = (b.node("router_logits", {"model_dim": d, "experts": experts}, [x], "router"), 0)
    routed = logits
    if bs.moe_balance_mode == "auxfree":
        routed = (b.node("auxfree_load_balancing", {"experts": experts, "top_k": top_k,
                                                    "bias_lr": bs.auxfree_bias_lr}, [logits]), 0)
    route = b.node("topk_route", {"top_k": top_k, "experts": experts, "score_fn": bs.router_score_fn}, [routed])
    disp_cfg = {"model_dim": d, "experts": experts, "mlp_mult": bs.mlp_multiplier, "multiple_of": bs.multiple_of}
    if bs.intermediate_size:
        disp_cfg["hidden_dim"] = bs.intermediate_size
    y = b.node("expert_dispatch", disp_cfg, [x, (route, 0), (route, 1)], "experts")
    out: Ref = (b.node("expert_combine", {}, [(y, 0)]), 0)
    if bs.shared_experts:
        shared = b.node("swiglu", {"model_dim": d, "mlp_mult": bs.mlp_multiplier * bs.shared_experts,
                                   "multiple_of": bs.multiple_of}, [x], "shared_expert")
        out = (b.node("residual_add", {"dim": d, "init_scale": 1.0}, [out, (shared, 0)]), 0)
    lb = b.node("load_balance_loss", {"experts": experts}, [logits, (route, 0), (route, 1)])
    aux: Ref = (b.node("loss_scale", {"coef": bs.router_aux_loss_coef}, [(lb, 0)]), 0)
    if bs.router_z_loss_coef > 0:
        z = b.node("router_z_loss", {}, [logits])
        aux = (b.node("aux_loss_add", {"coef": bs.router_z_loss_coef}, [aux, (z, 0)]), 0)
    return b.outputs(out, aux)


def _norm(b: GraphBuilder, x: Ref, spec: ModelSpec, eps: float | None = None, node_id: str | None = None) -> Ref:
    bs = spec.block_spec
    d = spec.model_dim
    if bs.norm_type == "rmsnorm":
        cfg = {"model_dim": d, "eps": eps if eps is not None else bs.norm_eps, "centered": bs.centered_rms_norm,
               "force_float32": bs.family == "muse_glimmer"}
        return (b.node("rms_norm", cfg, [x], node_id), 0)
    if bs.norm_type == "dyt":
        return (b.node("dyt", {"model_dim": d, "alpha_init": bs.dyt_alpha_init}, [x], node_id), 0)
    if bs.norm_type == "group_norm":
        return (b.node("group_norm", {"model_dim": d, "num_groups": bs.group_norm_groups}, [x], node_id), 0)
    return (b.node("layer_norm", {"model_dim": d, "eps": 1e-5}, [x], node_id), 0)


def _residual(b: GraphBuilder, x: Ref, delta: Ref, spec: ModelSpec) -> Ref:
    if spec.block_spec.residual_type == "mhc":
        return (b.node("manifold_hyper_connection", {"dim": spec.model_dim, "beta_init": 0.1}, [x, delta]), 0)
    return (b.node("residual_add", {"dim": spec.model_dim, "init_scale": 1.0}, [x, delta]), 0)


def build_routed_mlp_graph(spec: ModelSpec, experts: int) -> NeuronGraph:
    """(hidden, routing weights, routing indices) -> expert output: an MoE MLP whose routes come from
    outside the block (the semantic routers). Same shape as the reference's
    ``build_semantic_router_mlp_graph`` (``neuralfn/torch_templates.py:1414``)."""
    bs = spec.block_spec
    b = GraphBuilder("semantic_router_mlp")
    x, rw, ri = b.input("x"), b.input("routing_weights"), b.input("routing_indices")
    cfg = {"model_dim": spec.model_dim, "experts": experts, "mlp_mult": bs.mlp_multiplier, "multiple_of": bs.multiple_of}
    if bs.intermediate_size:
        cfg["hidden_dim"] = bs.intermediate_size
    y = b.node("expert_dispatch", cfg, [x, rw, ri], "dispatch")
    return b.outputs((b.node("expert_combine", {}, [(y, 0)], "combine"), 0))


def build_decoder_block_graph(spec: ModelSpec, layer_index: int = 0, *, cross: bool = False,
                              routed_experts: int = 0) -> NeuronGraph:
    """hidden -> hidden (dense) or (hidden, aux loss) for MoE blocks. ``cross``: second input
    ``context`` and a cross-attention sub-layer between self-attention and the MLP (decoder of an
    encoder-decoder stack). ``routed_experts`` > 0: inputs (x, routing_weights, routing_indices) and
    an externally routed MoE MLP with that many experts, no aux output."""
    bs = spec.block_spec
    b = GraphBuilder(f"block_{layer_index}")
    x = b.input("x")
    context = b.input("context") if cross else None
    routes = (b.input("routing_weights"), b.input("routing_indices")) if routed_experts else None
    sandwich = bs.norm_layout == "sandwich"
    attn_graph = build_dense_attention_graph(spec, layer_index)
    if bs.family == "jamba" and layer_index % 2 == 1:
        a_out: Ref = (b.node("mamba", {"model_dim": spec.model_dim}, [_norm(b, x, spec)], "mamba"), 0)
    elif bs.family == "ttt":
        n = _norm(b, x, spec)
        a_out = (b.node("ttt_linear", {"input_dim": spec.model_dim, "output_dim": spec.model_dim,
                                       "hidden_dim": bs.ttt_hidden_dim}, [n], "ttt"), 0)
    else:
        a_out = (b.subgraph(attn_graph, "attention", [_norm(b, x, spec, node_id="attn_norm")], "attention",
                            ["x"], ["y"]), 0)
    if sandwich:
        a_out = _norm(b, a_out, spec, bs.post_norm_eps, "post_attn_norm")
    h1 = _residual(b, x, a_out, spec)
    if context is not None:
        c_out: Ref = (b.subgraph(build_dense_attention_graph(spec, layer_index, cross=True), "cross_attention",
                                 [_norm(b, h1, spec, node_id="cross_attn_norm"), context], "cross_attention",
                                 ["x", "context"], ["y"]), 0)
        h1 = _residual(b, h1, c_out, spec)
    n2 = _norm(b, h1, spec, node_id="mlp_norm")
    aux: Ref | None = None
    if routes is not None:
        m_out = (b.subgraph(build_routed_mlp_graph(spec, routed_experts), "semantic_router_mlp", [n2, routes[0], routes[1]],
                            "mlp", ["x", "routing_weights", "routing_indices"], ["y"]), 0)
    elif bs.mlp_type == "moe":
        m = b.subgraph(build_moe_mlp_graph(spec), "moe_mlp", [n2], "mlp", ["x"], ["y", "aux_loss"])
        m_out, aux = (m, 0), (m, 1)
    else:
        m_out = (b.subgraph(build_dense_mlp_graph(spec), "mlp", [n2], "mlp", ["x"], ["y"]), 0)
    if sandwich:
        m_out = _norm(b, m_out, spec, bs.post_norm_eps, "post_mlp_norm")
    h2 = _residual(b, h1, m_out, spec)
    if bs.adapter_type == "randmap" and bs.adapter_dim > 0:
        h2 = (b.node("randmap_adapter", {"model_dim": spec.model_dim, "adapter_dim": bs.adapter_dim}, [h2]), 0)
    return b.outputs(h2, aux) if aux is not None else b.outputs(h2)


def __getattr__(name: str):
    # root/model-stage builders live in torch_templates_roots (imported lazily: it imports this module)
    from . import torch_templates_roots as _roots
    if hasattr(_roots, name):
        return getattr(_roots, name)
    raise AttributeError(name)

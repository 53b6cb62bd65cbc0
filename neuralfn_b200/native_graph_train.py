"""Preflight for training a *graph file* on a native engine.

``plan_native_graph_training(graph.json)`` reads one immutable byte snapshot of the file, parses
it strictly (no duplicate keys, no NaN / Infinity, bounded size), never executes any neuron
source stored in it, and decides whether the graph is exactly what a native engine implements:

1. the graph carries a ``template_spec`` (the model specification it was built from);
2. rebuilding a graph from that specification gives the same *shape hash* - a SHA-256 over the
   canonical structure (node module types and configurations, edges, nested variant libraries;
   ids, positions and trained state excluded) - so nothing was edited by hand;
3. the specification sits inside the native engine's envelope (family, block options, inactive
   fields at their defaults); every violation is reported as a *blocker*.

The result (``NativeGraphTrainPlan``) holds the selector (``gpt2``, ``gpt2_qknorm``, ``llama``
...), the route, the ``NativeTrainConfig`` fields and the equivalent ``nfn train`` argument
vector - or the list of blockers. ``materialize=True`` with a *new* ``artifact_dir`` writes the
sidecar files: ``source-graph.json`` (the exact bytes), ``native-training-plan.json``,
``native-training-proof.json`` (hashes and the checks that passed), ``compatibility-report.json``
and ``native-execution-manifest.json``. Unlike the reference, whose trainers do not consume the
lowered graph, the plan here is what ``run_native_training`` executes.

Behavioural counterpart: ``neuralfn/native_graph_train.py`` (``plan_native_graph_training``
:3077-3302, strict JSON :685-820, shape hashes :70-82 and ``_shape_hash`` :1838, selector
contracts :84-226, sidecars :3021-3076).
"""
from __future__ import annotations

import hashlib
import json
import math
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any

__all__ = ["NativeGraphTrainPlan", "GraphPreflightError", "strict_json_loads", "shape_hash", "plan_native_graph_training"]

MAX_GRAPH_BYTES = 256 * 1024 * 1024


class GraphPreflightError(ValueError):
    pass


def strict_json_loads(data: bytes) -> Any:
    """UTF-8 JSON without duplicate keys and without NaN / Infinity."""
    def pairs(items):
        out = {}
        for k, v in items:
            if k in out:
                raise GraphPreflightError(f"duplicate key {k!r}")
            out[k] = v
        return out

    def bad_constant(name):
        raise GraphPreflightError(f"non-finite number {name}")

    try:
        return json.loads(data.decode("utf-8"), object_pairs_hook=pairs, parse_constant=bad_constant)
    except UnicodeDecodeError as exc:
        raise GraphPreflightError("the graph file is not UTF-8") from exc
    except json.JSONDecodeError as exc:
        raise GraphPreflightError(f"invalid JSON: {exc}") from exc


def _canon(v: Any) -> Any:
    if isinstance(v, float):
        if not math.isfinite(v):
            raise GraphPreflightError("non-finite number in the graph")
        return repr(v)
    if isinstance(v, dict):
        return {k: _canon(v[k]) for k in sorted(v)}
    if isinstance(v, (list, tuple)):
        return [_canon(x) for x in v]
    return v


def _node_shape(node: dict, variants: dict, depth: int) -> Any:
    if depth > 16:
        raise GraphPreflightError("variant libraries nest too deeply")
    nd = node.get("neuron_def") or {}
    ref = nd.get("variant_ref")
    sub = nd.get("subgraph")
    if ref is not None and sub is None:
        sub = variants.get(ref if isinstance(ref, str) else json.dumps(ref, sort_keys=True))
    return {"kind": nd.get("kind"), "module_type": nd.get("module_type"), "config": _canon(nd.get("module_config") or {}),
            "inputs": [p.get("name") for p in nd.get("input_ports") or []], "outputs": [p.get("name") for p in nd.get("output_ports") or []],
            "subgraph": _graph_shape(sub, variants, depth + 1) if isinstance(sub, dict) else None}


def _graph_shape(g: dict, variants: dict, depth: int = 0) -> Any:
    nodes = g.get("nodes") or {}
    items = nodes.items() if isinstance(nodes, dict) else ((n.get("instance_id"), n) for n in nodes)
    order = {nid: i for i, (nid, _) in enumerate(sorted(items, key=lambda kv: str(kv[0])))}
    items = nodes.items() if isinstance(nodes, dict) else ((n.get("instance_id"), n) for n in nodes)
    shaped = [(str(nid), _node_shape(n, variants, depth)) for nid, n in sorted(items, key=lambda kv: str(kv[0]))]
    raw_edges = g.get("edges") or []
    raw_edges = list(raw_edges.values()) if isinstance(raw_edges, dict) else raw_edges
    edges = sorted((order.get(e.get("src_node"), -1), e.get("src_port", 0), order.get(e.get("dst_node"), -1), e.get("dst_port", 0))
                   for e in raw_edges)
    return {"nodes": shaped, "edges": edges, "inputs": [order.get(i, -1) for i in g.get("input_node_ids") or []],
            "outputs": [order.get(i, -1) for i in g.get("output_node_ids") or []]}


def shape_hash(graph_doc: dict) -> str:
    """SHA-256 of the graph's structure (what is connected to what, with which module types and
    configurations); instance positions, trained state and free-text fields do not enter."""
    lib = graph_doc.get("variant_library") or {}
    variants = {}
    if isinstance(lib, dict):
        for k, v in lib.items():
            variants[k] = v.get("graph", v) if isinstance(v, dict) else v
    payload = json.dumps(_canon(_graph_shape(graph_doc, variants)), sort_keys=True, separators=(",", ":"))
    return hashlib.sha256(payload.encode("utf-8")).hexdigest()


@dataclass
class NativeGraphTrainPlan:
    graph_path: str
    graph_sha256: str
    graph_bytes: int
    shape_sha256: str
    rebuilt_shape_sha256: str | None
    family: str | None
    selector: str | None
    route: str | None
    train_config: dict = field(default_factory=dict)
    trainer_argv: list[str] = field(default_factory=list)
    blockers: list[str] = field(default_factory=list)
    checks: list[str] = field(default_factory=list)
    artifact_dir: str | None = None

    @property
    def ok(self) -> bool:
        return not self.blockers

    def to_dict(self) -> dict:
        return asdict(self) | {"ok": self.ok}


def _gpt_selector(spec, blockers: list[str]) -> str | None:
    b = spec.block_spec
    if b.norm_type != "layernorm" or b.mlp_type != "gelu" or b.pos_encoding != "absolute":
        blockers.append("the GPT engine implements LayerNorm + GELU MLP + learned positions only")
    if b.num_kv_heads not in (None, b.num_heads):
        blockers.append("the GPT engine has no grouped-query attention")
    if b.attention_variant != "dense" or b.layer_attention_pattern:
        blockers.append("only dense causal attention is native for GPT graphs")
    if not spec.tie_embeddings:
        blockers.append("the GPT engine ties the head to the token embedding")
    if b.experts or b.adapter_type != "none" or b.compression != "none" or b.dropout_p:
        blockers.append("experts, adapters, compression and dropout are outside the GPT engine")
    if abs(b.mlp_multiplier - 4.0) > 1e-9 or b.intermediate_size not in (None, 4 * spec.model_dim):
        blockers.append("the GPT engine uses a 4x MLP")
    qk, cap, z = bool(b.use_qk_norm), spec.logit_softcap > 0, spec.z_loss_coef > 0
    table = {(False, False, False): "gpt2", (False, False, True): "gpt2_zloss", (False, True, False): "gpt2_softcap",
             (True, False, False): "gpt2_qknorm", (True, False, True): "gpt2_stable", (True, True, True): "gpt2_qknorm_softcap_zloss"}
    sel = table.get((qk, cap, z))
    if sel is None:
        blockers.append("this combination of QK norm / soft cap / z-loss has no native selector")
    return sel


def _llama_selector(spec, blockers: list[str]) -> str | None:
    b = spec.block_spec
    if b.norm_type != "rmsnorm" or b.mlp_type != "swiglu" or b.pos_encoding != "rope" or b.linear_bias:
        blockers.append("the Llama engine implements RMSNorm + SwiGLU + RoPE without biases")
    if b.rope_scaling:
        blockers.append("rotary scaling variants are not native")
    if b.attention_variant != "dense" or b.layer_attention_pattern:
        blockers.append("only dense causal attention is native for Llama graphs")
    if b.experts or b.adapter_type != "none" or b.compression != "none" or b.dropout_p:
        blockers.append("experts, adapters, compression and dropout are outside the Llama engine")
    return "llama"


def plan_native_graph_training(graph_path, artifact_dir=None, materialize: bool = False, **train_overrides) -> NativeGraphTrainPlan:
    path = Path(graph_path)
    data = path.read_bytes()  # ONE snapshot: everything below, including the sidecar copy, uses these bytes
    if len(data) > MAX_GRAPH_BYTES:
        raise GraphPreflightError("graph file too large")
    doc = strict_json_loads(data)
    if not isinstance(doc, dict) or "nodes" not in doc or "edges" not in doc:
        raise GraphPreflightError("not a graph document")
    plan = NativeGraphTrainPlan(str(path), hashlib.sha256(data).hexdigest(), len(data), shape_hash(doc), None, None, None, None)
    plan.checks.append("strict JSON: no duplicate keys, no non-finite numbers")
    tspec = (doc.get("torch_config") or {}).get("template_spec")
    if not isinstance(tspec, dict):
        plan.blockers.append("the graph carries no template_spec: it was not built from a model specification")
        return _finish(plan, data, artifact_dir, materialize)
    from .config import spec_from_dict
    from .serialization import graph_to_json
    from .torch_templates import build_gpt_root_graph
    try:
        spec = spec_from_dict(tspec)
        rebuilt = json.loads(graph_to_json(build_gpt_root_graph(spec)))
    except Exception as exc:
        plan.blockers.append(f"the template_spec does not build: {exc}")
        return _finish(plan, data, artifact_dir, materialize)
    plan.rebuilt_shape_sha256 = shape_hash(rebuilt)
    if plan.rebuilt_shape_sha256 != plan.shape_sha256:
        plan.blockers.append("the graph differs structurally from what its template_spec builds (edited by hand?)")
    else:
        plan.checks.append("shape hash equals the hash of the graph rebuilt from template_spec")
    fam = spec.block_spec.family
    plan.family = {"gpt2": "gpt", "gpt": "gpt", "nanogpt": "gpt", "llama": "llama"}.get(fam)
    if plan.family is None:
        plan.blockers.append(f"family {fam!r} trains through the tensor runtime (TorchTrainer), not a native engine")
        return _finish(plan, data, artifact_dir, materialize)
    sel_blockers: list[str] = []
    plan.selector = _gpt_selector(spec, sel_blockers) if plan.family == "gpt" else _llama_selector(spec, sel_blockers)
    plan.blockers += sel_blockers
    if spec.template.kind not in ("", "pretrain", "lm", None) if hasattr(spec.template, "kind") else False:
        plan.blockers.append("only the plain language-model root is native (fine-tuning roots use the tensor runtime)")
    plan.route = "native-gpt" if plan.family == "gpt" else "native-llama"
    b = spec.block_spec
    cfg = {"base_model": plan.family, "template_name": plan.selector or "", "n_layer": spec.num_layers, "n_head": b.num_heads,
           "n_kv_head": b.num_kv_heads or 0, "d_model": spec.model_dim, "d_ff": b.intermediate_size or 0, "vocab_size": spec.vocab_size,
           "seq_len": spec.max_position_embeddings}
    cfg.update(train_overrides)
    plan.train_config = cfg
    if plan.ok:
        plan.checks.append(f"selector {plan.selector}: block options inside the {plan.route} envelope")
        argv = ["nfn", "train", "--base-model", plan.family, "--template-name", plan.selector]
        for k in ("n_layer", "n_head", "d_model", "vocab_size", "seq_len"):
            argv += [f"--{k.replace('_', '-')}", str(cfg[k])]
        for k, v in train_overrides.items():
            argv += [f"--{k.replace('_', '-')}", str(v)]
        plan.trainer_argv = argv
    return _finish(plan, data, artifact_dir, materialize)


def _finish(plan: NativeGraphTrainPlan, data: bytes, artifact_dir, materialize: bool) -> NativeGraphTrainPlan:
    if not materialize:
        return plan
    if artifact_dir is None:
        raise GraphPreflightError("materialize=True needs an artifact_dir")
    out = Path(artifact_dir)
    if out.exists():
        raise GraphPreflightError(f"{out} exists; sidecars are only written into a new directory")
    out.mkdir(parents=True)
    plan.artifact_dir = str(out)
    (out / "source-graph.json").write_bytes(data)
    dump = lambda name, obj: (out / name).write_text(json.dumps(obj, indent=2, sort_keys=True), encoding="utf-8")  # noqa: E731
    dump("native-training-plan.json", plan.to_dict())
    dump("native-training-proof.json", {"graph_sha256": plan.graph_sha256, "shape_sha256": plan.shape_sha256,
                                        "rebuilt_shape_sha256": plan.rebuilt_shape_sha256, "checks": plan.checks, "ok": plan.ok,
                                        "trainer_consumes_plan": True})
    dump("compatibility-report.json", {"family": plan.family, "selector": plan.selector, "route": plan.route, "blockers": plan.blockers})
    dump("native-execution-manifest.json", {"schema": "neuralfn_b200.native_graph_training.v1", "source_graph": "source-graph.json",
                                            "source_graph_sha256": plan.graph_sha256, "plan": "native-training-plan.json",
                                            "status": "ready" if plan.ok else "blocked"})
    return plan

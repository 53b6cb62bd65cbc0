"""Native Execution IR: a source-inert description of a tensor graph plus its weights as a raw tensor
bundle - what a native runtime needs to execute a model without importing the graph's Python.

``migrate_graph_to_native(graph | path, out_dir)`` writes into a NEW directory:

* ``native-execution-manifest.json`` (``neuralfn.native_execution_manifest`` v1): model identity
  (name, family / preset classification, graph SHA-256), the lowered topology (nodes with their
  stage type and JSON-safe configuration, edges with ports, a topological order), tensor specs
  (name, dtype, shape, byte offset, byte length, SHA-256), capabilities, the kernel ABI the bundle
  was written against, tokenizer / chat-template metadata and stop tokens;
* ``tensors.bin`` (``neuralfn.raw_tensor_bundle.v1``): the tensors back to back, little endian,
  each starting on a 64-byte boundary;
* ``compatibility-report.json``: per node whether the sm_100a kernel library covers its stage,
  and the blockers (function neurons carry Python source and are never executed or imported here:
  they are recorded by name and source digest only).

Module weights are read with ``torch.load(weights_only=True)``: nothing is unpickled into objects.
``load_native_bundle`` maps the bundle back into tensors and checks every digest.

Behavioural counterpart: ``neuralfn/native_ir.py:30-300, 1814-2300`` (``migrate_graph_to_native``,
the manifest and the raw tensor bundle) and ``neuralfn/_pt_migrate_worker.py``.
"""
from __future__ import annotations

import base64
import hashlib
import io
import json
import math
from pathlib import Path
from typing import Any

import numpy as np
import torch

__all__ = ["MANIFEST_SCHEMA", "BUNDLE_SCHEMA", "NativeMigrationError", "lower_graph", "compatibility_report", "migrate_graph_to_native",
           "load_native_bundle"]

MANIFEST_SCHEMA = "neuralfn.native_execution_manifest"
BUNDLE_SCHEMA = "neuralfn.raw_tensor_bundle.v1"
_ALIGN = 64
_DTYPE_NAMES = {torch.float32: "float32", torch.bfloat16: "bfloat16", torch.float16: "float16", torch.int64: "int64", torch.int32: "int32",
                torch.uint8: "uint8", torch.int8: "int8", torch.bool: "bool", torch.float64: "float64"}
_DTYPES = {v: k for k, v in _DTYPE_NAMES.items()}


class NativeMigrationError(ValueError):
    pass


def _json_safe(v: Any, path: str) -> Any:
    if v is None or isinstance(v, (bool, int, str)):
        return v
    if isinstance(v, float):
        if not math.isfinite(v):
            raise NativeMigrationError(f"{path}: non-finite number")
        return v
    if isinstance(v, (list, tuple)):
        return [_json_safe(x, f"{path}[{i}]") for i, x in enumerate(v)]
    if isinstance(v, dict):
        return {str(k): _json_safe(x, f"{path}.{k}") for k, x in v.items()}
    raise NativeMigrationError(f"{path}: {type(v).__name__} is not representable in the IR")


def lower_graph(graph) -> dict:
    """Source-inert topology of a graph (nested subgraphs included). Function neurons appear with
    the digest of their source, never with the source itself."""
    def lower(g, prefix: str) -> dict:
        nodes = []
        for nid, inst in g.nodes.items():
            nd = inst.neuron_def
            rec: dict[str, Any] = {"id": nid, "name": nd.name, "kind": nd.kind, "inputs": [p.name for p in nd.input_ports],
                                   "outputs": [p.name for p in nd.output_ports]}
            if nd.kind == "module":
                rec["stage"] = nd.module_type
                rec["config"] = _json_safe(dict(nd.module_config or {}), f"{prefix}{nid}.config")
                rec["has_state"] = bool(nd.module_state)
            elif nd.kind == "subgraph":
                rec["subgraph"] = lower(nd.subgraph, f"{prefix}{nid}/")
                if nd.variant_ref:
                    rec["variant_ref"] = dict(nd.variant_ref)
            else:
                rec["source_sha256"] = hashlib.sha256((nd.source_code or "").encode("utf-8")).hexdigest()
            nodes.append(rec)
        edges = [{"id": e.id, "src": e.src_node, "src_port": e.src_port, "dst": e.dst_node, "dst_port": e.dst_port, "weight": e.weight,
                  "bias": e.bias} for e in g.edges.values()]
        order = g.topological_order() if not g.has_cycles() else None
        return {"name": g.name, "runtime": g.runtime, "inputs": list(g.input_node_ids), "outputs": list(g.output_node_ids), "nodes": nodes,
                "edges": edges, "topological_order": order}
    return lower(graph, "")


def compatibility_report(ir: dict) -> dict:
    """Which nodes the kernel library covers natively, and what blocks a fully native execution."""
    from .tensor.stages_core import STAGE_REGISTRY
    native_hot = {"linear", "lm_head", "causal_self_attention", "fused_causal_self_attention", "scaled_dot_product_attention", "rms_norm", "layer_norm",
                  "swiglu", "token_cross_entropy", "expert_dispatch", "token_embedding", "rotary_embedding", "mlp", "glu"}
    rows, blockers = [], []

    def walk(g: dict, prefix: str) -> None:
        if g["topological_order"] is None:
            blockers.append(f"{prefix or 'root'}: the graph has cycles (iterative settling is scalar-runtime only)")
        for n in g["nodes"]:
            path = prefix + n["id"]
            if n["kind"] == "module":
                known = n["stage"] in STAGE_REGISTRY
                rows.append({"node": path, "stage": n["stage"], "known_stage": known, "native_kernels": n["stage"] in native_hot})
                if not known:
                    blockers.append(f"{path}: unknown stage type {n['stage']!r}")
            elif n["kind"] == "subgraph":
                walk(n["subgraph"], path + "/")
            else:
                rows.append({"node": path, "stage": None, "known_stage": False, "native_kernels": False})
                blockers.append(f"{path}: function neuron {n['name']!r} carries Python source; it is not executed natively")
    walk(ir, "")
    return {"schema": "neuralfn.native_compatibility_report.v1", "executable": not blockers, "blockers": blockers, "nodes": rows,
            "native_kernel_nodes": sum(r["native_kernels"] for r in rows), "total_nodes": len(rows)}


def _collect_tensors(graph) -> dict[str, torch.Tensor]:
    out: dict[str, torch.Tensor] = {}

    def walk(g, prefix: str) -> None:
        for nid, inst in g.nodes.items():
            nd = inst.neuron_def
            if nd.kind == "module" and nd.module_state:
                raw = base64.b64decode(nd.module_state.encode("ascii"))
                try:
                    sd = torch.load(io.BytesIO(raw), map_location="cpu", weights_only=True)
                except Exception as exc:  # anything but plain tensors is refused, not unpickled
                    raise NativeMigrationError(f"{prefix}{nid}: module state is not a plain tensor dictionary ({type(exc).__name__})") from None
                for k, v in sd.items():
                    if not isinstance(v, torch.Tensor):
                        raise NativeMigrationError(f"{prefix}{nid}.{k}: not a tensor")
                    out[f"{prefix}{nid}.{k}"] = v.detach().contiguous()
            elif nd.kind == "subgraph" and nd.subgraph is not None:
                walk(nd.subgraph, f"{prefix}{nid}/")
    walk(graph, "")
    return out


def migrate_graph_to_native(graph_or_path, out_dir, *, model_name: str | None = None, tokenizer: dict | None = None, chat_template: str | None = None,
                            stop_token_ids=(), extra_tensors: dict[str, torch.Tensor] | None = None) -> dict:
    """Lowers a graph (object, JSON text or path of a JSON file) and writes the bundle directory.
    Returns the manifest. ``out_dir`` must not exist."""
    from .ops.registry import coverage_summary
    from .serialization import graph_from_json, graph_to_json
    if isinstance(graph_or_path, (str, Path)) and Path(str(graph_or_path)).is_file():
        text = Path(graph_or_path).read_text(encoding="utf-8")
        graph = graph_from_json(text)
    elif isinstance(graph_or_path, str):
        text, graph = graph_or_path, graph_from_json(graph_or_path)
    else:
        graph, text = graph_or_path, graph_to_json(graph_or_path)
    out = Path(out_dir)
    if out.exists():
        raise NativeMigrationError(f"{out} exists; migration writes into a new directory")
    ir = lower_graph(graph)
    report = compatibility_report(ir)
    tensors = _collect_tensors(graph)
    for k, v in (extra_tensors or {}).items():
        if k in tensors:
            raise NativeMigrationError(f"tensor name {k!r} given twice")
        tensors[k] = v.detach().contiguous().cpu()
    family = preset = None
    tmpl = dict(dict(graph.torch_config or {}).get("template_spec", {}) or {})
    hint = tmpl.get("preset") or dict(tmpl.get("template", {}) or {}).get("name") or model_name or graph.name
    try:
        from .native_registry import classify_native_model
        spec, preset = classify_native_model(str(hint))
        family = spec.family
    except KeyError:
        pass
    staging = out.with_name(out.name + ".staging")
    if staging.exists():
        raise NativeMigrationError(f"{staging} exists (an earlier migration did not finish); remove it first")
    staging.mkdir(parents=True)
    specs, offset = [], 0
    with open(staging / "tensors.bin", "wb") as f:
        for name in sorted(tensors):
            t = tensors[name]
            if t.dtype not in _DTYPE_NAMES:
                raise NativeMigrationError(f"{name}: dtype {t.dtype} is not storable")
            pad = (-offset) % _ALIGN
            f.write(b"\0" * pad)
            offset += pad
            raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
            f.write(raw)
            specs.append({"name": name, "dtype": _DTYPE_NAMES[t.dtype], "shape": list(t.shape), "offset": offset, "nbytes": len(raw),
                          "sha256": hashlib.sha256(raw).hexdigest()})
            offset += len(raw)
    manifest = {"schema": MANIFEST_SCHEMA, "version": 1,
                "model": {"name": model_name or graph.name, "family": family, "preset": preset, "graph_sha256": hashlib.sha256(text.encode("utf-8")).hexdigest(),
                          "runtime": graph.runtime, "parameters": int(sum(int(np.prod(s["shape"])) if s["shape"] else 1 for s in specs))},
                "topology": ir,
                "tensors": {"schema": BUNDLE_SCHEMA, "file": "tensors.bin", "alignment": _ALIGN, "total_bytes": offset, "specs": specs},
                "capabilities": {"executable_natively": report["executable"], "native_kernel_nodes": report["native_kernel_nodes"],
                                 "total_nodes": report["total_nodes"]},
                "kernel_abi": {"library": "libnfn_b200_kernels", "target": "sm_100a", **coverage_summary()},
                "tokenizer": _json_safe(tokenizer or {}, "tokenizer"), "chat_template": chat_template,
                "stop_token_ids": [int(t) for t in stop_token_ids]}
    (staging / "compatibility-report.json").write_text(json.dumps(report, indent=2), encoding="utf-8")
    (staging / "source-graph.json").write_text(text, encoding="utf-8")
    (staging / "native-execution-manifest.json").write_text(json.dumps(manifest, indent=2), encoding="utf-8")
    staging.rename(out)
    return manifest


def load_native_bundle(directory) -> tuple[dict, dict[str, torch.Tensor]]:
    """(manifest, tensors) of a migrated directory; every tensor is checked against its digest and
    the specs must lie inside the bundle without overlapping."""
    root = Path(directory)
    manifest = json.loads((root / "native-execution-manifest.json").read_text(encoding="utf-8"))
    if manifest.get("schema") != MANIFEST_SCHEMA or manifest.get("version") != 1:
        raise NativeMigrationError("not a native execution manifest (version 1)")
    tz = manifest["tensors"]
    if tz.get("schema") != BUNDLE_SCHEMA or "/" in tz["file"] or tz["file"].startswith("."):
        raise NativeMigrationError("unknown tensor bundle")
    blob = np.fromfile(root / tz["file"], dtype=np.uint8)
    if blob.size != tz["total_bytes"]:
        raise NativeMigrationError("tensor bundle has the wrong size")
    out, cursor = {}, 0
    for s in sorted(tz["specs"], key=lambda r: r["offset"]):
        lo, n = int(s["offset"]), int(s["nbytes"])
        if lo < cursor or lo % tz["alignment"] or lo + n > blob.size or s["dtype"] not in _DTYPES:
            raise NativeMigrationError(f"tensor {s['name']!r} has a bad placement or dtype")
        raw = blob[lo:lo + n]
        if hashlib.sha256(raw.tobytes()).hexdigest() != s["sha256"]:
            raise NativeMigrationError(f"tensor {s['name']!r} does not match its digest")
        t = torch.from_numpy(raw.copy()).view(_DTYPES[s["dtype"]]) if n else torch.empty(0, dtype=_DTYPES[s["dtype"]])
        out[s["name"]] = t.reshape(s["shape"])
        cursor = lo + n
    return manifest, out

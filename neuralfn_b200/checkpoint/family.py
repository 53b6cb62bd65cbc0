"""Family (Llama) native checkpoint directories: a JSON document, one raw little-endian float32
parameter file and a DONE marker.

Layout of ``<dir>/``:
    checkpoint.json   format ``nfn-native-family-optimizer-checkpoint-v1``: family, template,
                      steps, and an ``inference_contract`` (schema
                      ``neuralfn.native_family_llama.inference_checkpoint`` v2) that names the
                      artifact (path, dtype float32, byte order little, contiguous row-major,
                      nbytes, sha256), the geometry, the fixed Llama semantics and the tensor
                      table (name, shape, offset, nbytes, sha256)
    model.f32         the tensors back to back in the canonical order
    DONE              the text ``done`` - written last; a directory without it is incomplete

Canonical order and shapes are a function of the geometry alone: token_embedding.weight,
final_norm.weight, lm_head.weight, then per layer attention_norm, q_proj, k_proj, v_proj,
attention_out, ffn_norm, ffn_gate_up [2, hidden, dim], ffn_down. Readers re-derive that table
and refuse anything that disagrees (sizes, offsets, digests, unknown semantics).

``save_family_llama_checkpoint`` / ``load_family_llama_checkpoint`` convert between this layout
and the engine's fused tensors (``wqkv`` = q | k | v rows, ``w_gate_up`` = gate rows | up rows).

Format contract: ``neuralfn/native_family_checkpoint.py:21-35, 247-273, 297-420``.
"""
from __future__ import annotations

import hashlib
import json
import os
from pathlib import Path
from typing import Any, Mapping

import torch

__all__ = ["FAMILY_OPTIMIZER_FORMAT", "LLAMA_INFERENCE_SCHEMA", "LLAMA_CHECKPOINT_FORMAT", "FamilyCheckpointError", "expected_llama_layout",
           "save_family_llama_checkpoint", "inspect_family_llama_checkpoint", "load_family_llama_checkpoint"]

FAMILY_OPTIMIZER_FORMAT = "nfn-native-family-optimizer-checkpoint-v1"
LLAMA_INFERENCE_SCHEMA = "neuralfn.native_family_llama.inference_checkpoint"
LLAMA_INFERENCE_VERSION = 2
LLAMA_CHECKPOINT_FORMAT = "neuralfn.native_family_llama.f32.v1"
LLAMA_SEMANTICS = {"norm_type": "rmsnorm", "mlp_type": "swiglu", "pos_encoding": "rope", "attention_variant": "dense", "residual_type": "add",
                   "linear_bias": False, "dropout_p": 0.0, "tie_embeddings": False}
_GEOMETRY_INTS = ("vocab_size", "padded_vocab_size", "model_dim", "hidden_dim", "num_layers", "num_heads", "num_kv_heads", "head_dim", "max_seq_len")


class FamilyCheckpointError(ValueError):
    pass


def expected_llama_layout(geometry: Mapping[str, Any]) -> list[tuple[str, tuple[int, ...]]]:
    d, h, L, vp = int(geometry["model_dim"]), int(geometry["hidden_dim"]), int(geometry["num_layers"]), int(geometry["padded_vocab_size"])
    kv = int(geometry["num_kv_heads"]) * int(geometry["head_dim"])
    out: list[tuple[str, tuple[int, ...]]] = [("token_embedding.weight", (vp, d)), ("final_norm.weight", (d,)), ("lm_head.weight", (vp, d))]
    for l in range(L):
        p = f"layers.{l}."
        out += [(p + "attention_norm.weight", (d,)), (p + "q_proj.weight", (d, d)), (p + "k_proj.weight", (kv, d)), (p + "v_proj.weight", (kv, d)),
                (p + "attention_out.weight", (d, d)), (p + "ffn_norm.weight", (d,)), (p + "ffn_gate_up.weight", (2, h, d)), (p + "ffn_down.weight", (d, h))]
    return out


def _geometry_of(cfg) -> dict[str, Any]:
    if cfg.n_head * cfg.head_dim != cfg.d_model:
        raise FamilyCheckpointError("the family format needs model_dim == num_heads * head_dim")
    if cfg.tie_embeddings or cfg.qk_norm or cfg.window:
        raise FamilyCheckpointError("the family format describes the plain Llama block (untied head, no QK norm, no window)")
    return {"vocab_size": cfg.vocab_size, "padded_vocab_size": cfg.padded_vocab, "model_dim": cfg.d_model, "hidden_dim": cfg.d_ff,
            "num_layers": cfg.n_layer, "num_heads": cfg.n_head, "num_kv_heads": cfg.n_kv_head, "head_dim": cfg.head_dim,
            "max_seq_len": cfg.max_seq_len, "rope_theta": float(cfg.rope_theta), "rope_scaling_factor": 1.0, "rms_norm_eps": float(cfg.norm_eps)}


def _split_engine_tensors(cfg, tensors: Mapping[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    d, kv, F = cfg.d_model, cfg.n_kv_head * cfg.head_dim, cfg.d_ff
    out = {"token_embedding.weight": tensors["tok_embeddings"], "final_norm.weight": tensors["norm"], "lm_head.weight": tensors["lm_head"]}
    for l in range(cfg.n_layer):
        p, q = f"layers.{l}.", f"layers.{l}."
        wqkv = tensors[q + "wqkv"].reshape(d + 2 * kv, d)
        out[p + "attention_norm.weight"] = tensors[q + "attn_norm"]
        out[p + "q_proj.weight"], out[p + "k_proj.weight"], out[p + "v_proj.weight"] = wqkv[:d], wqkv[d:d + kv], wqkv[d + kv:]
        out[p + "attention_out.weight"] = tensors[q + "wo"].reshape(d, d)
        out[p + "ffn_norm.weight"] = tensors[q + "ffn_norm"]
        out[p + "ffn_gate_up.weight"] = tensors[q + "w_gate_up"].reshape(2, F, d)
        out[p + "ffn_down.weight"] = tensors[q + "w_down"].reshape(d, F)
    return out


def save_family_llama_checkpoint(out_dir, cfg, tensors: Mapping[str, torch.Tensor], *, steps: int = 0, template_name: str = "llama",
                                 extra: dict | None = None) -> dict:
    """Writes a new directory (refuses to touch an existing one). ``tensors``: the engine's named
    tensors (any float dtype). Returns the JSON document."""
    out = Path(out_dir)
    if out.exists():
        raise FamilyCheckpointError(f"{out} exists; checkpoints are never overwritten")
    geometry = _geometry_of(cfg)
    named = _split_engine_tensors(cfg, tensors)
    staging = out.with_name(out.name + ".staging")
    staging.mkdir(parents=True)
    table, offset, whole = [], 0, hashlib.sha256()
    with open(staging / "model.f32", "xb") as f:
        for name, shape in expected_llama_layout(geometry):
            t = named[name].detach().to(torch.float32).cpu().contiguous()
            if tuple(t.shape) != shape:
                raise FamilyCheckpointError(f"{name}: shape {tuple(t.shape)} instead of {shape}")
            raw = t.numpy().astype("<f4", copy=False).tobytes()
            f.write(raw)
            whole.update(raw)
            table.append({"name": name, "source_name": name, "dtype": "float32", "shape": list(shape), "offset": offset, "nbytes": len(raw),
                          "sha256": hashlib.sha256(raw).hexdigest(), "role": "parameter", "byte_order": "little", "layout": "row_major"})
            offset += len(raw)
        f.flush()
        os.fsync(f.fileno())
    doc = {"format": FAMILY_OPTIMIZER_FORMAT, "model_family": "llama", "native_target": "llama", "template_name": template_name, "steps": int(steps),
           "inference_contract": {"schema": LLAMA_INFERENCE_SCHEMA, "version": LLAMA_INFERENCE_VERSION, "family": "llama", "preset": "llama",
                                  "checkpoint_kind": "live_full_architecture", "done_marker": "DONE",
                                  "artifact": {"format": LLAMA_CHECKPOINT_FORMAT, "path": "model.f32", "dtype": "float32", "byte_order": "little",
                                               "layout": "contiguous_row_major", "nbytes": offset, "sha256": whole.hexdigest()},
                                  "geometry": geometry, "semantics": dict(LLAMA_SEMANTICS), "training": {"train_seq_len": cfg.max_seq_len},
                                  "tensors": table}}
    doc.update(extra or {})
    (staging / "checkpoint.json").write_text(json.dumps(doc, indent=2, sort_keys=True), encoding="utf-8")
    (staging / "DONE").write_text("done\n", encoding="utf-8")
    os.rename(staging, out)
    return doc


def _safe_child(root: Path, rel: Any, what: str) -> Path:
    if not isinstance(rel, str) or not rel or os.path.isabs(rel) or ".." in Path(rel).parts:
        raise FamilyCheckpointError(f"{what} must be a relative path inside the checkpoint directory")
    p = root / rel
    if p.is_symlink():
        raise FamilyCheckpointError(f"{what} is a symbolic link")
    return p


def inspect_family_llama_checkpoint(ckpt_dir) -> dict:
    """Validates the directory end to end (document, marker, sizes, digests, layout re-derived
    from the geometry) and returns ``{"document", "geometry", "tensors", "path"}``."""
    root = Path(ckpt_dir)
    try:
        doc = json.loads((root / "checkpoint.json").read_text(encoding="utf-8"))
    except (OSError, json.JSONDecodeError) as exc:
        raise FamilyCheckpointError(f"cannot read {root / 'checkpoint.json'}: {exc}") from exc
    if doc.get("format") != FAMILY_OPTIMIZER_FORMAT or str(doc.get("model_family", "")).lower() != "llama":
        raise FamilyCheckpointError("not a Llama family checkpoint document")
    c = doc.get("inference_contract") or {}
    if c.get("schema") != LLAMA_INFERENCE_SCHEMA or c.get("version") != LLAMA_INFERENCE_VERSION or c.get("checkpoint_kind") != "live_full_architecture":
        raise FamilyCheckpointError("unsupported inference contract")
    marker = _safe_child(root, c.get("done_marker"), "done_marker")
    if not marker.is_file() or marker.read_text(encoding="utf-8").strip() != "done":
        raise FamilyCheckpointError("the DONE marker is missing: the checkpoint was not completely written")
    art = c.get("artifact") or {}
    if art.get("format") != LLAMA_CHECKPOINT_FORMAT or art.get("dtype") != "float32" or art.get("byte_order") != "little" or art.get("layout") != "contiguous_row_major":
        raise FamilyCheckpointError("unsupported artifact encoding")
    path = _safe_child(root, art.get("path"), "artifact.path")
    geometry = dict(c.get("geometry") or {})
    for k in _GEOMETRY_INTS:
        if not isinstance(geometry.get(k), int) or isinstance(geometry.get(k), bool) or geometry[k] < 1:
            raise FamilyCheckpointError(f"geometry.{k} must be a positive integer")
    if geometry["padded_vocab_size"] < geometry["vocab_size"] or geometry["model_dim"] != geometry["num_heads"] * geometry["head_dim"] or \
            geometry["num_heads"] % geometry["num_kv_heads"] or geometry["head_dim"] % 2:
        raise FamilyCheckpointError("inconsistent geometry")
    if dict(c.get("semantics") or {}) != LLAMA_SEMANTICS:
        raise FamilyCheckpointError("semantics differ from the Llama contract")
    if (c.get("training") or {}).get("train_seq_len") != geometry["max_seq_len"]:
        raise FamilyCheckpointError("training.train_seq_len must equal geometry.max_seq_len")
    layout = expected_llama_layout(geometry)
    table = c.get("tensors") or []
    if [t.get("name") for t in table] != [n for n, _ in layout]:
        raise FamilyCheckpointError("tensor table does not match the layout derived from the geometry")
    size = path.stat().st_size
    if size != art.get("nbytes"):
        raise FamilyCheckpointError(f"artifact holds {size} bytes, the document says {art.get('nbytes')}")
    whole, offset = hashlib.sha256(), 0
    with open(path, "rb") as f:
        for rec, (name, shape) in zip(table, layout):
            n = 4
            for s in shape:
                n *= s
            if rec.get("shape") != list(shape) or rec.get("offset") != offset or rec.get("nbytes") != n:
                raise FamilyCheckpointError(f"{name}: shape / offset / size disagree with the derived layout")
            raw = f.read(n)
            if len(raw) != n or hashlib.sha256(raw).hexdigest() != rec.get("sha256"):
                raise FamilyCheckpointError(f"{name}: bytes do not match the recorded digest")
            whole.update(raw)
            offset += n
    if offset != size or whole.hexdigest() != art.get("sha256"):
        raise FamilyCheckpointError("artifact digest mismatch")
    return {"document": doc, "geometry": geometry, "tensors": table, "path": path}


def load_family_llama_checkpoint(ckpt_dir):
    """Returns ``(LlamaConfig, engine tensors as bf16, document)`` after full validation."""
    import numpy as np

    from ..models.llama import LlamaConfig
    info = inspect_family_llama_checkpoint(ckpt_dir)
    g = info["geometry"]
    cfg = LlamaConfig(n_layer=g["num_layers"], n_head=g["num_heads"], n_kv_head=g["num_kv_heads"], d_model=g["model_dim"], d_ff=g["hidden_dim"],
                      vocab_size=g["vocab_size"], max_seq_len=g["max_seq_len"], rope_theta=g["rope_theta"], norm_eps=g["rms_norm_eps"])
    if cfg.padded_vocab != g["padded_vocab_size"]:
        cfg = LlamaConfig(**{**cfg.__dict__, "vocab_pad_to": 1, "vocab_size": g["padded_vocab_size"]})
    flat = np.memmap(info["path"], dtype="<f4", mode="r")
    named = {}
    for rec in info["tensors"]:
        a = np.asarray(flat[rec["offset"] // 4:(rec["offset"] + rec["nbytes"]) // 4]).reshape(rec["shape"])
        named[rec["name"]] = torch.from_numpy(a.copy())
    out = {"tok_embeddings": named["token_embedding.weight"], "norm": named["final_norm.weight"], "lm_head": named["lm_head.weight"]}
    for l in range(g["num_layers"]):
        p = f"layers.{l}."
        out[p + "attn_norm"] = named[p + "attention_norm.weight"]
        out[p + "wqkv"] = torch.cat([named[p + "q_proj.weight"], named[p + "k_proj.weight"], named[p + "v_proj.weight"]], 0)
        out[p + "wo"] = named[p + "attention_out.weight"]
        out[p + "ffn_norm"] = named[p + "ffn_norm.weight"]
        out[p + "w_gate_up"] = named[p + "ffn_gate_up.weight"].reshape(2 * g["hidden_dim"], g["model_dim"])
        out[p + "w_down"] = named[p + "ffn_down.weight"]
    return cfg, {k: v.to(torch.bfloat16) for k, v in out.items()}, info["document"]

"""Strict safetensors reader / writer and the ingestion of sharded Hugging Face checkpoints.

A safetensors file is an 8-byte little-endian header length, a JSON header mapping tensor names
to ``{dtype, shape, data_offsets}`` (plus an optional ``__metadata__`` string map), and the raw
little-endian tensor bytes. The reader here is deliberately strict: the header must be a JSON
object of bounded size without duplicate keys, every tensor must lie inside the data section,
sizes must equal shape x dtype width, the tensors must tile the data section without overlap or
gap, and only the dtypes listed below are accepted. Nothing is unpickled and nothing is executed.

A sharded checkpoint is a directory with ``model.safetensors.index.json`` (``weight_map``:
tensor name -> shard file); every shard listed must exist inside the directory, every tensor must
be found in the shard the index names, and no shard may carry tensors the index does not know.

``load_hf_llama_directory`` turns such a directory (or a single ``model.safetensors``) plus its
``config.json`` into an ``EngineConfig`` and the resident engine's fused tensors.

Behavioural counterpart: ``neuralfn/native_muse_glimmer_checkpoint.py`` (strict safetensors
index + shards -> native bf16 conversion, tensor contracts, manifest publishing).
"""
from __future__ import annotations

import json
import struct
from pathlib import Path
from typing import Mapping

import numpy as np
import torch

__all__ = ["SafetensorsError", "read_safetensors", "write_safetensors", "read_sharded_checkpoint", "load_hf_llama_directory",
           "export_hf_llama_directory"]

MAX_HEADER_BYTES = 100 * 1024 * 1024
_DTYPES = {"BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F32": (torch.float32, 4), "F64": (torch.float64, 8),
           "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
           "BOOL": (torch.bool, 1)}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


def _no_duplicates(pairs):
    out = {}
    for k, v in pairs:
        if k in out:
            raise SafetensorsError(f"duplicate key {k!r} in the header")
        out[k] = v
    return out


def _read_header(path: Path) -> tuple[dict, int, int]:
    size = path.stat().st_size
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise SafetensorsError(f"{path}: too short for a safetensors file")
        (hlen,) = struct.unpack("<Q", raw)
        if hlen < 2 or hlen > MAX_HEADER_BYTES or 8 + hlen > size:
            raise SafetensorsError(f"{path}: implausible header length {hlen}")
        try:
            header = json.loads(f.read(hlen).decode("utf-8"), object_pairs_hook=_no_duplicates)
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise SafetensorsError(f"{path}: header is not valid JSON: {exc}") from exc
    if not isinstance(header, dict):
        raise SafetensorsError(f"{path}: header must be a JSON object")
    return header, 8 + hlen, size


def read_safetensors(path, *, names: set[str] | None = None) -> tuple[dict[str, torch.Tensor], dict[str, str]]:
    """Returns (tensors, metadata). ``names`` restricts which tensors are materialised (all are validated)."""
    path = Path(path)
    header, data0, size = _read_header(path)
    meta = header.pop("__metadata__", {}) or {}
    if not isinstance(meta, dict) or any(not isinstance(k, str) or not isinstance(v, str) for k, v in meta.items()):
        raise SafetensorsError(f"{path}: __metadata__ must map strings to strings")
    spans = []
    for name, rec in header.items():
        if not isinstance(rec, dict) or set(rec) != {"dtype", "shape", "data_offsets"}:
            raise SafetensorsError(f"{path}: tensor {name!r} has a malformed record")
        if rec["dtype"] not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {rec['dtype']!r}")
        shape, offs = rec["shape"], rec["data_offsets"]
        if not isinstance(shape, list) or any(isinstance(d, bool) or not isinstance(d, int) or d < 0 for d in shape):
            raise SafetensorsError(f"{path}: tensor {name!r} has a bad shape")
        if not isinstance(offs, list) or len(offs) != 2 or any(isinstance(o, bool) or not isinstance(o, int) for o in offs):
            raise SafetensorsError(f"{path}: tensor {name!r} has bad offsets")
        n = _DTYPES[rec["dtype"]][1]
        for d in shape:
            n *= d
        if offs[0] < 0 or offs[1] - offs[0] != n or data0 + offs[1] > size:
            raise SafetensorsError(f"{path}: tensor {name!r} does not fit its offsets")
        spans.append((offs[0], offs[1], name))
    spans.sort()
    cursor = 0
    for lo, hi, name in spans:
        if lo != cursor:
            raise SafetensorsError(f"{path}: gap or overlap before tensor {name!r}")
        cursor = hi
    if data0 + cursor != size:
        raise SafetensorsError(f"{path}: {size - data0 - cursor} trailing bytes after the last tensor")
    flat = np.memmap(path, dtype=np.uint8, mode="r", offset=data0) if cursor else np.zeros(0, np.uint8)
    out = {}
    for lo, hi, name in spans:
        if names is not None and name not in names:
            continue
        rec = header[name]
        dt = _DTYPES[rec["dtype"]][0]
        buf = torch.from_numpy(np.array(flat[lo:hi], copy=True))
        out[name] = buf.view(dt).reshape(rec["shape"]) if hi > lo else torch.empty(rec["shape"], dtype=dt)
    return out, dict(meta)


def write_safetensors(path, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] | None = None) -> None:
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blobs, off = [], 0
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"dtype {t.dtype} cannot be stored")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    with open(path, "xb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for raw in blobs:
            f.write(raw)


def read_sharded_checkpoint(directory) -> dict[str, torch.Tensor]:
    """All tensors of a checkpoint directory (index + shards, or one ``model.safetensors``)."""
    root = Path(directory)
    index = root / "model.safetensors.index.json"
    if not index.is_file():
        single = root / "model.safetensors"
        if not single.is_file():
            raise SafetensorsError(f"{root} holds neither model.safetensors.index.json nor model.safetensors")
        return read_safetensors(single)[0]
    doc = json.loads(index.read_text(encoding="utf-8"), object_pairs_hook=_no_duplicates)
    wmap = doc.get("weight_map")
    if not isinstance(wmap, dict) or not wmap:
        raise SafetensorsError("the index has no weight_map")
    by_shard: dict[str, set[str]] = {}
    for name, shard in wmap.items():
        if not isinstance(shard, str) or "/" in shard or "\\" in shard or shard.startswith("."):
            raise SafetensorsError(f"shard name {shard!r} must be a plain file name")
        by_shard.setdefault(shard, set()).add(name)
    out: dict[str, torch.Tensor] = {}
    for shard, wanted in sorted(by_shard.items()):
        p = root / shard
        if not p.is_file() or p.is_symlink():
            raise SafetensorsError(f"shard {shard} is missing (or a symbolic link)")
        got, _ = read_safetensors(p)
        if set(got) != wanted:
            extra, missing = sorted(set(got) - wanted)[:3], sorted(wanted - set(got))[:3]
            raise SafetensorsError(f"shard {shard} disagrees with the index (unexpected {extra}, missing {missing})")
        out.update(got)
    return out


def load_hf_llama_directory(directory, *, max_batch: int = 1, max_seq: int | None = None):
    """(EngineConfig, tensors under the resident engine's names) for a Llama-style Hugging Face
    checkpoint directory: ``config.json`` + safetensors. Biases, rotary scaling variants and tied
    or extra tensors that the engine has no slot for are refused rather than dropped."""
    from ..serving.engine import EngineConfig
    root = Path(directory)
    hf = json.loads((root / "config.json").read_text(encoding="utf-8"))
    if hf.get("attention_bias") or hf.get("mlp_bias"):
        raise SafetensorsError("checkpoints with linear biases are not supported by the Llama engine layout")
    if hf.get("rope_scaling") not in (None, {}):
        raise SafetensorsError("rope_scaling variants need explicit rotary tables; load through the tensor runtime instead")
    d, L, H = int(hf["hidden_size"]), int(hf["num_hidden_layers"]), int(hf["num_attention_heads"])
    Hkv = int(hf.get("num_key_value_heads") or H)
    hd = int(hf.get("head_dim") or d // H)
    V, F = int(hf["vocab_size"]), int(hf["intermediate_size"])
    Vp = (V + 7) // 8 * 8
    tie = bool(hf.get("tie_word_embeddings", False))
    cfg = EngineConfig(family=1, n_layer=L, d_model=d, n_head=H, n_kv_head=Hkv, head_dim=hd, d_ff=F, vocab=V, padded_vocab=Vp,
                       max_seq=int(max_seq or hf.get("max_position_embeddings", 2048)), max_batch=max_batch, qk_norm=0, rope_hf=1,
                       rope_theta=float(hf.get("rope_theta", 10000.0)), norm_eps=float(hf.get("rms_norm_eps", 1e-5)), tie_embeddings=int(tie))
    sd = read_sharded_checkpoint(root)

    def take(name: str, shape: tuple[int, ...]) -> torch.Tensor:
        if name not in sd:
            raise SafetensorsError(f"tensor {name} is missing")
        t = sd.pop(name)
        if tuple(t.shape) != shape:
            raise SafetensorsError(f"{name}: shape {tuple(t.shape)} instead of {shape}")
        return t.to(torch.bfloat16)

    def pad_vocab(t: torch.Tensor) -> torch.Tensor:
        if Vp == V:
            return t
        return torch.cat([t, torch.zeros(Vp - V, d, dtype=t.dtype)], 0)

    out = {"tok_embeddings": pad_vocab(take("model.embed_tokens.weight", (V, d))), "norm": take("model.norm.weight", (d,))}
    if not tie:
        out["lm_head"] = pad_vocab(take("lm_head.weight", (V, d)))
    else:
        sd.pop("lm_head.weight", None)
    for l in range(L):
        p, q = f"model.layers.{l}.", f"layers.{l}."
        out[q + "attn_norm"] = take(p + "input_layernorm.weight", (d,))
        out[q + "wqkv"] = torch.cat([take(p + "self_attn.q_proj.weight", (H * hd, d)), take(p + "self_attn.k_proj.weight", (Hkv * hd, d)),
                                     take(p + "self_attn.v_proj.weight", (Hkv * hd, d))], 0)
        out[q + "wo"] = take(p + "self_attn.o_proj.weight", (d, H * hd))
        out[q + "ffn_norm"] = take(p + "post_attention_layernorm.weight", (d,))
        out[q + "w_gate_up"] = torch.cat([take(p + "mlp.gate_proj.weight", (F, d)), take(p + "mlp.up_proj.weight", (F, d))], 0)
        out[q + "w_down"] = take(p + "mlp.down_proj.weight", (d, F))
    leftovers = [k for k in sd if not k.endswith("rotary_emb.inv_freq")]
    if leftovers:
        raise SafetensorsError(f"tensors without a slot in the engine layout: {sorted(leftovers)[:4]}")
    return cfg, out


def export_hf_llama_directory(directory, cfg, params: Mapping[str, torch.Tensor], *, dtype=torch.bfloat16) -> None:
    """Writes ``config.json`` + ``model.safetensors`` with Hugging Face Llama tensor names from an
    unsharded parameter dictionary under this framework's names (``tok_embeddings``,
    ``layers.N.{attn_norm,wqkv,wo,ffn_norm,w_gate_up,w_down}``, ``norm``, ``lm_head``); ``cfg`` is a
    ``LlamaConfig``. The inverse of ``load_hf_llama_directory``; vocabulary padding rows are cut."""
    root = Path(directory)
    root.mkdir(parents=True, exist_ok=True)
    d, hd, H, Hkv, F, V = cfg.d_model, cfg.head_dim, cfg.n_head, cfg.n_kv_head, cfg.d_ff, cfg.vocab_size
    t = lambda x: x.detach().to(dtype).contiguous()  # noqa: E731
    out = {"model.embed_tokens.weight": t(params["tok_embeddings"][:V]), "model.norm.weight": t(params["norm"])}
    if not cfg.tie_embeddings:
        out["lm_head.weight"] = t(params["lm_head"][:V])
    for l in range(cfg.n_layer):
        p, q = f"model.layers.{l}.", f"layers.{l}."
        wqkv, wgu = params[q + "wqkv"], params[q + "w_gate_up"]
        out[p + "input_layernorm.weight"] = t(params[q + "attn_norm"])
        out[p + "self_attn.q_proj.weight"] = t(wqkv[:H * hd])
        out[p + "self_attn.k_proj.weight"] = t(wqkv[H * hd:(H + Hkv) * hd])
        out[p + "self_attn.v_proj.weight"] = t(wqkv[(H + Hkv) * hd:])
        out[p + "self_attn.o_proj.weight"] = t(params[q + "wo"])
        out[p + "post_attention_layernorm.weight"] = t(params[q + "ffn_norm"])
        out[p + "mlp.gate_proj.weight"] = t(wgu[:F])
        out[p + "mlp.up_proj.weight"] = t(wgu[F:])
        out[p + "mlp.down_proj.weight"] = t(params[q + "w_down"])
    hf = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": d, "num_hidden_layers": cfg.n_layer, "num_attention_heads": H,
          "num_key_value_heads": Hkv, "head_dim": hd, "intermediate_size": F, "vocab_size": V, "max_position_embeddings": cfg.max_seq_len,
          "rope_theta": cfg.rope_theta, "rms_norm_eps": cfg.norm_eps, "tie_word_embeddings": bool(cfg.tie_embeddings), "attention_bias": False,
          "mlp_bias": False, "torch_dtype": {torch.bfloat16: "bfloat16", torch.float16: "float16", torch.float32: "float32"}[dtype]}
    (root / "config.json").write_text(json.dumps(hf, indent=2), encoding="utf-8")
    target = root / "model.safetensors"
    if target.exists():
        target.unlink()
    write_safetensors(target, out, {"format": "pt"})

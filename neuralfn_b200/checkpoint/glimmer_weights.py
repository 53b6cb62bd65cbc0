"""Muse-Glimmer text weights from their published containers into this framework's tensors.

Two sources, one strict tensor contract each:

* a Hugging Face style safetensors directory (``model.safetensors.index.json`` + shards, or one
  ``model.safetensors``) with ``model.language_model.*`` names;
* GGUF files (``token_embd.weight``, ``blk.N.attn_q.weight`` ...; F32 / F16 / BF16 / Q4_K / Q5_K / Q6_K
  tensors are decoded to bf16).

Both produce the parameter dictionary of ``models.glimmer`` / the resident engine: ``tok_embeddings``,
per layer ``attn_norm`` ``wqkvg`` (q | k | v | gate rows) ``wo`` ``post_attn_norm`` ``mlp_norm``
``w_gate_up`` (gate rows then up rows) ``w_down`` ``post_mlp_norm``, then ``norm`` and ``lm_head``; the
vocabulary is zero-padded to the engine's row multiple. The four layer norms are stored as centred
weights in the source (scale = 1 + w) and are copied unchanged, since the kernels apply the same form.

Strictness: every contract tensor must be present exactly once with the contract's shape, shards must
agree with the index, and tensors outside the contract (vision tower, rotary tables aside) are an error
unless ``allow_extra_prefixes`` names them. ``inspect_*`` reads headers only.

``convert_glimmer_weights`` writes a named-tensor checkpoint directory (``weights_00000000.nfnw`` + manifest
+ ``DONE_00000000``) that ``nfn train --init-from`` / ``load_named_checkpoint`` and the decoders accept; an
existing output directory is never overwritten.

Reference: the tensor contracts of ``neuralfn/native_muse_glimmer_checkpoint.py:1127-1201`` (safetensors names,
shapes, centred-delta norms) and ``neuralfn/csrc/native_train/muse_glimmer_native_train.cpp:1230-1262`` (GGUF names).
The vision-tower contracts (``:1203-1300``) and LoRA attachment (``:580-948``) are not converted here.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass
from pathlib import Path

import torch

from .safetensors_io import SafetensorsError, _no_duplicates, _read_header, read_safetensors

__all__ = ["GlimmerGeometry", "TensorContract", "safetensors_contracts", "gguf_contracts", "inspect_glimmer_safetensors",
           "load_glimmer_safetensors", "load_glimmer_gguf", "to_serving_names", "convert_glimmer_weights"]


@dataclass(frozen=True)
class GlimmerGeometry:
    n_layer: int = 52
    d_model: int = 6656
    n_head: int = 32
    n_kv_head: int = 2
    head_dim: int = 128
    d_ff: int = 19968
    vocab_size: int = 202048
    vocab_pad_to: int = 128

    @property
    def q_width(self) -> int:
        return self.n_head * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.n_kv_head * self.head_dim

    @property
    def padded_vocab(self) -> int:
        return (self.vocab_size + self.vocab_pad_to - 1) // self.vocab_pad_to * self.vocab_pad_to

    @classmethod
    def from_json(cls, text_or_path: str) -> "GlimmerGeometry":
        p = Path(text_or_path)
        doc = json.loads(p.read_text() if p.is_file() else text_or_path)
        return cls(**{k: int(v) for k, v in doc.items() if k in cls.__dataclass_fields__})


@dataclass(frozen=True)
class TensorContract:
    source: str                 # name in the container
    part: str                   # which piece of which engine tensor it becomes, e.g. "layers.3.wqkvg:0"
    shape: tuple[int, ...]
    centered: bool = False


_PROJ = (("q", "wqkvg", 0), ("k", "wqkvg", 1), ("v", "wqkvg", 2), ("gate", "wqkvg", 3), ("o", "wo", 0),
         ("mlp_gate", "w_gate_up", 0), ("mlp_up", "w_gate_up", 1), ("mlp_down", "w_down", 0))
_NORMS = (("attn_norm", "input_layernorm", "attn_norm"), ("post_attn_norm", "post_attention_layernorm", "post_attention_norm"),
          ("mlp_norm", "pre_feedforward_layernorm", "ffn_norm"), ("post_mlp_norm", "post_feedforward_layernorm", "post_ffw_norm"))


def _proj_shapes(g: GlimmerGeometry) -> dict[str, tuple[int, int]]:
    return {"q": (g.q_width, g.d_model), "k": (g.kv_width, g.d_model), "v": (g.kv_width, g.d_model), "gate": (g.q_width, g.d_model),
            "o": (g.d_model, g.q_width), "mlp_gate": (g.d_ff, g.d_model), "mlp_up": (g.d_ff, g.d_model), "mlp_down": (g.d_model, g.d_ff)}


def safetensors_contracts(g: GlimmerGeometry) -> list[TensorContract]:
    hf = {"q": "self_attn.q_proj", "k": "self_attn.k_proj", "v": "self_attn.v_proj", "gate": "self_attn.gate_proj", "o": "self_attn.o_proj",
          "mlp_gate": "mlp.gate_proj", "mlp_up": "mlp.up_proj", "mlp_down": "mlp.down_proj"}
    shapes = _proj_shapes(g)
    out = [TensorContract("model.language_model.embed_tokens.weight", "tok_embeddings:0", (g.vocab_size, g.d_model))]
    for l in range(g.n_layer):
        pre = f"model.language_model.layers.{l}."
        for ours, theirs, _gg in _NORMS:
            out.append(TensorContract(pre + theirs + ".weight", f"layers.{l}.{ours}:0", (g.d_model,), centered=True))
        for key, ours, piece in _PROJ:
            out.append(TensorContract(pre + hf[key] + ".weight", f"layers.{l}.{ours}:{piece}", shapes[key]))
    out += [TensorContract("model.language_model.norm.weight", "norm:0", (g.d_model,)),
            TensorContract("lm_head.weight", "lm_head:0", (g.vocab_size, g.d_model))]
    return out


def gguf_contracts(g: GlimmerGeometry) -> list[TensorContract]:
    gg = {"q": "attn_q", "k": "attn_k", "v": "attn_v", "gate": "attn_gate", "o": "attn_output", "mlp_gate": "ffn_gate", "mlp_up": "ffn_up",
          "mlp_down": "ffn_down"}
    shapes = _proj_shapes(g)
    out = [TensorContract("token_embd.weight", "tok_embeddings:0", (g.vocab_size, g.d_model))]
    for l in range(g.n_layer):
        for ours, _hf, theirs in _NORMS:
            out.append(TensorContract(f"blk.{l}.{theirs}.weight", f"layers.{l}.{ours}:0", (g.d_model,), centered=True))
        for key, ours, piece in _PROJ:
            out.append(TensorContract(f"blk.{l}.{gg[key]}.weight", f"layers.{l}.{ours}:{piece}", shapes[key]))
    out += [TensorContract("output_norm.weight", "norm:0", (g.d_model,)), TensorContract("output.weight", "lm_head:0", (g.vocab_size, g.d_model))]
    return out


# weightless per-head norms ship as all-ones vectors in GGUF exports; they carry no information and are skipped
_GGUF_IGNORED_SUFFIXES = (".attn_q_norm.weight", ".attn_k_norm.weight")
_SAFETENSORS_IGNORED_SUFFIXES = ("rotary_emb.inv_freq",)


def _assemble(g: GlimmerGeometry, pieces: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """part name -> tensor ("name:piece") into whole engine tensors, vocabulary padded."""
    groups: dict[str, dict[int, torch.Tensor]] = {}
    for part, t in pieces.items():
        name, piece = part.rsplit(":", 1)
        groups.setdefault(name, {})[int(piece)] = t
    out = {}
    for name, parts in groups.items():
        t = parts[0] if len(parts) == 1 else torch.cat([parts[i] for i in range(len(parts))], 0)
        if name in ("tok_embeddings", "lm_head") and g.padded_vocab > g.vocab_size:
            t = torch.cat([t, torch.zeros(g.padded_vocab - g.vocab_size, t.shape[1], dtype=t.dtype)], 0)
        out[name] = t.contiguous()
    return out


def _shard_map(root: Path) -> dict[str, Path]:
    """tensor name -> shard file, from the index (validated) or the single file."""
    index = root / "model.safetensors.index.json"
    if not index.is_file():
        single = root / "model.safetensors"
        if not single.is_file():
            raise SafetensorsError(f"{root} holds neither model.safetensors.index.json nor model.safetensors")
        header, _, _ = _read_header(single)
        return {k: single for k in header if k != "__metadata__"}
    doc = json.loads(index.read_text(encoding="utf-8"), object_pairs_hook=_no_duplicates)
    wmap = doc.get("weight_map")
    if not isinstance(wmap, dict) or not wmap:
        raise SafetensorsError("the index has no weight_map")
    out = {}
    for name, shard in wmap.items():
        if not isinstance(shard, str) or "/" in shard or "\\" in shard or shard.startswith("."):
            raise SafetensorsError(f"shard name {shard!r} must be a plain file name")
        p = root / shard
        if not p.is_file() or p.is_symlink():
            raise SafetensorsError(f"shard {shard} is missing (or a symbolic link)")
        out[name] = p
    return out


def inspect_glimmer_safetensors(directory, geometry: GlimmerGeometry | None = None, *, allow_extra_prefixes: tuple[str, ...] = ()) -> dict:
    """Header-only validation of a directory against the text contract. Returns a report; raises on a violation."""
    g = geometry or GlimmerGeometry()
    root = Path(directory)
    where = _shard_map(root)
    headers = {p: _read_header(p)[0] for p in sorted(set(where.values()))}
    contracts = safetensors_contracts(g)
    wanted = {c.source: c for c in contracts}
    missing = sorted(set(wanted) - set(where))
    if missing:
        raise SafetensorsError(f"{len(missing)} contract tensors are missing, first: {missing[0]}")
    extra = [k for k in where if k not in wanted and not k.endswith(_SAFETENSORS_IGNORED_SUFFIXES) and not k.startswith(allow_extra_prefixes or ("\0",))]
    if extra:
        raise SafetensorsError(f"{len(extra)} tensors outside the text contract, first: {sorted(extra)[0]} (name their prefix in allow_extra_prefixes to skip them)")
    dtypes: dict[str, int] = {}
    payload = 0
    for name, c in wanted.items():
        entry = headers[where[name]].get(name)
        if entry is None:
            raise SafetensorsError(f"the index places {name} in {where[name].name}, whose header does not list it")
        if tuple(entry.get("shape", ())) != c.shape:
            raise SafetensorsError(f"{name}: shape {tuple(entry.get('shape', ()))} instead of {c.shape}")
        dtypes[entry["dtype"]] = dtypes.get(entry["dtype"], 0) + 1
        lo, hi = entry["data_offsets"]
        payload += hi - lo
    n_params = sum(int(torch.tensor(c.shape).prod()) for c in contracts)
    return {"status": "ok", "geometry": asdict(g), "tensors": len(contracts), "parameters": n_params, "payload_bytes": payload,
            "dtypes": dtypes, "shards": sorted(p.name for p in headers)}


def load_glimmer_safetensors(directory, geometry: GlimmerGeometry | None = None, *, dtype=torch.bfloat16,
                             allow_extra_prefixes: tuple[str, ...] = ()) -> dict[str, torch.Tensor]:
    g = geometry or GlimmerGeometry()
    inspect_glimmer_safetensors(directory, g, allow_extra_prefixes=allow_extra_prefixes)
    where = _shard_map(Path(directory))
    wanted = {c.source: c for c in safetensors_contracts(g)}
    pieces: dict[str, torch.Tensor] = {}
    for shard in sorted(set(where.values())):
        names = {n for n, p in where.items() if p == shard and n in wanted}
        got, _ = read_safetensors(shard, names=names)
        for n in names:
            pieces[wanted[n].part] = got[n].to(dtype)
    return _assemble(g, pieces)


def load_glimmer_gguf(paths, geometry: GlimmerGeometry | None = None, *, dtype=torch.bfloat16) -> dict[str, torch.Tensor]:
    """One or more GGUF files (a split export) -> engine tensors; K-quant blocks are decoded."""
    from .gguf import GGUFFile
    g = geometry or GlimmerGeometry()
    wanted = {c.source: c for c in gguf_contracts(g)}
    pieces: dict[str, torch.Tensor] = {}
    for path in ([paths] if isinstance(paths, (str, Path)) else list(paths)):
        with GGUFFile(path) as f:
            for name, t in f.tensors.items():
                if name.endswith(_GGUF_IGNORED_SUFFIXES):
                    continue
                c = wanted.get(name)
                if c is None:
                    raise ValueError(f"{path}: tensor {name} is outside the Muse-Glimmer text contract")
                if tuple(t.shape) != c.shape:
                    raise ValueError(f"{name}: shape {tuple(t.shape)} instead of {c.shape}")
                if c.part in pieces:
                    raise ValueError(f"{name} appears in more than one file")
                pieces[c.part] = torch.from_numpy(f.dequantize(name).copy()).to(dtype)
    missing = sorted(c.source for c in wanted.values() if c.part not in pieces)
    if missing:
        raise ValueError(f"{len(missing)} contract tensors are missing from the GGUF files, first: {missing[0]}")
    return _assemble(g, pieces)


def to_serving_names(params: dict[str, torch.Tensor], g: GlimmerGeometry) -> dict[str, torch.Tensor]:
    """The unsharded dictionary ``serving.tp_glimmer.TPGlimmerDecoder(full_params=...)`` takes (projections apart)."""
    q, kv = g.q_width, g.kv_width
    out = {"embed": params["tok_embeddings"], "head": params["lm_head"], "final_norm": params["norm"]}
    for l in range(g.n_layer):
        p = f"layers.{l}."
        w, gu = params[p + "wqkvg"], params[p + "w_gate_up"]
        out.update({p + "wq": w[:q], p + "wk": w[q:q + kv], p + "wv": w[q + kv:q + 2 * kv], p + "wg": w[q + 2 * kv:],
                    p + "w_gate": gu[:g.d_ff], p + "w_up": gu[g.d_ff:]})
        for k in ("attn_norm", "wo", "post_attn_norm", "mlp_norm", "w_down", "post_mlp_norm"):
            out[p + k] = params[p + k]
    return out


def convert_glimmer_weights(source, output_dir, geometry: GlimmerGeometry | None = None, *, gguf: bool = False,
                            allow_extra_prefixes: tuple[str, ...] = ()) -> dict:
    """Writes ``output_dir`` (must not exist) as a named-tensor checkpoint at step 0. Returns the manifest."""
    from .named import write_named_tensors
    g = geometry or GlimmerGeometry()
    out = Path(output_dir)
    if out.exists():
        raise FileExistsError(f"{out} exists; converted checkpoints are never overwritten")
    params = load_glimmer_gguf(source, g) if gguf else load_glimmer_safetensors(source, g, allow_extra_prefixes=allow_extra_prefixes)
    out.mkdir(parents=True)
    name = "weights_00000000.nfnw"
    sha = write_named_tensors(out / name, params, {"model_family": "muse-glimmer", "geometry": asdict(g), "step": 0,
                                                   "source_format": "gguf" if gguf else "safetensors"})
    manifest = {"format": "neuralfn_b200.named_checkpoint", "model_family": "muse-glimmer", "geometry": asdict(g), "step": 0,
                "tensors": len(params), "parameters": sum(t.numel() for t in params.values()), "files": {name: sha}}
    (out / "manifest.json").write_text(json.dumps(manifest, indent=2))
    (out / "DONE_00000000").write_text(json.dumps({name: sha}))
    return manifest

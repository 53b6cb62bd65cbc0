"""Dense GPT checkpoints in the reference's on-disk formats, so files interchange:

* ``model_%08d.bin``       256 x int32 header ``[20240326, 5, T, V, L, H, C, Vp, 0...]`` + bf16
  tensors in the order ``wte, wpe, per layer {ln_1.w, ln_1.b, c_attn.w[3C,C], c_attn.b,
  c_proj.w, c_proj.b, ln_2.w, ln_2.b, c_fc.w[4C,C], c_fc.b, mlp.c_proj.w[C,4C],
  mlp.c_proj.b}, ln_f.w, ln_f.b`` (reader: ``neuralfn/native_dense_checkpoint.py:171-313``)
* ``parameters_%08d.bin``  32 x int64 header ``[20260711, 1, step, T, V, L, H, C, Vp, n_tensors,
  n_elements, grad_accum, micro_steps]`` + fp32 master weights, same order
* ``optimizer_%08d.bin``   32 x int64 header ``[20260710, 1, step, T, V, L, H, C, Vp, n_tensors,
  2*n_elements, grad_accum, micro_steps]`` + per tensor ``m`` then ``v`` (fp32)
  (writers: ``nfn_gpt2_native_train.cpp:29053-29550``)
* ``DONE_%08d``            written last.

Added for the data-parallel sharded optimizer: ``optimizer_%08d.rank%05d.bin`` (one per
rank: 32 x int64 header ``[20260712, 1, step, T, V, L, H, C, Vp, rank, world, lo, shard,
n_total]`` + the rank's fp32 ``master, m, v`` slices of the flat layout) with
``optimizer_%08d.manifest.json`` naming every shard and its SHA-256;
``consolidate_sharded_optimizer`` rebuilds the single-file forms from them.
A ``model_%08d.variant.json`` sidecar records what the v5 header cannot (qk-norm,
soft-cap, z-loss, eps values).
"""
from __future__ import annotations

import json
import struct
from dataclasses import asdict
from pathlib import Path

import torch
import torch.distributed as dist

from ..models.gpt2 import FlatLayout, GPT2Config, gpt2_param_specs
from .container import peek_header, read_container, write_container

MODEL_MAGIC, MODEL_VERSION, MODEL_HEADER_BYTES = 20240326, 5, 1024
PARAMS_MAGIC, OPTIM_MAGIC, SHARD_MAGIC, STATE_HEADER_BYTES = 20260711, 20260710, 20260712, 256

__all__ = ["read_moa_sidecar", "write_dense_model", "read_dense_model", "inspect_dense_model", "save_dense_checkpoint", "load_dense_checkpoint",
           "consolidate_sharded_optimizer", "latest_step"]


def _geometry(cfg: GPT2Config) -> list[int]:
    return [cfg.max_seq_len, cfg.vocab_size, cfg.n_layer, cfg.n_head, cfg.d_model, cfg.padded_vocab]


def _model_header(cfg: GPT2Config) -> bytes:
    h = [0] * 256
    h[0], h[1] = MODEL_MAGIC, MODEL_VERSION
    h[2:8] = _geometry(cfg)
    return struct.pack("<256i", *h)


def _state_header(magic: int, step: int, cfg: GPT2Config, *rest: int) -> bytes:
    h = [magic, 1, step, *_geometry(cfg), *rest]
    return struct.pack("<32q", *(h + [0] * (32 - len(h))))


def _ordered_views(cfg: GPT2Config, layout: FlatLayout, flat: torch.Tensor) -> list[torch.Tensor]:
    return [layout.view(flat, s.name) for s in gpt2_param_specs(cfg)]


def write_dense_model(path, cfg: GPT2Config, layout: FlatLayout, params_bf16: torch.Tensor) -> str:
    """bf16 flat parameter buffer -> ``model_*.bin``. Returns the file SHA-256."""
    flat = params_bf16.detach().to("cpu", torch.bfloat16).contiguous()
    return write_container(path, _model_header(cfg), _ordered_views(cfg, layout, flat))


def inspect_dense_model(path) -> dict:
    raw, size = peek_header(path, MODEL_HEADER_BYTES)
    h = struct.unpack("<256i", raw)
    if h[0] != MODEL_MAGIC or h[1] != MODEL_VERSION:
        raise ValueError("not a dense GPT checkpoint at version 5")
    T, V, L, H, C, Vp = h[2:8]
    if min(T, V, L, H, C) <= 0 or Vp < V or C % H:
        raise ValueError("dense checkpoint has invalid model geometry")
    cfg = GPT2Config(n_layer=L, n_head=H, d_model=C, vocab_size=V, max_seq_len=T)
    if cfg.padded_vocab != Vp:
        cfg = GPT2Config(n_layer=L, n_head=H, d_model=C, vocab_size=V, max_seq_len=T, vocab_pad_to=_pad_quantum(V, Vp))
    n = sum(s.numel for s in gpt2_param_specs(cfg))
    if size != MODEL_HEADER_BYTES + 2 * n:
        raise ValueError("dense checkpoint file size does not match its version-5 geometry")
    return {"max_seq_len": T, "vocab_size": V, "num_layers": L, "num_heads": H, "channels": C, "padded_vocab_size": Vp,
            "parameter_count": n, "file_size": size, "config": cfg}


def _pad_quantum(V: int, Vp: int) -> int:
    for q in (128, 64, 256, 512, 1024, 32, 16, 8, 1):
        if (V + q - 1) // q * q == Vp:
            return q
    raise ValueError(f"cannot express padded vocab {Vp} for vocab {V}")


def read_dense_model(path, variant: dict | None = None) -> tuple[GPT2Config, dict[str, torch.Tensor], str]:
    """-> (config, name -> bf16 CPU tensor, file sha256). The variant sidecar next to the
    file (or ``variant``) restores qk-norm / soft-cap / z-loss settings."""
    info = inspect_dense_model(path)
    cfg: GPT2Config = info["config"]
    side = Path(str(path)[:-4] + ".variant.json")
    if variant is None and side.exists():
        variant = json.loads(side.read_text())
    if variant:
        cfg = GPT2Config(**{**asdict(cfg), **{k: v for k, v in variant.items() if k in asdict(cfg)}})
    specs = gpt2_param_specs(cfg)
    tensors = [torch.empty(s.shape, dtype=torch.bfloat16) for s in specs]
    _, sha = read_container(path, MODEL_HEADER_BYTES, tensors)
    named = {s.name: t for s, t in zip(specs, tensors)}
    diff_meta = Path(str(path)[:-4] + ".diff.json")
    if getattr(cfg, "differential", False) and diff_meta.exists():
        import numpy as np
        meta = json.loads(diff_meta.read_text())
        lam = np.frombuffer((diff_meta.parent / meta["parameters"]).read_bytes(), dtype="<f4")
        for l in range(cfg.n_layer):
            slot = torch.zeros(8, dtype=torch.bfloat16)
            slot[0] = float(lam[l])
            named[f"h.{l}.attn.diff_lambda"] = slot
    return cfg, named, sha


def latest_step(directory) -> int | None:
    steps = sorted(int(p.name[5:]) for p in Path(directory).glob("DONE_*") if p.name[5:].isdigit())
    return steps[-1] if steps else None


def _all_gather_flat(shard: torch.Tensor, world: int) -> torch.Tensor:
    if world == 1:
        return shard
    full = torch.empty(shard.numel() * world, dtype=shard.dtype, device=shard.device)
    dist.all_gather_into_tensor(full, shard.contiguous())
    return full


def save_dense_checkpoint(trainer, out_dir, step: int | None = None, *, sharded_optimizer: bool | None = None,
                          grad_accum: int = 1) -> dict:
    """Collective over the trainer's ranks. Writes model + fp32 parameters + optimizer
    (single-file when ``sharded_optimizer`` is false: the shards are all-gathered first;
    rank-sharded files + manifest otherwise, the default for world > 1) + ``DONE``.
    Returns {file name: sha256} on rank 0."""
    cfg, layout, opt = trainer.cfg, trainer.layout, trainer.opt
    world, rank = opt.world, opt.rank
    step = opt.step_count if step is None else step
    sharded = (world > 1) if sharded_optimizer is None else sharded_optimizer
    out = Path(out_dir)
    if rank == 0:
        out.mkdir(parents=True, exist_ok=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize() if trainer.device.type == "cuda" else None
    digests: dict[str, str] = {}
    specs = gpt2_param_specs(cfg)
    n_el = sum(s.numel for s in specs)
    if rank == 0:
        name = f"model_{step:08d}.bin"
        digests[name] = write_dense_model(out / name, cfg, layout, trainer.bufs.params)
        (out / f"model_{step:08d}.variant.json").write_text(json.dumps(
            {k: getattr(cfg, k) for k in ("qk_norm", "qk_norm_eps", "logit_softcap", "z_loss", "ln_eps", "mlp_mult", "vocab_pad_to",
                                          "differential", "diff_lambda_init", "diff_norm_eps")}))
    if sharded:
        name = f"optimizer_{step:08d}.rank{rank:05d}.bin"
        hdr = _state_header(SHARD_MAGIC, step, cfg, rank, world, opt.lo, opt.shard, layout.n_total)
        sha = write_container(out / name, hdr, [opt.master, opt.m, opt.v])
        entries = [None] * world
        if world > 1:
            dist.all_gather_object(entries, {"rank": rank, "file": name, "sha256": sha, "lo": opt.lo, "shard": opt.shard})
        else:
            entries = [{"rank": 0, "file": name, "sha256": sha, "lo": 0, "shard": opt.shard}]
        if rank == 0:
            manifest = {"schema": "neuralfn_b200.dense_sharded_optimizer.v1", "step": step, "world_size": world,
                        "n_total": layout.n_total, "geometry": _geometry(cfg), "shards": entries}
            (out / f"optimizer_{step:08d}.manifest.json").write_text(json.dumps(manifest, indent=2))
            digests.update({e["file"]: e["sha256"] for e in entries})
    else:
        master, m, v = (_all_gather_flat(t, world).cpu() for t in (opt.master, opt.m, opt.v))
        if rank == 0:
            name = f"parameters_{step:08d}.bin"
            digests[name] = write_container(out / name, _state_header(PARAMS_MAGIC, step, cfg, len(specs), n_el, grad_accum, step * grad_accum),
                                            _ordered_views(cfg, layout, master))
            name = f"optimizer_{step:08d}.bin"
            mv = [t for a, b in zip(_ordered_views(cfg, layout, m), _ordered_views(cfg, layout, v)) for t in (a, b)]
            digests[name] = write_container(out / name, _state_header(OPTIM_MAGIC, step, cfg, len(specs), 2 * n_el, grad_accum, step * grad_accum), mv)
    if getattr(cfg, "differential", False):
        digests.update(_write_diff_sidecars(out, step, cfg, layout, opt, world, rank))
    if getattr(cfg, "moa_activations", ()) and rank == 0:
        digests.update(_write_moa_sidecar(out, step, cfg, getattr(trainer.engine, "activation", cfg.moa_activations[0]), digests))
    if world > 1:
        dist.barrier()
    if rank == 0:
        (out / f"DONE_{step:08d}").write_text(json.dumps(digests, sort_keys=True))
    return digests


DIFF_SCHEMA = "neuralfn_b200.gpt2_diff.sidecar.v1"
MOA_SCHEMA = "neuralfn.native_dense_moa.inference_checkpoint"


def _write_moa_sidecar(out: Path, step: int, cfg: GPT2Config, selected: str, digests: dict[str, str]) -> dict[str, str]:
    """Mixture-of-activations runs: ``model_<step>.moa.json`` names the activation in effect when the model file was written
    (inference must apply the same one), the candidates and the probe interval; schema and file name as the reference's
    (``nfn_gpt2_native_train.cpp:3985-3987,4303-4330``)."""
    import hashlib
    model = f"model_{step:08d}.bin"
    meta = {"schema": MOA_SCHEMA, "version": 1, "preset": "gpt2_moa", "checkpoint_kind": "trained_dense_v5",
            "model": {"path": model, "format": "neuralfn.native_dense_gpt.v5", "nbytes": (out / model).stat().st_size, "sha256": digests.get(model, "")},
            "done_marker": f"DONE_{step:08d}",
            "selection": {"activation": selected, "candidates": list(cfg.moa_activations), "interval": cfg.moa_interval},
            "geometry": {"max_seq_len": cfg.max_seq_len, "vocab_size": cfg.vocab_size, "padded_vocab_size": cfg.padded_vocab, "num_layers": cfg.n_layer,
                         "model_dim": cfg.d_model, "num_heads": cfg.n_head, "head_dim": cfg.head_dim, "mlp_hidden_dim": cfg.mlp_mult * cfg.d_model}}
    raw = json.dumps(meta, indent=2).encode()
    name = f"model_{step:08d}.moa.json"
    (out / name).write_bytes(raw)
    return {name: hashlib.sha256(raw).hexdigest()}


def read_moa_sidecar(directory, step: int) -> dict:
    """The selection record of a mixture-of-activations checkpoint; refuses a file whose model digest does not match."""
    d = Path(directory)
    path = d / f"model_{step:08d}.moa.json"
    if not path.exists():
        raise FileNotFoundError(f"{path.name} is missing: a gpt2_moa checkpoint needs its activation record")
    meta = json.loads(path.read_text())
    if meta.get("schema") != MOA_SCHEMA or meta.get("selection", {}).get("activation") not in meta.get("selection", {}).get("candidates", []):
        raise ValueError(f"{path.name}: not a mixture-of-activations record")
    done = json.loads((d / f"DONE_{step:08d}").read_text())
    if meta["model"].get("sha256") and done.get(meta["model"]["path"]) != meta["model"]["sha256"]:
        raise ValueError(f"{path.name} describes a different model file")
    return meta


def _diff_values(cfg: GPT2Config, layout: FlatLayout, flat: torch.Tensor) -> torch.Tensor:
    """[n_layer] fp32: element 0 of every layer's lambda slot of a full flat fp32 buffer."""
    return torch.stack([layout.view(flat, f"h.{l}.attn.diff_lambda")[0] for l in range(cfg.n_layer)]).float().cpu()


def _write_diff_sidecars(out: Path, step: int, cfg: GPT2Config, layout: FlatLayout, opt, world: int, rank: int) -> dict[str, str]:
    """Differential variant: the learned lambdas are no tensors of the dense model file. Their fp32
    values and AdamW moments go to ``diff_parameters_<step>.bin`` / ``diff_optimizer_<step>.bin`` (raw
    little-endian fp32, one value per layer; moments as m then v) with ``model_<step>.diff.json``
    describing them (file names as the reference's, ``nfn_gpt2_native_train.cpp:4402-4430``)."""
    import hashlib
    master, m, v = (_all_gather_flat(t, world).cpu() for t in (opt.master, opt.m, opt.v))
    if rank != 0:
        return {}
    lam, lm, lv = (_diff_values(cfg, layout, t) for t in (master, m, v))
    digests = {}
    for name, payload in ((f"diff_parameters_{step:08d}.bin", lam), (f"diff_optimizer_{step:08d}.bin", torch.cat([lm, lv]))):
        raw = payload.numpy().astype("<f4").tobytes()
        (out / name).write_bytes(raw)
        digests[name] = hashlib.sha256(raw).hexdigest()
    meta = {"schema": DIFF_SCHEMA, "step": step, "layers": cfg.n_layer, "lambda_init": cfg.diff_lambda_init,
            "norm_eps": cfg.diff_norm_eps, "dtype": "float32", "parameters": f"diff_parameters_{step:08d}.bin",
            "optimizer": f"diff_optimizer_{step:08d}.bin", "sha256": digests}
    (out / f"model_{step:08d}.diff.json").write_text(json.dumps(meta, indent=2))
    return digests


def _load_diff_sidecars(d: Path, step: int, cfg: GPT2Config, layout: FlatLayout, trainer, restored: dict) -> None:
    """Restores lambdas (bf16 parameters, fp32 master) and their moments from the sidecars. A checkpoint
    of the differential variant without them is refused: silently re-initialised lambdas would change the model."""
    import hashlib
    import numpy as np
    meta_path = d / f"model_{step:08d}.diff.json"
    if not meta_path.exists():
        raise FileNotFoundError(f"{meta_path.name} is missing: a gpt2_diff checkpoint needs its differential sidecars")
    meta = json.loads(meta_path.read_text())
    if meta.get("schema") != DIFF_SCHEMA or int(meta["layers"]) != cfg.n_layer or int(meta["step"]) != step:
        raise ValueError("differential sidecar metadata does not match this model / step")
    opt = trainer.opt
    lo, hi = opt.lo, opt.lo + opt.shard

    def read(name: str, count: int) -> torch.Tensor:
        raw = (d / name).read_bytes()
        if hashlib.sha256(raw).hexdigest() != meta["sha256"][name] or len(raw) != 4 * count:
            raise ValueError(f"{name}: size or checksum does not match {meta_path.name}")
        return torch.from_numpy(np.frombuffer(raw, dtype="<f4").copy())

    lam = read(meta["parameters"], cfg.n_layer)
    mv = read(meta["optimizer"], 2 * cfg.n_layer)
    params = trainer.bufs.params
    for l in range(cfg.n_layer):
        name = f"h.{l}.attn.diff_lambda"
        off = layout.offsets[name]
        layout.view(params, name)[0] = lam[l].to(params.dtype)
        if lo <= off < hi:                       # this rank owns the slot's first element
            opt.master[off - lo] = lam[l]
            if restored.get("moments"):
                opt.m[off - lo] = mv[l]
                opt.v[off - lo] = mv[cfg.n_layer + l]
    restored["diff_sidecars"] = True


def _read_state(path, magic: int, cfg: GPT2Config, tensors: list[torch.Tensor]) -> tuple[int, ...]:
    raw, _ = read_container(path, STATE_HEADER_BYTES, tensors)
    h = struct.unpack("<32q", raw)
    if h[0] != magic or h[1] != 1 or list(h[3:9]) != _geometry(cfg):
        raise ValueError(f"{Path(path).name}: magic/version/geometry does not match the model")
    return h


def consolidate_sharded_optimizer(directory, step: int, cfg: GPT2Config) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Rebuilds the full flat fp32 ``(master, m, v)`` from rank-sharded optimizer files,
    checking each shard's SHA-256 against the manifest."""
    d = Path(directory)
    man = json.loads((d / f"optimizer_{step:08d}.manifest.json").read_text())
    if man["geometry"] != _geometry(cfg):
        raise ValueError("sharded optimizer manifest belongs to a different model geometry")
    n_total = man["n_total"]
    full = [torch.zeros(n_total, dtype=torch.float32) for _ in range(3)]
    for e in sorted(man["shards"], key=lambda e: e["rank"]):
        parts = [torch.empty(e["shard"], dtype=torch.float32) for _ in range(3)]
        raw, sha = read_container(d / e["file"], STATE_HEADER_BYTES, parts)
        h = struct.unpack("<32q", raw)
        if h[0] != SHARD_MAGIC or h[2] != step or h[9] != e["rank"] or h[10] != man["world_size"] or sha != e["sha256"]:
            raise ValueError(f"{e['file']}: header or checksum does not match the manifest")
        for dst, src in zip(full, parts):
            dst[e["lo"]:e["lo"] + e["shard"]] = src
    return tuple(full)


def load_dense_checkpoint(trainer, directory, step: int | None = None) -> dict:
    """Restores a trainer (any world size that matches the files' sharding, or any world
    size at all for single-file optimizers). A model-only checkpoint is a warm start:
    master weights are the bf16 weights, moments reset - the reference's behaviour
    (``nfn_gpt2_native_train.cpp:1134``). Returns what was restored."""
    d = Path(directory)
    step = latest_step(d) if step is None else step
    if step is None:
        raise FileNotFoundError(f"no completed checkpoint (DONE_*) under {d}")
    cfg, layout, opt = trainer.cfg, trainer.layout, trainer.opt
    cfg_file, tensors, _ = read_dense_model(d / f"model_{step:08d}.bin")
    if _geometry(cfg_file) != _geometry(cfg):
        raise ValueError("checkpoint geometry does not match the trainer's model")
    flat = torch.zeros(layout.n_total, dtype=torch.bfloat16)
    for name, t in tensors.items():
        layout.view(flat, name).copy_(t)
    trainer.bufs.params.copy_(flat)
    restored = {"step": step, "model": True, "master": False, "moments": False}
    lo, hi = opt.lo, opt.lo + opt.shard
    man = d / f"optimizer_{step:08d}.manifest.json"
    if man.exists():
        m = json.loads(man.read_text())
        if m["world_size"] == opt.world:
            e = next(e for e in m["shards"] if e["rank"] == opt.rank)
            parts = [torch.empty(opt.shard, dtype=torch.float32) for _ in range(3)]
            raw, sha = read_container(d / e["file"], STATE_HEADER_BYTES, parts)
            h = struct.unpack("<32q", raw)
            # the shard's own header must describe this step, rank, world and slice: a manifest that points
            # at a shard of another step (with a matching digest entry) must not load silently
            if (h[0] != SHARD_MAGIC or h[2] != step or h[9] != opt.rank or h[10] != opt.world or e["lo"] != opt.lo
                    or e["shard"] != opt.shard or sha != e["sha256"]):
                raise ValueError(f"{e['file']}: header or checksum does not match the manifest / this rank's shard")
        else:  # re-shard through the consolidated form
            parts = []
            for t in consolidate_sharded_optimizer(d, step, cfg):
                # the saving world padded the flat buffer to a multiple of 8 * its size; this world pads
                # to its own multiple. Only padding differs, so cut or zero-extend to this layout's length.
                if t.numel() < layout.n_total:
                    t = torch.cat([t, torch.zeros(layout.n_total - t.numel(), dtype=t.dtype)])
                parts.append(t[:layout.n_total][lo:hi])
        for dst, src in zip((opt.master, opt.m, opt.v), parts):
            dst.copy_(src)
        restored.update(master=True, moments=True)
    else:
        specs = gpt2_param_specs(cfg)
        pfile, ofile = d / f"parameters_{step:08d}.bin", d / f"optimizer_{step:08d}.bin"
        if pfile.exists():
            full = torch.zeros(layout.n_total, dtype=torch.float32)
            _read_state(pfile, PARAMS_MAGIC, cfg, _ordered_views(cfg, layout, full))
            opt.master.copy_(full[lo:hi])
            restored["master"] = True
        else:
            opt.master.copy_(flat[lo:hi].float())
        if ofile.exists():
            fm, fv = torch.zeros(layout.n_total, dtype=torch.float32), torch.zeros(layout.n_total, dtype=torch.float32)
            # the file interleaves m and v per tensor; read into per-tensor temporaries
            tmp = [torch.empty(s.shape, dtype=torch.float32) for s in specs for _ in (0, 1)]
            _read_state(ofile, OPTIM_MAGIC, cfg, tmp)
            for i, s in enumerate(specs):
                layout.view(fm, s.name).copy_(tmp[2 * i])
                layout.view(fv, s.name).copy_(tmp[2 * i + 1])
            opt.m.copy_(fm[lo:hi])
            opt.v.copy_(fv[lo:hi])
            restored["moments"] = True
        else:
            opt.m.zero_()
            opt.v.zero_()
    if getattr(cfg, "differential", False):
        _load_diff_sidecars(d, step, cfg, layout, trainer, restored)
    if getattr(cfg, "moa_activations", ()):
        trainer.engine.activation = read_moa_sidecar(d, step)["selection"]["activation"]
        restored["moa_activation"] = trainer.engine.activation
    opt.step_count = step if restored["moments"] else 0
    return restored

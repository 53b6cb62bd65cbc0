"""Self-describing checkpoints for model families without a fixed legacy layout (Llama-style
engines, MoE, ...): ``weights_%08d.nfnw`` = ``NFNNAMED`` magic, u64 length of a JSON header
(model config, tensor names / shapes / dtype, in file order), zero padding to a multiple of
256 bytes, then the tensors back to back; ``state_%08d.rank%05d.nfns`` = the rank's fp32
``master, m, v`` shards of the flat layout behind the same kind of header. Written through
the exclusive, checksummed container writer; a ``DONE_%08d`` file lists every SHA-256.
"""
from __future__ import annotations

import json
import struct
from dataclasses import asdict, is_dataclass
from pathlib import Path

import torch
import torch.distributed as dist

from .container import peek_header, read_container, write_container

MAGIC = b"NFNNAMED"
__all__ = ["write_named_tensors", "read_named_tensors", "save_named_checkpoint", "load_named_checkpoint"]


def _header(meta: dict) -> bytes:
    body = json.dumps(meta, sort_keys=True).encode()
    raw = MAGIC + struct.pack("<Q", len(body)) + body
    return raw + b"\0" * (-len(raw) % 256)


def _read_header(path) -> tuple[dict, int]:
    head, _ = peek_header(path, 16)
    if head[:8] != MAGIC:
        raise ValueError(f"{path}: not a named-tensor checkpoint")
    n = struct.unpack("<Q", head[8:16])[0]
    total = (16 + n + 255) // 256 * 256
    raw, _ = peek_header(path, total)
    return json.loads(raw[16:16 + n]), total


def write_named_tensors(path, tensors: dict[str, torch.Tensor], meta: dict | None = None) -> str:
    items = [(k, v.detach().to("cpu").contiguous()) for k, v in tensors.items()]
    table = [{"name": k, "shape": list(v.shape), "dtype": str(v.dtype).replace("torch.", "")} for k, v in items]
    return write_container(path, _header({"tensors": table, **(meta or {})}), [v for _, v in items])


def read_named_tensors(path) -> tuple[dict[str, torch.Tensor], dict, str]:
    meta, hbytes = _read_header(path)
    out = {t["name"]: torch.empty(t["shape"], dtype=getattr(torch, t["dtype"])) for t in meta["tensors"]}
    _, sha = read_container(path, hbytes, list(out.values()))
    return out, meta, sha


def save_named_checkpoint(trainer, out_dir, step: int | None = None) -> dict:
    """Collective. bf16 weights by name (rank 0) + every rank's optimizer shard."""
    opt, layout = trainer.opt, trainer.layout
    step = opt.step_count if step is None else step
    out = Path(out_dir)
    if opt.rank == 0:
        out.mkdir(parents=True, exist_ok=True)
    if opt.world > 1:
        dist.barrier()
    if trainer.device.type == "cuda":
        torch.cuda.synchronize()
    cfg = trainer.cfg
    meta = {"config": asdict(cfg) if is_dataclass(cfg) else dict(vars(cfg)), "config_class": type(cfg).__name__, "step": step}
    digests = {}
    if opt.rank == 0:
        flat = trainer.bufs.params.detach().cpu()
        name = f"weights_{step:08d}.nfnw"
        digests[name] = write_named_tensors(out / name, {s.name: layout.view(flat, s.name) for s in cfg.param_specs()}, meta)
    name = f"state_{step:08d}.rank{opt.rank:05d}.nfns"
    sha = write_named_tensors(out / name, {"master": opt.master, "m": opt.m, "v": opt.v},
                              {**meta, "rank": opt.rank, "world_size": opt.world, "lo": opt.lo, "shard": opt.shard, "n_total": layout.n_total})
    entries = [None] * opt.world
    if opt.world > 1:
        dist.all_gather_object(entries, (name, sha))
    else:
        entries = [(name, sha)]
    digests.update(dict(entries))
    if opt.world > 1:
        dist.barrier()
    if opt.rank == 0:
        (out / f"DONE_{step:08d}").write_text(json.dumps(digests, sort_keys=True))
    return digests


def load_named_checkpoint(trainer, directory, step: int | None = None, *, weights_only: bool = False) -> dict:
    """``weights_only``: start a new run from the saved weights (fresh moments, step 0), as post-training does."""
    from .dense import latest_step
    d = Path(directory)
    step = latest_step(d) if step is None else step
    if step is None:
        raise FileNotFoundError(f"no completed checkpoint (DONE_*) under {d}")
    opt, layout = trainer.opt, trainer.layout
    digests = json.loads((d / f"DONE_{step:08d}").read_text())
    tensors, meta, sha = read_named_tensors(d / f"weights_{step:08d}.nfnw")
    if sha != digests[f"weights_{step:08d}.nfnw"]:
        raise ValueError("weights file does not match the checksum recorded at save time")
    flat = torch.zeros(layout.n_total, dtype=torch.bfloat16)
    for s in trainer.cfg.param_specs():
        if tuple(tensors[s.name].shape) != tuple(s.shape):
            raise ValueError(f"checkpoint tensor {s.name} has shape {tuple(tensors[s.name].shape)}, the model expects {tuple(s.shape)}")
        layout.view(flat, s.name).copy_(tensors[s.name])
    trainer.bufs.params.copy_(flat)
    restored = {"step": step, "model": True, "moments": False}
    sfile = d / f"state_{step:08d}.rank{opt.rank:05d}.nfns"
    if sfile.exists() and not weights_only:
        st, smeta, _ = read_named_tensors(sfile)
        if smeta["world_size"] != opt.world or smeta["shard"] != opt.shard:
            raise ValueError("optimizer state was saved for a different world size")
        opt.master.copy_(st["master"])
        opt.m.copy_(st["m"])
        opt.v.copy_(st["v"])
        opt.step_count = step
        restored["moments"] = True
    else:
        opt.master.copy_(flat[opt.lo:opt.lo + opt.shard].float())
        opt.m.zero_()
        opt.v.zero_()
        opt.step_count = 0
    return restored

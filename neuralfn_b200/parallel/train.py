"""Training driver for the model-parallel families: tensor-parallel Llama (``--parallel tp``) and
expert-parallel MoE Llama (``--parallel ep``). One process per GPU under ``torch.distributed.run``
(or one process alone); CPU ranks on gloo run the same code with PyTorch fallbacks.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m neuralfn_b200.parallel.train \
        --parallel tp --model llama3_8b --dataset /data/fineweb10B --batch-size 4 --seq-len 4096 --max-steps 1000 --output-dir runs/tp

* ``tp``: every rank of the group sees the SAME batch (rows are split inside the model);
* ``ep``: every rank draws its OWN batches (data parallel around the expert-parallel layers).

Progress goes to stdout as JSON lines (``train_step``, ``checkpoint``, ``complete``), the format the
``nfn`` dashboard reads. A checkpoint is a directory ``step_%08d/`` with one safetensors file per
rank (named fp32 master tensors of that rank's shard plus the flat AdamW moments), ``manifest.json``
written last by rank 0; ``--resume`` continues from the newest complete one, data cursor included.

Reference counterpart: the per-family native trainers launched by ``cli/nfn.py`` (single GPU there).
"""
from __future__ import annotations

import argparse
import json
import os
import time
from dataclasses import asdict
from pathlib import Path

import torch
import torch.distributed as dist

__all__ = ["main", "save_parallel_checkpoint", "load_parallel_checkpoint"]


def _emit(rank: int, **ev) -> None:
    if rank == 0:
        print(json.dumps(ev), flush=True)


def _check_device_status(device, what: str) -> None:
    """Raise when a kernel recorded an error (a bounded wait that ran out) since the last check."""
    if torch.device(device).type != "cuda":
        return
    from ..ops import _lib
    _lib.assert_status_ok(what)


def save_parallel_checkpoint(trainer, out_dir: Path, step: int, extra: dict) -> Path:
    from ..checkpoint.safetensors_io import write_safetensors
    mdl = trainer.model
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    d = out_dir / f"step_{step:08d}"
    d.mkdir(parents=True, exist_ok=True)
    tensors = {f"master.{n}": v.detach().cpu() for n, v in mdl.layout.views(trainer.master).items()}
    tensors["adam.m"], tensors["adam.v"] = trainer.m.detach().cpu(), trainer.v.detach().cpu()
    path = d / f"rank{rank:03d}.safetensors"
    if path.exists():
        path.unlink()
    write_safetensors(path, tensors, {"step": str(step), "rank": str(rank), "world": str(world)})
    if dist.is_initialized():
        dist.barrier()
    if rank == 0:
        (d / "manifest.json").write_text(json.dumps({"schema": "neuralfn_b200.parallel_checkpoint.v1", "step": step, "world": world,
                                                     "optimizer_step": trainer.step_count, **extra}, indent=2))
    return d


def load_parallel_checkpoint(trainer, out_dir: Path) -> dict | None:
    """Restores the newest complete checkpoint under ``out_dir`` (same world size); returns its manifest."""
    from ..checkpoint.safetensors_io import read_safetensors
    done = sorted(p.parent for p in out_dir.glob("step_*/manifest.json"))
    if not done:
        return None
    d = done[-1]
    man = json.loads((d / "manifest.json").read_text())
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    if man["world"] != world:
        raise ValueError(f"checkpoint was written by {man['world']} ranks, this job has {world}")
    tensors, _ = read_safetensors(d / f"rank{rank:03d}.safetensors")
    mdl = trainer.model
    with torch.no_grad():
        for n, v in mdl.layout.views(trainer.master).items():
            v.copy_(tensors[f"master.{n}"])
        trainer.m.copy_(tensors["adam.m"])
        trainer.v.copy_(tensors["adam.v"])
        mdl.params.detach().copy_(trainer.master.to(mdl.dtype))
    trainer.step_count = int(man["optimizer_step"])
    return man


def main(argv=None) -> int:
    from ..bench.tp_llama_bench import MODELS
    ap = argparse.ArgumentParser(prog="neuralfn_b200.parallel.train")
    ap.add_argument("--parallel", choices=["tp", "ep"], required=True)
    ap.add_argument("--model", default="tiny", help="tp: " + " | ".join(sorted(MODELS)) + "; ep: ignored (use the --n-* flags)")
    ap.add_argument("--n-layer", type=int, default=4)
    ap.add_argument("--n-head", type=int, default=8)
    ap.add_argument("--n-kv-head", type=int, default=4)
    ap.add_argument("--d-model", type=int, default=512)
    ap.add_argument("--vocab-size", type=int, default=50304)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--expert-hidden", type=int, default=1024)
    ap.add_argument("--router-score", default="softmax", choices=["softmax", "sigmoid", "sqrt_softplus"])
    ap.add_argument("--balance-coef", type=float, default=0.01)
    ap.add_argument("--router-z-coef", type=float, default=1e-3)
    ap.add_argument("--dataset", default="")
    ap.add_argument("--batch-size", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--max-steps", type=int, default=100)
    ap.add_argument("--learning-rate", type=float, default=3e-4)
    ap.add_argument("--warmup-steps", type=int, default=20)
    ap.add_argument("--weight-decay", type=float, default=0.1)
    ap.add_argument("--max-grad-norm", type=float, default=1.0)
    ap.add_argument("--progress-every", type=int, default=10)
    ap.add_argument("--checkpoint-every", type=int, default=0)
    ap.add_argument("--output-dir", default="")
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--seed", type=int, default=1337)
    ap.add_argument("--tp-size", type=int, default=0, help="--parallel tp: ranks per tensor-parallel group (0 = all); the rest is data parallel (TP x DP mesh)")
    ap.add_argument("--device", default="auto", choices=["auto", "cuda", "cpu"])
    a = ap.parse_args(argv)

    cuda = a.device == "cuda" or (a.device == "auto" and torch.cuda.is_available())
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(dev)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl" if cuda else "gloo")
    from .dp import AdamWConfig
    opt = AdamWConfig(lr=a.learning_rate, warmup_steps=a.warmup_steps, total_steps=a.max_steps, weight_decay=a.weight_decay, max_grad_norm=a.max_grad_norm)
    if a.parallel == "tp":
        from ..models.llama import LlamaConfig
        from .tp import TensorParallelContext
        from .tp_llama import TPLlama, TPLlamaTrainer
        cfg = LlamaConfig(max_seq_len=a.seq_len, vocab_pad_to=128, **MODELS[a.model])
        tp_size = a.tp_size or world
        if world > 1 and tp_size != world:
            from .tp_llama import tp_dp_mesh
            tp_group, dp_group, _t, dp_index = tp_dp_mesh(tp_size)
            model = TPLlama(cfg, TensorParallelContext(dev, tp_group), seed=a.seed, dp_group=dp_group)
            data_rank, data_world = dp_index, world // tp_size          # every tensor-parallel group reads its own batches
        else:
            model = TPLlama(cfg, TensorParallelContext(dev), seed=a.seed)
            data_rank, data_world = 0, 1
        trainer = TPLlamaTrainer(model, opt)
    else:
        from .moe_llama import EPMoELlama, FlatAdamWTrainer, MoELlamaConfig
        cfg = MoELlamaConfig(n_layer=a.n_layer, n_head=a.n_head, n_kv_head=a.n_kv_head, d_model=a.d_model, n_experts=a.experts, top_k=a.top_k,
                             expert_hidden=a.expert_hidden, vocab_size=a.vocab_size, max_seq_len=a.seq_len, score_fn=a.router_score,
                             balance_coef=a.balance_coef, router_z_coef=a.router_z_coef)
        model = EPMoELlama(cfg, dev, seed=a.seed)
        trainer = FlatAdamWTrainer(model, opt)
        data_rank, data_world = rank, world

    sampler = None
    if a.dataset:
        from ..data import TokenDataset
        ds = TokenDataset(a.dataset, allow_train_as_val=True)
        if ds.max_token("train") >= cfg.vocab_size:
            raise ValueError(f"dataset holds token id {ds.max_token('train')} but the vocabulary is {cfg.vocab_size}")
        sampler = ds.sampler("train", a.seq_len, a.batch_size, data_rank, data_world)
        batches = iter(sampler)
    else:
        gen = torch.Generator().manual_seed(a.seed + 17 * data_rank)

        def synthetic():
            while True:
                t = torch.randint(0, cfg.vocab_size, (a.batch_size, a.seq_len + 1), generator=gen)
                yield t[:, :-1], t[:, 1:]
        batches = synthetic()

    out_dir = Path(a.output_dir) if a.output_dir else None
    start = 0
    if a.resume and out_dir is not None:
        man = load_parallel_checkpoint(trainer, out_dir)
        if man is not None:
            start = int(man["step"])
            if sampler is not None:
                sampler.seek(start)
                batches = iter(sampler)
            _emit(rank, event="resumed", step=start)
    tokens_per_step = a.batch_size * a.seq_len * data_world
    t0 = last = time.perf_counter()
    loss = None
    for step in range(start + 1, a.max_steps + 1):
        tok, tgt = next(batches)
        loss = trainer.step(torch.as_tensor(tok).to(dev, non_blocking=True), torch.as_tensor(tgt).to(dev, non_blocking=True))
        if a.progress_every and (step % a.progress_every == 0 or step == a.max_steps):
            val = float(loss)  # the only host synchronisation of the loop
            now = time.perf_counter()
            n = min(a.progress_every, step - start)
            _emit(rank, event="train_step", step=step, loss=val, tokens_per_second=n * tokens_per_step / max(now - last, 1e-9),
                  grad_norm=float(trainer.clip[1]))
            last = now
        if out_dir is not None and a.checkpoint_every and (step % a.checkpoint_every == 0 or step == a.max_steps):
            _check_device_status(dev, f"checkpoint at step {step}")  # never publish a step that ran on timed-out waits
            d = save_parallel_checkpoint(trainer, out_dir, step, {"parallel": a.parallel, "config": asdict(cfg)})
            _emit(rank, event="checkpoint", step=step, path=str(d))
    if cuda:
        torch.cuda.synchronize()
    _emit(rank, event="complete", status="ok", steps=a.max_steps - start, final_loss=None if loss is None else float(loss),
          train_compute_tokens_per_second=(a.max_steps - start) * tokens_per_step / max(time.perf_counter() - t0, 1e-9), world_size=world,
          parallel=a.parallel)
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

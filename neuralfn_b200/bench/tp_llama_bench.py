"""Tensor-parallel Llama training throughput (one TP group = all ranks of the job).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        -m neuralfn_b200.bench.tp_llama_bench --model llama3_8b --batch 4 --seq 4096 --steps 5 --warmup 3 [--impl fused|nccl]

Every step is forward + backward + gradient all-reduce of the replicated tensors + clipping norm +
AdamW, on synthetic tokens and randomly initialised weights. Timed with CUDA events per rank, the
maximum over ranks is reported; rank 0 prints one JSON line. ``--impl nccl`` swaps the fused
GEMM+collective kernels for NCCL all-gather / reduce-scatter around the plain GEMM (the baseline
the fused kernels are measured against).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

MODELS = {
    "llama3_8b": dict(n_layer=32, n_head=32, n_kv_head=8, d_model=4096, d_ff=14336, vocab_size=128256, rope_theta=500000.0),
    "llama_1b": dict(n_layer=16, n_head=32, n_kv_head=8, d_model=2048, d_ff=8192, vocab_size=128256, rope_theta=500000.0),
    "tiny": dict(n_layer=2, n_head=8, n_kv_head=8, d_model=512, d_ff=2048, vocab_size=4096, rope_theta=10000.0),
}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3_8b", choices=sorted(MODELS))
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (0 = the model's own)")
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="fused", choices=["fused", "nccl"])
    a = ap.parse_args(argv)

    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from ..models.llama import LlamaConfig
    from ..ops import _lib
    from ..parallel.dp import AdamWConfig
    from ..parallel.tp import TensorParallelContext
    from ..parallel.tp_llama import TPLlama, TPLlamaTrainer

    spec = dict(MODELS[a.model])
    if a.layers:
        spec["n_layer"] = a.layers
    cfg = LlamaConfig(max_seq_len=a.seq, vocab_pad_to=128, **spec)
    tp = TensorParallelContext(dev, impl=a.impl)
    model = TPLlama(cfg, tp)
    trainer = TPLlamaTrainer(model, AdamWConfig(lr=3e-4, warmup_steps=10, total_steps=1000))
    g = torch.Generator(device=dev).manual_seed(1234)  # the same tokens on every rank
    batches = [(torch.randint(0, cfg.vocab_size, (a.batch, a.seq), device=dev, generator=g),
                torch.randint(0, cfg.vocab_size, (a.batch, a.seq), device=dev, generator=g)) for _ in range(4)]
    losses = []
    for i in range(a.warmup):
        losses.append(trainer.step(*batches[i % 4]))
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        losses.append(trainer.step(*batches[i % 4]))
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    status = _lib.status_read_reset()
    n_params = sum(s.numel for s in model.layout.order if s.decay and not s.name.startswith(("tok_", "lm_"))) * world \
        + 2 * cfg.padded_vocab * cfg.d_model
    tokens = a.batch * a.seq
    flops = 6.0 * (n_params - cfg.padded_vocab * cfg.d_model) * tokens + 12.0 * cfg.n_layer * cfg.d_model * a.seq * tokens * 0.5
    if rank == 0:
        print(json.dumps({"metric": "train_tokens_per_second", "value": round(tokens / (ms.item() / 1e3), 1), "unit": "tokens/s",
                          "ms_per_step": round(ms.item(), 3), "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "impl": a.impl,
                          "model_tflops_per_gpu": round(flops / (ms.item() / 1e3) / world / 1e12, 1), "dtype": "bf16", "data": "synthetic",
                          "loss_first": round(float(losses[0]), 4), "loss_last": round(float(losses[-1]), 4), "device_status": status,
                          "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2**30, 1),
                          "config": {"model": a.model, "layers": cfg.n_layer, "params": n_params, "global_batch": a.batch, "seq_len": a.seq,
                                     "parallelism": f"tp{world}+sp"}}), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

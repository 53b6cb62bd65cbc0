"""Tensor-parallel decode throughput: Llama shapes and the Glimmer ~29B shape (greedy, random weights, synthetic prompt).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29512 \
        -m neuralfn_b200.bench.tp_decode_bench --model llama3_8b --batch 32 --context 1024 --steps 64 --warmup 8 [--no-graph] [--impl fused|nccl]

Prefills ``context`` tokens per row, then times ``steps`` decode steps (all rows advance one token
per step) with CUDA events on every rank; the maximum over ranks is reported by rank 0 as one JSON
line. ``--impl nccl`` replaces the fused all-reduce + residual + norm kernel by an NCCL all-reduce
followed by separate element-wise kernels.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .tp_llama_bench import MODELS


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3_8b", choices=sorted(MODELS) + ["glimmer_29b", "glimmer_tiny"])
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--impl", default="fused", choices=["fused", "nccl"])
    a = ap.parse_args(argv)
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from ..models.llama import LlamaConfig
    from ..ops import _lib
    from ..parallel.tp import TensorParallelContext
    from ..serving.tp_decode import TPLlamaDecoder

    cap = a.context + a.steps + a.warmup + 8
    glimmer = a.model.startswith("glimmer")
    if glimmer:
        # the ~29B decoder shape of the Glimmer family: 48 layers, 6656 wide, 32 query / 2 KV heads of 128, gated attention,
        # sandwich norms, three 4096-token sliding-window rotary layers then one global position-free layer, SwiGLU 24576
        from ..presets_glimmer import glimmer_benchmark_shape
        from ..serving.tp_glimmer import GlimmerTPConfig, TPGlimmerDecoder
        over = dict(n_layer=a.layers) if a.layers else {}
        if a.model == "glimmer_tiny":
            cfg = GlimmerTPConfig(n_layer=a.layers or 4, d_model=1024, n_head=8, n_kv_head=2, head_dim=128, d_ff=4096, vocab_size=32000, window=256)
        else:
            cfg = GlimmerTPConfig.from_spec(glimmer_benchmark_shape(), **over)
        dec = TPGlimmerDecoder(cfg, TensorParallelContext(dev, impl=a.impl), max_batch=a.batch, max_seq=cap, use_graph=not a.no_graph)
    else:
        spec = dict(MODELS[a.model])
        if a.layers:
            spec["n_layer"] = a.layers
        cfg = LlamaConfig(max_seq_len=cap, vocab_pad_to=128, **spec)
        dec = TPLlamaDecoder(cfg, TensorParallelContext(dev, impl=a.impl), max_batch=a.batch, max_seq=cap, use_graph=not a.no_graph)
    prompt = torch.randint(0, cfg.vocab_size, (a.batch, a.context), device=dev, generator=torch.Generator(device=dev).manual_seed(7))
    e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    e[0].record()
    dec.prefill(prompt)
    e[1].record()
    for _ in range(a.warmup):
        dec.step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e[2].record()
    for _ in range(a.steps):
        dec.step()
    e[3].record()
    torch.cuda.synchronize()
    t = torch.tensor([e[2].elapsed_time(e[3]) / a.steps, e[0].elapsed_time(e[1])], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    status = _lib.status_read_reset()
    if rank == 0:
        hd = cfg.head_dim
        if glimmer:
            per_rank_weight_bytes = 2 * (cfg.n_layer * ((2 * dec.Hq + 2 * dec.Hkv) * hd * cfg.d_model + dec.Hq * hd * cfg.d_model
                                                         + 3 * dec.Fl * cfg.d_model) + dec.Vl * cfg.d_model)
            ctx_mid = a.context + a.warmup + a.steps / 2
            kv_bytes = sum(2 * 2 * dec.Hkv * hd * min(ctx_mid, c) * a.batch for c in dec.caps)
        else:
            per_rank_weight_bytes = 2 * (cfg.n_layer * ((cfg.n_head + 2 * cfg.n_kv_head) * hd * cfg.d_model + cfg.n_head * hd * cfg.d_model
                                                         + 3 * cfg.d_ff * cfg.d_model) + cfg.padded_vocab * cfg.d_model) / world
            kv_bytes = 2 * 2 * cfg.n_layer * (cfg.n_kv_head // world) * hd * (a.context + a.warmup + a.steps / 2) * a.batch
        ms = t[0].item()
        print(json.dumps({"metric": "decode_tokens_per_second", "value": round(a.batch / (ms / 1e3), 1), "unit": "tokens/s", "ms_per_step": round(ms, 4),
                          "prefill_ms": round(t[1].item(), 2),
                          "prefill_tokens_per_second": round(a.batch * a.context / (t[1].item() / 1e3), 1), "n_gpus": world, "batch": a.batch, "context": a.context, "steps": a.steps,
                          "warmup": a.warmup, "graph": not a.no_graph, "impl": a.impl, "dtype": "bf16", "data": "synthetic",
                          "hbm_gbs_per_gpu": round((per_rank_weight_bytes + kv_bytes) / (ms / 1e3) / 1e9, 1), "device_status": status,
                          "config": {"model": a.model, "layers": cfg.n_layer, "parallelism": f"tp{world}"}}), flush=True)
    dec.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

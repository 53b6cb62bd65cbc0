"""Expert-parallel MoE layer, forward + backward (router, top-k, exchange, experts, combine).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29513 \
        -m neuralfn_b200.bench.ep_moe_bench --tokens 32768 --dim 2048 --experts 64 --hidden 1024 --top-k 8 --steps 5 --warmup 3

Every rank holds ``tokens`` rows of its own and ``experts / world`` experts. A step is router GEMM
-> softmax top-k (renormalised) -> ``ExpertParallelFFN`` -> a scalar loss (mean of outputs plus the
density balance loss and the router z-loss) -> backward into x, the router and the experts. Timed
with CUDA events per rank; rank 0 prints the maximum over ranks as one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768, help="token rows per rank")
    ap.add_argument("--dim", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--exchange", choices=("peer", "nccl"), default="peer",
                    help="peer: rows travel by this framework's pull kernels over peer memory; nccl: all_to_all_single (the baseline)")
    ap.add_argument("--capacity-factor", type=float, default=2.0, help="--exchange peer: receive capacity in units of tokens * top_k")
    a = ap.parse_args(argv)
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from ..ops import _lib
    from ..parallel.ep_train import ExpertParallelFFN
    from ..tensor import kernel_bridge as KB

    layer = ExpertParallelFFN(a.dim, a.hidden, a.experts, device=dev, dtype=torch.bfloat16)
    exchange = None
    if a.exchange == "peer":
        from ..parallel.ep_fused_train import PeerExchange, fused_expert_parallel_ffn
        exchange = PeerExchange(a.experts, a.top_k, a.dim, a.tokens, dev, capacity_factor=min(a.capacity_factor, world))
    g = torch.Generator(device=dev).manual_seed(11 + rank)
    w_router = (torch.randn(a.experts, a.dim, device=dev, generator=g) * 0.02).to(torch.bfloat16).requires_grad_(True)
    x = torch.randn(a.tokens, a.dim, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)

    def step():
        for t in (x, w_router, *layer.parameters()):
            t.grad = None
        logits = KB.linear(x, w_router).float()
        scores = torch.softmax(logits, -1)
        w, idx = scores.topk(a.top_k, -1)
        w = w / w.sum(-1, keepdim=True)
        y = fused_expert_parallel_ffn(x, w, idx, layer.w1, layer.w2, layer.w3, exchange) if exchange is not None else layer(x, w, idx)
        balance = a.experts * scores.mean(0).pow(2).sum()
        zloss = torch.logsumexp(logits, -1).pow(2).mean()
        loss = y.float().mean() + 0.01 * balance + 1e-3 * zloss
        loss.backward()
        return loss

    for _ in range(a.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    status = _lib.status_read_reset()
    if rank == 0:
        flops = 3 * 2.0 * a.tokens * a.top_k * 3 * a.dim * a.hidden  # fwd + 2x bwd of the three expert products, per rank
        sec = ms.item() / 1e3
        print(json.dumps({"metric": "moe_layer_train_tokens_per_second", "value": round(a.tokens * world / sec, 1), "unit": "tokens/s",
                          "ms_per_step": round(ms.item(), 3), "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "dtype": "bf16",
                          "expert_tflops_per_gpu": round(flops / sec / 1e12, 1), "loss": round(float(loss), 5), "device_status": status, "exchange": a.exchange,
                          "row_bytes_exchanged_per_gpu_per_step": 4 * a.tokens * a.top_k * a.dim * 2 * (world - 1) // max(world, 1),
                          "config": {"tokens_per_gpu": a.tokens, "d_model": a.dim, "experts": a.experts, "expert_hidden": a.hidden,
                                     "top_k": a.top_k, "parallelism": f"ep{world}"}}), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

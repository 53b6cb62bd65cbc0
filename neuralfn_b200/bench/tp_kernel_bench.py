"""Stand-alone timing of the fused compute + collective kernels at the per-rank shapes of a tensor-parallel
Llama-3-8B step, against their library pairing and against a roofline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29517 \
        -m neuralfn_b200.bench.tp_kernel_bench --tokens 16384 --iters 20

Cases (world W, sequence-parallel rows M / W per rank, d = 4096, ffn 14336):

* ``ag_gemm``   all-gather of the activations -> GEMM with a column-parallel weight (QKV and gate|up shapes);
* ``gemm_rs``   GEMM with a row-parallel weight -> reduce-scatter (attention output and down shapes);
* ``allreduce`` the decode-sized all-reduce + residual + RMS norm (32 x 4096 rows), peer loads and multimem.

Each case runs ``iters`` times per implementation (``fused``: one kernel over peer memory; ``nccl``: the NCCL
collective and this framework's GEMM as two launches), timed with CUDA events on the launching stream
after warm-up, maximum over ranks. The roofline time of a case is the larger of FLOPs / the measured GEMM
peak and the bytes every GPU must receive over NVLink / the measured peer-copy rate (770 GB/s per
direction); ``roofline_fraction`` is that time over the measured one. The GEMM operands of a case (64 - 470 MB with
the output) are re-used between iterations. The all-reduce is timed twice: as eager calls (host-paced) and as 16 calls on
two alternating buffers inside a replayed CUDA graph, which is how a decode step issues it.

The reference has no tensor parallelism; the shapes are those of its Llama-3-8B template
(``neuralfn/config.py`` ``llama3_8b`` geometry: d 4096, 32 / 8 heads, ffn 14336).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0      # measured peer copy, per direction per GPU


def _time(fn, iters: int, warmup: int, dev) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(dev)
    if dist.is_initialized():
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize(dev)
    t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384, help="rows of the whole group (sequence-parallel: tokens / W per rank)")
    ap.add_argument("--dim", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--kv-dim", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--peak-tflops", type=float, default=0.0, help="GEMM peak for the roofline (default: MEASURED_PEAKS.json, else 1590)")
    a = ap.parse_args(argv)
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from ..ops import _lib
    from ..parallel.tp import TensorParallelContext
    peak = a.peak_tflops
    if not peak:
        try:
            here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
            peak = float(json.load(open(os.path.join(here, "MEASURED_PEAKS.json")))["bf16_tflops"])
        except Exception:
            peak = 1590.0
    bf = torch.bfloat16
    M, d, W = a.tokens, a.dim, world
    rows = M // W
    g = torch.Generator(device=dev).manual_seed(3 + rank)
    rnd = lambda *s: (torch.randn(*s, device=dev, generator=g) * 0.05).to(bf)  # noqa: E731
    results = []

    def record(case, shape, impl, ms, flops, link_bytes):
        t_flops, t_link = flops / (peak * 1e12), link_bytes / (NVLINK_GBS * 1e9)
        roof = max(t_flops, t_link)
        results.append({"case": case, "shape": shape, "impl": impl, "ms": round(ms, 4), "tflops_per_gpu": round(flops / ms / 1e9, 1),
                        "nvlink_gbs_in": round(link_bytes / ms / 1e6, 1), "roofline_ms": round(roof * 1e3, 4),
                        "bound": "gemm" if t_flops >= t_link else "nvlink", "roofline_fraction": round(roof * 1e3 / ms, 3)})

    for impl in ("fused", "nccl"):
        ctx = TensorParallelContext(dev, impl=impl)
        # all-gather -> GEMM: x_local [rows, d], weight [N / W, d]
        for name, n_full in (("qkv", d + 2 * a.kv_dim), ("gate_up", 2 * a.ffn)):
            nl = n_full // W // 8 * 8
            x, w = rnd(rows, d), rnd(nl, d)
            ms = _time(lambda: ctx.column_linear(x, w), a.iters, a.warmup, dev)
            record("ag_gemm", f"{name}: {M}x{nl}x{d}", impl, ms, 2.0 * M * nl * d, (W - 1) * rows * d * 2)
        # GEMM -> reduce-scatter: x [M, K / W], weight [d, K / W]
        for name, k_full in (("attn_out", d), ("down", a.ffn)):
            kl = k_full // W // 8 * 8
            x, w = rnd(M, kl), rnd(d, kl)
            ms = _time(lambda: ctx.row_linear(x, w), a.iters, a.warmup, dev)
            record("gemm_rs", f"{name}: {M}x{d}x{kl}", impl, ms, 2.0 * M * d * kl, (W - 1) * rows * d * 2)
        # decode all-reduce + residual + RMS norm
        B = 32
        resid, nw = rnd(B, d), rnd(d)
        variants = (("peer", False), ("multimem", True)) if impl == "fused" else (("nccl", False),)
        for vname, mc in variants:
            if impl == "fused":
                part, sym = ctx.partial_buffer(B, d)
                part.copy_(rnd(B, d))
            else:
                part, sym = rnd(B, d), None
            ms = _time(lambda: ctx.allreduce_resid_norm(part, sym, resid=resid, norm_weight=nw, use_multicast=mc), a.iters * 10, a.warmup, dev)
            record("allreduce_resid_norm", f"{B}x{d}", vname, ms, 0.0, (W - 1) * B * d * 2)
            if impl == "fused":
                # the same call as a decode step issues it: K calls on two alternating buffers inside one CUDA graph, replayed
                # (no host work between launches); the device-side epoch moves on by K before every replay
                Kc = 16
                part2, sym2 = ctx.partial_buffer(B, d)
                part2.copy_(part)
                bufs = ((part, sym), (part2, sym2))

                def body():
                    for i in range(Kc):
                        ctx.allreduce_resid_norm(*bufs[i % 2], resid=resid, norm_weight=nw, use_multicast=mc)
                body()
                torch.cuda.synchronize(dev)
                side = torch.cuda.Stream(dev)
                side.wait_stream(torch.cuda.current_stream(dev))
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.stream(side):
                    with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                        body()
                torch.cuda.current_stream(dev).wait_stream(side)
                ctx.advance_epoch_on_device(-Kc)              # capture advanced the host epoch without running anything

                def replay():
                    ctx.advance_epoch_on_device(Kc)
                    graph.replay()
                ms = _time(replay, a.iters, a.warmup, dev) / Kc
                record("allreduce_resid_norm", f"{B}x{d} (in a CUDA graph, per call)", vname, ms, 0.0, (W - 1) * B * d * 2)
                # where the time goes inside one launch: device-side timestamps of CTA 0 (signal, peers arrived, rows done, end)
                import ctypes
                stamps = torch.zeros(5, dtype=torch.int64, device=dev)
                lib = _lib.load()
                lib.nfn_allreduce_set_trace(ctypes.c_void_p(stamps.data_ptr()))
                phases = torch.zeros(4, dtype=torch.float64)
                n_tr = 20
                for i in range(n_tr):
                    if world > 1:
                        dist.barrier()
                    ctx.allreduce_resid_norm(*bufs[i % 2], resid=resid, norm_weight=nw, use_multicast=mc)
                    torch.cuda.synchronize(dev)
                    t = stamps.cpu().double()
                    phases += (t[1:] - t[:-1]) / n_tr
                lib.nfn_allreduce_set_trace(ctypes.c_void_p(0))
                results[-1]["phases_us"] = {k: round(float(v) / 1e3, 2) for k, v in zip(("signal", "wait_for_peers", "rows", "tail"), phases)}
    torch.cuda.synchronize(dev)
    status = _lib.status_read_reset()
    if rank == 0:
        print(json.dumps({"bench": "tp_kernels", "n_gpus": W, "gemm_peak_tflops": peak, "nvlink_gbs_per_direction": NVLINK_GBS,
                          "device_status": status, "iters": a.iters, "results": results}), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

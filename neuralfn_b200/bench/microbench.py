"""Isolated kernel timing harness (CUDA events, L2 flushed between iterations).

    python -m neuralfn_b200.bench.microbench gemm --m 16384 --n 2304 --k 768
    python -m neuralfn_b200.bench.microbench attention_fwd --batch 16 --heads 12 --seq 1024 --head-dim 64
    python -m neuralfn_b200.bench.microbench all            # the shapes of the GPT-2 124M step

Each case prints one JSON line: median milliseconds over ``--iters`` timed launches (after
``--warmup``), achieved TFLOP/s or GB/s from the algorithmic work, and - when ``--peak-tflops``
/ ``--peak-gbs`` are given - the fraction of that peak. Counterpart of the reference's
``linear_backward_bench.cpp`` / ``lm_head_backward_bench.cpp`` harnesses.
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys

import torch


def _flush_buffer(dev):
    return torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device=dev)  # larger than the 126 MB L2


def time_kernel(fn, iters: int, warmup: int, flush) -> float:
    for _ in range(max(3, warmup)):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush.zero_()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        stop.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(stop))
    return statistics.median(times)


def _report(name, ms, *, flops=0.0, bytes_=0.0, args=None, extra=None):
    out = {"kernel": name, "ms": round(ms, 5)}
    if flops:
        out["tflops"] = round(flops / ms / 1e9, 2)
        if args.peak_tflops:
            out["frac_of_peak_tflops"] = round(out["tflops"] / args.peak_tflops, 3)
    if bytes_:
        out["gbs"] = round(bytes_ / ms / 1e6, 1)
        if args.peak_gbs:
            out["frac_of_peak_gbs"] = round(out["gbs"] / args.peak_gbs, 3)
    out.update(extra or {})
    print(json.dumps(out), flush=True)
    return out


def case_gemm(args, m=None, n=None, k=None, a_mn=False, b_mn=False, tag="gemm"):
    from neuralfn_b200.ops.gemm import gemm
    dev = torch.device("cuda")
    m, n, k = m or args.m, n or args.n, k or args.k
    a = torch.randn((k, m) if a_mn else (m, k), device=dev).bfloat16()
    b = torch.randn((k, n) if b_mn else (n, k), device=dev).bfloat16()
    out = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
    ws = torch.empty(32 * 1024 * 1024, device=dev, dtype=torch.float32) if (a_mn or m <= 256) else None  # split-K: weight gradients, skinny decode products
    if getattr(args, "skinny_impl", -1) >= 0:
        from neuralfn_b200.ops import _lib
        _lib.load().nfn_gemm_skinny_set_impl(int(args.skinny_impl))
    ms = time_kernel(lambda: gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, workspace=ws), args.iters, args.warmup, args.flush)
    return _report(tag, ms, flops=2.0 * m * n * k, bytes_=2.0 * (m * k + n * k + m * n), args=args,
                   extra={"m": m, "n": n, "k": k, "a_mn": a_mn, "b_mn": b_mn})


def case_skinny(args):
    """Decode-sized products of a Glimmer 29B layer at TP 4 (32 rows): the mma.sync weight-streaming kernel against the tcgen05
    split-K path, as fractions of the copy bandwidth."""
    from neuralfn_b200.ops import _lib
    from neuralfn_b200.ops.gemm import gemm
    dev = torch.device("cuda")
    L = _lib.load()
    ws = torch.empty(32 * 1024 * 1024, device=dev, dtype=torch.float32)
    out = []
    for m, n, k in ((32, 2304, 6656), (32, 6656, 1024), (32, 12288, 6656), (32, 6656, 6144), (8, 12288, 6656), (64, 12288, 6656), (32, 4096, 4096)):
        a = torch.randn(m, k, device=dev).bfloat16()
        w = torch.randn(n, k, device=dev).bfloat16()
        c = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
        for impl in ((3, 2, 0) if m <= 32 else (2, 0)):
            old = L.nfn_gemm_skinny_set_impl(impl)
            ms = time_kernel(lambda: gemm(a, w, out=c, workspace=ws), args.iters, args.warmup, args.flush)  # L2 flushed between calls
            L.nfn_gemm_skinny_set_impl(old)
            out.append(_report({3: "skinny_mma_resident_cluster", 2: "skinny_mma", 0: "skinny_tcgen05_splitk"}[impl], ms, flops=2.0 * m * n * k, bytes_=2.0 * (n * k + m * k + m * n), args=args,
                               extra={"m": m, "n": n, "k": k}))
    return out


def case_grouped_k(args):
    """Weight gradients of all experts of an MoE layer (d = --k columns of the token buffer, hidden --n, --experts experts, --m rows
    in the expert-sorted buffer, split unevenly): one grouped launch against one TN GEMM per expert."""
    from neuralfn_b200.ops.gemm import gemm, gemm_grouped_k
    dev = torch.device("cuda")
    E, rows_total, d, h = args.experts, args.m, args.k, args.n
    g = torch.Generator(device=dev).manual_seed(0)
    w = torch.rand(E, device=dev, generator=g) + 0.2
    counts = (w / w.sum() * rows_total * 0.97).int().tolist()
    offs = [0]
    for c in counts:
        offs.append(offs[-1] + (c + 127) // 128 * 128)
    xs = torch.zeros(offs[-1], d, device=dev, dtype=torch.bfloat16)
    dh = (torch.randn(offs[-1], h, device=dev, generator=g) * 0.1).bfloat16()
    for e, c in enumerate(counts):
        xs[offs[e]:offs[e] + c] = (torch.randn(c, d, device=dev, generator=g) * 0.1).bfloat16()
    group_rows = torch.tensor(offs, device=dev, dtype=torch.int32)
    dw = torch.empty(E, d, h, device=dev, dtype=torch.bfloat16)
    flops = 2.0 * sum(counts) * d * h

    def loop():
        for e, c in enumerate(counts):
            gemm(xs[offs[e]:offs[e] + c], dh[offs[e]:offs[e] + c], a_mn=True, b_mn=True, out=dw[e])
    extra = {"experts": E, "rows": offs[-1], "d": d, "h": h}
    out = [_report("grouped_k", time_kernel(lambda: gemm_grouped_k(xs, dh, group_rows, dw), args.iters, args.warmup, args.flush), flops=flops, args=args, extra=extra)]
    if not args.no_baseline:
        out.append(_report("per_expert_loop", time_kernel(loop, args.iters, args.warmup, args.flush), flops=flops, args=args, extra=extra))
    return out


def case_attention(args, backward=False):
    from neuralfn_b200.ops import kernels as K
    dev = torch.device("cuda")
    B, H, T, D = args.batch, args.heads, args.seq, args.head_dim
    Hkv = args.kv_heads or H
    q = torch.randn(B * T, H * D, device=dev).bfloat16()
    k = torch.randn(B * T, Hkv * D, device=dev).bfloat16()
    v = torch.randn(B * T, Hkv * D, device=dev).bfloat16()
    o, lse = K.attention_forward(q, k, v, B=B, T=T, n_q_heads=H, n_kv_heads=Hkv, head_dim=D, causal=True)
    flops = 4.0 * B * H * T * T * D / 2  # causal
    if not backward:
        ms = time_kernel(lambda: K.attention_forward(q, k, v, B=B, T=T, n_q_heads=H, n_kv_heads=Hkv, head_dim=D, causal=True, out=o, lse=lse),
                         args.iters, args.warmup, args.flush)
        return _report("attention_fwd", ms, flops=flops, args=args, extra={"B": B, "H": H, "Hkv": Hkv, "T": T, "D": D})
    do = torch.randn_like(o)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    delta = torch.empty(B, H, T, device=dev)
    acc = torch.empty(B * T, H * D, device=dev)
    ms = time_kernel(lambda: K.attention_backward(do, q, k, v, o, lse, B=B, T=T, n_q_heads=H, n_kv_heads=Hkv, head_dim=D, causal=True,
                                                  dq=dq, dk=dk, dv=dv, delta=delta, dq_accum=acc), args.iters, args.warmup, args.flush)
    return _report("attention_bwd", ms, flops=2.5 * flops, args=args, extra={"B": B, "H": H, "Hkv": Hkv, "T": T, "D": D})


def case_cross_entropy(args):
    from neuralfn_b200.ops import kernels as K
    dev = torch.device("cuda")
    rows, V = args.batch * args.seq, args.vocab
    Vp = (V + 127) // 128 * 128
    src = torch.randn(rows, Vp, device=dev).bfloat16()
    logits = torch.empty_like(src)
    tgt = torch.randint(0, V, (rows,), device=dev, dtype=torch.int32)
    row_loss, mean = torch.empty(rows, device=dev), torch.zeros(1, device=dev)

    def run():
        logits.copy_(src)  # the kernel overwrites logits with gradients
        K.cross_entropy(logits, tgt, vocab=V, cap=30.0, z_coef=1e-4, grad_scale=1.0 / rows, loss_scale=1.0 / rows, write_grad=True,
                        row_loss=row_loss, mean_loss=mean)

    copy_ms = time_kernel(lambda: logits.copy_(src), args.iters, args.warmup, args.flush)
    ms = time_kernel(run, args.iters, args.warmup, args.flush) - copy_ms
    return _report("cross_entropy_fwd_bwd", ms, bytes_=2.0 * rows * Vp * 2, args=args, extra={"rows": rows, "vocab": V})


def case_norm(args):
    from neuralfn_b200.ops import kernels as K
    dev = torch.device("cuda")
    rows, C = args.batch * args.seq, args.k
    x = torch.randn(rows, C, device=dev).bfloat16()
    w, b = torch.ones(C, device=dev).bfloat16(), torch.zeros(C, device=dev).bfloat16()
    y, mean, rstd = torch.empty_like(x), torch.empty(rows, device=dev), torch.empty(rows, device=dev)
    ms = time_kernel(lambda: K.norm_forward(x, w, b, eps=1e-5, mode=K.NORM_LAYER, out=y, mean=mean, rstd=rstd), args.iters, args.warmup, args.flush)
    return _report("layernorm_fwd", ms, bytes_=2.0 * rows * C * 2, args=args, extra={"rows": rows, "C": C})


def case_adamw(args):
    from neuralfn_b200.ops import kernels as K
    dev = torch.device("cuda")
    n = args.params
    master, m, v = (torch.zeros(n, device=dev) for _ in range(3))
    grads = torch.randn(n, device=dev).bfloat16()
    params = torch.empty(n, device=dev, dtype=torch.bfloat16)
    hyper = torch.zeros(K.HYPER_SIZE, device=dev)
    hyper[K.HP_LR], hyper[K.HP_BETA1], hyper[K.HP_BETA2], hyper[K.HP_EPS] = 1e-3, 0.9, 0.95, 1e-8
    hyper[K.HP_BC1], hyper[K.HP_BC2], hyper[K.HP_GRAD_SCALE], hyper[K.HP_MAX_NORM] = 0.1, 0.05, 1.0, 0.0
    clip = torch.ones(2, device=dev)
    ms = time_kernel(lambda: K.adamw_flat(master, m, v, grads, params, n, hyper, clip), args.iters, args.warmup, args.flush)
    return _report("adamw_flat", ms, bytes_=n * (3 * 4 * 2 + 2 + 2.0), args=args, extra={"params": n})


def case_decode_attention(args):
    from neuralfn_b200.ops import infer as I
    dev = torch.device("cuda")
    B, Hq, Hkv, D, ctx = args.batch, args.heads, args.kv_heads or 1, args.head_dim, args.seq
    kc = torch.randn(B, Hkv, ctx, D, device=dev).bfloat16()
    vc = torch.randn(B, Hkv, ctx, D, device=dev).bfloat16()
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, device=dev).bfloat16()
    lengths = torch.full((B,), ctx, dtype=torch.int32, device=dev)
    ws = I.DecodeAttentionWorkspace(B, Hq, Hkv, D, dev)
    cos, sin = I.rope_tables(ctx, D, device=dev)
    out = torch.empty(B, Hq * D, device=dev, dtype=torch.bfloat16)
    ms = time_kernel(lambda: I.decode_attention(qkv, kc, vc, lengths, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=D, workspace=ws, cos=cos,
                                                sin=sin, qk_norm=True, out=out), args.iters, args.warmup, args.flush)
    return _report("decode_attention", ms, bytes_=2.0 * B * Hkv * ctx * D * 2, args=args, extra={"B": B, "Hq": Hq, "Hkv": Hkv, "ctx": ctx, "D": D})


def case_kquant_gemv(args):
    from neuralfn_b200.ops import infer as I
    from neuralfn_b200.quant import kquant
    dev = torch.device("cuda")
    N, Kd, B = args.n, args.k, min(args.batch, 8)
    raw = torch.from_numpy(kquant.random_blocks(12, N * Kd // 256, seed=0)).to(dev).reshape(-1)
    x = torch.randn(B, Kd, device=dev).bfloat16()
    out = torch.empty(B, N, device=dev, dtype=torch.bfloat16)
    ms = time_kernel(lambda: I.kquant_gemv(12, raw, x, N, out=out), args.iters, args.warmup, args.flush)
    return _report("q4_k_gemv", ms, bytes_=float(raw.numel()), flops=2.0 * B * N * Kd, args=args, extra={"B": B, "N": N, "K": Kd})



def case_gemm_kquant(args):
    """Prefill product over Q4_K weights, dequantisation fused into the GEMM pipeline, against the
    two-step path (dequantise to bf16, then the bf16 GEMM)."""
    from neuralfn_b200.ops import infer as I
    from neuralfn_b200.ops.gemm import gemm
    from neuralfn_b200.quant import kquant
    dev = torch.device("cuda")
    M, N, Kd = args.m, args.n, args.k
    raw = torch.from_numpy(kquant.random_blocks(12, N * Kd // 256, seed=0)).to(dev).reshape(-1)
    x = torch.randn(M, Kd, device=dev).bfloat16()
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    wbuf = torch.empty(N * Kd, device=dev, dtype=torch.bfloat16)
    ms = time_kernel(lambda: I.gemm_kquant(12, x, raw, N, out=out), args.iters, args.warmup, args.flush)
    two = time_kernel(lambda: gemm(x, I.dequant_kquant(12, raw, out=wbuf).view(N, Kd), out=out), args.iters, args.warmup, args.flush)
    return _report("q4_k_gemm_fused_dequant", ms, bytes_=float(raw.numel()) + 2.0 * M * (Kd + N), flops=2.0 * M * N * Kd, args=args,
                   extra={"m": M, "n": N, "k": Kd, "two_step_ms": round(two, 5)})


def case_block_attention(args):
    """Speculative verification block (16 rows per sequence) against a bf16 KV cache."""
    from neuralfn_b200.ops import infer as I
    dev = torch.device("cuda")
    B, Hq, Hkv, D, ctx, R = args.batch, args.heads, args.kv_heads or 1, args.head_dim, args.seq, 16
    kc = torch.randn(B, Hkv, ctx + 128, D, device=dev).bfloat16()
    vc = torch.randn(B, Hkv, ctx + 128, D, device=dev).bfloat16()
    qkv = torch.randn(B * R, (Hq + 2 * Hkv) * D, device=dev).bfloat16()
    lengths = torch.full((B,), ctx, dtype=torch.int32, device=dev)
    ws = I.BlockAttentionWorkspace(B, R, Hq, Hkv, D, dev)
    out = torch.empty(B * R, Hq * D, device=dev, dtype=torch.bfloat16)
    ms = time_kernel(lambda: I.block_attention(qkv, kc, vc, lengths, rows=R, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=D, workspace=ws, out=out),
                     args.iters, args.warmup, args.flush)
    return _report("block_attention_16_rows", ms, bytes_=2.0 * B * Hkv * ctx * D * 2, flops=4.0 * B * Hq * R * ctx * D, args=args,
                   extra={"B": B, "Hq": Hq, "Hkv": Hkv, "ctx": ctx, "D": D, "rows": R})


def case_turboquant_attention(args):
    """Decode attention over TurboQuant records (3.5 bits per coordinate)."""
    from neuralfn_b200.quant.turboquant import TurboQuantCodec, TurboQuantKVCache, default_outlier_indices
    dev = torch.device("cuda")
    B, Hq, Hkv, D, ctx = args.batch, args.heads, args.kv_heads or 1, args.head_dim, args.seq
    codec = TurboQuantCodec(D, profile="mse-3.5", seed=0, outlier_indices=default_outlier_indices(D))
    cache = TurboQuantKVCache(codec, B, Hkv, ctx, dev)
    cache.k.copy_(torch.randint(0, 255, cache.k.shape, dtype=torch.uint8, device=dev))
    cache.v.copy_(torch.randint(0, 255, cache.v.shape, dtype=torch.uint8, device=dev))
    cache.k.view(torch.float32)[..., 0] = 1.0  # finite norms
    cache.v.view(torch.float32)[..., 0] = 1.0
    cache._len_host = [ctx] * B
    cache.lengths.fill_(ctx)
    q = torch.randn(B, Hq * D, device=dev).bfloat16()
    ms = time_kernel(lambda: cache.attention(q, Hq), args.iters, args.warmup, args.flush)
    return _report("turboquant_decode_attention", ms, bytes_=float(B * ctx * cache.bytes_per_token), args=args,
                   extra={"B": B, "Hq": Hq, "Hkv": Hkv, "ctx": ctx, "D": D, "bytes_per_token": cache.bytes_per_token})



def case_engine_decode(args):
    """Resident-engine decode throughput on Llama-3-8B layer shapes (8 of the 32 layers, so that the
    weights stay a few GB): tokens/s for the whole batch and the weight bytes streamed per second."""
    import time

    from neuralfn_b200.serving import EngineConfig, ResidentEngine
    L, d, Hq, Hkv, hd, F, V = 8, 4096, 32, 8, 128, 14336, 32000
    B, ctx = max(1, args.batch), args.seq
    cfg = EngineConfig(family=1, n_layer=L, d_model=d, n_head=Hq, n_kv_head=Hkv, head_dim=hd, d_ff=F, vocab=V, padded_vocab=V,
                       max_seq=ctx + 80, max_batch=B, qk_norm=0, rope_hf=1, rope_theta=500000.0, norm_eps=1e-5, tie_embeddings=0)
    eng = ResidentEngine(cfg)
    g = torch.Generator().manual_seed(0)
    w = {n: (torch.ones(k) if n.endswith("norm") else torch.randn(k, generator=g) * 0.02).bfloat16() for n, k in eng.expected_tensors().items()}
    eng.load_named_tensors(w)
    weight_bytes = 2 * sum(k for n, k in eng.expected_tensors().items() if n != "tok_embeddings")
    prompt = torch.randint(0, V, (ctx,), generator=g).tolist()
    last = {b: eng.prefill(b, prompt) for b in range(B)}
    for _ in range(8):
        last = eng.decode(last)
    torch.cuda.synchronize()
    steps = 48
    t0 = time.perf_counter()
    for _ in range(steps):
        last = eng.decode(last)
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / steps
    return _report("engine_decode_llama8b_shape_8_layers", dt * 1e3, bytes_=float(weight_bytes), args=args,
                   extra={"batch": B, "context": ctx, "tokens_per_second": round(B / dt, 1), "ms_per_step": round(dt * 1e3, 3),
                          "kernel_launches_per_step": eng.launches // (steps + 8 + B) if hasattr(eng, "launches") else None})


CASES = {"gemm": case_gemm, "attention_fwd": case_attention, "attention_bwd": lambda a: case_attention(a, True),
         "cross_entropy": case_cross_entropy, "norm": case_norm, "adamw": case_adamw, "decode_attention": case_decode_attention,
         "skinny": case_skinny, "grouped_k": case_grouped_k, "kquant_gemv": case_kquant_gemv, "gemm_kquant": case_gemm_kquant, "block_attention": case_block_attention,
         "turboquant_attention": case_turboquant_attention, "engine_decode": case_engine_decode}


def run_all(args):
    M = 16 * 1024
    res = []
    for (n, k) in ((2304, 768), (768, 768), (3072, 768), (768, 3072), (50304, 768)):
        res.append(case_gemm(args, M, n, k, tag="gemm_fwd"))
    for (n, k) in ((768, 2304), (768, 3072), (3072, 768)):
        res.append(case_gemm(args, M, n, k, b_mn=True, tag="gemm_dx"))
    for (m, n) in ((2304, 768), (3072, 768), (768, 3072), (50304, 768)):
        res.append(case_gemm(args, m, n, M, a_mn=True, b_mn=True, tag="gemm_dw"))
    res.append(case_attention(args))
    res.append(case_attention(args, True))
    res.append(case_cross_entropy(args))
    res.append(case_norm(args))
    res.append(case_adamw(args))
    return res


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case", choices=sorted(CASES) + ["all"])
    ap.add_argument("--m", type=int, default=16384)
    ap.add_argument("--n", type=int, default=2304)
    ap.add_argument("--k", type=int, default=768)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--kv-heads", type=int, default=0)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--vocab", type=int, default=50257)
    ap.add_argument("--params", type=int, default=124 * 1000 * 1000)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--experts", type=int, default=16, help="grouped_k case")
    ap.add_argument("--no-baseline", action="store_true", help="grouped_k case: skip the per-expert loop (profiler captures)")
    ap.add_argument("--skinny-impl", type=int, default=-1, help="gemm case: nfn_gemm_skinny_set_impl mode for products with 3 - 64 rows (-1: the default)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--peak-tflops", type=float, default=0.0, help="measured bf16 GEMM peak to report fractions against")
    ap.add_argument("--peak-gbs", type=float, default=0.0, help="measured HBM copy bandwidth to report fractions against")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("microbench needs a CUDA device", file=sys.stderr)
        return 2
    args.flush = _flush_buffer(torch.device("cuda"))
    if args.case == "all":
        run_all(args)
    else:
        CASES[args.case](args)
    from neuralfn_b200.ops import _lib
    _lib.assert_status_ok("microbench")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

"""Tensor-parallel linears: host logic on gloo ranks (CPU), the fused kernel with a single
rank (one GPU), and fused vs oracle across two GPUs (skipped with fewer than two)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _full_problem(world, rows, K, N, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(world * rows, K, generator=g) * 0.5
    w = torch.randn(N, K, generator=g) * 0.05
    b = torch.randn(N, generator=g) * 0.1
    return x, w, b


def _worker(rank, world, port, backend, impl, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group(backend, rank=rank, world_size=world)
    try:
        from neuralfn_b200.parallel.tp import TensorParallelContext
        dev = torch.device("cuda", rank) if backend == "nccl" else torch.device("cpu")
        if backend == "nccl":
            torch.cuda.set_device(dev)
        dt = torch.bfloat16 if backend == "nccl" else torch.float32
        ctx = TensorParallelContext(dev, impl=impl)
        rows, K, N = 256, 512, 768
        x, w, b = _full_problem(world, rows, K, N)
        errs = {}
        # column-parallel: sequence-sharded x, weight rows split across ranks
        nl = N // world
        xl = x[rank * rows:(rank + 1) * rows].to(dev, dt)
        wl = w[rank * nl:(rank + 1) * nl].to(dev, dt).contiguous()
        bl = b[rank * nl:(rank + 1) * nl].to(dev, dt).contiguous()
        for rep in range(3):  # repeated calls exercise epochs and buffer alternation
            y = ctx.column_linear(xl, wl, bias=bl, act="gelu")
        ref = torch.nn.functional.gelu(x @ w[rank * nl:(rank + 1) * nl].T + b[rank * nl:(rank + 1) * nl], approximate="tanh")
        errs["column"] = float((y.float().cpu() - ref).abs().max())
        # sharded weight gathered into the GEMM
        y = ctx.gathered_weight_linear(x[:384].to(dev, dt), wl, bias=b.to(dev, dt))
        errs["gathered_weight"] = float((y.float().cpu() - (x[:384] @ w.T + b)).abs().max())
        # row-parallel: K split across ranks, output rows scattered
        kl = K // world
        xk = x[:, rank * kl:(rank + 1) * kl].to(dev, dt).contiguous()
        wk = w[:, rank * kl:(rank + 1) * kl].to(dev, dt).contiguous()
        resid = x[rank * rows:(rank + 1) * rows, :N] if N <= K else torch.zeros(rows, N)
        resid = torch.randn(rows, N, generator=torch.Generator().manual_seed(5 + rank))
        for rep in range(3):
            y = ctx.row_linear(xk, wk, bias=b.to(dev, dt), resid=resid.to(dev, dt))
        ref = (x @ w.T + b)[rank * rows:(rank + 1) * rows] + resid
        errs["row"] = float((y.float().cpu() - ref).abs().max())
        # decode-sized all-reduce + residual + RMS norm (plain peer loads, then multicast if offered)
        B, Nd = 32, 1664
        parts = [torch.randn(B, Nd, generator=torch.Generator().manual_seed(20 + r)) for r in range(world)]
        res0 = torch.randn(B, Nd, generator=torch.Generator().manual_seed(40))
        nw = 1 + 0.1 * torch.randn(Nd, generator=torch.Generator().manual_seed(41))
        total = sum(p.to(dt).float() for p in parts) + res0.to(dt).float()
        total = total.to(dt).float()
        ref = total * torch.rsqrt(total.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.to(dt).float()
        for it, mc in enumerate((False, True, False)):
            if impl == "fused":
                buf, sym = ctx.partial_buffer(B, Nd)
                buf.copy_(parts[rank].to(dev, dt))
            else:
                buf, sym = parts[rank].to(dev, dt), None
            resid = res0.to(dev, dt).clone()
            y = ctx.allreduce_resid_norm(buf, sym, resid=resid, norm_weight=nw.to(dev, dt), use_multicast=mc)
            errs[f"allreduce{it}"] = max(float((y.float().cpu() - ref).abs().max()), float((resid.float().cpu() - total).abs().max()))
        if backend == "nccl":
            torch.cuda.synchronize()
            from neuralfn_b200.ops import _lib
            errs["status"] = _lib.status_read_reset()
        out_q.put((rank, errs))
    finally:
        dist.destroy_process_group()


def _run(world, backend, impl):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, backend, impl, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return dict(results)


def test_torch_impl_on_two_gloo_ranks():
    res = _run(2, "gloo", "torch")
    for rank, errs in res.items():
        assert errs["column"] < 1e-4 and errs["gathered_weight"] < 1e-4 and errs["row"] < 1e-4, (rank, errs)
        assert max(errs[f"allreduce{i}"] for i in range(3)) < 1e-4, (rank, errs)


@pytest.mark.gpu
@pytest.mark.parametrize("impl", ["fused", "nccl"])
def test_single_rank_paths_on_one_gpu(impl):
    from neuralfn_b200.ops import _lib
    from neuralfn_b200.parallel.tp import TensorParallelContext
    dev = torch.device("cuda", 0)
    ctx = TensorParallelContext(dev, impl=impl)
    x, w, b = _full_problem(1, 384, 512, 2304, seed=3)
    xd, wd, bd = x.to(dev).bfloat16(), w.to(dev).bfloat16(), b.to(dev).bfloat16()
    ref = xd.float() @ wd.float().T + bd.float()
    y = ctx.column_linear(xd, wd, bias=bd, act="silu")
    torch.testing.assert_close(y.float(), torch.nn.functional.silu(ref), atol=3e-2, rtol=3e-2)
    y = ctx.gathered_weight_linear(xd, wd, bias=bd)
    torch.testing.assert_close(y.float(), ref, atol=3e-2, rtol=3e-2)
    resid = torch.randn(384, 2304, device=dev).bfloat16()
    for _ in range(2):
        y = ctx.row_linear(xd, wd, bias=bd, resid=resid)
    torch.testing.assert_close(y.float(), ref + resid.float(), atol=5e-2, rtol=3e-2)
    if impl == "fused":
        buf, sym = ctx.partial_buffer(32, 6656)
        buf.copy_(torch.randn(32, 6656, device=dev))
        r0 = torch.randn(32, 6656, device=dev).bfloat16()
        resid = r0.clone()
        nw = (0.1 * torch.randn(6656, device=dev)).bfloat16()
        y = ctx.allreduce_resid_norm(buf, sym, bias=None, resid=resid, norm_weight=nw, centered=True)
        tot = (buf.float() + r0.float()).bfloat16().float()
        torch.testing.assert_close(resid.float(), tot, atol=0, rtol=0)
        ref = tot * torch.rsqrt(tot.pow(2).mean(-1, keepdim=True) + 1e-6) * (1 + nw.float())
        torch.testing.assert_close(y.float(), ref, atol=3e-2, rtol=2e-2)
    torch.cuda.synchronize()
    assert _lib.status_read_reset() == 0


@pytest.mark.gpu
def test_fused_matches_oracle_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    res = _run(2, "nccl", "fused")
    for rank, errs in res.items():
        assert errs["status"] == 0, (rank, errs)
        assert errs["column"] < 0.06 and errs["gathered_weight"] < 0.06 and errs["row"] < 0.08, (rank, errs)
        assert max(errs[f"allreduce{i}"] for i in range(3)) < 0.08, (rank, errs)

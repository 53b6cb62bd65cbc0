"""Self-check of the fused compute + collective kernels inside an already initialised process group.

``run_fused_check()`` exercises, on small shapes and against fp32 PyTorch oracles computed from the
same seeds on every rank:

* all-gather -> GEMM (``nfn_gemm_tp`` mode AG_A) through ``TensorParallelContext.column_linear``,
* parameter all-gather -> GEMM (AG_B) through ``gathered_weight_linear``,
* GEMM -> reduce-scatter (RS) through ``row_linear``,
* one-shot all-reduce + residual + RMS norm (``nfn_allreduce_resid_norm``), with plain peer loads,
* expert-parallel dispatch (pull), grouped expert GEMMs and combine (``nfn_moe_ep_*``),

and finally reads the device status word (bounded waits that ran out leave a code there). It needs no
launcher of its own: ``bench.py --gpus N`` calls it before the timed region on every multi-GPU run, so
the kernels are proven on the same ranks, over the same NVLink fabric, that produce the scaling
numbers. Returns a small dict (``{"status": "ok", "max_err": {...}}``); raises on a mismatch.

The reference has no counterpart (it has neither tensor nor expert parallelism); the oracles are the
unsharded products.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

__all__ = ["run_fused_check"]


def _rand(shape, seed, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def run_fused_check(device: torch.device | None = None, *, moe: bool = True) -> dict:
    """Collective over the default process group (world 1 works too: the kernels then run their
    single-rank paths). All ranks must call it."""
    from ..ops import _lib
    from .tp import TensorParallelContext

    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    dev = device or torch.device("cuda", torch.cuda.current_device())
    bf = torch.bfloat16
    errs: dict[str, float] = {}
    ctx = TensorParallelContext(dev, impl="fused")

    # shapes every world size from 1 to 8 accepts: the gathered-weight product needs N / world to be a multiple of the
    # 128-column tile, the reduce-scatter needs K / world to be a multiple of 8
    rows, K, N = 256, 64 * max(world, 8), 128 * world * (3 if world <= 2 else 1)
    x = _rand((world * rows, K), 0, 0.5)
    w = _rand((N, K), 1, 0.05)
    b = _rand((N,), 2, 0.1)
    xq, wq, bq = x.to(bf).float(), w.to(bf).float(), b.to(bf).float()  # what the kernels actually see

    # ---- all-gather -> GEMM (sequence-sharded activations, column-parallel weight) ----
    nl = N // world
    xl = x[rank * rows:(rank + 1) * rows].to(dev, bf)
    wl = w[rank * nl:(rank + 1) * nl].to(dev, bf).contiguous()
    bl = b[rank * nl:(rank + 1) * nl].to(dev, bf).contiguous()
    for _ in range(2):  # the second call exercises the epoch / buffer alternation
        y = ctx.column_linear(xl, wl, bias=bl, act="gelu")
    ref = torch.nn.functional.gelu(xq @ wq[rank * nl:(rank + 1) * nl].T + bq[rank * nl:(rank + 1) * nl], approximate="tanh")
    errs["ag_gemm"] = float((y.float().cpu() - ref).abs().max())

    # ---- parameter all-gather -> GEMM ----
    y = ctx.gathered_weight_linear(x[:384].to(dev, bf), wl, bias=b.to(dev, bf))
    errs["param_ag_gemm"] = float((y.float().cpu() - (xq[:384] @ wq.T + bq)).abs().max())

    # ---- GEMM -> reduce-scatter (row-parallel weight) ----
    kl = K // world
    xk = x[:, rank * kl:(rank + 1) * kl].to(dev, bf).contiguous()
    wk = w[:, rank * kl:(rank + 1) * kl].to(dev, bf).contiguous()
    resid = _rand((rows, N), 5 + rank)
    for _ in range(2):
        y = ctx.row_linear(xk, wk, bias=b.to(dev, bf), resid=resid.to(dev, bf))
    ref = (xq @ wq.T + bq)[rank * rows:(rank + 1) * rows] + resid.to(bf).float()
    errs["gemm_rs"] = float((y.float().cpu() - ref).abs().max())

    # ---- one-shot all-reduce + residual + RMS norm (decode-sized) ----
    B, Nd = 32, 1664
    parts = [_rand((B, Nd), 20 + r) for r in range(world)]
    res0 = _rand((B, Nd), 40)
    nw = 1 + 0.1 * _rand((Nd,), 41)
    total = (sum(p.to(bf).float() for p in parts) + res0.to(bf).float()).to(bf).float()
    ref = total * torch.rsqrt(total.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.to(bf).float()
    buf, sym = ctx.partial_buffer(B, Nd)
    buf.copy_(parts[rank].to(dev, bf))
    resid_d = res0.to(dev, bf).clone()
    y = ctx.allreduce_resid_norm(buf, sym, resid=resid_d, norm_weight=nw.to(dev, bf), use_multicast=False)
    errs["allreduce_resid_norm"] = max(float((y.float().cpu() - ref).abs().max()), float((resid_d.float().cpu() - total).abs().max()))

    # ---- expert-parallel MoE: pull dispatch, grouped GEMMs, pull combine ----
    if moe:
        from ..ops.moe import moe_reference
        from .ep import ExpertParallelMoE
        E, k, D, F, T = 8, 2, 256, 256, 300
        if E % world == 0:
            g = torch.Generator().manual_seed(0)
            wr = (torch.randn(E, D, generator=g) * 0.2).to(bf).to(dev)
            wgu = (torch.randn(E, 2 * F, D, generator=g) * 0.05).to(bf).to(dev)
            wd = (torch.randn(E, D, F, generator=g) * 0.05).to(bf).to(dev)
            El = E // world
            layer = ExpertParallelMoE(E, k, D, F, T, dev)
            g = torch.Generator().manual_seed(100 + rank)
            worst = 0.0
            for it in range(2):
                xt = (torch.randn(T - 7 * it, D, generator=g) * 0.5).to(bf).to(dev)
                rs = torch.randn(xt.shape[0], D, generator=g).to(bf).to(dev)
                out = layer.forward(xt, wr, wgu[rank * El:(rank + 1) * El].contiguous(), wd[rank * El:(rank + 1) * El].contiguous(), resid=rs)
                refm = moe_reference(xt, wr, wgu, wd, k, resid=rs)
                # a token whose top-k choice flips under bf16 rounding gets a different expert; count rows, not elements
                worst = max(worst, float(((out.float() - refm).abs().amax(-1) > 0.08).float().mean()))
            errs["moe_ep_bad_row_fraction"] = worst

    torch.cuda.synchronize(dev)
    status = _lib.status_read_reset()
    limits = {"ag_gemm": 0.06, "param_ag_gemm": 0.06, "gemm_rs": 0.08, "allreduce_resid_norm": 0.06, "moe_ep_bad_row_fraction": 0.02}
    bad = {k_: v for k_, v in errs.items() if not (v <= limits[k_])}
    flag = torch.tensor([1 if (bad or status) else 0], device=dev)
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    if int(flag.item()):
        raise RuntimeError(f"fused collective kernels failed their self-check on rank {rank}: errors {errs}, device status {status}")
    return {"status": "ok", "world": world, "max_err": {k_: round(v, 5) for k_, v in errs.items()}}

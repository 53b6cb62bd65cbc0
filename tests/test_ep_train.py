"""Expert-parallel MoE FFN with gradients: two gloo ranks against the unsharded PyTorch experts;
on two GPUs the same with the native grouped GEMMs underneath."""
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


def _data(rank, T, d, E, k):
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(T, d, generator=g)
    logits = torch.randn(T, E, generator=g)
    w, idx = torch.softmax(logits, -1).topk(k, -1)
    return x, w / w.sum(-1, keepdim=True), idx, torch.randn(T, d, generator=g)


def _worker(rank, world, port, backend, out_q, exchange="library"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dist.init_process_group(backend, rank=rank, world_size=world)
    try:
        from neuralfn_b200.parallel.ep_train import ExpertParallelFFN
        from neuralfn_b200.tensor.stages_moe import grouped_swiglu_experts
        cuda = backend == "nccl"
        dev = torch.device("cuda", rank) if cuda else torch.device("cpu")
        if cuda:
            torch.cuda.set_device(dev)
        dt = torch.bfloat16 if cuda else torch.float32
        d, h, E, k = 128, 192, 4, 2
        Ts = [96, 160]  # ranks hold different numbers of tokens
        g = torch.Generator().manual_seed(7)
        full = [torch.randn(E, d, h, generator=g) * 0.05, torch.randn(E, h, d, generator=g) * 0.05, torch.randn(E, d, h, generator=g) * 0.05]
        layer = ExpertParallelFFN(d, h, E, device=dev, dtype=dt)
        layer.load_full(*[t.to(dev, dt) for t in full])
        x, w, idx, dout = _data(rank, Ts[rank], d, E, k)
        xg = x.to(dev, dt).requires_grad_(True)
        wg = w.to(dev).requires_grad_(True)
        if exchange == "peer":
            # rows, gradients and per-row scalars through this framework's pull kernels; no library all-to-all
            from neuralfn_b200.ops import _lib
            from neuralfn_b200.parallel.ep_fused_train import PeerExchange, fused_expert_parallel_ffn
            ex = PeerExchange(E, k, d, max(Ts), dev)
            for _ in range(2):                      # twice: the buffers and epochs are reused by every layer / step
                xg.grad = wg.grad = layer.w1.grad = layer.w2.grad = layer.w3.grad = None
                y = fused_expert_parallel_ffn(xg, wg, idx.to(dev), layer.w1, layer.w2, layer.w3, ex)
                y.backward(dout.to(dev, dt))
            torch.cuda.synchronize()
            assert _lib.status_read_reset() == 0
        else:
            y = layer(xg, wg, idx.to(dev))
            y.backward(dout.to(dev, dt))
        # oracle: all experts in one process, both ranks' tokens (expert gradients add up over ranks)
        ref_w = [t.clone().requires_grad_(True) for t in full]
        mine = None
        for r in range(world):
            xr, wr, ir, dr = _data(r, Ts[r], d, E, k)
            xr, wr = xr.requires_grad_(True), wr.requires_grad_(True)
            yr = grouped_swiglu_experts(xr, ref_w[0], ref_w[1], ref_w[2], wr, ir)
            yr.backward(dr)
            if r == rank:
                mine = (yr.detach(), xr.grad, wr.grad)

        def rel(a, b):
            return float((a.float().cpu() - b).abs().max() / (b.abs().max() + 1e-9))

        lo = rank * layer.local
        errs = {"y": rel(y, mine[0]), "dx": rel(xg.grad, mine[1]), "dw": rel(wg.grad, mine[2]),
                "dw1": rel(layer.w1.grad, ref_w[0].grad[lo:lo + layer.local]), "dw2": rel(layer.w2.grad, ref_w[1].grad[lo:lo + layer.local]),
                "dw3": rel(layer.w3.grad, ref_w[2].grad[lo:lo + layer.local])}
        out_q.put((rank, errs))
    finally:
        dist.destroy_process_group()


def _run(world, backend, exchange="library"):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, backend, q, exchange)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return dict(res)


def test_expert_parallel_ffn_gradients_on_gloo():
    for rank, e in _run(2, "gloo").items():
        assert max(e.values()) < 1e-4, (rank, e)


@pytest.mark.gpu
def test_expert_parallel_ffn_gradients_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    for rank, e in _run(2, "nccl").items():
        assert max(e.values()) < 0.05, (rank, e)


@pytest.mark.gpu
def test_peer_memory_exchange_gradients_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    for rank, e in _run(2, "nccl", "peer").items():
        assert max(e.values()) < 0.05, (rank, e)


@pytest.mark.gpu
def test_peer_memory_exchange_gradients_on_one_gpu():
    """World of one: the same kernels with every peer pointer local."""
    from neuralfn_b200.ops import _lib
    from neuralfn_b200.parallel.ep_fused_train import PeerExchange, fused_expert_parallel_ffn
    from neuralfn_b200.tensor.stages_moe import grouped_swiglu_experts
    dev = torch.device("cuda", 0)
    d, h, E, k, T = 128, 192, 4, 2, 200
    g = torch.Generator().manual_seed(7)
    full = [torch.randn(E, d, h, generator=g) * 0.05, torch.randn(E, h, d, generator=g) * 0.05, torch.randn(E, d, h, generator=g) * 0.05]
    x, w, idx, dout = _data(0, T, d, E, k)
    ws = [t.to(dev, torch.bfloat16).requires_grad_(True) for t in full]
    xg, wg = x.to(dev, torch.bfloat16).requires_grad_(True), w.to(dev).requires_grad_(True)
    ex = PeerExchange(E, k, d, T, dev)
    y = fused_expert_parallel_ffn(xg, wg, idx.to(dev), ws[0], ws[1], ws[2], ex)
    y.backward(dout.to(dev, torch.bfloat16))
    torch.cuda.synchronize()
    assert _lib.status_read_reset() == 0
    ref_w = [t.clone().requires_grad_(True) for t in full]
    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    yr = grouped_swiglu_experts(xr, ref_w[0], ref_w[1], ref_w[2], wr, idx)
    yr.backward(dout)

    def rel(a, b):
        return float((a.float().cpu() - b).abs().max() / (b.abs().max() + 1e-9))

    errs = {"y": rel(y, yr.detach()), "dx": rel(xg.grad, xr.grad), "dw": rel(wg.grad, wr.grad), "dw1": rel(ws[0].grad, ref_w[0].grad),
            "dw2": rel(ws[1].grad, ref_w[1].grad), "dw3": rel(ws[2].grad, ref_w[2].grad)}
    assert max(errs.values()) < 0.05, errs

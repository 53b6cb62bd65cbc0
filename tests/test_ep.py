"""Expert-parallel MoE over peer memory: one rank (single GPU) and two ranks vs the fp32 oracle."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

E, K_, D, F_, T = 8, 2, 256, 256, 300


def _weights(dev):
    g = torch.Generator().manual_seed(0)
    wr = (torch.randn(E, D, generator=g) * 0.2).bfloat16().to(dev)
    wgu = (torch.randn(E, 2 * F_, D, generator=g) * 0.05).bfloat16().to(dev)
    wd = (torch.randn(E, D, F_, generator=g) * 0.05).bfloat16().to(dev)
    return wr, wgu, wd


def _check(layer, rank, world, dev):
    from neuralfn_b200.ops import _lib
    from neuralfn_b200.ops.moe import moe_reference
    wr, wgu, wd = _weights(dev)
    El = E // world
    g = torch.Generator().manual_seed(100 + rank)
    errs = []
    for it in range(3):
        x = (torch.randn(T - 7 * it, D, generator=g) * 0.5).bfloat16().to(dev)
        resid = torch.randn(x.shape[0], D, generator=g).bfloat16().to(dev)
        out = layer.forward(x, wr, wgu[rank * El:(rank + 1) * El].contiguous(), wd[rank * El:(rank + 1) * El].contiguous(), resid=resid)
        ref = moe_reference(x, wr, wgu, wd, K_, resid=resid)
        err = (out.float() - ref).abs().amax(-1)
        errs.append(float((err > 0.08).float().mean()))
    torch.cuda.synchronize()
    return max(errs), _lib.status_read_reset()


def test_single_rank_equals_oracle():
    from neuralfn_b200.parallel.ep import ExpertParallelMoE
    dev = torch.device("cuda", 0)
    layer = ExpertParallelMoE(E, K_, D, F_, T, dev)
    bad, status = _check(layer, 0, 1, dev)
    assert status == 0 and bad < 0.02, (bad, status)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    try:
        from neuralfn_b200.parallel.ep import ExpertParallelMoE
        dev = torch.device("cuda", rank)
        layer = ExpertParallelMoE(E, K_, D, F_, T, dev)
        q.put((rank, *_check(layer, rank, world, dev)))
    finally:
        dist.destroy_process_group()


def test_two_ranks_equal_oracle():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, bad, status in res:
        assert status == 0 and bad < 0.02, (rank, bad, status)

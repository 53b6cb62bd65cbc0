"""MoE Llama with expert parallelism: loss and gradients of two gloo ranks (different batches) against
the single-process model holding every expert; a few optimizer steps; the GPU variant on two GPUs."""
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


def _cfg():
    from neuralfn_b200.parallel.moe_llama import MoELlamaConfig
    return MoELlamaConfig(n_layer=2, n_head=4, n_kv_head=2, d_model=128, n_experts=4, top_k=2, expert_hidden=192, vocab_size=384, max_seq_len=128)


def _batch(cfg, rank, B, T):
    g = torch.Generator().manual_seed(50 + rank)
    return torch.randint(0, cfg.vocab_size, (B, T), generator=g), torch.randint(0, cfg.vocab_size, (B, T), generator=g)


def _worker(rank, world, port, backend, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dist.init_process_group(backend, rank=rank, world_size=world)
    try:
        from neuralfn_b200.parallel.dp import AdamWConfig
        from neuralfn_b200.parallel.moe_llama import EPMoELlama, FlatAdamWTrainer, _is_expert, moe_llama_reference_loss
        cuda = backend == "nccl"
        dev = torch.device("cuda", rank) if cuda else torch.device("cpu")
        if cuda:
            torch.cuda.set_device(dev)
        cfg = _cfg()
        B, T = 2, 128 if cuda else 24
        model = EPMoELlama(cfg, dev, seed=3)
        full = model.full_state()
        tok, tgt = _batch(cfg, rank, B, T)
        loss = model.loss(tok.to(dev), tgt.to(dev))
        model.backward(loss)
        ref = {n: v.clone().requires_grad_(True) for n, v in full.items()}
        ref_losses = []
        for r in range(world):
            rt, rg = _batch(cfg, r, B, T)
            ref_losses.append(moe_llama_reference_loss(cfg, ref, rt, rg))
        (sum(ref_losses) / world).backward()
        El = cfg.n_experts // world
        worst, worst_name = 0.0, ""
        for n, v in model.p.items():
            want = ref[n].grad
            if _is_expert(n):
                want = want[rank * El:(rank + 1) * El]
            err = float((v.main_grad.float().cpu() - want).abs().max() / (want.abs().max() + 1e-8))
            if err > worst:
                worst, worst_name = err, n
        gn_ref = float(torch.sqrt(sum(v.grad.pow(2).sum() for v in ref.values())))
        errs = {"loss": abs(float(loss) - float(ref_losses[rank])), "grad_rel": worst, "worst": worst_name,
                "norm_rel": abs(float(model.grad_norm()) - gn_ref) / gn_ref}
        tr = FlatAdamWTrainer(model, AdamWConfig(lr=3e-3, warmup_steps=1, schedule="constant", weight_decay=0.0))
        losses = [float(tr.step(tok.to(dev), tgt.to(dev))) for _ in range(6)]
        errs["loss_drop"] = losses[0] - losses[-1]
        out_q.put((rank, errs))
    finally:
        dist.destroy_process_group()


def _run(world, backend):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, backend, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return dict(res)


def test_ep_moe_llama_matches_single_process_model_on_gloo():
    for rank, e in _run(2, "gloo").items():
        assert e["loss"] < 1e-4 and e["grad_rel"] < 2e-3 and e["norm_rel"] < 1e-3, (rank, e)
        assert e["loss_drop"] > 0.05, (rank, e)


@pytest.mark.gpu
def test_ep_moe_llama_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    for rank, e in _run(2, "nccl").items():
        assert e["loss"] < 0.05 and e["norm_rel"] < 0.1, (rank, e)
        assert e["loss_drop"] > 0.05, (rank, e)

"""Tensor-parallel Llama: loss and gradients of two gloo ranks against the unsharded PyTorch
model, and a few optimizer steps (CPU); the fused-kernel path on two GPUs against the same oracle."""
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
    from neuralfn_b200.models.llama import LlamaConfig
    return LlamaConfig(n_layer=2, n_head=4, n_kv_head=2, d_model=256, d_ff=512, vocab_size=500, max_seq_len=256, vocab_pad_to=128)


def _full_params(cfg, seed=3):
    from neuralfn_b200.models.gpt2 import FlatLayout
    from neuralfn_b200.models.llama import init_llama_params_, llama_param_specs
    layout = FlatLayout(llama_param_specs(cfg))
    flat = torch.zeros(layout.n_total)
    init_llama_params_(cfg, layout, flat, seed)
    views = layout.views(flat)
    g = torch.Generator().manual_seed(seed + 1)
    for n, v in views.items():  # make the norm weights non-trivial
        if n.endswith("norm"):
            v.add_(0.1 * torch.randn(v.shape, generator=g))
    return {n: v.clone() for n, v in views.items()}


def _worker(rank, world, port, backend, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dist.init_process_group(backend, rank=rank, world_size=world)
    try:
        from neuralfn_b200.models.llama import llama_reference_forward
        from neuralfn_b200.parallel.dp import AdamWConfig
        from neuralfn_b200.parallel.tp import TensorParallelContext
        from neuralfn_b200.parallel.tp_llama import TPLlama, TPLlamaTrainer, shard_llama_params
        cuda = backend == "nccl"
        dev = torch.device("cuda", rank) if cuda else torch.device("cpu")
        if cuda:
            torch.cuda.set_device(dev)
        cfg = _cfg()
        full = _full_params(cfg)
        B, T = 2, 256 if cuda else 32
        g = torch.Generator().manual_seed(11)
        tokens = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
        targets = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
        # oracle: unsharded fp32 model
        ref = {n: v.clone().requires_grad_(True) for n, v in full.items()}
        ref_loss, _ = llama_reference_forward(cfg, ref, tokens, targets)
        ref_loss.backward()
        ref_grads = shard_llama_params(cfg, {n: v.grad for n, v in ref.items()}, rank, world)

        tp = TensorParallelContext(dev)
        model = TPLlama(cfg, tp, full_params=full)
        loss = model.loss(tokens.to(dev), targets.to(dev))
        model.backward(loss)
        total = loss.detach().float().clone()
        dist.all_reduce(total)
        errs = {"loss": abs(float(total) - float(ref_loss))}
        worst = 0.0
        for n, gref in ref_grads.items():
            got = model.p[n].main_grad.float().cpu()
            worst = max(worst, float((got - gref).abs().max() / (gref.abs().max() + 1e-8)))
        errs["grad_rel"] = worst
        gn_ref = torch.sqrt(sum(v.grad.pow(2).sum() for v in ref.values()))
        errs["norm_rel"] = abs(float(model.grad_norm()) - float(gn_ref)) / float(gn_ref)
        # the gathered shards are the unsharded model again
        back = model.full_state()
        errs["roundtrip"] = max(float((back[n] - full[n]).abs().max()) for n in full) if not cuda else 0.0
        tr = TPLlamaTrainer(model, AdamWConfig(lr=3e-3, warmup_steps=1, schedule="constant", weight_decay=0.0))
        losses = [float(tr.step(tokens.to(dev), targets.to(dev))) for _ in range(6)]
        errs["loss_drop"] = losses[0] - losses[-1]
        errs["impl"] = tp.impl
        if cuda:
            from neuralfn_b200.ops import _lib
            errs["status"] = _lib.status_read_reset()
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
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return dict(res)


def test_tp_llama_matches_unsharded_model_on_gloo():
    for rank, e in _run(2, "gloo").items():
        assert e["impl"] == "torch"
        assert e["loss"] < 1e-4 and e["grad_rel"] < 1e-3 and e["norm_rel"] < 1e-4 and e["roundtrip"] == 0.0, (rank, e)
        assert e["loss_drop"] > 0.05, (rank, e)


@pytest.mark.gpu
def test_tp_llama_fused_kernels_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    for rank, e in _run(2, "nccl").items():
        assert e["impl"] == "fused"
        assert e["loss"] < 0.03 and e["grad_rel"] < 0.06 and e["norm_rel"] < 0.03, (rank, e)
        assert e["loss_drop"] > 0.05, (rank, e)


@pytest.mark.gpu
def test_tp_llama_single_gpu_runs_the_fused_path():
    from neuralfn_b200.models.llama import llama_reference_forward
    from neuralfn_b200.parallel.tp import TensorParallelContext
    from neuralfn_b200.parallel.tp_llama import TPLlama
    cfg = _cfg()
    full = _full_params(cfg)
    g = torch.Generator().manual_seed(11)
    tokens = torch.randint(0, cfg.vocab_size, (2, 256), generator=g)
    targets = torch.randint(0, cfg.vocab_size, (2, 256), generator=g)
    ref = {n: v.clone().requires_grad_(True) for n, v in full.items()}
    ref_loss, _ = llama_reference_forward(cfg, ref, tokens, targets)
    ref_loss.backward()
    model = TPLlama(cfg, TensorParallelContext(torch.device("cuda", 0)), full_params=full)
    loss = model.loss(tokens.cuda(), targets.cuda())
    model.backward(loss)
    assert abs(float(loss) - float(ref_loss)) < 0.03
    for n, v in ref.items():
        got = model.p[n].main_grad.float().cpu()
        assert float((got - v.grad).abs().max() / (v.grad.abs().max() + 1e-8)) < 0.06, n


def test_export_and_reload_hf_llama_directory(tmp_path):
    from neuralfn_b200.checkpoint.safetensors_io import export_hf_llama_directory, load_hf_llama_directory
    cfg = _cfg()
    full = _full_params(cfg)
    export_hf_llama_directory(tmp_path / "hf", cfg, full, dtype=torch.float32)
    ecfg, tensors = load_hf_llama_directory(tmp_path / "hf", max_batch=2, max_seq=64)
    assert ecfg.n_layer == cfg.n_layer and ecfg.n_kv_head == cfg.n_kv_head and ecfg.vocab == cfg.vocab_size
    for n in ("layers.1.wqkv", "layers.0.w_gate_up", "layers.1.w_down", "norm"):
        assert torch.equal(tensors[n].float(), full[n].to(torch.bfloat16).float()), n
    assert torch.equal(tensors["tok_embeddings"][:cfg.vocab_size].float(), full["tok_embeddings"][:cfg.vocab_size].to(torch.bfloat16).float())


def _mesh_worker(rank, world, port, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from neuralfn_b200.models.llama import llama_reference_forward
        from neuralfn_b200.parallel.dp import AdamWConfig
        from neuralfn_b200.parallel.tp import TensorParallelContext
        from neuralfn_b200.parallel.tp_llama import TPLlama, TPLlamaTrainer, shard_llama_params, tp_dp_mesh
        tp_group, dp_group, t, d = tp_dp_mesh(2)
        cfg = _cfg()
        full = _full_params(cfg)
        B, T = 2, 32
        batches = []
        for r in range(2):                                   # one batch per replica
            g = torch.Generator().manual_seed(40 + r)
            batches.append((torch.randint(0, cfg.vocab_size, (B, T), generator=g), torch.randint(0, cfg.vocab_size, (B, T), generator=g)))
        # oracle: the unsharded model on both replicas' batches, gradients averaged
        ref = {n: v.clone().requires_grad_(True) for n, v in full.items()}
        ref_loss = sum(llama_reference_forward(cfg, ref, tok, tgt)[0] for tok, tgt in batches) / 2
        ref_loss.backward()
        ref_grads = shard_llama_params(cfg, {n: v.grad for n, v in ref.items()}, t, 2)
        model = TPLlama(cfg, TensorParallelContext(torch.device("cpu"), tp_group), full_params=full, dp_group=dp_group)
        tok, tgt = batches[d]
        loss = model.loss(tok, tgt)
        model.backward(loss)
        worst = max(float((model.p[n].main_grad.float() - gref).abs().max() / (gref.abs().max() + 1e-8)) for n, gref in ref_grads.items())
        mean_loss = float(model.reduce_loss(loss.detach().clone()))
        tr = TPLlamaTrainer(model, AdamWConfig(lr=3e-3, warmup_steps=1, schedule="constant", weight_decay=0.0))
        losses = [float(tr.step(tok, tgt)) for _ in range(5)]
        digest = float(model.params.detach().double().sum())
        out_q.put((rank, {"t": t, "d": d, "grad_rel": worst, "loss_err": abs(mean_loss - float(ref_loss)), "drop": losses[0] - losses[-1], "digest": digest}))
    finally:
        dist.destroy_process_group()


def test_tp2_x_dp2_mesh_matches_the_unsharded_model_on_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_mesh_worker, args=(r, 4, port, q)) for r in range(4)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted((e["t"], e["d"]) for e in res.values()) == [(0, 0), (0, 1), (1, 0), (1, 1)]
    for rank, e in res.items():
        assert e["grad_rel"] < 1e-3 and e["loss_err"] < 1e-4 and e["drop"] > 0.03, (rank, e)
    # replicas of one shard stay bit-identical after the optimizer steps
    assert res[0]["digest"] == res[2]["digest"] and res[1]["digest"] == res[3]["digest"]

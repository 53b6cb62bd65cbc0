"""Tensor-parallel Glimmer decoder: gloo ranks (PyTorch fallbacks) and GPUs (fused kernels) against the
unsharded fp32 restatement of the block. Covers sliding-window ring caches shorter than the prompt,
position-free global layers, gated attention, sandwich norms, replicated KV heads and CUDA-graph decode."""
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


def _cfg(cuda: bool, n_kv: int):
    from neuralfn_b200.serving.tp_glimmer import GlimmerTPConfig
    if cuda:
        return GlimmerTPConfig(n_layer=4, d_model=256, n_head=4, n_kv_head=n_kv, head_dim=64, d_ff=512, vocab_size=500, window=64,
                               vocab_pad_to=128)
    return GlimmerTPConfig(n_layer=4, d_model=64, n_head=4, n_kv_head=n_kv, head_dim=16, d_ff=128, vocab_size=120, window=8, vocab_pad_to=64)


def _check(dec, cfg, full, prompt, n_new, cuda):
    """Teacher-forced: every token we produced must be the reference's arg-max (or a near tie under bf16)."""
    from neuralfn_b200.serving.tp_glimmer import glimmer_reference_logits
    got = dec.generate(prompt.to(dec.dev), n_new).cpu()
    seq, bad, worst = prompt.clone(), 0, 0.0
    for i in range(n_new):
        last = glimmer_reference_logits(cfg, full, seq)[:, -1]
        gap = last.max(-1).values - last.gather(-1, got[:, i:i + 1]).squeeze(-1)
        worst = max(worst, float(gap.max()))
        bad += int((gap > (0.25 if cuda else 1e-4)).sum())
        seq = torch.cat([seq, got[:, i:i + 1]], 1)
    return got, bad, worst


def _worker(rank, world, port, backend, n_kv, use_graph, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dist.init_process_group(backend, rank=rank, world_size=world)
    try:
        from neuralfn_b200.parallel.tp import TensorParallelContext
        from neuralfn_b200.serving.tp_glimmer import TPGlimmerDecoder, random_glimmer_params
        cuda = backend == "nccl"
        dev = torch.device("cuda", rank) if cuda else torch.device("cpu")
        if cuda:
            torch.cuda.set_device(dev)
        cfg = _cfg(cuda, n_kv)
        B, T, n_new = 2, (256 if cuda else 12), 6            # prompts longer than the window: the ring wraps during prefill
        full = random_glimmer_params(cfg, 3)
        dec = TPGlimmerDecoder(cfg, TensorParallelContext(dev), max_batch=B, max_seq=T + 16, full_params=full, use_graph=use_graph)
        prompt = torch.randint(0, cfg.vocab_size, (B, T), generator=torch.Generator().manual_seed(4))
        got, bad, worst = _check(dec, cfg, full, prompt, n_new, cuda)
        dec.set_sampling(temperature=0.8, top_k=16, top_p=0.9, seed=3)
        sampled = dec.generate(prompt.to(dev), 4).cpu()
        status = 0
        if cuda:
            from neuralfn_b200.ops import _lib
            status = _lib.status_read_reset()
        dec.close()
        out_q.put((rank, {"bad": bad, "worst": worst, "tokens": got.tolist(), "sampled": sampled.tolist(), "status": status,
                          "kv_local": dec.Hkv, "caps": dec.caps}))
    finally:
        dist.destroy_process_group()


def _run(world, backend, n_kv, use_graph=False):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, backend, n_kv, use_graph, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return res


@pytest.mark.parametrize("n_kv", [2, 1])
def test_two_gloo_ranks_match_the_unsharded_model(n_kv):
    res = _run(2, "gloo", n_kv)
    assert res[0]["tokens"] == res[1]["tokens"] and res[0]["sampled"] == res[1]["sampled"]
    for r in res.values():
        assert r["bad"] == 0, r
        assert r["kv_local"] == 1 and r["caps"] == [8, 8, 8, 28]            # three ring layers, one global


def test_single_rank_cpu_matches_the_unsharded_model():
    from neuralfn_b200.parallel.tp import TensorParallelContext
    from neuralfn_b200.serving.tp_glimmer import TPGlimmerDecoder, random_glimmer_params
    cfg = _cfg(False, 2)
    full = random_glimmer_params(cfg, 9)
    dec = TPGlimmerDecoder(cfg, TensorParallelContext(torch.device("cpu")), max_batch=3, max_seq=40, full_params=full)
    prompt = torch.randint(0, cfg.vocab_size, (3, 20), generator=torch.Generator().manual_seed(1))
    _got, bad, _worst = _check(dec, cfg, full, prompt, 10, False)
    assert bad == 0 and dec.Hkv == 2


def test_config_from_the_glimmer_benchmark_spec():
    from neuralfn_b200.presets_glimmer import glimmer_benchmark_shape
    from neuralfn_b200.serving.tp_glimmer import GlimmerTPConfig
    cfg = GlimmerTPConfig.from_spec(glimmer_benchmark_shape())
    assert (cfg.n_layer, cfg.d_model, cfg.n_head, cfg.n_kv_head, cfg.head_dim, cfg.d_ff) == (48, 6656, 32, 2, 128, 24576)
    assert cfg.window == 4096 and cfg.global_every == 4 and not cfg.is_local(3) and cfg.is_local(4)
    assert cfg.padded_vocab % 64 == 0 and cfg.logit_softcap == 30.0


@pytest.mark.gpu
@pytest.mark.parametrize("use_graph", [False, True])
def test_one_gpu_kernel_path(use_graph):
    from neuralfn_b200.ops import _lib
    from neuralfn_b200.parallel.tp import TensorParallelContext
    from neuralfn_b200.serving.tp_glimmer import TPGlimmerDecoder, random_glimmer_params
    cfg = _cfg(True, 2)
    full = random_glimmer_params(cfg, 3)
    dev = torch.device("cuda", 0)
    dec = TPGlimmerDecoder(cfg, TensorParallelContext(dev), max_batch=2, max_seq=288, full_params=full, use_graph=use_graph)
    prompt = torch.randint(0, cfg.vocab_size, (2, 256), generator=torch.Generator().manual_seed(4))
    _got, bad, worst = _check(dec, cfg, full, prompt, 8, True)
    dec.close()
    assert _lib.status_read_reset() == 0
    assert bad == 0, worst


@pytest.mark.gpu
@pytest.mark.parametrize("n_kv,use_graph", [(2, False), (1, True)])
def test_two_gpus_fused_kernels(n_kv, use_graph):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    res = _run(2, "nccl", n_kv, use_graph)
    assert res[0]["tokens"] == res[1]["tokens"] and res[0]["sampled"] == res[1]["sampled"]
    for r in res.values():
        assert r["status"] == 0 and r["bad"] == 0, r

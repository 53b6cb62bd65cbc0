"""Pipeline-parallel training (Llama and Glimmer engines) on two GPUs matches the single-GPU trainer step for step."""
import os
import socket
import zlib

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _cfg(family="llama"):
    if family == "glimmer":
        from neuralfn_b200.models.glimmer import GlimmerConfig
        return GlimmerConfig(n_layer=4, n_head=4, n_kv_head=2, head_dim=64, d_model=256, d_ff=512, vocab_size=512, max_seq_len=128, window=48,
                             global_every=2, output_multiplier=0.5)
    from neuralfn_b200.models.llama import LlamaConfig
    return LlamaConfig(n_layer=4, n_head=4, n_kv_head=2, d_model=256, d_ff=512, vocab_size=512, max_seq_len=128)


def _fill_by_name(tr):
    """Deterministic weights keyed by tensor name, so a stage and the whole model agree."""
    flat = torch.zeros(tr.layout.n_total)
    for s in tr.layout.order:
        g = torch.Generator().manual_seed(zlib.crc32(s.name.encode()))
        v = tr.layout.view(flat, s.name)
        v.copy_(torch.ones(s.shape) if s.init == "ones" else (torch.zeros(s.shape) if s.init == "zeros" else torch.randn(s.shape, generator=g) * 0.02))
    tr.opt.master.copy_(flat)
    tr.bufs.params.copy_(flat.bfloat16())


def _batches(steps, micro):
    g = torch.Generator().manual_seed(0)
    tok = [[torch.randint(0, 512, (2, 128), generator=g, dtype=torch.int32) for _ in range(micro)] for _ in range(steps)]
    return tok, [[torch.roll(t, -1, 1) for t in row] for row in tok]


MICRO = 3   # more micro-batches than stages: warm-up, steady 1F1B pairs and a cool-down all occur


def _worker(rank, world, port, q, family):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    try:
        from neuralfn_b200.parallel.dp import AdamWConfig
        from neuralfn_b200.parallel.pp import PipelineParallelTrainer
        tr = PipelineParallelTrainer(_cfg(family), 2, 128, AdamWConfig(lr=2e-3, warmup_steps=1, total_steps=20, weight_decay=0.0), micro_batches=MICRO)
        _fill_by_name(tr.inner)
        tok, tgt = _batches(4, MICRO)
        losses = [tr.train_step(tok[i], tgt[i]) for i in range(4)]
        tr.inner.check_status()
        names = [s.name for s in tr.layout.order]
        q.put((rank, losses, names))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("family", ["llama", "glimmer"])
def test_two_stage_pipeline_matches_single_gpu(tmp_path, family):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, family)) for r in range(2)]
    for p in procs:
        p.start()
    res = {r: (l, n) for r, l, n in (q.get(timeout=240) for _ in procs)}
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res[0][0] == res[1][0]
    qkv = "layers.2.wqkv" if family == "llama" else "layers.2.wqkvg"
    assert "tok_embeddings" in res[0][1] and "lm_head" in res[1][1] and qkv in res[1][1] and "layers.1.wo" in res[0][1]
    # single-GPU reference with the same weights, batches and accumulation
    from neuralfn_b200.parallel.dp import AdamWConfig
    from neuralfn_b200.trainers.dense_gpt import DenseGPTTrainer
    ref = DenseGPTTrainer(_cfg(family), 2, 128, AdamWConfig(lr=2e-3, warmup_steps=1, total_steps=20, weight_decay=0.0), grad_accum_steps=MICRO,
                          use_cuda_graph=False)
    _fill_by_name(ref)
    tok, tgt = _batches(4, MICRO)
    want = []
    for i in range(4):
        want.append(sum(ref.train_step(tok[i][m], tgt[i][m]) for m in range(MICRO)) / MICRO)
    # the stages clip by the whole model's gradient norm, like the single-GPU trainer
    assert max(abs(x - y) for x, y in zip(res[0][0], want)) < 0.05, (res[0][0], want)
    assert want[-1] < want[0] + 0.05          # four steps on random tokens: no divergence (progress is not the point here)

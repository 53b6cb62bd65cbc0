"""Llama-family engine (RMSNorm, RoPE, GQA, SwiGLU) vs. the fp32 PyTorch restatement, and a
short training run through the generic dense trainer."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(**kw):
    from neuralfn_b200.models.gpt2 import FlatLayout
    from neuralfn_b200.models.llama import LlamaConfig, LlamaEngine, init_llama_params_, llama_param_specs
    base = dict(n_layer=2, n_head=4, n_kv_head=2, d_model=256, d_ff=512, vocab_size=1000, max_seq_len=128)
    base.update(kw)
    cfg = LlamaConfig(**base)
    layout = FlatLayout(llama_param_specs(cfg))
    master = torch.empty(layout.n_total, device="cuda")
    init_llama_params_(cfg, layout, master, 0)
    g = torch.Generator(device="cuda").manual_seed(1)
    for s in layout.order:
        if not s.decay:
            layout.view(master, s.name).add_(torch.randn(s.shape, device="cuda", generator=g) * 0.05)
    params = master.to(torch.bfloat16)
    grads = torch.zeros_like(params)
    B, T = 2, 128
    eng = LlamaEngine(cfg, layout, params, grads, B, T)
    tok = torch.randint(0, cfg.vocab_size, (B, T), device="cuda")
    tgt = torch.randint(0, cfg.vocab_size, (B, T), device="cuda")
    eng.set_batch(tok, tgt)
    return cfg, layout, params, grads, eng, tok, tgt


@pytest.mark.parametrize("kw", [dict(), dict(qk_norm=True, tie_embeddings=True, window=48, logit_softcap=30.0, z_loss=1e-4,
                                             rope_convention="legacy"),
                                dict(n_head=2, n_kv_head=2, head_dim_override=128)])
def test_engine_matches_reference(kernel_lib, kw):
    from neuralfn_b200.models.llama import llama_reference_forward
    from neuralfn_b200.ops import _lib
    cfg, layout, params, grads, eng, tok, tgt = _setup(**kw)
    loss = eng.forward()
    eng.backward()
    _lib.assert_status_ok("llama engine")
    ref_p = {k: v.float().clone().requires_grad_(True) for k, v in layout.views(params).items()}
    ref_loss, _ = llama_reference_forward(cfg, ref_p, tok, tgt)
    ref_loss.backward()
    assert abs(loss.item() - ref_loss.item()) < 2e-2 * max(1.0, ref_loss.item())
    gv = layout.views(grads)
    bad = {}
    for name, ref in ref_p.items():
        denom = ref.grad.norm().item() + 1e-8
        rel = (gv[name].float() - ref.grad).norm().item() / denom
        if rel > 6e-2 and denom > 1e-4:
            bad[name] = (rel, denom)
    assert not bad, bad


def test_trainer_runs_llama_and_weights_load_into_the_inference_engine(kernel_lib):
    from neuralfn_b200.models.llama import LlamaConfig
    from neuralfn_b200.parallel.dp import AdamWConfig
    from neuralfn_b200.serving import EngineConfig, ResidentEngine
    from neuralfn_b200.trainers.dense_gpt import DenseGPTTrainer
    cfg = LlamaConfig(n_layer=2, n_head=4, n_kv_head=2, d_model=256, d_ff=512, vocab_size=512, max_seq_len=128)
    tr = DenseGPTTrainer(cfg, 4, 128, AdamWConfig(lr=3e-3, warmup_steps=2, total_steps=50, weight_decay=0.0), seed=3)
    torch.manual_seed(0)
    tok = torch.randint(0, 512, (4, 128))
    tgt = torch.roll(tok, -1, dims=1)
    losses = [tr.train_step(tok, tgt) for _ in range(14)]
    tr.check_status()
    assert losses[-1] < losses[0] - 0.5, losses
    # the trained weights drive the resident engine unchanged (same tensor names)
    eng = ResidentEngine(EngineConfig(family=1, n_layer=2, d_model=256, n_head=4, n_kv_head=2, head_dim=64, d_ff=512, vocab=512,
                                      padded_vocab=cfg.padded_vocab, max_seq=128, max_batch=2, rope_hf=1, norm_eps=cfg.norm_eps,
                                      tie_embeddings=0))
    eng.load_named_tensors({k: v.detach().cpu() for k, v in tr.layout.views(tr.bufs.params).items()})
    prompt = tok[0, :20].tolist()
    nxt = eng.prefill(0, prompt)
    tr.engine.set_batch(tok, tgt)
    tr.engine.forward(compute_grad_logits=False)
    ref = tr.engine.logits_view()[0, 19].float().cpu()
    assert (eng.last_logits(0) - ref).abs().max() < 0.25
    assert nxt == int(ref.argmax()) or (ref.max() - ref[nxt]) < 0.2

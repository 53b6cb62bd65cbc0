"""Resident inference engine vs plain PyTorch forwards: prefill logits, token-by-token decode
through the KV cache (greedy), continuous batching, both model families."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _gpt2_setup(qk_norm=False, softcap=0.0):
    from neuralfn_b200.models.gpt2 import FlatLayout, GPT2Config, gpt2_param_specs, init_gpt2_params_
    cfg = GPT2Config(n_layer=2, n_head=4, d_model=256, vocab_size=1000, max_seq_len=96, qk_norm=qk_norm, logit_softcap=softcap)
    layout = FlatLayout(gpt2_param_specs(cfg))
    master = torch.empty(layout.n_total)
    init_gpt2_params_(cfg, layout, master, seed=5)
    for s in gpt2_param_specs(cfg):  # make biases / norm weights non-trivial
        if not s.decay:
            layout.view(master, s.name).add_(0.05 * torch.randn(s.shape, generator=torch.Generator().manual_seed(len(s.name))))
    params = {n: v.bfloat16() for n, v in layout.views(master).items()}
    return cfg, params


@pytest.mark.parametrize("qk_norm,softcap", [(False, 0.0), (True, 30.0)])
def test_gpt2_family_prefill_and_decode_match_full_forward(qk_norm, softcap):
    from neuralfn_b200.models.gpt2 import reference_forward
    from neuralfn_b200.serving import EngineConfig, ResidentEngine
    cfg, params = _gpt2_setup(qk_norm, softcap)
    eng = ResidentEngine(EngineConfig.gpt2(cfg, max_batch=4))
    eng.load_named_tensors(params)
    dev_params = {k: v.cuda().float() for k, v in params.items()}
    prompts = {0: [5, 17, 900, 3, 44, 8, 120], 2: [7, 7, 7, 250]}
    seqs = {s: list(p) for s, p in prompts.items()}
    nxt = {}
    for slot, p in prompts.items():
        nxt[slot] = eng.prefill(slot, p)
        _, logits = reference_forward(cfg, dev_params, torch.tensor([p], device="cuda"))
        ref = logits[0, -1, :cfg.vocab_size].float().cpu()
        got = eng.last_logits(slot)
        assert (got - ref).abs().max() < 0.15, float((got - ref).abs().max())
        assert nxt[slot] == int(ref.argmax()) or (ref.max() - ref[nxt[slot]]) < 0.1
    for step in range(6):  # step 0 eager, step 1 captures the CUDA graph, later steps replay it
        for slot in seqs:
            seqs[slot].append(nxt[slot])
        nxt = eng.decode({slot: seqs[slot][-1] for slot in seqs})
        for slot in seqs:
            _, logits = reference_forward(cfg, dev_params, torch.tensor([seqs[slot]], device="cuda"))
            ref = logits[0, -1, :cfg.vocab_size].float().cpu()
            got = eng.last_logits(slot)
            assert (got - ref).abs().max() < 0.2, (step, slot, float((got - ref).abs().max()))
        assert eng.slot_length(0) == len(seqs[0])
    assert eng.launches > 0 and eng.device_bytes > 0


def _llama_ref(cfg, w, tokens):
    """fp32 reference: RMSNorm, hf rotary, GQA with optional sliding window, SwiGLU."""
    T = len(tokens)
    hd, Hq, Hkv = cfg.head_dim, cfg.n_head, cfg.n_kv_head
    x = w["tok_embeddings"][torch.tensor(tokens)]
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2).double() / hd))
    ang = torch.outer(torch.arange(T).double(), inv)
    cos, sin = ang.cos().float()[:, None], ang.sin().float()[:, None]

    def rms(v, wt, eps):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * wt

    def rope(v):
        a, b = v[..., :hd // 2], v[..., hd // 2:]
        return torch.cat((a * cos - b * sin, b * cos + a * sin), -1)

    for l in range(cfg.n_layer):
        h = rms(x, w[f"layers.{l}.attn_norm"], cfg.norm_eps)
        qkv = h @ w[f"layers.{l}.wqkv"].T
        q = qkv[:, :Hq * hd].view(T, Hq, hd)
        k = qkv[:, Hq * hd:(Hq + Hkv) * hd].view(T, Hkv, hd)
        v = qkv[:, (Hq + Hkv) * hd:].view(T, Hkv, hd)
        if cfg.qk_norm == 2:
            q = rms(q, w[f"layers.{l}.q_norm"], cfg.qk_norm_eps)
            k = rms(k, w[f"layers.{l}.k_norm"], cfg.qk_norm_eps)
        q, k = rope(q), rope(k)
        k = k.repeat_interleave(Hq // Hkv, 1)
        v = v.repeat_interleave(Hq // Hkv, 1)
        s = torch.einsum("thd,shd->hts", q, k) / math.sqrt(hd)
        i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
        mask = j <= i
        local = cfg.window > 0 and (cfg.global_every <= 0 or (l + 1) % cfg.global_every != 0)
        if local:
            mask = mask & (i - j < cfg.window)
        s = s.masked_fill(~mask, float("-inf"))
        a = torch.einsum("hts,shd->thd", s.softmax(-1), v).reshape(T, Hq * hd)
        x = x + a @ w[f"layers.{l}.wo"].T
        h = rms(x, w[f"layers.{l}.ffn_norm"], cfg.norm_eps)
        gu = h @ w[f"layers.{l}.w_gate_up"].T
        x = x + (F.silu(gu[:, :cfg.d_ff]) * gu[:, cfg.d_ff:]) @ w[f"layers.{l}.w_down"].T
    x = rms(x, w["norm"], cfg.norm_eps)
    head = w["tok_embeddings"] if cfg.tie_embeddings else w["lm_head"]
    return (x @ head.T)[:, :cfg.vocab]


@pytest.mark.parametrize("window,qk_norm,hd", [(0, 0, 64), (16, 2, 128)])
def test_llama_family_hybrid_cache_matches_reference(window, qk_norm, hd):
    from neuralfn_b200.serving import EngineConfig, ResidentEngine
    cfg = EngineConfig(family=1, n_layer=3, d_model=256, n_head=4, n_kv_head=2, head_dim=hd, d_ff=512, vocab=777, padded_vocab=784,
                       max_seq=80, max_batch=3, qk_norm=qk_norm, rope_hf=1, rope_theta=10000.0, norm_eps=1e-5, tie_embeddings=0,
                       window=window, global_every=3 if window else 0)
    eng = ResidentEngine(cfg)
    g = torch.Generator().manual_seed(1)
    w = {}
    for name, numel in eng.expected_tensors().items():
        if name.endswith("norm"):
            w[name] = (1 + 0.1 * torch.randn(numel, generator=g)).bfloat16()
        else:
            w[name] = (torch.randn(numel, generator=g) * 0.04).bfloat16()
    shapes = {"tok_embeddings": (784, 256), "lm_head": (784, 256)}
    for l in range(3):
        shapes.update({f"layers.{l}.wqkv": ((4 + 4) * hd, 256), f"layers.{l}.wo": (256, 4 * hd), f"layers.{l}.w_gate_up": (1024, 256),
                       f"layers.{l}.w_down": (256, 512)})
    eng.load_named_tensors(w)
    wf = {k: (v.float().view(*shapes[k]) if k in shapes else v.float()) for k, v in w.items()}
    seq = [3, 99, 501, 7, 7, 320, 64, 2, 11, 600, 13, 14, 15, 16, 17, 18, 19, 20, 21, 22]
    nxt = eng.prefill(1, seq)
    ref = _llama_ref(cfg, wf, seq)[-1]
    assert (eng.last_logits(1) - ref).abs().max() < 0.12
    for step in range(12):  # crosses the window size so the ring cache wraps
        seq.append(nxt)
        nxt = eng.decode({1: seq[-1]})[1]
        ref = _llama_ref(cfg, wf, seq)[-1]
        err = float((eng.last_logits(1) - ref).abs().max())
        assert err < 0.15, (step, err)


def test_generate_continuous_batching_is_order_independent():
    from neuralfn_b200.serving import EngineConfig, ResidentEngine, Sampling
    cfg, params = _gpt2_setup()
    eng = ResidentEngine(EngineConfig.gpt2(cfg, max_batch=2))
    eng.load_named_tensors(params)
    prompts = [[1, 2, 3], [400, 5], [9, 9, 9, 9, 9], [77], [5, 6, 7, 8]]
    a = eng.generate(prompts, max_new_tokens=6)
    b = [eng.generate([p], max_new_tokens=6)[0] for p in prompts]
    assert a == b and all(len(x) == 6 for x in a)
    c = eng.generate(prompts[:2], max_new_tokens=5, sampling=Sampling(temperature=1.0, top_k=20, seed=3))
    assert all(0 <= t < cfg.vocab_size for seq in c for t in seq)


def _glimmer_ref(cfg, w, tokens):
    """fp32 reference of the Glimmer block layout (see EngineConfig.glimmer)."""
    T = len(tokens)
    hd, Hq, Hkv, C, F_ = cfg.head_dim, cfg.n_head, cfg.n_kv_head, cfg.d_model, cfg.d_ff

    def rms(v, wt, eps, centered):
        y = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
        return y if wt is None else y * ((1 + wt) if centered else wt)

    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2).double() / hd))
    ang = torch.outer(torch.arange(T).double(), inv)
    cos, sin = ang.cos().float()[:, None], ang.sin().float()[:, None]

    def rope(v):
        a, b = v[..., :hd // 2], v[..., hd // 2:]
        return torch.cat((a * cos - b * sin, b * cos + a * sin), -1)

    x = rms(w["tok_embeddings"][torch.tensor(tokens)], None, cfg.norm_eps, False)
    for l in range(cfg.n_layer):
        local = (l + 1) % cfg.global_every != 0
        n = rms(x, w[f"layers.{l}.attn_norm"], cfg.norm_eps, True)
        p = n @ w[f"layers.{l}.wqkv"].T
        q = p[:, :Hq * hd].view(T, Hq, hd)
        k = p[:, Hq * hd:(Hq + Hkv) * hd].view(T, Hkv, hd)
        v = p[:, (Hq + Hkv) * hd:(Hq + 2 * Hkv) * hd].view(T, Hkv, hd)
        g = p[:, (Hq + 2 * Hkv) * hd:]
        q, k = rms(q, None, cfg.qk_norm_eps, False), rms(k, None, cfg.qk_norm_eps, False)
        if local:
            q, k = rope(q), rope(k)
        q = q * cfg.q_scale
        k, v = k.repeat_interleave(Hq // Hkv, 1), v.repeat_interleave(Hq // Hkv, 1)
        s = torch.einsum("thd,shd->hts", q, k) / math.sqrt(hd)
        i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
        mask = (j <= i) & ((i - j < cfg.window) if local else True)
        a = torch.einsum("hts,shd->thd", s.masked_fill(~mask, float("-inf")).softmax(-1), v).reshape(T, Hq * hd)
        a = a * torch.sigmoid(g)
        x = x + rms(a @ w[f"layers.{l}.wo"].T, w[f"layers.{l}.post_attn_norm"], cfg.post_norm_eps, True)
        m = rms(x, w[f"layers.{l}.ffn_norm"], cfg.norm_eps, True)
        gu = m @ w[f"layers.{l}.w_gate_up"].T
        f = (F.silu(gu[:, :F_]) * gu[:, F_:]) @ w[f"layers.{l}.w_down"].T
        x = x + rms(f, w[f"layers.{l}.post_ffn_norm"], cfg.post_norm_eps, True)
    logits = cfg.output_multiplier * (rms(x, w["norm"], cfg.norm_eps, False) @ w["lm_head"].T)
    return (cfg.logit_softcap * torch.tanh(logits / cfg.logit_softcap))[:, :cfg.vocab]


def test_glimmer_layout_matches_reference():
    from neuralfn_b200.serving import EngineConfig, ResidentEngine
    cfg = EngineConfig.glimmer(n_layer=4, d_model=256, n_head=4, n_kv_head=2, head_dim=128, d_ff=512, vocab=500, max_seq=64, window=12,
                               max_batch=2)
    eng = ResidentEngine(cfg)
    g = torch.Generator().manual_seed(2)
    w, shapes = {}, {"tok_embeddings": (512, 256), "lm_head": (512, 256)}
    for l in range(4):
        shapes.update({f"layers.{l}.wqkv": ((4 + 4 + 4) * 128, 256), f"layers.{l}.wo": (256, 512), f"layers.{l}.w_gate_up": (1024, 256),
                       f"layers.{l}.w_down": (256, 512)})
    for name, numel in eng.expected_tensors().items():
        if "norm" in name:
            w[name] = (0.1 * torch.randn(numel, generator=g)).bfloat16() if name != "norm" else (1 + 0.1 * torch.randn(numel, generator=g)).bfloat16()
        else:
            w[name] = (torch.randn(numel, generator=g) * 0.05).bfloat16()
    eng.load_named_tensors(w)
    wf = {k: (v.float().view(*shapes[k]) if k in shapes else v.float()) for k, v in w.items()}
    seq = [3, 99, 401, 7, 7, 320, 64, 2, 11, 450, 13, 14, 15, 16, 17, 18]
    nxt = eng.prefill(0, seq)
    ref = _glimmer_ref(cfg, wf, seq)[-1]
    assert (eng.last_logits(0) - ref).abs().max() < 0.1, float((eng.last_logits(0) - ref).abs().max())
    for step in range(10):
        seq.append(nxt)
        nxt = eng.decode({0: seq[-1]})[0]
        err = float((eng.last_logits(0) - _glimmer_ref(cfg, wf, seq)[-1]).abs().max())
        assert err < 0.12, (step, err)


def _small_llama_engine(window=0, max_batch=3, hd=64, max_seq=96):
    from neuralfn_b200.serving import EngineConfig, ResidentEngine
    cfg = EngineConfig(family=1, n_layer=3, d_model=256, n_head=4, n_kv_head=2, head_dim=hd, d_ff=512, vocab=777, padded_vocab=784,
                       max_seq=max_seq, max_batch=max_batch, qk_norm=2, rope_hf=1, rope_theta=10000.0, norm_eps=1e-5, tie_embeddings=0,
                       window=window, global_every=3 if window else 0)
    eng = ResidentEngine(cfg)
    g = torch.Generator().manual_seed(5)
    w = {}
    for name, numel in eng.expected_tensors().items():
        w[name] = ((1 + 0.1 * torch.randn(numel, generator=g)) if name.endswith("norm") else torch.randn(numel, generator=g) * 0.04).bfloat16()
    eng.load_named_tensors(w)
    return eng


@pytest.mark.parametrize("window,hd", [(0, 64), (16, 128)])
def test_verify_matches_sequential_decode_and_commit_is_prefix_exact(window, hd):
    eng = _small_llama_engine(window, hd=hd)
    eng.enable_verify(8)
    prompt = [3, 99, 501, 7, 7, 320, 64, 2, 11, 600, 13, 14, 15, 16, 17, 18, 19, 20, 21, 22]
    # slot 1: plain greedy decoding is the oracle
    t = eng.prefill(1, prompt)
    oracle, logits = [t], []
    for _ in range(7):
        t = eng.decode({1: t})[1]
        oracle.append(t)
        logits.append(eng.last_logits(1))
    # slot 0: verify the oracle's first 6 tokens as one block: every row must predict the next oracle token
    first = eng.prefill(0, prompt)
    assert first == oracle[0]
    got = eng.verify({0: oracle[:6]})[0]
    for r in range(6):
        lv = eng.verify_logits(0, r)
        assert float((lv - logits[r]).abs().max()) < 0.12, r
        assert int(lv.argmax()) == got[r]                             # the device argmax is the argmax of the row it returns
        assert float(logits[r][oracle[r + 1]] - logits[r][got[r]]) < 0.25  # and at worst a near-tie of the oracle's choice
    assert eng.slot_length(0) == len(prompt)  # nothing was appended yet
    # accept 4 rows, then continue with single-token decoding on the oracle's tokens: same logits as the oracle saw
    eng.commit({0: 4})
    assert eng.slot_length(0) == len(prompt) + 4
    assert float((eng.last_logits(0) - logits[3]).abs().max()) < 0.12
    for i in range(4, 7):
        eng.decode({0: oracle[i]})
        assert float((eng.last_logits(0) - logits[i]).abs().max()) < 0.12, i


def test_append_truncate_and_fork():
    eng = _small_llama_engine(0)
    prompt = list(range(5, 45))
    full_next = eng.prefill(0, prompt)
    ref = eng.last_logits(0)
    # the same tokens through prefill(…20) + append(20 more, in chunks of 8)
    eng.prefill(1, prompt[:20])
    nxt = eng.append(1, prompt[20:], chunk=8)
    assert eng.slot_length(1) == 40
    assert float(ref[full_next] - ref[nxt]) < 0.25
    assert float((eng.last_logits(1) - ref).abs().max()) < 0.12
    # fork the first 30 tokens into slot 2 and finish there
    eng.fork(0, 2, 30)
    assert eng.slot_length(2) == 30
    eng.append(2, prompt[30:])
    assert float((eng.last_logits(2) - ref).abs().max()) < 0.12
    # truncate slot 0 to 30 tokens and replay the tail
    eng.truncate(0, 30)
    eng.append(0, prompt[30:])
    assert float((eng.last_logits(0) - ref).abs().max()) < 0.12
    with pytest.raises(Exception):
        eng.truncate(0, 1000)

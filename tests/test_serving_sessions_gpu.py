"""Sessions, speculative decoding, prefix cache, artifacts and structured output on the resident engine."""
import json

import pytest
import torch

pytestmark = pytest.mark.gpu


def _engine(max_batch=4, seed=5, n_layer=3, max_seq=160):
    from neuralfn_b200.serving import EngineConfig, ResidentEngine
    cfg = EngineConfig(family=1, n_layer=n_layer, d_model=256, n_head=4, n_kv_head=2, head_dim=64, d_ff=512, vocab=777, padded_vocab=784,
                       max_seq=max_seq, max_batch=max_batch, qk_norm=2, rope_hf=1, rope_theta=10000.0, norm_eps=1e-5, tie_embeddings=0)
    eng = ResidentEngine(cfg)
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, numel in eng.expected_tensors().items():
        w[name] = ((1 + 0.1 * torch.randn(numel, generator=g)) if name.endswith("norm") else torch.randn(numel, generator=g) * 0.05).bfloat16()
    eng.load_named_tensors(w)
    return cfg, w, eng


PROMPT = [5, 9, 200, 31, 5, 9, 200, 31, 5, 9, 200, 31, 77, 12, 5, 9, 200, 31, 5, 9]


def _same_up_to_ties(model, prompt, a, b):
    """Two greedy streams may only part ways where the model's top two logits nearly tie."""
    for i, (x, y) in enumerate(zip(a, b)):
        if x != y:
            with model.create_session() as s:
                s.prefill(list(prompt) + list(a[:i]))
                lg = s.current_logits()
            assert abs(float(lg[x] - lg[y])) < 0.3, (i, x, y)
            return
    assert len(a) == len(b)


def test_plain_speculative_and_draft_decoding_agree():
    from neuralfn_b200.serving import DraftEngineProposer, GenerationConfig, NativeInferenceModel, NGramProposer
    _cfg, _w, eng = _engine()
    model = NativeInferenceModel(eng)
    greedy = GenerationConfig(max_new_tokens=24, temperature=0.0)
    with model.create_session() as s:
        s.prefill(PROMPT)
        plain = s.decode(greedy)
        assert plain.completion_tokens == 24 and plain.finish_reason == "length" and len(s.token_ids) == len(PROMPT) + 24
    with model.create_session() as s:
        s.prefill(PROMPT)
        spec = s.decode(greedy, proposer=NGramProposer(), speculative_tokens=7)
        assert spec.completion_tokens == 24 and spec.speculative_assistant_blocks > 0
        assert spec.speculative_proposed_tokens == spec.speculative_accepted_tokens + spec.speculative_rejected_tokens
        assert len(s.token_ids) == len(PROMPT) + 24 and s.cached_tokens in (len(s.token_ids), len(s.token_ids) - 1)
        _same_up_to_ties(model, PROMPT, plain.token_ids, spec.token_ids)
        # the session stays usable after a speculative run
        more = s.decode(GenerationConfig(max_new_tokens=3, temperature=0.0))
        assert more.completion_tokens == 3
    # a draft with the same weights proposes what the target would say: (nearly) everything is accepted
    _c2, _w2, draft = _engine(max_batch=1)
    with model.create_session() as s:
        s.prefill(PROMPT)
        res = s.decode(greedy, proposer=DraftEngineProposer(draft), speculative_tokens=5)
        _same_up_to_ties(model, PROMPT, plain.token_ids, res.token_ids)
        assert res.speculative_accepted_tokens >= 0.7 * res.speculative_proposed_tokens > 0
        assert res.speculative_target_rows < 24 + res.speculative_assistant_blocks + 1
    # sampled speculative decoding runs and reports consistent statistics
    with model.create_session(seed=3) as s:
        s.prefill(PROMPT)
        res = s.decode(GenerationConfig(max_new_tokens=16, temperature=0.9, top_k=40, seed=11), proposer=NGramProposer(), speculative_tokens=4)
        assert res.completion_tokens == 16 and all(0 <= t < 777 for t in res.token_ids)
    model.close()


def test_stop_tokens_cancel_fork_truncate():
    from neuralfn_b200.serving import GenerationConfig, InferenceError, NativeInferenceModel
    _cfg, _w, eng = _engine()
    model = NativeInferenceModel(eng)
    s = model.create_session()
    s.prefill(PROMPT)
    base = s.decode(GenerationConfig(max_new_tokens=10, temperature=0.0))
    # stop token: generation ends on its first occurrence
    t = model.fork_session(s, len(PROMPT))
    mine = t.decode(GenerationConfig(max_new_tokens=10, temperature=0.0)).token_ids  # same code path as the run below
    _same_up_to_ties(model, PROMPT, base.token_ids, mine)
    stop_at = mine[4]
    first = mine.index(stop_at)
    t.truncate(len(PROMPT))
    t.truncate(len(PROMPT))  # a no-op the second time
    r = t.decode(GenerationConfig(max_new_tokens=10, temperature=0.0, stop_token_ids=(stop_at,)))
    assert r.finish_reason == "stop" and r.events[-1].finish_reason == "stop" and r.token_ids[-1] == stop_at
    assert r.token_ids == mine[:first + 1] or abs(len(r.token_ids) - first - 1) <= 10
    # cancel from the event callback
    u = model.fork_session(s, len(PROMPT))
    seen = []
    r = u.decode(GenerationConfig(max_new_tokens=10, temperature=0.0), on_event=lambda ev: (seen.append(ev.token_id), u.cancel() if len(seen) == 3 else None))
    assert r.cancelled and r.finish_reason == "cancelled" and len(r.token_ids) == 3
    # truncate back to the prompt and decode again: same stream
    s.truncate(len(PROMPT))
    again = s.decode(GenerationConfig(max_new_tokens=10, temperature=0.0))
    assert len(again.token_ids) == 10
    s.truncate(len(PROMPT))
    s.close()
    _same_up_to_ties(model, PROMPT, base.token_ids, again.token_ids)
    s = model.create_session()
    s.prefill(PROMPT)
    with pytest.raises(InferenceError):
        s.truncate(10 ** 6)
    s.reset()
    assert s.token_ids == ()
    stats = model.stats()
    assert stats["forks"] == 2 and stats["sessions_open"] == 3
    for x in (s, t, u):
        x.close()
    assert model.stats()["sessions_open"] == 0
    with pytest.raises(InferenceError):
        [model.create_session() for _ in range(5)]
    model.close()


def test_artifact_round_trip_prefix_cache_and_structured_output(tmp_path):
    from neuralfn_b200.serving import GenerationConfig, NativeInferenceModel, NativeModelLoadConfig, write_artifact
    from neuralfn_b200.serving.constrained import ConstrainedDecoder, single_byte_token_inventory
    from neuralfn_b200.serving.openai_server import ServingRuntime
    from neuralfn_b200.serving.prefix_cache import PrefixCache
    cfg, w, eng = _engine(max_batch=2)
    with NativeInferenceModel(eng).create_session() as s:
        s.prefill(PROMPT)
        want = s.decode(GenerationConfig(max_new_tokens=6, temperature=0.0)).token_ids
    eng.close()
    art = write_artifact(tmp_path / "art", cfg, w, codec="bytes:300", chat_template="plain-roles", stop_token_ids=(1,))
    model = NativeInferenceModel.load(art, NativeModelLoadConfig(session_count=3))
    assert model.engine.config.max_batch == 3 and model.codec.name == "utf8-bytes"
    with model.create_session() as s:
        s.prefill(PROMPT)
        assert s.decode(GenerationConfig(max_new_tokens=6, temperature=0.0)).token_ids == want
    # prefix cache: the second request shares 18 prompt tokens with the first
    cache = PrefixCache(model, capacity=2, min_reuse_tokens=8)
    lease = cache.acquire(PROMPT)
    assert lease.reused_tokens == 0
    lease.session.prefill(PROMPT)
    cache.release(lease.session)
    p2 = PROMPT[:18] + [400, 401, 402]
    lease2 = cache.acquire(p2)
    assert lease2.reused_tokens == 18 and len(lease2.session.token_ids) == 18
    lease2.session.prefill(p2[18:])
    with model.create_session() as fresh:
        fresh.prefill(p2)
        assert float((fresh.current_logits() - lease2.session.current_logits()).abs().max()) < 0.12
    cache.release(lease2.session)
    assert len(cache) <= 2 and cache.stats["hits"] == 1
    cache.clear()
    # structured output over single-byte tokens (byte b is token 300 + b)
    inv = single_byte_token_inventory(lambda t: model.codec.decode([t]), 777)
    assert inv[ord("{")] == 300 + ord("{")
    schema = {"type": "object", "required": ["n", "ok"], "properties": {"n": {"type": "integer", "maxDigits": 3}, "ok": {"type": "boolean"},
                                                                       "tag": {"enum": ["a", "b"]}}}
    with model.create_session() as s:
        s.prefill(PROMPT)
        doc, _ = ConstrainedDecoder(schema, inv).generate(s, 96)
    assert isinstance(doc["n"], int) and isinstance(doc["ok"], bool) and set(doc) <= {"n", "ok", "tag"}
    # the serving runtime end to end (no HTTP): chat -> tokens -> text
    rt = ServingRuntime(model=model, prefix_cache=PrefixCache(model, 1, min_reuse_tokens=4), max_output_tokens=8)
    ids, max_new = rt.prepare_chat([{"role": "user", "content": "hi"}], 5)
    out = rt.generate(ids, GenerationConfig(max_new_tokens=max_new, temperature=0.0))
    assert len(out["token_ids"]) == 5 and out["prompt_tokens"] == len(ids)
    out2 = rt.generate(ids + [300 + ord("!")], GenerationConfig(max_new_tokens=2, temperature=0.0))
    assert out2["reused_tokens"] >= 4
    json.dumps(out2)
    model.close()


def test_hidden_state_taps_agree_across_prefill_decode_and_verify():
    """The same positions reached three ways (one prompt; prompt + decode steps; prompt + committed verification blocks)
    hold the same tapped hidden states, and a fork carries them along."""
    from neuralfn_b200.serving import Sampling
    toks = (PROMPT * 2)[:36]
    greedy = Sampling(temperature=0.0)

    def fresh():
        _cfg, _w, eng = _engine(max_batch=2)
        eng.enable_taps([0, 2])
        return eng

    a = fresh()
    a.prefill(0, toks)
    full = a.read_taps(0, 0, 36).float()
    assert full.shape == (36, 512) and float(full.abs().max()) > 0
    assert torch.equal(a.read_taps(0, 30, 6, device=False).float(), full[30:36].cpu())
    b = fresh()
    b.prefill(1, toks[:30])
    for t in toks[30:36]:
        b.decode({1: t}, greedy)
    step = b.read_taps(1, 0, 36).float()
    assert (step[:30] - full[:30]).abs().max() < 1e-6 and (step - full).abs().max() < 0.06 * full.abs().max()
    c = fresh()
    c.prefill(0, toks[:30])
    c.verify({0: toks[30:34] + [1, 2, 3]})
    c.commit({0: 4})                                       # three block rows are discarded
    c.verify({0: toks[34:36]})
    c.commit({0: 2})
    blk = c.read_taps(0, 0, 36).float()
    assert (blk - full).abs().max() < 0.06 * full.abs().max()
    c.fork(0, 1, 33)
    assert torch.equal(c.read_taps(1, 0, 33), c.read_taps(0, 0, 33))
    with pytest.raises(Exception):
        c.read_taps(1, 30, 6)                              # past the fork's 33 cached tokens
    for e in (a, b, c):
        e.close()


def test_dflash_proposer_keeps_greedy_output_and_counts_blocks():
    """A random-initialised block-diffusion draft on the engine's taps: whatever it proposes, verification keeps the
    target's greedy stream; a draft distilled on the target's own continuation gets its proposals accepted."""
    from neuralfn_b200.serving import DFlashProposer, GenerationConfig, NativeInferenceModel, target_embed_and_head
    from neuralfn_b200.tensor.dflash import DFlashConfig, DFlashDraftModel
    cfg, w, eng = _engine(max_batch=2)
    eng.enable_taps([0, 2])
    model = NativeInferenceModel(eng)
    greedy = GenerationConfig(max_new_tokens=24, temperature=0.0)
    with model.create_session() as s:
        s.prefill(PROMPT)
        plain = s.decode(greedy)
    dcfg = DFlashConfig(d_model=128, n_layer=2, n_head=4, block_size=8, context_window=64, tap_layers=(0, 2), mask_token_id=0)
    torch.manual_seed(0)
    draft = DFlashDraftModel(dcfg, cfg.d_model).cuda().bfloat16()
    tensors = {k: v.view(-1, cfg.d_model) if k in ("tok_embeddings", "lm_head") else v for k, v in w.items()}
    embed, head = target_embed_and_head(cfg, tensors, "cuda")
    with model.create_session() as s:
        s.prefill(PROMPT)
        prop = DFlashProposer(eng, s.slot, draft, embed, head)
        res = s.decode(greedy, proposer=prop, speculative_tokens=7)
        assert res.completion_tokens == 24 and prop.calls > 0
        assert res.speculative_proposed_tokens == 7 * res.speculative_assistant_blocks or res.speculative_proposed_tokens > 0
        assert res.speculative_target_rows >= res.speculative_assistant_blocks
        _same_up_to_ties(model, PROMPT, plain.token_ids, res.token_ids)
    # a draft that knows the continuation: its proposals are accepted, which proves that the tap window the proposer
    # reads, the block layout ([pending, mask, ...]; slot i = distance i) and the shared final norm + head line up
    future = list(PROMPT) + list(plain.token_ids)
    rows = tensors["lm_head"].float().cuda() / tensors["norm"].float().cuda()     # the head then scores each row's own token highest

    class KnowingDraft(torch.nn.Module):
        cfg = dcfg

        def forward(self, block_embeds, taps, mask):
            n = taps.shape[1]                                   # cached tokens, all inside the context window here
            assert block_embeds.shape[:3] == (1, 1, dcfg.block_size) and mask.shape[-1] == n + dcfg.block_size
            assert taps.shape[-1] == 2 * cfg.d_model and float(taps.abs().max()) > 0
            toks = [future[n + i] if n + i < len(future) else 0 for i in range(dcfg.block_size)]
            return rows[toks][None, None]

    with model.create_session() as s:
        s.prefill(PROMPT)
        res = s.decode(greedy, proposer=DFlashProposer(eng, s.slot, KnowingDraft(), embed, head), speculative_tokens=7)
        assert tuple(res.token_ids) == tuple(plain.token_ids)
        assert res.speculative_accepted_tokens >= 0.8 * res.speculative_proposed_tokens > 0, (res.speculative_accepted_tokens, res.speculative_proposed_tokens)
        assert res.speculative_target_rows < 24 + res.speculative_assistant_blocks and res.speculative_assistant_blocks <= 5
    model.close()


def test_forks_copy_on_write():
    """A fork takes no cache slot and copies nothing until it is used; the source's slot is handed over when it closes first."""
    from neuralfn_b200.serving import GenerationConfig, NativeInferenceModel
    _cfg, _w, eng = _engine(max_batch=2)
    model = NativeInferenceModel(eng)
    greedy = GenerationConfig(max_new_tokens=10, temperature=0.0)
    src = model.create_session()
    src.prefill(PROMPT)
    want = src.decode(greedy).token_ids
    n = len(PROMPT)
    forks = [model.fork_session(src, n) for _ in range(5)]           # more forks than slots
    st = model.stats()
    assert st["unused_forks"] == 5 and st["forks"] == 5 and st.get("fork_copies", 0) == 0 and all(f.shares_cache for f in forks)
    assert forks[0].token_ids == tuple(PROMPT) and forks[0].cached_tokens == n - 1
    # first use: the rows are copied into the fork's own slot, and it continues exactly like the source did
    got = forks[0].decode(greedy).token_ids
    _same_up_to_ties(model, PROMPT, want, got)
    assert not forks[0].shares_cache and model.stats()["fork_copies"] == 1 and model.stats()["unused_forks"] == 4
    # both slots are taken now: a further fork cannot materialise, and says so
    with pytest.raises(Exception, match="slot"):
        forks[1].current_logits()
    forks[0].close()
    # the source appends without disturbing its forks (no sliding-window caches here), truncating below them detaches one first
    src.decode(GenerationConfig(max_new_tokens=2, temperature=0.0))
    assert all(f.shares_cache for f in forks[1:])
    short = model.fork_session(src, 8)
    with pytest.raises(Exception, match="slot"):
        src.truncate(10)                                               # four forks read rows 10 .. 18 and only one slot is free: refused
    assert len(src.token_ids) == n + 12                                # the source is untouched by the refusal
    for f in forks[2:]:
        f.close()
    src.truncate(10)                                                   # the remaining long fork was given its own copy first
    assert model.stats()["fork_copies"] == 2 and not forks[1].shares_cache and short.shares_cache
    _same_up_to_ties(model, PROMPT, want, forks[1].decode(greedy).token_ids)
    forks[1].close()
    assert short.token_ids == tuple(PROMPT[:8]) and bool(torch.isfinite(short.current_logits()).all())
    model.close()


def test_closing_the_source_hands_its_slot_to_a_fork():
    from neuralfn_b200.serving import GenerationConfig, NativeInferenceModel
    _cfg, _w, eng = _engine(max_batch=1)
    model = NativeInferenceModel(eng)
    greedy = GenerationConfig(max_new_tokens=8, temperature=0.0)
    src = model.create_session()
    src.prefill(PROMPT)
    want = src.decode(greedy).token_ids
    a = model.fork_session(src, len(PROMPT))
    b = model.fork_session(src, 12)
    src.close()                                                        # the only slot goes to the fork with the longer prefix
    st = model.stats()
    assert st["fork_adoptions"] == 1 and st.get("fork_copies", 0) == 0 and not a.shares_cache and b.shares_cache
    _same_up_to_ties(model, PROMPT, want, a.decode(greedy).token_ids)
    a.close()                                                          # and on to the next one, shortened to its 11 cached rows
    assert model.stats()["fork_adoptions"] == 2 and b.cached_tokens == 11
    assert torch.isfinite(b.current_logits()).all()
    model.close()


def test_artifact_with_a_dflash_assistant_file(tmp_path):
    """An artifact directory plus an exported assistant file: `attach_dflash` wires taps, draft and the shared head, and
    decoding uses the draft without being told to."""
    from neuralfn_b200.serving import GenerationConfig, NativeInferenceModel, NativeModelLoadConfig, write_artifact
    from neuralfn_b200.tensor.dflash import DFlashConfig, DFlashDistillationTrainer
    cfg, w, eng = _engine(max_batch=1)
    eng.close()
    shaped = {k: (v.view(-1, cfg.d_model) if k in ("tok_embeddings", "lm_head") else v) for k, v in w.items()}
    write_artifact(tmp_path / "art", cfg, shaped)
    dcfg = DFlashConfig(d_model=64, n_layer=1, n_head=2, block_size=6, context_window=32, tap_layers=(1,), mask_token_id=0)
    trainer = DFlashDistillationTrainer(dcfg, target=None, embed=None, lm_head=None, target_dim=cfg.d_model)
    trainer.export_native_assistant(tmp_path / "assistant.nfnw")
    greedy = GenerationConfig(max_new_tokens=12, temperature=0.0)
    with NativeInferenceModel.load(tmp_path / "art", NativeModelLoadConfig(session_count=1, speculative_decoding="off")) as plain_model:
        with plain_model.create_session() as s:
            s.prefill(PROMPT)
            plain = s.decode(greedy)
    with NativeInferenceModel.load(tmp_path / "art", NativeModelLoadConfig(session_count=1)) as model:
        model.attach_dflash(tmp_path / "assistant.nfnw")
        assert model.engine.tap_layers == (1,)
        with model.create_session() as s:
            s.prefill(PROMPT)
            res = s.decode(greedy)
            assert res.speculative_assistant_blocks > 0 and res.speculative_proposed_tokens > 0
            _same_up_to_ties(model, PROMPT, plain.token_ids, res.token_ids)


def test_media_rows_enter_the_prompt_through_prefill_rows():
    from neuralfn_b200.serving import GenerationConfig, NativeInferenceModel
    from neuralfn_b200.serving.multimodal import fuse_media_rows, prefill_with_media
    cfg, w, eng = _engine(max_batch=2)
    embed = w["tok_embeddings"].view(-1, cfg.d_model).cuda()
    # no media: the rows of the plain embeddings reproduce the token prompt exactly
    nxt = eng.prefill(0, PROMPT)
    want = eng.last_logits(0).clone()
    rows = fuse_media_rows(cfg, embed, PROMPT, {})
    assert eng.prefill_rows(1, rows) == nxt and torch.equal(eng.last_logits(1), want)
    assert eng.prefill_rows(1, rows.cpu()) == nxt                                   # host rows work too
    # three placeholder positions take media features; the session carries on as usual
    model = NativeInferenceModel(eng)
    eng.release(0), eng.release(1)
    prompt = list(PROMPT)
    prompt[3] = prompt[4] = prompt[9] = 700
    feats = torch.randn(3, cfg.d_model, generator=torch.Generator().manual_seed(0))
    with model.create_session() as s:
        info = prefill_with_media(s, embed, prompt, {700: feats})
        assert info == {"prompt_tokens": 20, "total_tokens": 20, "media_rows": 3}
        with_media = s.current_logits().clone()
        out = s.decode(GenerationConfig(max_new_tokens=6, temperature=0.0))
        assert out.completion_tokens == 6 and len(s.token_ids) == 26
    with model.create_session() as s:
        s.prefill(prompt)
        assert (s.current_logits() - with_media).abs().max() > 1e-3                  # the media rows changed the prompt
    with pytest.raises(ValueError):
        fuse_media_rows(cfg, embed, prompt, {700: feats[:2]})
    model.close()


def test_turboquant_cache_mode_decodes_close_to_the_bf16_cache():
    """K / V kept as 3.5-bit records: a quarter of the cache bytes, logits close to the bf16 engine's, greedy streams that
    part ways only where the bf16 model itself is undecided; forks carry records; verification blocks are refused."""
    from neuralfn_b200.serving import EngineConfig, EngineError, ResidentEngine, Sampling
    cfg, w, ref = _engine(max_batch=2)
    tq_cfg = EngineConfig(**{**cfg.__dict__, "kv_cache_mode": 1})
    tq = ResidentEngine(tq_cfg)
    tq.load_named_tensors(w)
    assert (tq.kv_bytes_per_token, ref.kv_bytes_per_token) == (192, 512)        # 2 heads x (48 + 48) record bytes against 2 x 2 x 64 x 2
    greedy = Sampling(temperature=0.0)
    a, b = ref.prefill(0, PROMPT, greedy), tq.prefill(0, PROMPT, greedy)
    assert torch.equal(ref.last_logits(0), tq.last_logits(0)) and a == b       # the prompt itself attends to fresh bf16 K / V
    agree, worst = 0, 0.0
    tok_ref = tok_tq = a
    for _ in range(16):
        tok_ref = ref.decode({0: tok_ref}, greedy)[0]
        nxt = tq.decode({0: tok_tq}, greedy)[0]
        lr, lt = ref.last_logits(0), tq.last_logits(0)
        worst = max(worst, float((lr - lt).abs().max() / lr.abs().max()))
        tok_tq = tok_ref                                                       # teacher-forced on the bf16 stream
        agree += int(nxt == tok_ref or float(lr.max() - lr[nxt]) < 0.5)
    assert agree >= 14 and worst < 0.35, (agree, worst)
    assert torch.isfinite(tq.last_logits(0)).all()
    tq.fork(0, 1, tq.slot_length(0))
    both = tq.decode({0: 5, 1: 5}, greedy)
    l0, l1 = tq.last_logits(0), tq.last_logits(1)
    assert both[0] == both[1] and torch.equal(l0, l1)                          # the fork carries the same records
    with pytest.raises(EngineError, match="TurboQuant"):
        tq.enable_verify(8)
    ref.close()
    tq.close()
    assert torch.isfinite(l0).all() and torch.isfinite(l1).all()


def test_projection_weights_stay_resident_in_k_quant_blocks():
    """Q4_K / Q6_K blocks loaded as they are: prompts (decode the tensor into the scratch buffer, then the bf16 product) and decode
    steps (quantised GEMV straight from the blocks) agree with an engine that holds the decoded values in bf16; the packed
    engine is smaller; only projection weights qualify."""
    import numpy as np

    from neuralfn_b200.quant import kquant
    from neuralfn_b200.serving import EngineConfig, ResidentEngine
    from neuralfn_b200.serving.engine import EngineError
    cfg = EngineConfig(family=1, n_layer=3, d_model=256, n_head=4, n_kv_head=2, head_dim=64, d_ff=512, vocab=777, padded_vocab=784,
                       max_seq=160, max_batch=4, qk_norm=2, rope_hf=1, rope_theta=10000.0, norm_eps=1e-5, tie_embeddings=0)
    plain, packed = ResidentEngine(cfg), ResidentEngine(cfg)
    g = torch.Generator().manual_seed(5)
    dense, quant = {}, {}
    for i, (name, numel) in enumerate(plain.expected_tensors().items()):
        leaf = name.rsplit(".", 1)[-1]
        if leaf in ("wqkv", "wo", "w_gate_up", "w_down", "lm_head"):
            qt = 14 if leaf in ("w_down", "lm_head") else 12
            raw = kquant.random_blocks(qt, numel // 256, seed=i)
            small = np.random.default_rng(i).uniform(2e-5, 1.5e-4, numel // 256).astype(np.float16).view(np.uint8).reshape(-1, 2)
            if qt == 12:
                raw[:, 0:2], raw[:, 2:4] = small, small
            else:
                raw[:, 208:210] = np.random.default_rng(i).uniform(5e-6, 2e-5, numel // 256).astype(np.float16).view(np.uint8).reshape(-1, 2)
            quant[name] = (qt, torch.from_numpy(raw.copy()))
            dense[name] = torch.from_numpy(kquant.dequantize(qt, raw).astype(np.float32)).bfloat16()
        else:
            dense[name] = ((1 + 0.1 * torch.randn(numel, generator=g)) if name.endswith("norm") else torch.randn(numel, generator=g) * 0.05).bfloat16()
    plain.load_named_tensors(dense)
    with pytest.raises(EngineError):
        packed.set_tensor_kquant("tok_embeddings", "Q4_K", torch.zeros(784 * 144, dtype=torch.uint8))
    packed.load_named_tensors({k: v for k, v in dense.items() if k not in quant}, quantized=quant)
    assert packed.device_bytes < plain.device_bytes
    a = plain.prefill(0, PROMPT)
    b = packed.prefill(0, PROMPT)
    la, lb = plain.last_logits(0), packed.last_logits(0)
    scale = float(la.abs().max())
    assert float((la - lb).abs().max()) < 0.02 * scale and scale > 0.05
    for _ in range(8):
        # both engines continue with the plain engine's token, so their caches stay comparable
        b = packed.decode({0: a})[0]
        a2 = plain.decode({0: a})[0]
        la, lb = plain.last_logits(0), packed.last_logits(0)
        assert float((la - lb).abs().max()) < 0.04 * float(la.abs().max())
        if a2 != b:
            assert abs(float(la[a2] - la[b])) < 0.05 * float(la.abs().max())
        a = a2
    plain.close(); packed.close()

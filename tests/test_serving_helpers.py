"""CPU checks of the serving helpers around the resident engine: media fusion rows, the shared target head, the DFlash
proposer (on a stand-in engine that serves stored taps) and the mixture-of-activations record."""
import json

import pytest
import torch

from neuralfn_b200.serving.engine import EngineConfig
from neuralfn_b200.serving.inference import DFlashProposer, InferenceError, target_embed_and_head
from neuralfn_b200.serving.multimodal import fuse_media_rows


def _cfg(**kw):
    base = dict(family=1, n_layer=2, d_model=32, n_head=2, n_kv_head=1, head_dim=16, d_ff=64, vocab=50, padded_vocab=56, max_seq=64, max_batch=2,
                norm_eps=1e-5, tie_embeddings=0)
    base.update(kw)
    return EngineConfig(**base)


def test_media_rows_replace_placeholders_in_order_and_are_normalised_like_embeddings():
    cfg = _cfg(embed_norm=1)
    g = torch.Generator().manual_seed(0)
    embed = torch.randn(56, 32, generator=g).bfloat16()
    ids = [3, 40, 7, 40, 40, 9]
    feats = torch.randn(3, 32, generator=g) * 5
    rows = fuse_media_rows(cfg, embed, ids, {40: feats}).float()
    rms = lambda x: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5)  # noqa: E731
    assert torch.allclose(rows[0], rms(embed[3].float()), atol=2e-2) and torch.allclose(rows[[1, 3, 4]], rms(feats), atol=2e-2)
    assert rows.shape == (6, 32) and abs(float(rows.pow(2).mean(-1).sqrt().mean()) - 1.0) < 0.02
    plain = fuse_media_rows(_cfg(), embed, ids, {})
    assert torch.equal(plain, embed[torch.tensor(ids)])                      # no norm, no media: the embedding rows themselves
    already = fuse_media_rows(cfg, embed, ids, {40: feats}, features_normalised=True).float()
    assert torch.allclose(already[1], feats[0].bfloat16().float(), atol=1e-6)
    with pytest.raises(ValueError, match="placeholders"):
        fuse_media_rows(cfg, embed, ids, {40: feats[:2]})


def test_target_head_is_final_norm_projection_multiplier_and_cap():
    cfg = _cfg(logit_softcap=5.0, output_multiplier=0.5)
    g = torch.Generator().manual_seed(1)
    t = {"tok_embeddings": torch.randn(56, 32, generator=g), "lm_head": torch.randn(56, 32, generator=g), "norm": 1 + 0.1 * torch.randn(32, generator=g)}
    embed, head = target_embed_and_head(cfg, t, "cpu")
    h = torch.randn(4, 32, generator=g)
    want = (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5) * t["norm"]).bfloat16() @ t["lm_head"].bfloat16().T
    want = 5.0 * torch.tanh(want.float()[:, :50] * 0.5 / 5.0)
    assert embed.shape == (56, 32) and torch.allclose(head(h), want, atol=1e-5)
    tied = target_embed_and_head(_cfg(tie_embeddings=1), {k: v for k, v in t.items() if k != "lm_head"}, "cpu")[1]
    assert tied(h).shape == (4, 50)
    with pytest.raises(InferenceError):
        target_embed_and_head(_cfg(family=0), t, "cpu")


class _TapEngine:
    """Serves taps the way the resident engine does: [n, taps * d] for cached positions of a slot."""

    def __init__(self, taps, layers):
        self.taps, self.tap_layers, self.reads = taps, tuple(layers), []

    def slot_length(self, slot):
        return self.taps.shape[0]

    def read_taps(self, slot, pos0, n):
        self.reads.append((slot, pos0, n))
        return self.taps[pos0:pos0 + n]


def test_dflash_proposer_reads_the_context_window_and_proposes_block_minus_one_tokens():
    from neuralfn_b200.tensor.dflash import DFlashConfig, DFlashDraftModel
    dcfg = DFlashConfig(d_model=16, n_layer=1, n_head=2, block_size=5, context_window=6, tap_layers=(0, 1), mask_token_id=0)
    torch.manual_seed(0)
    draft = DFlashDraftModel(dcfg, 32)
    cfg = _cfg()
    g = torch.Generator().manual_seed(2)
    t = {"tok_embeddings": torch.randn(56, 32, generator=g), "lm_head": torch.randn(56, 32, generator=g), "norm": torch.ones(32)}
    embed, head = target_embed_and_head(cfg, t, "cpu")
    eng = _TapEngine(torch.randn(10, 64, generator=g).bfloat16(), (0, 1))
    prop = DFlashProposer(eng, 1, draft.bfloat16(), embed, head)
    history = list(range(1, 11)) + [42]                                      # ten cached tokens and the pending one
    toks, q = prop.propose(history, 7)
    assert q is None and len(toks) == 4 and all(0 <= x < 50 for x in toks)   # block_size - 1 proposals, inside the vocabulary
    assert eng.reads == [(1, 4, 6)]                                          # the last context_window cached positions
    assert prop.propose(history, 2) == (toks[:2], None) and prop.calls == 2
    assert prop.propose(history[:5], 3) == ([], None)                        # history and cache disagree: nothing is proposed
    with pytest.raises(InferenceError, match="taps"):
        DFlashProposer(_TapEngine(eng.taps, (1, 2)), 0, draft, embed, head)


def test_mixture_of_activations_record_round_trip(tmp_path):
    from neuralfn_b200.checkpoint.dense import _write_moa_sidecar, read_moa_sidecar
    from neuralfn_b200.models.gpt2 import GPT2Config
    cfg = GPT2Config.variant("gpt2_moa", n_layer=2, n_head=2, d_model=64, vocab_size=100, max_seq_len=32)
    (tmp_path / "model_00000007.bin").write_bytes(b"x" * 33)
    digests = {"model_00000007.bin": "ab" * 32}
    digests.update(_write_moa_sidecar(tmp_path, 7, cfg, "relu2", digests))
    (tmp_path / "DONE_00000007").write_text(json.dumps(digests))
    rec = read_moa_sidecar(tmp_path, 7)
    assert rec["selection"] == {"activation": "relu2", "candidates": ["gelu", "relu", "silu", "relu2"], "interval": 50}
    assert rec["model"]["nbytes"] == 33 and rec["geometry"]["mlp_hidden_dim"] == 256 and rec["schema"] == "neuralfn.native_dense_moa.inference_checkpoint"
    (tmp_path / "DONE_00000007").write_text(json.dumps({**digests, "model_00000007.bin": "cd" * 32}))
    with pytest.raises(ValueError, match="different model"):
        read_moa_sidecar(tmp_path, 7)
    with pytest.raises(FileNotFoundError):
        read_moa_sidecar(tmp_path, 8)

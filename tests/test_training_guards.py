"""Host-side guards of the training loops: device-status checks before anything is published, and
the pinned staging ring that keeps queued host-to-device copies from seeing a later step's values."""
import pytest
import torch


class _BadTrainer:
    """A trainer whose device status word reports a timed-out wait."""
    def check_status(self):
        from neuralfn_b200.ops._lib import KernelLibraryError
        raise KernelLibraryError("dense gpt step: device status 5 (wait_peer)")


def test_no_checkpoint_is_written_when_the_device_status_is_bad(tmp_path):
    from neuralfn_b200.native_train import save_checkpoint_checked
    from neuralfn_b200.ops._lib import KernelLibraryError
    with pytest.raises(KernelLibraryError, match="wait_peer"):
        save_checkpoint_checked(_BadTrainer(), tmp_path / "ckpt", 3, dense_format=True)
    assert not (tmp_path / "ckpt").exists() or not list((tmp_path / "ckpt").glob("DONE_*"))


def test_pinned_ring_rotates_slots_and_keeps_values():
    from neuralfn_b200.utils.pinned import PinnedRing
    ring = PinnedRing(4, torch.float32, slots=3)
    dst = torch.zeros(4)
    seen = []
    for step in range(7):
        buf = ring.upload(dst, [float(step), 1.0, 2.0])
        seen.append(buf.data_ptr())
        assert dst[:3].tolist() == [float(step), 1.0, 2.0] and ring.last is buf
    assert len(set(seen)) == 3 and seen[0] == seen[3] == seen[6]  # three slots, used round-robin


@pytest.mark.gpu
def test_unsynchronised_steps_use_their_own_hyper_parameters():
    """N optimizer steps queued without any synchronisation must equal the same N steps with a
    synchronise after each: every queued hyper-parameter copy has to see its own step's values."""
    from neuralfn_b200.models.gpt2 import GPT2Config
    from neuralfn_b200.parallel.dp import AdamWConfig
    from neuralfn_b200.trainers.dense_gpt import DenseGPTTrainer
    cfg = GPT2Config.variant("gpt2", n_layer=1, n_head=2, d_model=128, vocab_size=512, max_seq_len=128)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, 512, (4 * 128,), generator=g, dtype=torch.int32).pin_memory()
    tgt = torch.randint(0, 512, (4 * 128,), generator=g, dtype=torch.int32).pin_memory()
    masters = []
    for sync in (True, False):
        tr = DenseGPTTrainer(cfg, 4, 128, AdamWConfig(lr=1e-2, warmup_steps=10, total_steps=40), seed=5, device="cuda:0")
        tr.upload(tok, tgt)
        for _ in range(24):
            tr.step_on_device_batch()
            if sync:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        tr.check_status()
        masters.append(tr.opt.master.clone())
    assert torch.equal(masters[0], masters[1])


@pytest.mark.gpu
def test_status_word_set_from_the_host_stops_a_checkpoint(tmp_path, kernel_lib):
    from neuralfn_b200.models.gpt2 import GPT2Config
    from neuralfn_b200.native_train import save_checkpoint_checked
    from neuralfn_b200.ops import _lib
    from neuralfn_b200.trainers.dense_gpt import DenseGPTTrainer
    cfg = GPT2Config.variant("gpt2", n_layer=1, n_head=2, d_model=128, vocab_size=512, max_seq_len=128)
    tr = DenseGPTTrainer(cfg, 2, 128, device="cuda:0")
    assert kernel_lib.nfn_status_set(5) == 0   # what a peer wait that ran out leaves behind
    with pytest.raises(_lib.KernelLibraryError):
        save_checkpoint_checked(tr, tmp_path / "ckpt", 1, dense_format=True)
    assert not list(tmp_path.glob("ckpt/DONE_*"))
    assert _lib.status_read_reset() == 0        # the failed check consumed the code


def test_stage_timer_report_uses_the_reference_field_names():
    from neuralfn_b200.utils.stage_timing import StageTimer
    clock = {"block_forward": 2.0, "block_forward.attention.qkv": 0.5}
    t = StageTimer(enabled=True, time_fn=lambda name: clock[name])
    for step in range(3):
        with t.stage("block_forward"):
            with t.stage("block_forward.attention.qkv"):
                pass
        t.next_step()
    rep = t.report()
    assert rep["stage_timing_enabled"] and rep["stage_timing_event_count"] == 6
    rec = {r["name"]: r for r in rep["stage_timing"]}
    q = rec["block_forward.attention.qkv"]
    assert set(q) == {"name", "total_ms", "count", "avg_ms", "first_step_total_ms", "first_step_count", "first_step_avg_ms",
                      "steady_state_total_ms", "steady_state_count", "steady_state_avg_ms"}
    assert q["count"] == 3 and q["first_step_count"] == 1 and q["steady_state_count"] == 2 and abs(q["avg_ms"] - 0.5) < 1e-9
    off = StageTimer(enabled=False)
    with off.stage("anything"):
        pass
    assert off.report()["stage_timing"] == []


@pytest.mark.gpu
def test_stage_timing_covers_a_training_step(monkeypatch):
    monkeypatch.setenv("NFN_NATIVE_GPT_STAGE_TIMING", "1")
    from neuralfn_b200.models.gpt2 import GPT2Config
    from neuralfn_b200.trainers.dense_gpt import DenseGPTTrainer
    cfg = GPT2Config.variant("gpt2_qknorm_softcap_zloss", n_layer=2, n_head=2, d_model=128, vocab_size=512, max_seq_len=128)
    tr = DenseGPTTrainer(cfg, 2, 128, device="cuda:0")
    assert tr.timer.enabled and not tr.use_cuda_graph
    tok = torch.randint(0, 512, (2 * 128,), dtype=torch.int32)
    for _ in range(3):
        tr.train_step(tok, tok)
    rep = tr.timer.report()
    names = {r["name"] for r in rep["stage_timing"]}
    for want in ("token_upload", "block_forward", "block_forward.attention.qkv", "block_forward.attention.sdpa", "lm_head_backward.ce",
                 "block_backward.attn_sdpa", "block_backward.mlp_fc.dweight_bias", "embedding_backward", "adamw_update"):
        assert want in names, want
    fwd = next(r for r in rep["stage_timing"] if r["name"] == "block_forward")
    assert fwd["count"] == 3 * cfg.n_layer and fwd["first_step_count"] == cfg.n_layer and fwd["total_ms"] > 0

"""Native data readers: shard formats, sequential sampler order, resume, rank striding,
prefetch ring, structured records. Pure CPU (reference coverage: tests/test_native_token_shards*.py)."""
import numpy as np
import pytest
import torch

from neuralfn_b200.data import (ByteDataset, PrefetchingLoader, RecordReader, TokenDataset, write_legacy_shard,
                                write_ppo_prompt_records, write_preference_records, write_sft_records, write_v2_shard)
from neuralfn_b200.data._rt import NativeRuntimeError, sha256_file


def _mk_token_dir(tmp_path, n0=1000, n1=700, nval=400, v2=False):
    rng = np.random.default_rng(0)
    a, b, c = (rng.integers(0, 5000, n) for n in (n0, n1, nval))
    if v2:
        write_v2_shard(tmp_path / "fineweb_train_000000.bin", a, 5000)
        write_v2_shard(tmp_path / "fineweb_train_000001.bin", b, 5000)
        write_v2_shard(tmp_path / "fineweb_val_000000.bin", c, 5000, split="validation")
    else:
        write_legacy_shard(tmp_path / "fineweb_train_000000.bin", a, with_header=True)
        write_legacy_shard(tmp_path / "fineweb_train_000001.bin", b, with_header=False)
        write_legacy_shard(tmp_path / "fineweb_val_000000.bin", c)
    return a, b, c


def _expected_windows(shards, T):
    toks, tgts = [], []
    for s in shards:
        for i in range((len(s) - 1) // T):
            toks.append(s[i * T:i * T + T])
            tgts.append(s[i * T + 1:i * T + T + 1])
    return np.stack(toks), np.stack(tgts)


@pytest.mark.parametrize("v2", [False, True])
def test_sequential_order_matches_window_definition(tmp_path, v2):
    a, b, c = _mk_token_dir(tmp_path, v2=v2)
    ds = TokenDataset(tmp_path)
    info = ds.describe(seq_len=64, batch_size=4, train_batch_tokens=1024)
    assert info["train_tokens"] == 1700 and info["val_tokens"] == 400
    assert info["train_shards"][0]["header_bytes"] == 512
    assert info["batch_plan"]["grad_accum_steps"] == 4 and info["batch_plan"]["train_sequences"] == 15 + 10
    assert ds.max_token() == max(a.max(), b.max())
    etok, etgt = _expected_windows([a, b], 64)
    s = ds.sampler("train", 64, 4)
    assert s.total_batches == 25 // 4
    got = list(s)
    assert len(got) == 6
    for i, (tok, tgt) in enumerate(got):
        np.testing.assert_array_equal(tok.numpy(), etok[4 * i:4 * i + 4])
        np.testing.assert_array_equal(tgt.numpy(), etgt[4 * i:4 * i + 4])
    assert s.next() is None
    assert s.next(wrap=True) is not None and s.position == 1


def test_seek_resume_and_rank_striding(tmp_path):
    a, b, _ = _mk_token_dir(tmp_path)
    ds = TokenDataset(tmp_path)
    etok, _ = _expected_windows([a, b], 32)
    full = ds.sampler("train", 32, 2)
    batches = [t.clone() for t, _ in full]
    full.seek(3)
    np.testing.assert_array_equal(full.next()[0].numpy(), batches[3].numpy())
    full.seek(len(batches) + 1)  # modulo, like the reference's seek_batch
    np.testing.assert_array_equal(full.next()[0].numpy(), batches[1].numpy())
    r0, r1 = ds.sampler("train", 32, 2, rank=0, world=2), ds.sampler("train", 32, 2, rank=1, world=2)
    assert r0.total_batches == len(etok) // 4
    t0, t1 = r0.next()[0].numpy(), r1.next()[0].numpy()
    np.testing.assert_array_equal(np.concatenate([t0, t1]), etok[:4])


def test_prefetch_ring_yields_sampler_order_and_wraps(tmp_path):
    a, b, _ = _mk_token_dir(tmp_path)
    ds = TokenDataset(tmp_path)
    ref = [t.clone() for t, _ in ds.sampler("train", 32, 4)]
    s = ds.sampler("train", 32, 4)
    loader = PrefetchingLoader(s, slots=3, pin=False)
    for i in range(2 * len(ref) + 1):
        tok, _ = next(loader)
        assert loader.batch_index == i
        np.testing.assert_array_equal(tok.numpy(), ref[i % len(ref)].numpy())
    loader.close()


def test_validation_fallbacks_and_errors(tmp_path):
    rng = np.random.default_rng(1)
    write_legacy_shard(tmp_path / "fineweb_train_000000.bin", rng.integers(0, 100, 300))
    with pytest.raises(NativeRuntimeError, match="validation"):
        TokenDataset(tmp_path)
    ds = TokenDataset(tmp_path, allow_train_as_val=True)
    assert ds.tokens("val") == 300
    bad = tmp_path / "bad"
    bad.mkdir()
    write_v2_shard(bad / "fineweb_train_000000.bin", rng.integers(0, 100, 300), 100)
    raw = bytearray((bad / "fineweb_train_000000.bin").read_bytes())
    raw[500] = 7  # reserved header byte
    (bad / "fineweb_train_000000.bin").write_bytes(bytes(raw))
    with pytest.raises(NativeRuntimeError, match="reserved"):
        TokenDataset(bad, require_validation=False)
    with pytest.raises(NativeRuntimeError, match=">= vocab"):
        write_v2_shard(bad / "x.bin", [5, 200], 100)
    with pytest.raises(NativeRuntimeError, match="not found"):
        TokenDataset(tmp_path / "nope")


def test_byte_dataset(tmp_path):
    data = np.frombuffer(b"hello native byte shards, hello again!" * 20, dtype=np.uint8)
    (tmp_path / "bytes_train.bin").write_bytes(data.tobytes())
    (tmp_path / "bytes_val.bin").write_bytes(data[:200].tobytes())
    ds = ByteDataset(tmp_path)
    tok, tgt = ds.sampler("train", 16, 2).next()
    np.testing.assert_array_equal(tok.numpy().ravel(), data[:32])
    np.testing.assert_array_equal(tgt.numpy().ravel()[:16], data[1:17])


def _sft_arrays(n, T, vocab, rng):
    ids = rng.integers(1, vocab, (n, T))
    tg = np.roll(ids, -1, axis=1)
    mask = np.zeros((n, T), np.float32)
    mask[:, T // 2:] = 1.0
    tg = np.where(mask > 0, tg, -100)
    seg = np.zeros((n, T), np.int32)
    seg[:, T // 2:] = 1
    return ids, tg, mask, seg


def test_structured_records_roundtrip(tmp_path):
    rng = np.random.default_rng(2)
    ids, tg, mask, seg = _sft_arrays(5, 16, 300, rng)
    write_sft_records(tmp_path / "sft_train_000.sft", ids, tg, mask, seg, vocab_size=300)
    r = RecordReader(tmp_path, "sft", "train", batch_size=2)
    assert r.total_batches == 2 and r.seq_len == 16 and r.describe()["records"] == 5
    b0, b1 = r.next(), r.next()
    assert r.next() is None
    np.testing.assert_array_equal(b1["input_ids"].numpy(), ids[2:4])
    np.testing.assert_array_equal(b0["targets"].numpy(), tg[:2])
    np.testing.assert_array_equal(b0["loss_mask"].numpy(), mask[:2])
    np.testing.assert_array_equal(b0["sequence_ids"].numpy(), seg[:2])
    r.seek(1)
    np.testing.assert_array_equal(r.next()["input_ids"].numpy(), ids[2:4])

    ids2, tg2, mask2, seg2 = _sft_arrays(5, 16, 300, rng)
    write_preference_records(tmp_path / "preference_train_000.preference",
                             dict(input_ids=ids, targets=tg, loss_mask=mask, sequence_ids=seg),
                             dict(input_ids=ids2, targets=tg2, loss_mask=mask2, sequence_ids=seg2), vocab_size=300)
    p = RecordReader(tmp_path, "preference", "train", batch_size=2).next()
    np.testing.assert_array_equal(p["chosen_input_ids"].numpy(), ids[:2])
    np.testing.assert_array_equal(p["rejected_targets"].numpy(), tg2[:2])

    pm = np.zeros((3, 8), np.float32)
    pm[:, :5] = 1
    pids = np.where(pm > 0, rng.integers(1, 300, (3, 8)), 0)
    write_ppo_prompt_records(tmp_path / "ppo_prompt_train_000.ppo_prompt", pids, pm, vocab_size=300)
    q = RecordReader(tmp_path, "ppo_prompt", "train", batch_size=3).next()
    np.testing.assert_array_equal(q["input_ids"].numpy(), pids)
    np.testing.assert_array_equal(q["attention_mask"].numpy(), pm)

    bad_mask = mask.copy()
    bad_mask[0, 0] = 1.0  # mask on an ignored (-100) target
    with pytest.raises(NativeRuntimeError):
        write_sft_records(tmp_path / "sft_train_001.sft", ids, tg, bad_mask, seg, vocab_size=300)
    assert not (tmp_path / "sft_train_001.sft").exists()


def test_sha256(tmp_path):
    import hashlib
    blob = bytes(range(256)) * 1000 + b"tail"
    (tmp_path / "blob").write_bytes(blob)
    assert sha256_file(tmp_path / "blob") == hashlib.sha256(blob).hexdigest()


def test_dataset_manager_prepares_verifies_and_loads(tmp_path):
    from neuralfn_b200.data import TokenDataset, TokenSampler
    from neuralfn_b200.data.manager import DatasetError, DatasetManager
    src = tmp_path / "corpus.txt"
    src.write_text("\n\n".join(f"document number {i} says hello to the world" for i in range(40)), encoding="utf-8")
    mgr = DatasetManager(tmp_path / "cache")
    man = mgr.prepare_text("tiny", [src], tokenizer="bytes", val_fraction=0.1, shard_tokens=600, document_separator=[0])
    assert man["vocab_size"] == 256 and man["val_tokens"] > 0 and len([s for s in man["shards"] if s["split"] == "train"]) >= 2
    assert mgr.list() == [{"name": "tiny", "variants": ["bytes"]}] and mgr.info("tiny")["train_tokens"] == man["train_tokens"]
    mgr.verify("tiny")
    with pytest.raises(DatasetError):
        mgr.prepare_text("tiny", [src], tokenizer="bytes")
    ds = TokenDataset(str(mgr.path("tiny")))
    assert ds.tokens("train") == man["train_tokens"] and ds.tokens("val") == man["val_tokens"]
    x, y = TokenSampler(ds, "train", 16, 2).next()
    assert x.shape == (2, 16) and (x[:, 1:] == y[:, :-1]).all() and int(x.max()) < 256
    # a flipped byte in a shard is caught
    shard = mgr.path("tiny") / man["shards"][0]["file"]
    raw = bytearray(shard.read_bytes())
    raw[-1] ^= 1
    shard.write_bytes(bytes(raw))
    with pytest.raises(DatasetError):
        mgr.verify("tiny")
    mgr.delete("tiny")
    assert mgr.list() == []

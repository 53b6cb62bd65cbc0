"""GGUF writer -> reader round trip with K-quant, F16, BF16 and F32 tensors and metadata."""
import numpy as np
import pytest

from neuralfn_b200.checkpoint.gguf import GGUFFile, write_gguf
from neuralfn_b200.quant import kquant


def test_roundtrip_metadata_and_tensors(tmp_path):
    rng = np.random.default_rng(0)
    w = rng.normal(size=(6, 512)).astype(np.float32)
    q4 = kquant.quantize_q4_k(w).tobytes()
    q6 = kquant.quantize_q6_k(w).tobytes()
    f16 = w.astype("<f2").tobytes()
    bf16 = (w.view(np.uint32) >> 16).astype("<u2").tobytes()
    meta = {"general.architecture": "llama", "llama.block_count": 2, "llama.rope.freq_base": 10000.0, "general.name": "tiny",
            "tokenizer.ggml.tokens": ["a", "b", "c"], "llama.flag": True}
    write_gguf(tmp_path / "m.gguf", meta, {"blk.0.attn_q.weight": (12, (6, 512), q4), "blk.0.ffn_down.weight": (14, (6, 512), q6),
                                           "token_embd.weight": (1, (6, 512), f16), "output_norm.weight": (0, (512,), w[0].tobytes()),
                                           "x.bf16": (30, (6, 512), bf16)})
    with GGUFFile(tmp_path / "m.gguf") as g:
        assert g.version == 3 and g.metadata["llama.block_count"] == 2 and g.metadata["tokenizer.ggml.tokens"] == ["a", "b", "c"]
        assert g.metadata["llama.flag"] is True and abs(g.metadata["llama.rope.freq_base"] - 10000.0) < 1e-3
        assert g.tensors["blk.0.attn_q.weight"].shape == (6, 512) and g.tensors["blk.0.attn_q.weight"].type_name == "Q4_K"
        assert g.raw("blk.0.attn_q.weight").tobytes() == q4 and g.data_start % 32 == 0
        assert np.abs(g.dequantize("blk.0.attn_q.weight") - w).mean() < 0.08
        assert np.abs(g.dequantize("blk.0.ffn_down.weight") - w).mean() < 0.02
        assert np.allclose(g.dequantize("token_embd.weight"), w, atol=2e-3)
        assert np.array_equal(g.dequantize("output_norm.weight"), w[0])
        assert np.allclose(g.dequantize("x.bf16"), w, atol=2e-2)
        assert g.summary()["tensors"] == 5


def test_rejects_bad_files(tmp_path):
    (tmp_path / "bad.gguf").write_bytes(b"NOPE" + b"\0" * 64)
    with pytest.raises(ValueError, match="not a GGUF"):
        GGUFFile(tmp_path / "bad.gguf")
    write_gguf(tmp_path / "t.gguf", {}, {"w": (12, (1, 256), kquant.random_blocks(12, 1).tobytes())})
    raw = (tmp_path / "t.gguf").read_bytes()
    (tmp_path / "t.gguf").write_bytes(raw[:-40])
    with pytest.raises(ValueError, match="past the end"):
        GGUFFile(tmp_path / "t.gguf")


def test_packed_rows_of_one_type_concatenate_without_decoding(tmp_path):
    """``packed`` hands out the blocks as stored (what the resident engine keeps for a K-quant projection); the q | k | v pieces of
    a fused projection are rows of super-blocks, so joining the bytes equals quantising the joined rows."""
    rng = np.random.default_rng(1)
    q, k = rng.normal(size=(4, 512)).astype(np.float32), rng.normal(size=(2, 512)).astype(np.float32)
    write_gguf(tmp_path / "m.gguf", {"general.architecture": "llama"},
               {"blk.0.attn_q.weight": (12, (4, 512), kquant.quantize_q4_k(q).tobytes()),
                "blk.0.attn_k.weight": (12, (2, 512), kquant.quantize_q4_k(k).tobytes())})
    with GGUFFile(tmp_path / "m.gguf") as g:
        (tq, bq), (tk, bk) = g.packed("blk.0.attn_q.weight"), g.packed("blk.0.attn_k.weight")
        assert tq == tk == 12 and bq.dtype == np.uint8 and bq.size == 4 * 2 * kquant.BLOCK_BYTES[12]
        fused = np.concatenate([bq, bk])
        want = np.concatenate([g.dequantize("blk.0.attn_q.weight"), g.dequantize("blk.0.attn_k.weight")])
        assert np.array_equal(kquant.dequantize(12, fused).reshape(6, 512), want)

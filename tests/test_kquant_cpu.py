"""Host-side K-quant and NF4 oracles: encoders and decoders agree, packed scales round-trip."""
import numpy as np

from neuralfn_b200.quant import kquant


def test_scale_min_packing_roundtrip():
    rng = np.random.default_rng(0)
    d, m = rng.integers(0, 64, (50, 8), dtype=np.uint8), rng.integers(0, 64, (50, 8), dtype=np.uint8)
    d2, m2 = kquant._scales_mins(kquant._pack_scales_mins(d, m))
    assert np.array_equal(d, d2) and np.array_equal(m, m2)


def test_q4_k_and_q6_k_quantisers_are_close():
    w = np.random.default_rng(1).normal(size=256 * 40).astype(np.float32)
    q4 = kquant.dequantize_q4_k(kquant.quantize_q4_k(w).tobytes())
    q6 = kquant.dequantize_q6_k(kquant.quantize_q6_k(w).tobytes())
    assert np.abs(q4 - w).mean() < 0.08 and np.abs(q4 - w).max() < 0.5
    assert np.abs(q6 - w).mean() < 0.02 and np.abs(q6 - w).max() < 0.2
    assert kquant.quantize_q4_k(w).shape == (40, 144) and kquant.quantize_q6_k(w).shape == (40, 210)


def test_q5_k_decoder_uses_the_high_bits():
    raw = kquant.random_blocks(13, 4, seed=3)
    a = kquant.dequantize_q5_k(raw.tobytes())
    raw2 = raw.copy()
    raw2[:, 16:48] ^= 0xFF  # flip every high bit
    b = kquant.dequantize_q5_k(raw2.tobytes())
    assert a.shape == (1024,) and np.all(np.abs(a - b) > 0)


def test_nf4_roundtrip_error():
    w = np.random.default_rng(2).normal(size=64 * 30).astype(np.float32)
    codes, absmax = kquant.nf4_encode(w)
    back = kquant.nf4_decode(codes, absmax)
    assert codes.dtype == np.uint8 and codes.size == w.size // 2
    assert np.abs(back - w).mean() < 0.12
    # low nibble holds the even element (the layout of the tensor-runtime nf4_linear stage)
    assert np.isclose(kquant.NF4_TABLE[codes[0] & 0xF] * absmax[0], back[0])

"""TurboQuant codec: numpy oracle properties (CPU) and the device kernels against it (GPU)."""
import numpy as np
import pytest
import torch

from neuralfn_b200.quant.turboquant import (TurboQuantCodec, TurboQuantError, default_outlier_indices, deterministic_random_rotation,
                                            lloyd_max_centroids, pack_mixed_bit_indices, unpack_mixed_bit_indices)


def test_rotation_centroids_and_packing():
    R = deterministic_random_rotation(16, 3)
    assert np.allclose(R @ R.T, np.eye(16), atol=1e-12) and np.array_equal(R, deterministic_random_rotation(16, 3))
    assert not np.allclose(R, deterministic_random_rotation(16, 4))
    c = lloyd_max_centroids(64, 3)
    assert len(c) == 8 and np.all(np.diff(c) > 0) and np.allclose(c, -c[::-1]) and abs(c[-1]) < 1
    widths = [4, 3, 2, 8, 1, 3, 4, 3]
    idx = [9, 5, 3, 200, 1, 0, 15, 7]
    packed = pack_mixed_bit_indices(idx, widths)
    assert len(packed) == (sum(widths) + 7) // 8 and unpack_mixed_bit_indices(packed, widths) == tuple(idx)
    with pytest.raises(TurboQuantError):
        pack_mixed_bit_indices([8], [3])
    with pytest.raises(TurboQuantError):
        TurboQuantCodec(16, outlier_indices=[0, 1])


@pytest.mark.parametrize("profile", ["mse-3.5", "qjl-3.5"])
def test_codec_accuracy(profile):
    rng = np.random.default_rng(0)
    D = 64
    codec = TurboQuantCodec(D, profile=profile, seed=1, outlier_indices=default_outlier_indices(D))
    assert codec.value_layout.index_bytes == D * 7 // 16 and codec.value_layout.record_bytes % 16 == 0
    rel_v, err_ip = [], []
    for _ in range(40):
        x, q = rng.normal(size=D), rng.normal(size=D)
        rv = codec.encode(x, key=False)
        rel_v.append(np.linalg.norm(codec.decode(rv, key=False) - x) / np.linalg.norm(x))
        rk = codec.encode(x, key=True)
        err_ip.append(codec.key_inner_product(q, rk) - q @ x)
    assert np.mean(rel_v) < 0.2                       # ~3.5 bits per coordinate
    assert np.std(err_ip) < (0.25 if profile == "mse-3.5" else 0.45) * np.sqrt(D)  # |q||x| ~ D: a few per cent
    if profile == "qjl-3.5":
        assert abs(np.mean(err_ip)) < 0.6             # the sign sketch removes the bias
        assert len(codec.encode(rng.normal(size=D), key=True)["signs"]) == D // 8
    zero = codec.encode(np.zeros(D), key=True)
    assert zero["norm"] == 0.0 and codec.key_inner_product(rng.normal(size=D), zero) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("profile,D,Hq,Hkv", [("mse-3.5", 128, 8, 2), ("qjl-3.5", 128, 4, 4), ("qjl-3.5", 64, 8, 1), ("mse-3.5", 64, 2, 2)])
def test_device_encode_and_attention_match_the_oracle(kernel_lib, profile, D, Hq, Hkv):
    from neuralfn_b200.ops import _lib
    from neuralfn_b200.quant.turboquant import TurboQuantKVCache
    torch.manual_seed(2)
    dev = "cuda"
    codec = TurboQuantCodec(D, profile=profile, seed=5, outlier_indices=default_outlier_indices(D))
    B, cap, steps = 2, 24, 30  # the ring wraps
    cache = TurboQuantKVCache(codec, B, Hkv, cap, dev)
    ks, vs = [], []
    for t in range(steps):
        k = torch.randn(B, Hkv * D, device=dev).bfloat16()
        v = torch.randn(B, Hkv * D, device=dev).bfloat16()
        if t < 7:
            cache.append(k[:1], v[:1], [0])  # sequence 1 starts later
            k[1], v[1] = 0, 0
        else:
            cache.append(k, v)
        ks.append(k.float().cpu().numpy())
        vs.append(v.float().cpu().numpy())
    _lib.assert_status_ok("turboquant encode")
    # device records == oracle records (up to centroid ties): compare through the decoded values and scores
    krec, vrec = cache.k.cpu().numpy(), cache.v.cpu().numpy()
    q = torch.randn(B, Hq * D, device=dev).bfloat16()
    out = cache.attention(q, Hq).float().cpu().numpy()
    _lib.assert_status_ok("turboquant attention")
    qn, G = q.float().cpu().numpy(), Hq // Hkv
    for b in range(B):
        toks = [t for t in range(steps) if (b == 0 or t >= 7)][-cap:]
        for hk in range(Hkv):
            keys = [codec.encode(ks[t][b, hk * D:(hk + 1) * D], key=True) for t in toks]
            vals = [codec.encode(vs[t][b, hk * D:(hk + 1) * D], key=False) for t in toks]
            # one record byte for byte (norm and packed indices; a tie may flip a single field)
            n_b = len([t for t in range(steps) if (b == 0 or t >= 7)])
            slot = (n_b - 1) % cap
            want = np.frombuffer(codec.record_bytes_of(vals[-1], key=False), dtype=np.uint8)
            assert np.count_nonzero(vrec[b, hk, slot] != want) <= 2
            for g in range(G):
                h = hk * G + g
                ref = codec.attention_oracle(qn[b, h * D:(h + 1) * D], keys, vals, D ** -0.5)
                assert np.abs(out[b, h * D:(h + 1) * D] - ref).max() < 0.03, (b, h)
    # per vector at D = 128: 64 of 256 bytes (80 for a QJL key with its sign bits and residual norm)
    assert cache.bytes_per_token <= (0.29 if D == 128 else 0.4) * (2 * Hkv * D * 2)

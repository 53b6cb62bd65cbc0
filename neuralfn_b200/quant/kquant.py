"""GGUF K-quant super-blocks on the host: numpy dequantisation oracles (Q4_K, Q5_K, Q6_K),
block builders for tests and tools, and NF4 encode/decode.

Layouts (256 weights per super-block, little endian, as published with ggml):
  Q4_K 144 B: half d, half dmin, u8 scales[12], u8 qs[128]
  Q5_K 176 B: half d, half dmin, u8 scales[12], u8 qh[32], u8 qs[128]
  Q6_K 210 B: u8 ql[128], u8 qh[64], i8 scales[16], half d
The reference imports these in ``neuralfn/native_muse_glimmer_checkpoint.py`` and decodes
them on the device in ``kernels.cu:1324-2015``.
"""
from __future__ import annotations

import numpy as np

QK_K = 256
GGML_TYPE = {"F32": 0, "F16": 1, "Q4_K": 12, "Q5_K": 13, "Q6_K": 14, "BF16": 30}
BLOCK_BYTES = {12: 144, 13: 176, 14: 210}

__all__ = ["QK_K", "GGML_TYPE", "BLOCK_BYTES", "dequantize", "dequantize_q4_k", "dequantize_q5_k", "dequantize_q6_k",
           "quantize_q4_k", "quantize_q6_k", "random_blocks", "NF4_TABLE", "nf4_encode", "nf4_decode"]


def _scales_mins(sc: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """(n, 12) packed bytes -> two (n, 8) arrays of 6-bit scales and mins."""
    sc = sc.astype(np.uint8)
    d, m = np.empty(sc.shape[:-1] + (8,), np.uint8), np.empty(sc.shape[:-1] + (8,), np.uint8)
    d[..., :4] = sc[..., 0:4] & 63
    m[..., :4] = sc[..., 4:8] & 63
    d[..., 4:] = (sc[..., 8:12] & 0xF) | ((sc[..., 0:4] >> 6) << 4)
    m[..., 4:] = (sc[..., 8:12] >> 4) | ((sc[..., 4:8] >> 6) << 4)
    return d, m


def _pack_scales_mins(d: np.ndarray, m: np.ndarray) -> np.ndarray:
    out = np.zeros(d.shape[:-1] + (12,), np.uint8)
    out[..., 0:4] = (d[..., :4] & 63) | ((d[..., 4:] >> 4) << 6)
    out[..., 4:8] = (m[..., :4] & 63) | ((m[..., 4:] >> 4) << 6)
    out[..., 8:12] = (d[..., 4:] & 0xF) | ((m[..., 4:] & 0xF) << 4)
    return out


def dequantize_q4_k(raw: np.ndarray) -> np.ndarray:
    b = np.frombuffer(raw, np.uint8).reshape(-1, 144)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32)
    dmin = b[:, 2:4].copy().view(np.float16).astype(np.float32)
    sc, mn = _scales_mins(b[:, 4:16])
    qs = b[:, 16:].reshape(-1, 4, 32)
    q = np.stack([qs & 0xF, qs >> 4], axis=2).reshape(-1, 8, 32).astype(np.float32)
    return (d[:, :, None] * sc[:, :, None].astype(np.float32) * q - dmin[:, :, None] * mn[:, :, None].astype(np.float32)).reshape(-1)


def dequantize_q5_k(raw: np.ndarray) -> np.ndarray:
    b = np.frombuffer(raw, np.uint8).reshape(-1, 176)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32)
    dmin = b[:, 2:4].copy().view(np.float16).astype(np.float32)
    sc, mn = _scales_mins(b[:, 4:16])
    qh = b[:, 16:48]
    qs = b[:, 48:].reshape(-1, 4, 32)
    lo, hi = (qs & 0xF).astype(np.int32), (qs >> 4).astype(np.int32)
    for j in range(4):
        lo[:, j] += ((qh >> (2 * j)) & 1).astype(np.int32) << 4
        hi[:, j] += ((qh >> (2 * j + 1)) & 1).astype(np.int32) << 4
    q = np.stack([lo, hi], axis=2).reshape(-1, 8, 32).astype(np.float32)
    return (d[:, :, None] * sc[:, :, None].astype(np.float32) * q - dmin[:, :, None] * mn[:, :, None].astype(np.float32)).reshape(-1)


def dequantize_q6_k(raw: np.ndarray) -> np.ndarray:
    b = np.frombuffer(raw, np.uint8).reshape(-1, 210)
    ql = b[:, :128].reshape(-1, 2, 64)
    qh = b[:, 128:192].reshape(-1, 2, 32)
    sc = b[:, 192:208].copy().view(np.int8).reshape(-1, 2, 8).astype(np.float32)
    d = b[:, 208:210].copy().view(np.float16).astype(np.float32)
    q = np.empty((b.shape[0], 2, 4, 32), np.int32)
    q[:, :, 0] = (ql[:, :, :32] & 0xF) | (((qh >> 0) & 3) << 4)
    q[:, :, 1] = (ql[:, :, 32:] & 0xF) | (((qh >> 2) & 3) << 4)
    q[:, :, 2] = (ql[:, :, :32] >> 4) | (((qh >> 4) & 3) << 4)
    q[:, :, 3] = (ql[:, :, 32:] >> 4) | (((qh >> 6) & 3) << 4)
    q = (q - 32).astype(np.float32)
    # element l of run r uses scale index (l // 16) + 2 r
    idx = (np.arange(32) // 16)[None, :] + 2 * np.arange(4)[:, None]
    s = sc[:, :, idx]  # (n, 2, 4, 32)
    return (d[:, :, None, None] * s * q).reshape(-1)


def dequantize(ggml_type: int, raw: np.ndarray) -> np.ndarray:
    return {12: dequantize_q4_k, 13: dequantize_q5_k, 14: dequantize_q6_k}[ggml_type](raw)


def quantize_q4_k(w: np.ndarray) -> np.ndarray:
    """Simple (min/max per sub-block) Q4_K encoder - good enough for tests and synthetic
    checkpoints; returns uint8 [n_blocks, 144]."""
    x = np.asarray(w, np.float32).reshape(-1, 8, 32)
    mn = np.minimum(x.min(-1), 0.0)
    scale = (x.max(-1) - mn) / 15.0
    d = np.maximum(scale.max(-1), 1e-12) / 63.0
    dmin = np.maximum((-mn).max(-1), 1e-12) / 63.0
    d16, dmin16 = d.astype(np.float16), dmin.astype(np.float16)
    d, dmin = d16.astype(np.float32), dmin16.astype(np.float32)
    sc = np.clip(np.rint(scale / d[:, None]), 0, 63).astype(np.uint8)
    mq = np.clip(np.rint(-mn / dmin[:, None]), 0, 63).astype(np.uint8)
    eff = np.maximum(d[:, None] * sc, 1e-30)
    q = np.clip(np.rint((x + (dmin[:, None] * mq)[:, :, None]) / eff[:, :, None]), 0, 15).astype(np.uint8).reshape(-1, 4, 2, 32)
    out = np.zeros((x.shape[0], 144), np.uint8)
    out[:, 0:2] = d16.view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = dmin16.view(np.uint8).reshape(-1, 2)
    out[:, 4:16] = _pack_scales_mins(sc, mq)
    out[:, 16:] = (q[:, :, 0] | (q[:, :, 1] << 4)).reshape(-1, 128)
    return out


def quantize_q6_k(w: np.ndarray) -> np.ndarray:
    x = np.asarray(w, np.float32).reshape(-1, 16, 16)
    amax = np.abs(x).max(-1)
    d = np.maximum(amax.max(-1), 1e-12) / (32.0 * 127.0)
    d16 = d.astype(np.float16)
    d = d16.astype(np.float32)
    sc = np.clip(np.rint(amax / 32.0 / d[:, None]), -128, 127).astype(np.int8)
    eff = d[:, None] * sc.astype(np.float32)
    eff = np.where(eff == 0, 1e-30, eff)
    q = (np.clip(np.rint(x / eff[:, :, None]), -32, 31) + 32).astype(np.uint8).reshape(-1, 2, 4, 32)
    out = np.zeros((x.shape[0], 210), np.uint8)
    ql = np.empty((x.shape[0], 2, 64), np.uint8)
    ql[:, :, :32] = (q[:, :, 0] & 0xF) | ((q[:, :, 2] & 0xF) << 4)
    ql[:, :, 32:] = (q[:, :, 1] & 0xF) | ((q[:, :, 3] & 0xF) << 4)
    qh = (q[:, :, 0] >> 4) | ((q[:, :, 1] >> 4) << 2) | ((q[:, :, 2] >> 4) << 4) | ((q[:, :, 3] >> 4) << 6)
    out[:, :128] = ql.reshape(-1, 128)
    out[:, 128:192] = qh.reshape(-1, 64)
    out[:, 192:208] = sc.view(np.uint8)
    out[:, 208:210] = d16.view(np.uint8).reshape(-1, 2)
    return out


def random_blocks(ggml_type: int, n_blocks: int, seed: int = 0) -> np.ndarray:
    """Random but well-formed super-blocks (finite small scales) for decoder tests."""
    rng = np.random.default_rng(seed)
    nb = BLOCK_BYTES[ggml_type]
    raw = rng.integers(0, 256, (n_blocks, nb), dtype=np.uint8)
    d = rng.uniform(1e-3, 2e-2, n_blocks).astype(np.float16).view(np.uint8).reshape(-1, 2)
    if ggml_type in (12, 13):
        raw[:, 0:2] = d
        raw[:, 2:4] = rng.uniform(1e-3, 2e-2, n_blocks).astype(np.float16).view(np.uint8).reshape(-1, 2)
    else:
        raw[:, 208:210] = d
    return raw


# ---- NF4 -------------------------------------------------------------------------------------
NF4_TABLE = np.array([-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
                      -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
                      0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
                      0.7229568362236023, 1.0], np.float32)


def nf4_encode(w: np.ndarray, group: int = 64) -> tuple[np.ndarray, np.ndarray]:
    """-> (codes uint8 [n/2], low nibble = even element; absmax fp32 [n/group])."""
    x = np.asarray(w, np.float32).reshape(-1, group)
    absmax = np.maximum(np.abs(x).max(-1), 1e-12).astype(np.float32)
    idx = np.abs((x / absmax[:, None])[..., None] - NF4_TABLE).argmin(-1).astype(np.uint8).reshape(-1, 2)
    return idx[:, 0] | (idx[:, 1] << 4), absmax


def nf4_decode(codes: np.ndarray, absmax: np.ndarray, group: int = 64) -> np.ndarray:
    idx = np.stack([codes & 0xF, codes >> 4], axis=1).reshape(-1)
    return (NF4_TABLE[idx].reshape(-1, group) * absmax[:, None]).reshape(-1)

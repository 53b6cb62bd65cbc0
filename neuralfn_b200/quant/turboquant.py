"""TurboQuant KV-cache compression: codec (numpy oracle + batched torch encoder) and the device
record layout that ``csrc/kernels/turboquant.cu`` attends over.

Per head vector x of dimension D:
  * MSE part - store ||x|| (fp32) and, for the unit vector rotated by a fixed orthogonal
    matrix R, the index of the nearest Lloyd-Max centroid per coordinate. The "3.5-bit"
    profiles give a fixed half of the coordinates (the model-level *outlier* channels) 4 bits
    and the rest 3 bits; indices are packed as consecutive little-endian bit fields.
  * QJL part (keys of profile ``qjl-3.5`` only) - the MSE fields shrink by one bit each, and one
    bit per coordinate stores the sign of S (u - u_mse) for a fixed Gaussian matrix S, plus the
    residual norm; it corrects query-key inner products only:
        <q, k> ~= ||k|| * ( <R q, c> + sqrt(pi/2)/D * ||r|| * <S q, signs> ).
    Values always use the MSE path.
Attention never rebuilds a cache matrix: the query is rotated once, scores are taken against
centroid indices, the output accumulates in rotated space and is rotated back once.

R and S come from a SHA-256 counter stream (key ``neuralfn-turboquant-v1:<seed>:<domain>``,
16-byte little-endian counter, first 8 digest bytes -> uniform, Box-Muller with the cosine
branch first), R by two-pass modified Gram-Schmidt over successive Gaussian columns - the
construction of the reference oracle (``neuralfn/turboquant.py:59-131``), so that seeds mean
the same matrices in both implementations. Centroids: Lloyd-Max for the density
(1 - x^2)^((D-3)/2) on [-1, 1] (``:146-207``); packing ``:210-262``; codec ``:298-475``.

Device record (one per token and kv head, 16-byte aligned):
    [ norm fp32 | residual_norm fp32 (qjl keys) | sign bits D/8 bytes (qjl keys) | packed indices ] padded.
"""
from __future__ import annotations

import hashlib
import math
from dataclasses import dataclass
from functools import lru_cache
from typing import Iterable, Sequence

import numpy as np
import torch

__all__ = ["PROFILES", "TurboQuantError", "deterministic_random_rotation", "deterministic_qjl_projection", "lloyd_max_centroids",
           "pack_mixed_bit_indices", "unpack_mixed_bit_indices", "TurboQuantCodec", "TurboQuantLayout", "TurboQuantKVCache",
           "default_outlier_indices"]

PROFILES = ("mse-3.5", "qjl-3.5")


class TurboQuantError(ValueError):
    pass


def _gaussians(seed: int, domain: str, count: int) -> np.ndarray:
    """``count`` standard normals from the SHA-256 counter stream."""
    key = f"neuralfn-turboquant-v1:{seed}:{domain}".encode("utf-8")
    n_u = 2 * ((count + 1) // 2)
    u = np.empty(n_u, dtype=np.float64)
    for c in range(n_u):
        d = hashlib.sha256(key + c.to_bytes(16, "little")).digest()
        u[c] = (int.from_bytes(d[:8], "little") + 0.5) / float(1 << 64)
    radius = np.sqrt(-2.0 * np.log(u[0::2]))
    angle = 2.0 * math.pi * u[1::2]
    out = np.empty(n_u, dtype=np.float64)
    out[0::2] = radius * np.cos(angle)
    out[1::2] = radius * np.sin(angle)
    return out[:count]


@lru_cache(maxsize=32)
def deterministic_random_rotation(dimension: int, seed: int) -> np.ndarray:
    """Orthogonal [D, D] matrix; ``rotated = R @ x``."""
    if dimension < 2:
        raise TurboQuantError("dimension must be at least 2")
    g = _gaussians(seed, f"rotation:{dimension}", dimension * dimension).reshape(dimension, dimension)
    cols: list[np.ndarray] = []
    for c in range(dimension):
        v = g[c].copy()
        for _ in range(2):
            for b in cols:
                v -= float(v @ b) * b
        n = float(np.sqrt(v @ v))
        if n <= 1e-14:
            raise TurboQuantError(f"rotation became singular at column {c}")
        cols.append(v / n)
    return np.stack(cols, axis=1)  # R[row][col] = cols[col][row]


@lru_cache(maxsize=32)
def deterministic_qjl_projection(dimension: int, seed: int) -> np.ndarray:
    return _gaussians(seed, f"qjl:{dimension}", dimension * dimension).reshape(dimension, dimension)


@lru_cache(maxsize=64)
def lloyd_max_centroids(dimension: int, bit_width: int, quadrature_points: int = 16384, iterations: int = 80) -> np.ndarray:
    if not 1 <= bit_width <= 8:
        raise TurboQuantError("bit_width must be in 1..8")
    levels = 1 << bit_width
    pts = -1.0 + (np.arange(quadrature_points) + 0.5) * (2.0 / quadrature_points)
    logw = (dimension - 3.0) / 2.0 * np.log1p(-(pts * pts))
    w = np.exp(logw - logw.max())
    cum = np.cumsum(w)
    targets = (np.arange(levels) + 0.5) * cum[-1] / levels
    cent = pts[np.minimum(np.searchsorted(cum, targets, side="left"), quadrature_points - 1)].copy()
    for _ in range(iterations):
        bounds = (cent[:-1] + cent[1:]) * 0.5
        bucket = np.searchsorted(bounds, pts, side="right")
        sums = np.bincount(bucket, weights=pts * w, minlength=levels)
        mass = np.bincount(bucket, weights=w, minlength=levels)
        new = np.where(mass > 0, sums / np.where(mass > 0, mass, 1.0), cent)
        delta = float(np.abs(new - cent).max())
        cent = new
        if delta < 1e-13:
            break
    half = levels // 2
    mag = (np.abs(cent[:half]) + np.abs(cent[::-1][:half])) * 0.5
    cent[:half] = -mag
    cent[::-1][:half] = mag
    return cent


def pack_mixed_bit_indices(indices: Sequence[int], bit_widths: Sequence[int]) -> bytes:
    if len(indices) != len(bit_widths):
        raise TurboQuantError("indices and bit_widths differ in length")
    acc = avail = 0
    out = bytearray()
    for i, (idx, wd) in enumerate(zip(indices, bit_widths)):
        if not 1 <= wd <= 8 or not 0 <= int(idx) < (1 << wd):
            raise TurboQuantError(f"field {i} does not fit {wd} bits")
        acc |= int(idx) << avail
        avail += wd
        while avail >= 8:
            out.append(acc & 0xFF)
            acc >>= 8
            avail -= 8
    if avail:
        out.append(acc & 0xFF)
    return bytes(out)


def unpack_mixed_bit_indices(packed: bytes, bit_widths: Sequence[int]) -> tuple[int, ...]:
    raw = bytes(packed)
    if len(raw) != (sum(bit_widths) + 7) // 8:
        raise TurboQuantError("packed payload has the wrong length")
    acc = int.from_bytes(raw, "little")
    out = []
    for wd in bit_widths:
        out.append(acc & ((1 << wd) - 1))
        acc >>= wd
    if acc:
        raise TurboQuantError("non-zero padding bits")
    return tuple(out)


def default_outlier_indices(dimension: int) -> tuple[int, ...]:
    """Every other channel: a fixed, model-independent choice for tests and fresh caches."""
    return tuple(range(0, dimension, 2))


@dataclass(frozen=True)
class TurboQuantLayout:
    """Byte layout of one device record."""
    dimension: int
    qjl: bool            # record carries residual norm + sign bits (keys of qjl-3.5)
    bit_widths: tuple[int, ...]

    @property
    def index_bytes(self) -> int:
        return (sum(self.bit_widths) + 7) // 8

    @property
    def header_bytes(self) -> int:
        return 4 + ((4 + self.dimension // 8) if self.qjl else 0)

    @property
    def record_bytes(self) -> int:
        # one spare word after the indices lets the kernel read bit fields with a two-word funnel shift
        return (self.header_bytes + self.index_bytes + 4 + 15) // 16 * 16


class TurboQuantCodec:
    def __init__(self, dimension: int, *, profile: str = "mse-3.5", seed: int = 0, outlier_indices: Iterable[int] | None = None) -> None:
        if dimension < 2 or dimension % 2:
            raise TurboQuantError("3.5-bit profiles need an even dimension >= 2")
        profile = str(profile).strip().lower()
        if profile not in PROFILES:
            raise TurboQuantError("profile must be mse-3.5 or qjl-3.5")
        if outlier_indices is None:
            raise TurboQuantError("3.5-bit profiles need a fixed model-level outlier_indices set")
        outliers = tuple(sorted(set(int(i) for i in outlier_indices)))
        if len(outliers) != dimension // 2 or any(not 0 <= i < dimension for i in outliers):
            raise TurboQuantError(f"exactly {dimension // 2} distinct outlier channels inside the head dimension are required")
        self.dimension, self.profile, self.seed, self.outlier_indices = dimension, profile, seed, outliers
        oset = set(outliers)
        self.value_bit_widths = tuple(4 if i in oset else 3 for i in range(dimension))
        self.key_bit_widths = tuple(w - 1 for w in self.value_bit_widths) if profile == "qjl-3.5" else self.value_bit_widths
        self.rotation = deterministic_random_rotation(dimension, seed)
        self.qjl_projection = deterministic_qjl_projection(dimension, seed) if profile == "qjl-3.5" else None
        self.key_layout = TurboQuantLayout(dimension, profile == "qjl-3.5", self.key_bit_widths)
        self.value_layout = TurboQuantLayout(dimension, False, self.value_bit_widths)

    def centroids(self, width: int) -> np.ndarray:
        return lloyd_max_centroids(self.dimension, width)

    # -- numpy oracle (one vector) ---------------------------------------------------------
    def _quantise(self, unit: np.ndarray, widths: Sequence[int]) -> tuple[np.ndarray, np.ndarray]:
        rot = self.rotation @ unit
        idx = np.empty(self.dimension, dtype=np.int64)
        q = np.empty(self.dimension, dtype=np.float64)
        for wd in set(widths):
            sel = np.array([w == wd for w in widths])
            cb = self.centroids(wd)
            j = np.abs(rot[sel, None] - cb[None, :]).argmin(axis=1)
            idx[sel], q[sel] = j, cb[j]
        return idx, q

    def encode(self, vector: Sequence[float], *, key: bool) -> dict:
        x = np.asarray(vector, dtype=np.float64)
        if x.shape != (self.dimension,) or not np.isfinite(x).all():
            raise TurboQuantError(f"a vector of {self.dimension} finite numbers is required")
        widths = self.key_bit_widths if key else self.value_bit_widths
        norm = float(np.sqrt(x @ x))
        unit = x / norm if norm > 0 else np.zeros_like(x)
        idx, q = self._quantise(unit, widths)
        rec = {"norm": float(np.float32(norm)), "indices": pack_mixed_bit_indices(idx.tolist(), widths), "qjl": False}
        if key and self.profile == "qjl-3.5":
            resid = unit - self.rotation.T @ q
            signs = (self.qjl_projection @ resid) >= 0.0
            rec.update(qjl=True, residual_norm=float(np.float32(np.sqrt(resid @ resid))), signs=np.packbits(signs, bitorder="little").tobytes())
        return rec

    def decode(self, rec: dict, *, key: bool) -> np.ndarray:
        """The MSE reconstruction (what values use; keys only for inspection)."""
        widths = self.key_bit_widths if key else self.value_bit_widths
        idx = unpack_mixed_bit_indices(rec["indices"], widths)
        q = np.array([self.centroids(w)[i] for i, w in zip(idx, widths)])
        return rec["norm"] * (self.rotation.T @ q)

    def key_inner_product(self, query: Sequence[float], rec: dict) -> float:
        qv = np.asarray(query, dtype=np.float64)
        widths = self.key_bit_widths
        idx = unpack_mixed_bit_indices(rec["indices"], widths)
        c = np.array([self.centroids(w)[i] for i, w in zip(idx, widths)])
        base = float((self.rotation @ qv) @ c)
        if not rec.get("qjl"):
            return rec["norm"] * base
        signs = np.unpackbits(np.frombuffer(rec["signs"], dtype=np.uint8), bitorder="little")[:self.dimension].astype(np.float64) * 2 - 1
        corr = math.sqrt(math.pi / 2.0) / self.dimension * rec["residual_norm"] * float((self.qjl_projection @ qv) @ signs)
        return rec["norm"] * (base + corr)

    def attention_oracle(self, query: Sequence[float], keys: list[dict], values: list[dict], scale: float) -> np.ndarray:
        s = np.array([self.key_inner_product(query, k) for k in keys]) * scale
        p = np.exp(s - s.max())
        p /= p.sum()
        return sum(pi * self.decode(v, key=False) for pi, v in zip(p, values))

    # -- device side -----------------------------------------------------------------------
    def record_bytes_of(self, rec: dict, *, key: bool) -> bytes:
        lay = self.key_layout if key else self.value_layout
        out = bytearray(lay.record_bytes)
        out[0:4] = np.float32(rec["norm"]).tobytes()
        off = 4
        if lay.qjl:
            out[4:8] = np.float32(rec["residual_norm"]).tobytes()
            out[8:8 + self.dimension // 8] = rec["signs"]
            off = 8 + self.dimension // 8
        out[off:off + lay.index_bytes] = rec["indices"]
        return bytes(out)

    def device_tables(self, device) -> dict[str, torch.Tensor]:
        """Constant tables the kernels read: rotation, projection, centroids (2..4 bits, 16 slots
        each), and per-coordinate bit offsets / widths for keys and values."""
        cents = np.zeros((5, 16), dtype=np.float32)
        for wd in (2, 3, 4):
            cents[wd, :1 << wd] = self.centroids(wd)

        def offsets(widths):
            off = np.concatenate([[0], np.cumsum(widths)[:-1]])
            return np.stack([off, np.asarray(widths)], axis=1).astype(np.int32)

        t = {"rotation": torch.tensor(self.rotation, dtype=torch.float32), "centroids": torch.tensor(cents),
             "key_fields": torch.tensor(offsets(self.key_bit_widths)), "value_fields": torch.tensor(offsets(self.value_bit_widths))}
        t["projection"] = torch.tensor(self.qjl_projection if self.qjl_projection is not None else np.zeros((1, 1)), dtype=torch.float32)
        return {k: v.contiguous().to(device) for k, v in t.items()}


class TurboQuantKVCache:
    """Compressed K/V records on the device for ``n_seq`` sequences: ``append`` encodes one new
    token per listed sequence (ring rows ``position % cap``), ``attention`` runs one decode
    query per sequence over the compressed records."""

    def __init__(self, codec: TurboQuantCodec, n_seq: int, n_kv_heads: int, cap: int, device) -> None:
        import ctypes as C

        from ..ops import _lib
        self.codec, self.n_seq, self.n_kv_heads, self.cap = codec, n_seq, n_kv_heads, cap
        self.device = torch.device(device)
        self.tables = codec.device_tables(self.device)
        kb, vb = codec.key_layout.record_bytes, codec.value_layout.record_bytes
        self.k = torch.zeros(n_seq, n_kv_heads, cap, kb, dtype=torch.uint8, device=self.device)
        self.v = torch.zeros(n_seq, n_kv_heads, cap, vb, dtype=torch.uint8, device=self.device)
        self.lengths = torch.zeros(n_seq, dtype=torch.int32, device=self.device)
        self._len_host = [0] * n_seq

        class _Tables(C.Structure):
            _fields_ = [("rotation", C.c_void_p), ("projection", C.c_void_p), ("centroids", C.c_void_p), ("key_fields", C.c_void_p),
                        ("value_fields", C.c_void_p), ("D", C.c_int), ("qjl", C.c_int), ("key_rec_bytes", C.c_int), ("value_rec_bytes", C.c_int)]
        t = self.tables
        self._c = _Tables(t["rotation"].data_ptr(), t["projection"].data_ptr(), t["centroids"].data_ptr(), t["key_fields"].data_ptr(),
                          t["value_fields"].data_ptr(), codec.dimension, int(codec.profile == "qjl-3.5"), kb, vb)
        self._C, self._lib = C, _lib

    @property
    def bytes_per_token(self) -> int:
        return self.n_kv_heads * (self.k.shape[-1] + self.v.shape[-1])

    def append(self, k: torch.Tensor, v: torch.Tensor, seqs: Sequence[int] | None = None) -> None:
        """k, v: bf16 [rows, n_kv_heads * D] - one new token for each sequence in ``seqs``
        (default: sequences 0 .. rows-1)."""
        C, L = self._C, self._lib.load()
        rows = k.shape[0]
        seqs = list(range(rows)) if seqs is None else [int(s) for s in seqs]
        seq = torch.tensor(seqs, dtype=torch.int32, device=self.device)
        slot = torch.tensor([self._len_host[s] % self.cap for s in seqs], dtype=torch.int32, device=self.device)
        st = C.c_void_p(self._lib.stream_ptr())
        for x, rec, is_key in ((k, self.k, 1), (v, self.v, 0)):
            assert x.dtype == torch.bfloat16 and x.shape == (rows, self.n_kv_heads * self.codec.dimension) and x.stride(1) == 1
            rc = L.nfn_turboquant_encode(C.byref(self._c), C.c_void_p(x.data_ptr()), C.c_longlong(x.stride(0)), C.c_void_p(seq.data_ptr()),
                                         C.c_void_p(slot.data_ptr()), C.c_int(rows), C.c_int(self.n_kv_heads), C.c_int(self.cap), C.c_int(is_key),
                                         C.c_void_p(rec.data_ptr()), st)
            self._lib.check(rc, "nfn_turboquant_encode")
        for s in seqs:
            self._len_host[s] += 1
        self.lengths.copy_(torch.tensor(self._len_host, dtype=torch.int32), non_blocking=False)

    def attention(self, q: torch.Tensor, n_q_heads: int, scale: float | None = None) -> torch.Tensor:
        """q: bf16 [n_seq, n_q_heads * D] -> bf16 [n_seq, n_q_heads * D]."""
        C, L = self._C, self._lib.load()
        D = self.codec.dimension
        assert q.dtype == torch.bfloat16 and q.shape == (self.n_seq, n_q_heads * D) and q.stride(1) == 1
        out = torch.empty_like(q)
        rc = L.nfn_turboquant_attention(C.byref(self._c), C.c_void_p(q.data_ptr()), C.c_int(q.stride(0)), C.c_void_p(self.k.data_ptr()),
                                        C.c_void_p(self.v.data_ptr()), C.c_void_p(self.lengths.data_ptr()), C.c_void_p(out.data_ptr()),
                                        C.c_int(out.stride(0)), C.c_int(self.n_seq), C.c_int(n_q_heads), C.c_int(self.n_kv_heads), C.c_int(self.cap),
                                        C.c_float(D ** -0.5 if scale is None else scale), C.c_void_p(self._lib.stream_ptr()))
        self._lib.check(rc, "nfn_turboquant_attention")
        return out

    def reset(self, seq: int) -> None:
        self._len_host[seq] = 0
        self.lengths[seq] = 0

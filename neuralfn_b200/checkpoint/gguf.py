"""GGUF v3 reader / writer: metadata key-values, tensor directory, memory-mapped tensor data,
K-quant (Q4_K / Q5_K / Q6_K) / F16 / BF16 / F32 tensors.

``GGUFFile(path)`` parses the header without touching tensor data; ``raw(name)`` returns the
stored bytes (uint8 view of the mapping, ready for the device GEMV / dequantisation
kernels), ``dequantize(name)`` the fp32 values through the numpy oracles. ``write_gguf`` builds
files for tests and tools. Layout per the public GGUF specification: magic ``GGUF``, u32
version, u64 tensor count, u64 kv count, kv pairs, tensor infos, padding to
``general.alignment`` (default 32), tensor data. Dimensions are stored innermost first.
Import path of the reference: ``neuralfn/native_muse_glimmer_checkpoint.py`` (K-quant GGUF).
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import numpy as np

from ..quant import kquant

__all__ = ["GGUFFile", "GGUFTensor", "write_gguf"]

MAGIC = b"GGUF"
# value types of the key-value section
T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 = range(13)
_SCALAR = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f", T_BOOL: "<?", T_U64: "<Q",
           T_I64: "<q", T_F64: "<d"}
# ggml tensor types handled here: type id -> (elements per block, bytes per block)
_TENSOR = {0: (1, 4), 1: (1, 2), 30: (1, 2), 12: (256, 144), 13: (256, 176), 14: (256, 210)}
_TYPE_NAME = {0: "F32", 1: "F16", 30: "BF16", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K"}


@dataclass
class GGUFTensor:
    name: str
    shape: tuple[int, ...]   # outermost first (numpy order)
    ggml_type: int
    offset: int              # from the start of the data section
    nbytes: int

    @property
    def type_name(self) -> str:
        return _TYPE_NAME.get(self.ggml_type, f"type{self.ggml_type}")


class _Reader:
    def __init__(self, buf) -> None:
        self.buf, self.pos = buf, 0

    def take(self, fmt: str):
        v = struct.unpack_from(fmt, self.buf, self.pos)[0]
        self.pos += struct.calcsize(fmt)
        return v

    def string(self) -> str:
        n = self.take("<Q")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8")
        self.pos += n
        return s

    def value(self, t: int):
        if t in _SCALAR:
            return self.take(_SCALAR[t])
        if t == T_STR:
            return self.string()
        if t == T_ARR:
            et, n = self.take("<I"), self.take("<Q")
            return [self.value(et) for _ in range(n)]
        raise ValueError(f"unknown GGUF value type {t}")


class GGUFFile:
    def __init__(self, path) -> None:
        self.path = Path(path)
        self._f = open(self.path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        r = _Reader(self._mm)
        if bytes(self._mm[:4]) != MAGIC:
            raise ValueError(f"{self.path}: not a GGUF file")
        r.pos = 4
        self.version = r.take("<I")
        if self.version not in (2, 3):
            raise ValueError(f"unsupported GGUF version {self.version}")
        n_tensors, n_kv = r.take("<Q"), r.take("<Q")
        self.metadata: dict[str, Any] = {}
        for _ in range(n_kv):
            key = r.string()
            self.metadata[key] = r.value(r.take("<I"))
        self.tensors: dict[str, GGUFTensor] = {}
        for _ in range(n_tensors):
            name = r.string()
            nd = r.take("<I")
            dims = [r.take("<Q") for _ in range(nd)]
            gt, off = r.take("<I"), r.take("<Q")
            if gt not in _TENSOR:
                raise ValueError(f"{name}: unsupported ggml tensor type {gt}")
            per, bpb = _TENSOR[gt]
            numel = int(np.prod(dims)) if dims else 1
            if dims and dims[0] % per:
                raise ValueError(f"{name}: innermost dimension {dims[0]} is not a multiple of the block size {per}")
            self.tensors[name] = GGUFTensor(name, tuple(reversed(dims)), gt, off, numel // per * bpb)
        self.alignment = int(self.metadata.get("general.alignment", 32))
        self.data_start = (r.pos + self.alignment - 1) // self.alignment * self.alignment
        for t in self.tensors.values():
            if self.data_start + t.offset + t.nbytes > len(self._mm):
                raise ValueError(f"{t.name}: tensor data runs past the end of the file")

    def close(self) -> None:
        if getattr(self, "_mm", None) is not None:
            self._mm.close()
            self._f.close()
            self._mm = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def raw(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        return np.frombuffer(self._mm, dtype=np.uint8, count=t.nbytes, offset=self.data_start + t.offset)

    def packed(self, name: str) -> tuple[int, np.ndarray]:
        """(ggml type, the tensor's bytes as stored): what ``ResidentEngine.set_tensor_kquant`` takes for a Q4_K / Q5_K / Q6_K
        projection weight (rows of K / 256 super-blocks back to back). Row-wise pieces of one type (q | k | v) can be
        concatenated along the rows without decoding."""
        return self.tensors[name].ggml_type, self.raw(name).copy()      # a copy: it outlives the mapping

    def dequantize(self, name: str) -> np.ndarray:
        """fp32 values in the tensor's logical shape."""
        t = self.tensors[name]
        raw = self.raw(name)
        if t.ggml_type == 0:
            out = raw.view("<f4").astype(np.float32)
        elif t.ggml_type == 1:
            out = raw.view("<f2").astype(np.float32)
        elif t.ggml_type == 30:
            out = (raw.view("<u2").astype(np.uint32) << 16).view(np.float32)
        else:
            out = kquant.dequantize(t.ggml_type, raw.tobytes())
        return out.reshape(t.shape)

    def summary(self) -> dict:
        by_type: dict[str, int] = {}
        for t in self.tensors.values():
            by_type[t.type_name] = by_type.get(t.type_name, 0) + t.nbytes
        return {"version": self.version, "tensors": len(self.tensors), "bytes_by_type": by_type,
                "architecture": self.metadata.get("general.architecture"), "alignment": self.alignment}


def _kv_bytes(key: str, value) -> bytes:
    def s(x: str) -> bytes:
        b = x.encode("utf-8")
        return struct.pack("<Q", len(b)) + b

    def typed(v) -> tuple[int, bytes]:
        if isinstance(v, bool):
            return T_BOOL, struct.pack("<?", v)
        if isinstance(v, int):
            return (T_U32, struct.pack("<I", v)) if 0 <= v < 2 ** 32 else (T_I64, struct.pack("<q", v))
        if isinstance(v, float):
            return T_F32, struct.pack("<f", v)
        if isinstance(v, str):
            return T_STR, s(v)
        if isinstance(v, (list, tuple)):
            if not v:
                return T_ARR, struct.pack("<IQ", T_U32, 0)
            et, _ = typed(v[0])
            return T_ARR, struct.pack("<IQ", et, len(v)) + b"".join(typed(e)[1] for e in v)
        raise TypeError(f"cannot store {type(v).__name__} in GGUF metadata")

    t, payload = typed(value)
    return s(key) + struct.pack("<I", t) + payload


def write_gguf(path, metadata: dict[str, Any], tensors: dict[str, tuple[int, tuple[int, ...], bytes]], alignment: int = 32) -> None:
    """``tensors``: name -> (ggml type id, logical shape outermost first, raw bytes)."""
    meta = dict(metadata)
    meta.setdefault("general.alignment", alignment)
    head = MAGIC + struct.pack("<IQQ", 3, len(tensors), len(meta)) + b"".join(_kv_bytes(k, v) for k, v in meta.items())
    infos, blobs, off = b"", [], 0
    for name, (gt, shape, raw) in tensors.items():
        nb = name.encode("utf-8")
        dims = tuple(reversed(shape))
        infos += struct.pack("<Q", len(nb)) + nb + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", gt, off)
        pad = -len(raw) % alignment
        blobs.append(bytes(raw) + b"\0" * pad)
        off += len(raw) + pad
    body = head + infos
    body += b"\0" * (-len(body) % alignment)
    Path(path).write_bytes(body + b"".join(blobs))

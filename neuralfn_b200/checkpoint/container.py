"""Header + segments checkpoint files through the native container writer (exclusive
create, staged + fsync, exact-size reads, SHA-256 of the file returned)."""
from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Sequence

import numpy as np
import torch

from ..data import _rt

__all__ = ["write_container", "read_container", "peek_header", "publish_dir"]


def _host_bytes(t) -> tuple[int, int, object]:
    """(address, nbytes, keep-alive) of a contiguous host array / tensor."""
    if isinstance(t, torch.Tensor):
        t = t.detach()
        if t.device.type != "cpu":
            t = t.cpu()
        t = t.contiguous()
        return t.data_ptr(), t.numel() * t.element_size(), t
    a = np.ascontiguousarray(t)
    return a.ctypes.data, a.nbytes, a


def write_container(path, header: bytes, segments: Sequence) -> str:
    """Writes ``header`` followed by every segment; returns the file's SHA-256."""
    keep = [_host_bytes(s) for s in segments]
    n = len(keep)
    ptrs = (C.c_void_p * max(n, 1))(*[k[0] for k in keep])
    sizes = (C.c_uint64 * max(n, 1))(*[k[1] for k in keep])
    sha = C.create_string_buffer(65)
    hb = C.create_string_buffer(header, len(header))
    _rt.check(_rt.lib().nfn_ckpt_write(str(path).encode(), C.cast(hb, C.c_void_p), len(header), ptrs, sizes, n, sha), "ckpt_write")
    return sha.value.decode()


def read_container(path, header_bytes: int, segments: Sequence[torch.Tensor]) -> tuple[bytes, str]:
    """Fills the given contiguous CPU tensors in order; returns (header, sha256)."""
    for s in segments:
        assert s.device.type == "cpu" and s.is_contiguous()
    n = len(segments)
    ptrs = (C.c_void_p * max(n, 1))(*[s.data_ptr() for s in segments])
    sizes = (C.c_uint64 * max(n, 1))(*[s.numel() * s.element_size() for s in segments])
    sha = C.create_string_buffer(65)
    hb = C.create_string_buffer(max(header_bytes, 1))
    _rt.check(_rt.lib().nfn_ckpt_read(str(path).encode(), C.cast(hb, C.c_void_p), header_bytes, ptrs, sizes, n, sha), "ckpt_read")
    return hb.raw[:header_bytes], sha.value.decode()


def peek_header(path, header_bytes: int) -> tuple[bytes, int]:
    hb = C.create_string_buffer(header_bytes)
    size = C.c_uint64(0)
    _rt.check(_rt.lib().nfn_ckpt_peek(str(path).encode(), C.cast(hb, C.c_void_p), header_bytes, C.byref(size)), "ckpt_peek")
    return hb.raw, int(size.value)


def publish_dir(staging: Path, final: Path) -> None:
    _rt.check(_rt.lib().nfn_ckpt_publish_dir(str(staging).encode(), str(final).encode()), "ckpt_publish_dir")

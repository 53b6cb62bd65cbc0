"""ctypes binding of ``libnfn_b200_kernels.so`` (the sm_100a kernel library).

The library is a plain C ABI: raw device pointers in, CUDA stream in, ``int``
status out. Nothing here falls back to PyTorch: when a CUDA device is present
and the shared object is missing or fails to load, importing an op raises.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

_LIB = None
_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libnfn_b200_kernels.so"


class KernelLibraryError(RuntimeError):
    pass


class GemmArgs(ctypes.Structure):
    _fields_ = [
        ("a", ctypes.c_void_p), ("b", ctypes.c_void_p), ("c", ctypes.c_void_p),
        ("m", ctypes.c_int), ("n", ctypes.c_int), ("k", ctypes.c_int),
        ("lda", ctypes.c_int), ("ldb", ctypes.c_int), ("ldc", ctypes.c_int),
        ("a_mn", ctypes.c_int), ("b_mn", ctypes.c_int),
        ("flags", ctypes.c_int),
        ("alpha", ctypes.c_float), ("act_param", ctypes.c_float),
        ("bias", ctypes.c_void_p),
        ("aux_in", ctypes.c_void_p), ("ld_aux_in", ctypes.c_int),
        ("aux_out", ctypes.c_void_p), ("ld_aux_out", ctypes.c_int),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_longlong), ("split_k", ctypes.c_int),
    ]


def lib_path() -> Path:
    return Path(os.environ.get("NFN_B200_KERNEL_LIB", _LIB_PATH))


def available() -> bool:
    return lib_path().exists()


def load():
    """Load (once) and return the kernel library handle."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not path.exists():
        raise KernelLibraryError(
            f"{path} is missing: build it with `python -m neuralfn_b200.ops._build` "
            "(nvcc cross-compiles sm_100a without a GPU)")
    lib = ctypes.CDLL(str(path))
    lib.nfn_last_error.restype = ctypes.c_char_p
    lib.nfn_abi_version.restype = ctypes.c_int
    _LIB = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().nfn_last_error()
        raise KernelLibraryError(f"{what} failed (rc={rc}): {msg.decode() if msg else ''}")


def stream_ptr() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream


def launch_count() -> int:
    """Kernels launched by the library in this process so far (host-side counter;
    launches replayed from a CUDA graph are not seen by it)."""
    lib = load()
    lib.nfn_launch_count.restype = ctypes.c_longlong
    return int(lib.nfn_launch_count())


def status_read_reset() -> int:
    """Synchronise and return the first error code any kernel recorded (0 = ok)."""
    return int(load().nfn_status_read_reset())


STATUS_NAMES = {
    0: "ok", 1: "wait_full", 2: "wait_empty", 3: "wait_tmem_full", 4: "wait_tmem_empty",
    5: "wait_peer", 6: "bad_args", 7: "wait_misc",
}


def assert_status_ok(what: str = "kernel") -> None:
    code = status_read_reset()
    if code != 0:
        raise KernelLibraryError(f"{what}: device status {code} ({STATUS_NAMES.get(code, '?')})")

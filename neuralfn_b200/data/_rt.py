"""ctypes loader for the host-side native runtime (``libnfn_b200_runtime.so``)."""
from __future__ import annotations

import ctypes as C
from functools import lru_cache
from pathlib import Path

_LIB = Path(__file__).resolve().parent.parent / "lib" / "libnfn_b200_runtime.so"


class NativeRuntimeError(RuntimeError):
    pass


@lru_cache(maxsize=1)
def lib() -> C.CDLL:
    if not _LIB.exists():
        from ..ops import _build
        _build.build_runtime()
    L = C.CDLL(str(_LIB))
    vp, cp, i32, i64, u32, u64 = C.c_void_p, C.c_char_p, C.c_int, C.c_int64, C.c_uint32, C.c_uint64
    sig = {
        "nfn_rt_last_error": (cp, []),
        "nfn_rt_sha256_file": (i32, [cp, C.c_char_p]),
        "nfn_rt_sha256": (i32, [vp, u64, C.c_char_p]),
        "nfn_rt_preset_count": (i32, []),
        "nfn_rt_preset_name": (cp, [i32]),
        "nfn_rt_preset_family": (cp, [cp]),
        "nfn_dataset_open": (vp, [cp, i32, i32, i32]),
        "nfn_dataset_close": (None, [vp]),
        "nfn_dataset_json": (i32, [vp, i64, i64, i64, C.c_char_p, i32]),
        "nfn_dataset_tokens": (i64, [vp, i32]),
        "nfn_dataset_max_token": (i64, [vp, i32]),
        "nfn_sampler_open": (vp, [vp, i32, i64, i64, i32, i32]),
        "nfn_sampler_close": (None, [vp]),
        "nfn_sampler_total_batches": (i64, [vp]),
        "nfn_sampler_position": (i64, [vp]),
        "nfn_sampler_seek": (i32, [vp, i64]),
        "nfn_sampler_reset": (None, [vp]),
        "nfn_sampler_next_i32": (i32, [vp, vp, vp, i64]),
        "nfn_sampler_next_wrap_i32": (i32, [vp, vp, vp, i64]),
        "nfn_prefetcher_open": (vp, [vp, i32, C.POINTER(vp), C.POINTER(vp), i64]),
        "nfn_prefetcher_acquire": (i32, [vp, C.POINTER(i64)]),
        "nfn_prefetcher_release": (i32, [vp, i32]),
        "nfn_prefetcher_close": (None, [vp]),
        "nfn_write_legacy_shard": (i32, [cp, vp, u64, i32]),
        "nfn_write_v2_shard": (i32, [cp, vp, u64, u32, cp, cp, cp, cp, cp]),
        "nfn_records_open": (vp, [cp, i32, i32, i32, i64, i32, i32]),
        "nfn_records_close": (None, [vp]),
        "nfn_records_json": (i32, [vp, C.c_char_p, i32]),
        "nfn_records_total_batches": (i64, [vp]),
        "nfn_records_seq_len": (i64, [vp]),
        "nfn_records_seek": (i32, [vp, i64]),
        "nfn_records_reset": (None, [vp]),
        "nfn_records_next": (i32, [vp, vp, vp, vp, vp, i64]),
        "nfn_write_records": (i32, [cp, i32, u64, u32, u32, u32, cp, cp, cp, cp, vp, u64]),
        "nfn_ckpt_write": (i32, [cp, vp, u64, C.POINTER(vp), C.POINTER(u64), i32, C.c_char_p]),
        "nfn_ckpt_read": (i32, [cp, vp, u64, C.POINTER(vp), C.POINTER(u64), i32, C.c_char_p]),
        "nfn_ckpt_peek": (i32, [cp, vp, u64, C.POINTER(u64)]),
        "nfn_ckpt_publish_dir": (i32, [cp, cp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args
    return L


def last_error() -> str:
    return (lib().nfn_rt_last_error() or b"").decode("utf-8", "replace")


def check(rc: int, what: str) -> int:
    if rc < 0:
        raise NativeRuntimeError(f"{what}: {last_error()}")
    return rc


def handle(ptr, what: str):
    if not ptr:
        raise NativeRuntimeError(f"{what}: {last_error()}")
    return ptr


def read_json(fn, *args) -> dict:
    import json
    need = check(fn(*args, None, 0), "json")
    buf = C.create_string_buffer(need + 1)
    check(fn(*args, buf, need + 1), "json")
    return json.loads(buf.value.decode())


def shipped_presets() -> dict[str, str]:
    """Preset name -> family, as compiled into the host runtime."""
    L = lib()
    names = [L.nfn_rt_preset_name(i).decode() for i in range(L.nfn_rt_preset_count())]
    return {n: L.nfn_rt_preset_family(n.encode()).decode() for n in names}


def sha256_file(path: str) -> str:
    out = C.create_string_buffer(65)
    check(lib().nfn_rt_sha256_file(str(path).encode(), out), "sha256_file")
    return out.value.decode()

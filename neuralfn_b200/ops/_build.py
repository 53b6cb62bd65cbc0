"""In-tree build of the sm_100a kernel library and the native runtime pieces.

``build_kernels()`` compiles every ``.cu`` under ``csrc/kernels`` with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` into
``neuralfn_b200/lib/libnfn_b200_kernels.so``. nvcc cross-compiles without a GPU,
so the build runs on CPU-only machines; the resulting ``.so`` is what the GPU
machine loads. Objects are rebuilt only when their source (or a header) changed.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent.parent
KERNEL_SRC = PKG / "csrc" / "kernels"
RUNTIME_SRC = PKG / "csrc" / "runtime"
ENGINE_SRC = PKG / "csrc" / "engine"
LIB_DIR = PKG / "lib"
OBJ_DIR = PKG / "lib" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
]


def _extra_flags() -> list[str]:
    """Extra nvcc flags from ``NFN_EXTRA_NVCC_FLAGS`` (for instance ``-DNFN_KERNEL_TIMERS`` to compile
    the per-role cycle counters into the GEMM and attention kernels). They are part of the object
    digests, so changing them rebuilds."""
    return os.environ.get("NFN_EXTRA_NVCC_FLAGS", "").split()


def _nvcc() -> str:
    for cand in (os.environ.get("NFN_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NFN_NVCC")


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(str(p.name).encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS + _extra_flags()).encode())
    return h.hexdigest()


def _compile_one(src: Path, obj: Path, extra: list[str], verbose: bool) -> str:
    lang = ["-x", "cu"] if src.suffix == ".cpp" else []
    cmd = [_nvcc(), *NVCC_FLAGS, *_extra_flags(), *extra, *lang, "-I", str(KERNEL_SRC), "-I", str(ENGINE_SRC), "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return proc.stderr if verbose else ""


def build_kernels(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile the CUDA kernel library; returns the path of the shared object."""
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    out = LIB_DIR / "libnfn_b200_kernels.so"
    # the resident inference engine (host C++ driving the kernels) lives in the same library,
    # so it shares the library's CUDA runtime instance and needs no extra link step
    sources = sorted(KERNEL_SRC.glob("*.cu")) + sorted(ENGINE_SRC.glob("*.cpp"))
    headers = sorted(list(KERNEL_SRC.glob("*.h")) + list(KERNEL_SRC.glob("*.cuh")) + list(KERNEL_SRC.glob("*.inc")) +
                     list(ENGINE_SRC.glob("*.h")))
    hdr_digest = _digest(headers)
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    jobs = []
    objs = []
    for src in sources:
        obj = OBJ_DIR / (src.stem + ".o")
        stamp = OBJ_DIR / (src.stem + ".sha")
        want = hashlib.sha256((hdr_digest + _digest([src])).encode()).hexdigest()
        objs.append(obj)
        if not force and obj.exists() and stamp.exists() and stamp.read_text() == want:
            continue
        jobs.append((src, obj, stamp, want))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            futs = {ex.submit(_compile_one, s, o, extra, ptxas_info): (s, st, w) for s, o, st, w in jobs}
            for fut in concurrent.futures.as_completed(futs):
                s, st, w = futs[fut]
                log = fut.result()
                st.write_text(w)
                if verbose:
                    print(f"[build] {s.name}", file=sys.stderr)
                if ptxas_info and log:
                    print(log, file=sys.stderr)
    if jobs or not out.exists():
        cmd = [_nvcc(), "-shared", "-o", str(out), *map(str, objs),
               "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    return out


def build_runtime(force: bool = False, verbose: bool = False) -> list[Path]:
    """Compile the host-side native runtime (C++): one shared object per file
    group under ``csrc/runtime`` (token shards, checkpoint writers, resident
    inference engine). Pure g++, no CUDA needed."""
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    outs = []
    if not RUNTIME_SRC.exists():
        return outs
    sources = sorted(RUNTIME_SRC.glob("*.cpp"))
    if not sources:
        return outs
    headers = sorted(RUNTIME_SRC.glob("*.h"))
    out = LIB_DIR / "libnfn_b200_runtime.so"
    stamp = OBJ_DIR / "runtime.sha"
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    want = _digest(sources + headers)
    if force or not out.exists() or not stamp.exists() or stamp.read_text() != want:
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-Wextra", "-pthread",
               "-I", str(RUNTIME_SRC), "-I", str(KERNEL_SRC), "-o", str(out), *map(str, sources), "-ldl"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"g++ failed:\n{proc.stdout}\n{proc.stderr}")
        stamp.write_text(want)
        if verbose:
            print("[build] runtime", file=sys.stderr)
    outs.append(out)
    return outs


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force=force, verbose=verbose)
    build_runtime(force=force, verbose=verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    if "--ptxas" in sys.argv:
        build_kernels(force=True, verbose=True, ptxas_info=True)

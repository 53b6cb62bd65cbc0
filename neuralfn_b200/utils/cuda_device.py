"""Which GPU to use when the caller did not say: the one with no compute processes and the most
free memory. Reads only (NVML through ``pynvml`` when present, else ``nvidia-smi`` queries);
never changes a device setting.

Behavioural counterpart: ``neuralfn/native_cuda_device.py`` (an ``nvidia-smi``-based picker of a
dedicated GPU).
"""
from __future__ import annotations

import os
import shutil
import subprocess
from dataclasses import dataclass

__all__ = ["GpuInfo", "list_gpus", "pick_dedicated_gpu"]


@dataclass(frozen=True)
class GpuInfo:
    index: int
    name: str
    memory_total_mib: int
    memory_used_mib: int
    compute_processes: int

    @property
    def memory_free_mib(self) -> int:
        return self.memory_total_mib - self.memory_used_mib


def _via_nvml() -> list[GpuInfo] | None:
    try:
        import pynvml  # type: ignore
        pynvml.nvmlInit()
    except Exception:
        return None
    try:
        out = []
        for i in range(pynvml.nvmlDeviceGetCount()):
            h = pynvml.nvmlDeviceGetHandleByIndex(i)
            mem = pynvml.nvmlDeviceGetMemoryInfo(h)
            try:
                procs = len(pynvml.nvmlDeviceGetComputeRunningProcesses(h))
            except Exception:
                procs = 0
            name = pynvml.nvmlDeviceGetName(h)
            out.append(GpuInfo(i, name.decode() if isinstance(name, bytes) else str(name), mem.total >> 20, mem.used >> 20, procs))
        return out
    except Exception:
        return None
    finally:
        try:
            pynvml.nvmlShutdown()
        except Exception:
            pass


def parse_nvidia_smi_csv(text: str) -> list[GpuInfo]:
    """Rows of ``index, name, memory.total, memory.used`` (``--format=csv,noheader,nounits``)."""
    out = []
    for line in text.strip().splitlines():
        parts = [p.strip() for p in line.split(",")]
        if len(parts) < 4 or not parts[0].isdigit():
            continue
        out.append(GpuInfo(int(parts[0]), parts[1], int(float(parts[2])), int(float(parts[3])), 0))
    return out


def _via_smi() -> list[GpuInfo] | None:
    exe = shutil.which("nvidia-smi")
    if not exe:
        return None
    try:
        r = subprocess.run([exe, "--query-gpu=index,name,memory.total,memory.used", "--format=csv,noheader,nounits"], capture_output=True,
                           text=True, timeout=20)
    except Exception:
        return None
    return parse_nvidia_smi_csv(r.stdout) if r.returncode == 0 else None


def list_gpus() -> list[GpuInfo]:
    return _via_nvml() or _via_smi() or []


def pick_dedicated_gpu(gpus: list[GpuInfo] | None = None, *, min_free_mib: int = 0) -> int | None:
    """Index of the best candidate among the visible GPUs (``CUDA_VISIBLE_DEVICES`` is honoured when
    it lists plain indices), or None when there is none."""
    gpus = list_gpus() if gpus is None else gpus
    visible = os.environ.get("CUDA_VISIBLE_DEVICES", "")
    if visible and all(p.strip().isdigit() for p in visible.split(",")):
        allowed = {int(p) for p in visible.split(",")}
        gpus = [g for g in gpus if g.index in allowed]
    gpus = [g for g in gpus if g.memory_free_mib >= min_free_mib]
    if not gpus:
        return None
    return min(gpus, key=lambda g: (g.compute_processes, -g.memory_free_mib, g.index)).index

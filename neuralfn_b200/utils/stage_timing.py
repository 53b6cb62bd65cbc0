"""Per-stage CUDA-event timing and NVTX ranges for the native trainers.

Opt-in diagnostic (``NFN_NATIVE_GPT_STAGE_TIMING=1`` or ``StageTimer(enabled=True)``): every named
stage of a training step is bracketed by a pre-allocated CUDA event pair on the launching stream and,
when ``NFN_NVTX=1``, by an NVTX range of the same name, so the names show up in a timeline profiler.
Stage names are nested with dots (``block_forward.attention.qkv``, ``block_backward.mlp_fc.dinput``)
and the report uses the field names of the reference trainer's ``stage_timing`` JSON block
(``name, total_ms, count, avg_ms, first_step_*, steady_state_*``;
``neuralfn/csrc/native_gpt2/nfn_gpt2_native_train.cpp:19656-19760, 30535-30556``). Events are resolved
lazily (``collect()``), so recording does not synchronise the stream. A step recorded under a CUDA
graph cannot be timed stage by stage, which is why the trainer runs eagerly while this is on - the
same trade the reference makes (its stage timing is a diagnostic mode, not the benchmark mode).
"""
from __future__ import annotations

import contextlib
import os
from dataclasses import dataclass, field

__all__ = ["StageTimer", "stage_timing_requested"]


def stage_timing_requested() -> bool:
    return os.environ.get("NFN_NATIVE_GPT_STAGE_TIMING", "") in ("1", "true", "TRUE")


@dataclass
class _Record:
    name: str
    total_ms: float = 0.0
    count: int = 0
    first_step_total_ms: float = 0.0
    first_step_count: int = 0
    steady_state_total_ms: float = 0.0
    steady_state_count: int = 0

    def public(self) -> dict:
        avg = lambda t, c: (t / c) if c else 0.0  # noqa: E731
        return {"name": self.name, "total_ms": self.total_ms, "count": self.count, "avg_ms": avg(self.total_ms, self.count),
                "first_step_total_ms": self.first_step_total_ms, "first_step_count": self.first_step_count,
                "first_step_avg_ms": avg(self.first_step_total_ms, self.first_step_count),
                "steady_state_total_ms": self.steady_state_total_ms, "steady_state_count": self.steady_state_count,
                "steady_state_avg_ms": avg(self.steady_state_total_ms, self.steady_state_count)}


@dataclass
class StageTimer:
    enabled: bool = field(default_factory=stage_timing_requested)
    nvtx: bool = field(default_factory=lambda: os.environ.get("NFN_NVTX", "") == "1")
    max_events: int = 65536
    time_fn: object = None   # tests inject a fake clock: callable(name) -> milliseconds

    def __post_init__(self) -> None:
        self.records: dict[str, _Record] = {}
        self._pending: list[tuple[str, int, object, object]] = []
        self._free: list[tuple[object, object]] = []
        self.step = 0
        self.dropped = 0
        self.event_pairs_created = 0

    # ------------------------------------------------------------------------------------
    def _pair(self):
        if self._free:
            return self._free.pop()
        import torch
        self.event_pairs_created += 1
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    @contextlib.contextmanager
    def stage(self, name: str):
        if not self.enabled:
            yield
            return
        if self.time_fn is not None:  # CPU tests
            yield
            self._add(name, self.step, float(self.time_fn(name)))
            return
        import torch
        if self.nvtx:
            torch.cuda.nvtx.range_push(name)
        if len(self._pending) >= self.max_events:
            self.dropped += 1
            try:
                yield
            finally:
                if self.nvtx:
                    torch.cuda.nvtx.range_pop()
            return
        a, b = self._pair()
        a.record()
        try:
            yield
        finally:
            b.record()
            if self.nvtx:
                torch.cuda.nvtx.range_pop()
            self._pending.append((name, self.step, a, b))

    def next_step(self) -> None:
        """Marks the end of an optimizer step (step 0 is the "first step" bucket)."""
        self.step += 1

    def _add(self, name: str, step: int, ms: float) -> None:
        r = self.records.setdefault(name, _Record(name))
        r.total_ms += ms
        r.count += 1
        if step == 0:
            r.first_step_total_ms += ms
            r.first_step_count += 1
        else:
            r.steady_state_total_ms += ms
            r.steady_state_count += 1

    def collect(self) -> None:
        """Resolve recorded event pairs (synchronises the device once)."""
        if not self._pending:
            return
        import torch
        torch.cuda.synchronize()
        for name, step, a, b in self._pending:
            self._add(name, step, a.elapsed_time(b))
            self._free.append((a, b))
        self._pending.clear()

    def report(self) -> dict:
        """The ``timing`` sub-block of the training report."""
        if self.time_fn is None:
            self.collect()
        return {"stage_timing_enabled": self.enabled, "stage_timing_event_count": sum(r.count for r in self.records.values()),
                "stage_timing_dropped_event_count": self.dropped, "stage_timing_event_pair_create_count": self.event_pairs_created,
                "stage_timing": [r.public() for r in self.records.values()]}

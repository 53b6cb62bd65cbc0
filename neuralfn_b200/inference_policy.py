"""Process-wide compute policy for generation: a temperature of exactly zero asks for *strict*
execution - deterministic algorithms, no TF32, no reduced-precision reductions, no autocast - and
anything else runs with the standard fast settings.

The strict settings are process-global switches of the tensor runtime, so requests are ordered by
a readers / writer gate: standard generations share it, a strict generation holds it alone, and a
waiting strict request stops new standard ones from entering (no starvation).

``CUBLAS_WORKSPACE_CONFIG`` only takes effect when cuBLAS initialises, hence
``prepare_inference_process_environment()`` has to run before the first CUDA use of a process that
may later serve a strict request; this module imports no tensor library itself.

The resident sm_100a engine needs none of those switches: its decode path has no atomics and no
data-dependent reduction order (split-K slices and attention splits are merged in index order), so
equal inputs give equal tokens in either mode; the policy record says so for telemetry.

Behavioural counterpart: ``neuralfn/inference_policy.py:23-572``.
"""
from __future__ import annotations

import math
import os
import sys
import threading
from contextlib import contextmanager
from dataclasses import asdict, dataclass
from typing import Any, Iterator

__all__ = ["DETERMINISTIC_CUBLAS_WORKSPACE_CONFIG", "prepare_inference_process_environment", "validate_inference_temperature",
           "temperature_uses_strict_inference", "InferenceConcurrencyGate", "INFERENCE_CONCURRENCY_GATE", "InferenceComputePolicy",
           "STANDARD_INFERENCE_POLICY", "STRICT_INFERENCE_POLICY", "compute_policy_payload", "inference_execution",
           "validate_strict_graph_support"]

DETERMINISTIC_CUBLAS_WORKSPACE_CONFIG = ":4096:8"
_LOSSY_COMPRESSIONS = frozenset({"int8", "int4", "nf4", "fp8", "mxfp4", "mxfp8", "nvfp4", "ternary", "kquant", "q4_k", "q5_k", "q6_k"})


def prepare_inference_process_environment() -> None:
    """Sets the cuBLAS workspace configuration that deterministic matmuls need. Idempotent; refuses
    when CUDA is already up with another value, because the setting would silently not apply."""
    want = DETERMINISTIC_CUBLAS_WORKSPACE_CONFIG
    torch_mod = sys.modules.get("torch")
    cuda = getattr(torch_mod, "cuda", None)
    started = bool(cuda is not None and getattr(cuda, "is_initialized", lambda: False)())
    if started and os.environ.get("CUBLAS_WORKSPACE_CONFIG") != want:
        raise RuntimeError(f"CUDA is already initialised without CUBLAS_WORKSPACE_CONFIG={want!r}; restart the process and prepare the "
                           "environment first")
    os.environ["CUBLAS_WORKSPACE_CONFIG"] = want


def validate_inference_temperature(value: Any) -> float:
    try:
        t = float(value)
    except (TypeError, ValueError):
        raise ValueError("temperature must be a finite number >= 0") from None
    if isinstance(value, bool) or not math.isfinite(t) or t < 0.0:
        raise ValueError("temperature must be a finite number >= 0")
    return t


def temperature_uses_strict_inference(value: Any) -> bool:
    return validate_inference_temperature(value) == 0.0


class InferenceConcurrencyGate:
    """Readers / writer lock with writer preference."""

    def __init__(self) -> None:
        self._cv = threading.Condition()
        self._shared = 0
        self._exclusive = False
        self._exclusive_waiting = 0

    @contextmanager
    def shared(self) -> Iterator[None]:
        with self._cv:
            self._cv.wait_for(lambda: not self._exclusive and self._exclusive_waiting == 0)
            self._shared += 1
        try:
            yield
        finally:
            with self._cv:
                self._shared -= 1
                self._cv.notify_all()

    @contextmanager
    def exclusive(self) -> Iterator[None]:
        with self._cv:
            self._exclusive_waiting += 1
            try:
                self._cv.wait_for(lambda: not self._exclusive and self._shared == 0)
                self._exclusive = True
            finally:
                self._exclusive_waiting -= 1
        try:
            yield
        finally:
            with self._cv:
                self._exclusive = False
                self._cv.notify_all()


INFERENCE_CONCURRENCY_GATE = InferenceConcurrencyGate()


@dataclass(frozen=True)
class InferenceComputePolicy:
    mode: str
    trigger: str | None
    deterministic_algorithms: bool
    autocast_disabled: bool
    tf32_disabled: bool
    reduced_precision_reductions_disabled: bool
    fast_math_disabled: bool

    @property
    def strict(self) -> bool:
        return self.mode == "strict"


STANDARD_INFERENCE_POLICY = InferenceComputePolicy("standard", None, False, False, False, False, False)
STRICT_INFERENCE_POLICY = InferenceComputePolicy("strict", "temperature_zero", True, True, True, True, True)


def compute_policy_payload(policy: InferenceComputePolicy, *, backend: str) -> dict[str, Any]:
    """The telemetry record attached to generation results (stable keys, version 1)."""
    return {"version": 1, "backend": str(backend), **asdict(policy)}


class _TorchSwitches:
    """Saves the process-global switches, applies the strict values, restores on exit."""

    def __init__(self, torch_module: Any) -> None:
        self.t = torch_module
        self.saved: list[tuple[Any, str, Any]] = []

    def _set(self, obj: Any, name: str, value: Any) -> None:
        if obj is not None and hasattr(obj, name):
            self.saved.append((obj, name, getattr(obj, name)))
            setattr(obj, name, value)

    def __enter__(self) -> "_TorchSwitches":
        t = self.t
        self.det = (t.are_deterministic_algorithms_enabled(), t.is_deterministic_algorithms_warn_only_enabled())
        t.use_deterministic_algorithms(True, warn_only=False)
        matmul = getattr(getattr(t.backends, "cuda", None), "matmul", None)
        self._set(matmul, "allow_tf32", False)
        self._set(matmul, "allow_fp16_reduced_precision_reduction", False)
        self._set(matmul, "allow_bf16_reduced_precision_reduction", False)
        cudnn = getattr(t.backends, "cudnn", None)
        self._set(cudnn, "allow_tf32", False)
        self._set(cudnn, "benchmark", False)
        self._set(cudnn, "deterministic", True)
        self.precision = t.get_float32_matmul_precision()
        t.set_float32_matmul_precision("highest")
        self.autocasts = [t.autocast(device_type=d, enabled=False) for d in ("cuda", "cpu")]
        for a in self.autocasts:
            a.__enter__()
        return self

    def __exit__(self, *exc) -> None:
        t = self.t
        for a in reversed(self.autocasts):
            a.__exit__(*exc)
        t.set_float32_matmul_precision(self.precision)
        for obj, name, value in reversed(self.saved):
            setattr(obj, name, value)
        t.use_deterministic_algorithms(self.det[0], warn_only=self.det[1])


@contextmanager
def inference_execution(temperature: Any, *, torch_module: Any | None = None, native_engine: bool = False) -> Iterator[InferenceComputePolicy]:
    """Wrap ONE whole generation (every forward, every token choice). Standard temperatures share
    the gate; temperature 0 takes it exclusively and, for the tensor runtime, flips the strict
    switches for the duration (``torch_module`` = the imported ``torch``). ``native_engine=True``
    marks a generation that runs on the resident engine only: strict needs no switches there."""
    if not temperature_uses_strict_inference(temperature):
        with INFERENCE_CONCURRENCY_GATE.shared():
            yield STANDARD_INFERENCE_POLICY
        return
    if native_engine:
        with INFERENCE_CONCURRENCY_GATE.exclusive():
            yield STRICT_INFERENCE_POLICY
        return
    if torch_module is None:
        raise RuntimeError("strict inference on the tensor runtime needs the imported torch module")
    cuda = getattr(torch_module, "cuda", None)
    if cuda is not None and cuda.is_available() and os.environ.get("CUBLAS_WORKSPACE_CONFIG") != DETERMINISTIC_CUBLAS_WORKSPACE_CONFIG:
        raise RuntimeError("strict inference needs prepare_inference_process_environment() before CUDA initialisation")
    with INFERENCE_CONCURRENCY_GATE.exclusive():
        with _TorchSwitches(torch_module):
            yield STRICT_INFERENCE_POLICY


def validate_strict_graph_support(graph: Any) -> None:
    """Fails closed when a graph states that it computes in a lossy format (compressed template,
    low-precision activations, quantised or low-bit module nodes, at any nesting depth)."""
    cfg = dict(getattr(graph, "torch_config", {}) or {})
    act = str(cfg.get("tile_cuda_activation_dtype", "") or "").strip().lower()
    if act not in ("", "none", "float32", "fp32"):
        raise RuntimeError(f"temperature 0 (strict) does not run with {act!r} activations; use float32")
    template = dict(dict(cfg.get("template_spec", {}) or {}).get("template", {}) or {})
    comp = str(template.get("compression", "none") or "none").strip().lower()
    if comp in _LOSSY_COMPRESSIONS:
        raise RuntimeError(f"temperature 0 (strict) does not run a graph compressed as {comp!r}")
    seen: set[int] = set()

    def walk(g: Any) -> None:
        if g is None or id(g) in seen:
            return
        seen.add(id(g))
        for node in getattr(g, "nodes", {}).values():
            nd = node.neuron_def
            mtype = str(getattr(nd, "module_type", "") or "").lower()
            if any(tag in mtype for tag in ("fp8", "mxfp", "nvfp4", "ternary", "bitlinear", "nf4", "kquant", "int8")):
                raise RuntimeError(f"temperature 0 (strict) does not run the low-precision stage {nd.module_type!r} (node {node.instance_id})")
            walk(getattr(nd, "subgraph", None))
        for versions in (getattr(g, "variant_library", {}) or {}).values():
            for sub in versions.values():
                walk(sub)

    walk(graph)

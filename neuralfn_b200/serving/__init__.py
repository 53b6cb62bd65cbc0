"""Serving: resident inference engine bindings, generation loop, HTTP endpoints."""
from .engine import (EngineConfig, EngineError, ResidentEngine, Sampling, resident_inference_abi_version,
                     resident_inference_capabilities)

__all__ = ["EngineConfig", "EngineError", "ResidentEngine", "Sampling", "resident_inference_abi_version",
           "resident_inference_capabilities"]

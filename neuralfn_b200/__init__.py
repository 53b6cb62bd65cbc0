"""neuralfn_b200: a B200-native (sm_100a) graph-neuron LLM framework.

Public names are resolved lazily so that importing the package does not pull in
torch or numpy (the scalar graph runtime and the CLI dispatcher stay light).
"""
from __future__ import annotations

import importlib

__version__ = "0.1.0"

_LAZY: dict[str, str] = {}


def _register(module: str, *names: str) -> None:
    for n in names:
        _LAZY[n] = module


def __getattr__(name: str):
    mod = _LAZY.get(name)
    if mod is None:
        raise AttributeError(f"module 'neuralfn_b200' has no attribute {name!r}")
    value = getattr(importlib.import_module(mod, __name__), name)
    globals()[name] = value
    return value


def __dir__():
    return sorted(list(globals()) + list(_LAZY))

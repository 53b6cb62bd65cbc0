"""Typed value slots of the scalar graph runtime.

A ``Port`` carries an optional closed range, an optional quantisation step and a
semantic dtype tag. ``condition`` is clamp-then-quantise; the executor applies it
to every edge value entering a port and to every value leaving a neuron.
Behavioural counterpart of the reference's ``neuralfn/port.py:9-67``; the JSON
form (``name, range, precision, dtype``) is identical.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Tuple

__all__ = ["Port"]


@dataclass(frozen=True)
class Port:
    name: str
    range: Optional[Tuple[float, float]] = None
    precision: Optional[float] = None
    dtype: str = "float"

    def __post_init__(self) -> None:
        if self.range is not None:
            lo, hi = self.range
            if not lo < hi:
                raise ValueError(f"Port '{self.name}': range low ({lo}) must be < high ({hi})")
        if self.precision is not None and not self.precision > 0:
            raise ValueError(f"Port '{self.name}': precision must be > 0")

    # -- value conditioning -------------------------------------------------
    def clamp(self, value: float) -> float:
        if self.range is None:
            return value
        lo, hi = self.range
        if value < lo:
            return lo
        if value > hi:
            return hi
        return value

    def quantize(self, value: float) -> float:
        step = self.precision
        if step is None:
            return value
        return round(value / step) * step

    def condition(self, value: float) -> float:
        return self.quantize(self.clamp(value))

    @property
    def is_transparent(self) -> bool:
        """True when conditioning is the identity (no range, no precision)."""
        return self.range is None and self.precision is None

    # -- JSON ---------------------------------------------------------------
    def to_dict(self) -> dict[str, Any]:
        return {
            "name": self.name,
            "range": None if self.range is None else [self.range[0], self.range[1]],
            "precision": self.precision,
            "dtype": self.dtype,
        }

    @classmethod
    def from_dict(cls, payload: dict[str, Any]) -> "Port":
        rng = payload.get("range")
        return cls(
            name=payload["name"],
            range=None if rng is None else (rng[0], rng[1]),
            precision=payload.get("precision"),
            dtype=payload.get("dtype", "float"),
        )

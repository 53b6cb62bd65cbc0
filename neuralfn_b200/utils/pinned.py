"""Pinned host staging for asynchronous host -> device copies issued every step.

``dst.copy_(pinned, non_blocking=True)`` only queues the copy; the host returns at once and
runs ahead of the GPU whenever it does not synchronise each step (kernel-only timing loops,
training loops that read the loss only every N steps). Rewriting the same pinned buffer for
step t + k while the copy of step t is still queued makes step t consume step t + k's values
(learning rate, bias corrections, tokens). ``PinnedRing`` rotates through a few pinned slots
and guards each one with a CUDA event recorded right after its copy: a slot is rewritten only
after the copy that last read it has executed.
"""
from __future__ import annotations

import torch

__all__ = ["PinnedRing"]


class PinnedRing:
    def __init__(self, numel: int, dtype: torch.dtype, slots: int = 4) -> None:
        pin = torch.cuda.is_available()
        self.slots = [torch.zeros(numel, dtype=dtype).pin_memory() if pin else torch.zeros(numel, dtype=dtype)
                      for _ in range(max(2, slots))]
        self.events: list = [None] * len(self.slots)
        self._next = 0
        self.last = self.slots[0]  # slot written by the most recent ``upload`` (for logging)
        self.waits = 0             # how often the host had to wait for a slot (test hook)

    def upload(self, dst: torch.Tensor, values) -> torch.Tensor:
        """Copy ``values`` (a tensor or a sequence of numbers, at most ``numel`` entries) into the
        next free slot and queue ``dst[:n] <- slot[:n]`` on the current stream."""
        i = self._next
        self._next = (i + 1) % len(self.slots)
        ev = self.events[i]
        if ev is not None and not ev.query():
            self.waits += 1
            ev.synchronize()
        buf = self.slots[i]
        src = values if isinstance(values, torch.Tensor) else torch.tensor(list(values), dtype=buf.dtype)
        n = src.numel()
        buf[:n].copy_(src.reshape(-1))
        dst.reshape(-1)[:n].copy_(buf[:n], non_blocking=True)
        if dst.is_cuda:
            if ev is None:
                ev = self.events[i] = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(dst.device))
        self.last = buf
        return buf

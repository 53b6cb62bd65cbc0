"""Bounded LRU cache of sealed session prefixes.

A finished request parks its session here instead of closing it. A new request asks for the
cached entry that shares the longest token prefix with its prompt, receives a *fork* of it
(device-to-device KV copy through ``NativeInferenceModel.fork_session``) and only prefills
the remainder. Entries are immutable while cached ("sealed"); a lease pins an entry while a
fork is being made so eviction cannot pull it away mid-copy. The cache never holds more than
``capacity`` sessions and always leaves ``reserve_slots`` engine slots for live requests.

Behavioural counterpart: ``neuralfn/_native_prefix_cache.py``.
"""
from __future__ import annotations

import threading
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Sequence

from .inference import InferenceError, NativeInferenceModel, NativeInferenceSession

__all__ = ["PrefixCache", "PrefixLease"]


@dataclass
class _Entry:
    key: int
    session: NativeInferenceSession
    tokens: tuple[int, ...]
    leases: int = 0
    hits: int = 0


@dataclass
class PrefixLease:
    """Result of ``acquire``: a fresh session and how many prompt tokens it already holds."""
    session: NativeInferenceSession
    reused_tokens: int
    entry_key: int | None = None


def _common_prefix(a: Sequence[int], b: Sequence[int]) -> int:
    n = min(len(a), len(b))
    i = 0
    while i < n and a[i] == b[i]:
        i += 1
    return i


class PrefixCache:
    def __init__(self, model: NativeInferenceModel, capacity: int = 4, *, reserve_slots: int = 1, min_reuse_tokens: int = 16) -> None:
        slots = model.engine.config.max_batch
        if capacity < 0 or reserve_slots < 1:
            raise ValueError("capacity >= 0 and reserve_slots >= 1 required")
        self.model = model
        self.capacity = max(0, min(capacity, slots - reserve_slots))
        self.min_reuse_tokens = min_reuse_tokens
        self._entries: "OrderedDict[int, _Entry]" = OrderedDict()
        self._next_key = 1
        self._lock = threading.RLock()
        self.stats = {"lookups": 0, "hits": 0, "reused_tokens": 0, "stored": 0, "evicted": 0}

    def __len__(self) -> int:
        return len(self._entries)

    # -- lookup ----------------------------------------------------------------------------
    def acquire(self, prompt: Sequence[int], seed: int | None = None) -> PrefixLease:
        """A session for ``prompt``: forked from the best cached prefix when one is worth it,
        otherwise fresh. The caller prefills ``prompt[lease.reused_tokens:]`` and owns the session."""
        prompt = [int(t) for t in prompt]
        with self._lock:
            self.stats["lookups"] += 1
            best, best_n = None, 0
            for e in self._entries.values():
                # never reuse the whole prompt: the last prompt token must be run to get logits
                n = min(_common_prefix(e.tokens, prompt), len(prompt) - 1)
                if n > best_n:
                    best, best_n = e, n
            if best is not None and best_n >= self.min_reuse_tokens:
                best.leases += 1
                try:
                    self._make_room_for_live()
                    child = self.model.fork_session(best.session, best_n, seed)
                except InferenceError:
                    child = None
                finally:
                    best.leases -= 1
                if child is not None:
                    best.hits += 1
                    self._entries.move_to_end(best.key)
                    self.stats["hits"] += 1
                    self.stats["reused_tokens"] += best_n
                    return PrefixLease(child, best_n, best.key)
            self._make_room_for_live()
            return PrefixLease(self.model.create_session(seed), 0, None)

    def _make_room_for_live(self) -> None:
        """Evicts least-recently-used unleased entries until the engine has a free slot."""
        while not self.model._free and self._evict_one():
            pass

    def _evict_one(self) -> bool:
        for key, e in self._entries.items():
            if e.leases == 0:
                del self._entries[key]
                e.session.close()
                self.stats["evicted"] += 1
                return True
        return False

    # -- store -----------------------------------------------------------------------------
    def release(self, session: NativeInferenceSession, *, keep: bool = True) -> None:
        """Hands a finished session back. With ``keep`` it is sealed and cached (its cached
        tokens become reusable); otherwise, or when the cache is disabled, it is closed."""
        with self._lock:
            if not keep or self.capacity == 0 or session.closed or session.cached_tokens < self.min_reuse_tokens:
                session.close()
                return
            tokens = tuple(session._tokens)
            for e in self._entries.values():
                if e.tokens[:len(tokens)] == tokens:  # an existing entry already covers this one
                    session.close()
                    return
            # drop entries that the new one fully covers
            for key in [k for k, e in self._entries.items() if e.leases == 0 and tokens[:len(e.tokens)] == e.tokens]:
                self._entries.pop(key).session.close()
                self.stats["evicted"] += 1
            while len(self._entries) >= self.capacity:
                if not self._evict_one():
                    session.close()
                    return
            session._pending = None
            key = self._next_key
            self._next_key += 1
            self._entries[key] = _Entry(key, session, tokens)
            self.stats["stored"] += 1

    def clear(self) -> None:
        with self._lock:
            for e in self._entries.values():
                e.session.close()
            self._entries.clear()

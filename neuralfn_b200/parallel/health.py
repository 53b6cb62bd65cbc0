"""Failure detection for multi-rank jobs, host side only: vote before commit, heartbeats through
the rendezvous store, a step watchdog, and a local launcher that ends every rank when one fails.

Nothing here touches a GPU. Device-side waits are bounded inside the kernels themselves (they
give up after a second, set the status word and return); these helpers cover what the host has
to notice: a rank that raised, exited, or stopped making progress.

* ``vote_all_ok`` - every rank contributes "I failed" (0/1) to a sum; all ranks learn the same
  answer before anyone commits a side effect (a checkpoint, an optimizer step after a shard
  check). The pattern of the reference's pipeline trainer (``muse_glimmer_native_train.cpp:
  6405-6412, 6458-6487``).
* ``Heartbeat`` - every rank publishes (step, wall time) under its key in the job's key-value
  store; ``stale_peers`` lists ranks whose last beat is older than a limit, so a rank can stop
  *between* steps instead of entering a collective its peer will never join.
* ``StepWatchdog`` - a daemon thread that fires a callback when ``beat()`` has not been called
  for ``timeout_s`` (a hung step on this rank).
* ``launch_local_ranks`` - starts one process per rank and, on the first non-zero exit, ends the
  others by PID (the reference launcher's kill-siblings rule, ``cli/nfn.py:3920-3928``).
"""
from __future__ import annotations

import json
import os
import signal
import subprocess
import sys
import threading
import time
from dataclasses import dataclass
from typing import Callable, Sequence

import torch
import torch.distributed as dist

__all__ = ["RankFailure", "vote_all_ok", "commit_if_all_ok", "Heartbeat", "StepWatchdog", "launch_local_ranks", "LaunchResult"]


class RankFailure(RuntimeError):
    """Some rank (possibly another one) reported a failure in a vote."""


def vote_all_ok(ok: bool, group=None, device: torch.device | str | None = None) -> tuple[bool, int]:
    """Returns (everyone ok, number of ranks that failed). Collective: every rank must call it,
    *including* the ones that failed - catch the local exception, vote, then re-raise."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return bool(ok), 0 if ok else 1
    if device is None:
        device = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([0 if ok else 1], dtype=torch.int32, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    failed = int(t.item())
    return failed == 0, failed


def commit_if_all_ok(prepare: Callable[[], object], commit: Callable[[object], None], group=None, device=None, what: str = "step") -> object:
    """Runs ``prepare`` (may raise), votes, and only when every rank succeeded runs ``commit``.
    Raises ``RankFailure`` on every rank otherwise; the local exception is chained."""
    err: BaseException | None = None
    value = None
    try:
        value = prepare()
    except Exception as exc:  # vote first, report afterwards
        err = exc
    ok, failed = vote_all_ok(err is None, group, device)
    if not ok:
        raise RankFailure(f"{what}: {failed} rank(s) failed; nothing was committed") from err
    commit(value)
    return value


class Heartbeat:
    """``store`` is any ``torch.distributed`` store (TCPStore, FileStore, HashStore)."""

    def __init__(self, store, rank: int, world: int, prefix: str = "nfn/hb") -> None:
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), json.dumps({"step": int(step), "t": time.time()}))

    def read(self, r: int) -> dict | None:
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return None
            return json.loads(bytes(self.store.get(self._key(r))).decode("utf-8"))
        except Exception:
            return None

    def stale_peers(self, max_age_s: float, now: float | None = None) -> list[int]:
        now = time.time() if now is None else now
        out = []
        for r in range(self.world):
            if r == self.rank:
                continue
            rec = self.read(r)
            if rec is None or now - float(rec["t"]) > max_age_s:
                out.append(r)
        return out

    def lagging_peers(self, step: int, max_lag_steps: int) -> list[int]:
        out = []
        for r in range(self.world):
            rec = self.read(r) if r != self.rank else None
            if rec is not None and step - int(rec["step"]) > max_lag_steps:
                out.append(r)
        return out


class StepWatchdog:
    def __init__(self, timeout_s: float, on_timeout: Callable[[float], None] | None = None, poll_s: float = 0.05) -> None:
        self.timeout_s, self.poll_s = float(timeout_s), poll_s
        self.on_timeout = on_timeout or self._default
        self.fired = False
        self._last = time.monotonic()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, name="nfn-step-watchdog", daemon=True)

    @staticmethod
    def _default(idle: float) -> None:
        print(json.dumps({"event": "watchdog_timeout", "idle_seconds": round(idle, 3), "pid": os.getpid()}), file=sys.stderr, flush=True)

    def start(self) -> "StepWatchdog":
        self._last = time.monotonic()
        self._thread.start()
        return self

    def beat(self) -> None:
        self._last = time.monotonic()

    def _run(self) -> None:
        while not self._stop.wait(self.poll_s):
            idle = time.monotonic() - self._last
            if idle > self.timeout_s and not self.fired:
                self.fired = True
                self.on_timeout(idle)

    def stop(self) -> None:
        self._stop.set()
        if self._thread.is_alive():
            self._thread.join(timeout=1.0)

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.stop()


@dataclass
class LaunchResult:
    exit_codes: list[int | None]
    first_failure: int | None   # rank that failed first (None: all succeeded)
    killed: list[int]           # ranks ended by the launcher

    @property
    def ok(self) -> bool:
        return self.first_failure is None and all(c == 0 for c in self.exit_codes)


def launch_local_ranks(argv: Sequence[str], world: int, *, env: dict | None = None, master_port: int = 29533, timeout_s: float | None = None,
                       grace_s: float = 3.0, poll_s: float = 0.05) -> LaunchResult:
    """Starts ``world`` copies of ``argv`` with RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR
    (127.0.0.1) / MASTER_PORT set. When one exits non-zero (or the overall timeout passes) the
    others get SIGTERM, then SIGKILL after ``grace_s`` - by PID, never by name."""
    procs: list[subprocess.Popen] = []
    base = dict(os.environ if env is None else env)
    for r in range(world):
        e = dict(base, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(master_port))
        procs.append(subprocess.Popen(list(argv), env=e))
    t0 = time.monotonic()
    first, killed = None, []
    while True:
        codes = [p.poll() for p in procs]
        bad = [r for r, c in enumerate(codes) if c not in (None, 0)]
        if bad and first is None:
            first = bad[0]
        timed_out = timeout_s is not None and time.monotonic() - t0 > timeout_s
        if first is not None or timed_out:
            live = [r for r, c in enumerate(codes) if c is None]
            for r in live:
                procs[r].send_signal(signal.SIGTERM)
            deadline = time.monotonic() + grace_s
            for r in live:
                try:
                    procs[r].wait(timeout=max(0.0, deadline - time.monotonic()))
                except subprocess.TimeoutExpired:
                    procs[r].kill()
                    procs[r].wait()
            killed = live
            if timed_out and first is None:
                first = live[0] if live else None
            break
        if all(c is not None for c in codes):
            break
        time.sleep(poll_s)
    return LaunchResult([p.poll() for p in procs], first, killed)

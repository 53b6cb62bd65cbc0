"""Failure detection on the host: CPU ranks over gloo, a key-value store, child processes.
No test here faults, traps or hangs a device."""
import os
import sys
import textwrap
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from neuralfn_b200.parallel.health import Heartbeat, RankFailure, StepWatchdog, commit_if_all_ok, launch_local_ranks, vote_all_ok


def _vote_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    committed = []

    def prepare():
        if rank == 1:
            raise ValueError("shard 3 failed its checksum")  # the injected failure: a host exception on one rank
        return rank * 10

    try:
        commit_if_all_ok(prepare, committed.append, what="shard check")
        outcome = "committed"
    except RankFailure as exc:
        outcome = f"refused:{type(exc.__cause__).__name__ if exc.__cause__ else 'None'}"
    # a second round in which everybody is fine still works after the failed vote
    ok, failed = vote_all_ok(True)
    with open(os.path.join(out_dir, f"r{rank}"), "w") as f:
        f.write(f"{outcome}|{len(committed)}|{ok}|{failed}")
    dist.destroy_process_group()


def test_vote_before_commit_refuses_on_every_rank(tmp_path):
    world = 3
    mp.spawn(_vote_worker, args=(world, 29641, str(tmp_path)), nprocs=world, join=True)
    got = [open(tmp_path / f"r{r}").read() for r in range(world)]
    assert got[0] == "refused:None|0|True|0" and got[2] == "refused:None|0|True|0"
    assert got[1] == "refused:ValueError|0|True|0"  # the failing rank keeps its own exception as the cause


def _missing_peer_worker(rank, world, port, out_dir):
    """Rank 1 leaves between steps without joining the next collective; rank 0 finds out on the
    host (heartbeat) and, if it tried the collective anyway, a short group timeout ends it."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world)
    hb.beat(0)
    dist.barrier()
    if rank == 1:
        return  # exits here, between steps, nothing in flight
    time.sleep(1.2)
    hb.beat(1)
    stale = hb.stale_peers(max_age_s=1.0)
    t0 = time.time()
    try:
        dist.all_reduce(torch.ones(1))
        err = "none"
    except Exception as exc:  # the short process-group timeout, or a connection error from the dead peer
        err = type(exc).__name__
    with open(os.path.join(out_dir, "r0"), "w") as f:
        f.write(f"{stale}|{err}|{time.time() - t0:.1f}")


def test_a_rank_that_left_is_seen_before_the_next_collective(tmp_path):
    mp.spawn(_missing_peer_worker, args=(2, 29643, str(tmp_path)), nprocs=2, join=True)
    stale, err, secs = open(tmp_path / "r0").read().split("|")
    assert stale == "[1]"
    assert err != "none" and float(secs) < 30


def test_heartbeat_and_watchdog_without_processes():
    store = dist.HashStore()
    a, b = Heartbeat(store, 0, 2), Heartbeat(store, 1, 2)
    assert a.stale_peers(1.0) == [1]  # never beat
    b.beat(5)
    a.beat(9)
    assert a.stale_peers(1.0) == [] and a.lagging_peers(9, 2) == [1] and a.lagging_peers(9, 4) == []
    assert a.stale_peers(1.0, now=time.time() + 5) == [1]
    fired = []
    with StepWatchdog(0.15, on_timeout=fired.append, poll_s=0.02) as wd:
        for _ in range(5):
            time.sleep(0.05)
            wd.beat()
        assert not fired
        time.sleep(0.4)
    assert len(fired) == 1 and fired[0] > 0.15 and wd.fired
    assert vote_all_ok(True) == (True, 0) and vote_all_ok(False) == (False, 1)


def test_launcher_ends_siblings_on_first_failure(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(textwrap.dedent("""
        import os, sys, time
        rank = int(os.environ["RANK"])
        assert os.environ["MASTER_ADDR"] == "127.0.0.1" and os.environ["WORLD_SIZE"] == "3"
        if rank == 1:
            time.sleep(0.3)
            sys.exit(7)
        time.sleep(60)
    """))
    t0 = time.time()
    res = launch_local_ranks([sys.executable, str(script)], 3, grace_s=2.0)
    assert time.time() - t0 < 20
    assert not res.ok and res.first_failure == 1 and res.exit_codes[1] == 7 and sorted(res.killed) == [0, 2]
    assert all(c is not None and c != 0 for c in (res.exit_codes[0], res.exit_codes[2]))
    ok_script = tmp_path / "ok.py"
    ok_script.write_text("import sys; sys.exit(0)\n")
    assert launch_local_ranks([sys.executable, str(ok_script)], 2).ok

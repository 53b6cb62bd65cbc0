"""Copy-on-write session forks, checked on the CPU with a stand-in for the resident engine that only records what the
session layer asks of it (which slot is copied where, shortened, released)."""
import pytest
import torch

from neuralfn_b200.serving import inference as inf


class _Cfg:
    max_batch, window, vocab, max_seq = 2, 0, 1000, 512


class _RecordingEngine:
    device_bytes = launches = 0

    def __init__(self, window=0, slots=2):
        self.config = _Cfg()
        self.config.window, self.config.max_batch = window, slots
        self.len, self.log = {}, []

    def prefill(self, slot, ids, sampling=None):
        self.len[slot] = len(ids)
        return 1

    def append(self, slot, ids):
        self.len[slot] += len(ids)
        return 1

    def decode(self, tokens, sampling=None):
        for s in tokens:
            self.len[s] = self.len.get(s, 0) + 1
        return {s: 1 for s in tokens}

    def fork(self, src, dst, n):
        self.log.append(("copy", src, dst, n))
        self.len[dst] = n

    def truncate(self, slot, n):
        self.log.append(("shorten", slot, n))
        self.len[slot] = n

    def release(self, slot):
        self.log.append(("release", slot))
        self.len[slot] = 0

    def slot_length(self, slot):
        return self.len.get(slot, 0)

    def last_logits(self, slot):
        return torch.zeros(4)

    def close(self):
        pass


def test_a_fork_costs_nothing_until_it_writes():
    eng = _RecordingEngine()
    m = inf.NativeInferenceModel(eng)
    src = m.create_session()
    src.prefill(list(range(20)))
    forks = [m.fork_session(src, 20) for _ in range(3)]
    assert m.stats()["unused_forks"] == 3 and all(f.shares_cache for f in forks) and eng.log == []
    assert forks[0].token_ids == tuple(range(20)) and forks[0].cached_tokens == 19
    forks[0].current_logits()                                     # runs the pending token: needs its own rows
    assert eng.log == [("copy", 0, 1, 19)] and m.stats()["fork_copies"] == 1 and not forks[0].shares_cache
    with pytest.raises(inf.InferenceError, match="slot"):
        forks[1].current_logits()                                 # both slots are taken
    src.prefill([7, 8])                                           # appending keeps the shared rows: nothing is copied
    assert len(eng.log) == 1 and forks[1].shares_cache
    eager = None
    forks[0].close()
    eager = m.fork_session(src, 5, lazy=False)
    assert eng.log[-1] == ("copy", 0, 1, 4) and not eager.shares_cache
    m.close()


def test_truncate_reset_and_sliding_windows_detach_first():
    eng = _RecordingEngine()
    m = inf.NativeInferenceModel(eng)
    src = m.create_session()
    src.prefill(list(range(20)))
    long, short = m.fork_session(src, 20), m.fork_session(src, 6)
    src.truncate(10)                                              # rows 0 .. 8 stay: only the long fork reads past them
    assert eng.log[0] == ("copy", 0, 1, 19) and not long.shares_cache and short.shares_cache
    long.close()
    src.reset()                                                   # everything goes: the short fork is copied out first
    assert ("copy", 0, 1, 5) in eng.log and not short.shares_cache
    m.close()
    # with sliding-window caches an append may wrap over shared rows, so forks are detached before it
    eng = _RecordingEngine(window=8)
    m = inf.NativeInferenceModel(eng)
    src = m.create_session()
    src.prefill(list(range(12)))
    f = m.fork_session(src, 12)
    src.prefill([1])
    assert eng.log == [("copy", 0, 1, 11)] and not f.shares_cache
    m.close()


def test_a_closing_source_hands_its_slot_down_the_line():
    eng = _RecordingEngine(slots=1)
    m = inf.NativeInferenceModel(eng)
    src = m.create_session()
    src.prefill(list(range(20)))
    a, b, c = m.fork_session(src, 20), m.fork_session(src, 12), m.fork_session(src, 16)
    grandchild = m.fork_session(b, 9)                             # a fork of an unused fork reads the same source
    assert grandchild._origin[0] is src
    src.close()                                                   # the fork with the longest prefix takes the slot, shortened to it
    assert eng.log == [("shorten", 0, 19)] and not a.shares_cache and a.slot == 0
    assert all(x.shares_cache and x._origin[0] is a for x in (b, c, grandchild))
    a.close()
    assert eng.log[-1] == ("shorten", 0, 15) and not c.shares_cache and b._origin[0] is c
    st = m.stats()
    assert st["fork_adoptions"] == 2 and st.get("fork_copies", 0) == 0 and st["unused_forks"] == 2
    c.close()
    b.close()                                                     # the last holder releases the slot for good
    assert grandchild.slot == 0 and eng.log[-1] == ("shorten", 0, 8)
    grandchild.close()
    assert eng.log[-1] == ("release", 0) and m.stats()["sessions_open"] == 0
    m.close()

"""1F1B pipeline schedule: structure per stage and freedom from deadlock under rendezvous semantics (CPU)."""
import pytest

from neuralfn_b200.parallel.pp import one_f_one_b_schedule, simulate_schedule, stage_layer_range


@pytest.mark.parametrize("world,micro", [(2, 1), (2, 2), (2, 5), (3, 3), (4, 2), (4, 8), (8, 16), (8, 3)])
def test_schedule_completes_and_matches_the_1f1b_bubble(world, micro):
    r = simulate_schedule(world, micro)
    assert r["peak_in_flight"] == [min(micro, world - s) for s in range(world)]
    # forward = 1 slot, backward = 2: the step takes (M + W - 1) forward + backward slots
    assert r["slots"] == 3 * (micro + world - 1)


def test_stage_programs():
    s0 = one_f_one_b_schedule(0, 2, 3)
    assert [a for a in s0 if a[0] != "comm"] == [("F", 0), ("F", 1), ("B", 0), ("F", 2), ("B", 1), ("B", 2)]
    assert ("comm", [("send", 1, "act", 1), ("recv", 1, "grad", 0)]) in s0          # the paired group of the steady phase
    last = one_f_one_b_schedule(1, 2, 3)
    assert [a for a in last if a[0] != "comm"] == [("F", 0), ("B", 0), ("F", 1), ("B", 1), ("F", 2), ("B", 2)]
    assert ("comm", [("send", 0, "grad", 0), ("recv", 0, "act", 1)]) in last
    solo = one_f_one_b_schedule(0, 1, 2)
    assert solo == [("F", 0), ("B", 0), ("F", 1), ("B", 1)]
    assert [stage_layer_range(10, r, 4) for r in range(4)] == [(0, 2), (2, 5), (5, 7), (7, 10)]


def test_simulator_detects_a_broken_schedule(monkeypatch):
    import neuralfn_b200.parallel.pp as pp
    good = pp.one_f_one_b_schedule

    def broken(rank, world, micro):
        acts = good(rank, world, micro)
        if rank == 0:       # split the paired group: stage 0 now sends the next activation before it posts the receive
            out = []
            for a in acts:
                if a[0] == "comm" and len(a[1]) == 2:
                    out += [("comm", [a[1][0]]), ("comm", [a[1][1]])]
                else:
                    out.append(a)
            return out
        return acts

    monkeypatch.setattr(pp, "one_f_one_b_schedule", broken)
    with pytest.raises(RuntimeError, match="deadlock"):
        pp.simulate_schedule(2, 3)

"""Failure detection without touching a GPU: the peer-memory protocol run by threads with injected faults (dropped,
delayed, duplicated flag writes; a rank that never starts), heartbeat deadlines, the step watchdog."""
import threading
import time

import torch

from spark_engine_b200.parallel import faults as F


def _run(world, arena, seq, budget, skip=()):
    xs = [torch.full((3, 8), float(r + 1)) for r in range(world)]
    res = [None] * world

    def work(r):
        res[r] = F.fake_allreduce(arena, r, xs[r], seq, budget)
    ths = [threading.Thread(target=work, args=(r,)) for r in range(world) if r not in skip]
    for t in ths:
        t.start()
    for t in ths:
        t.join()
    return res, xs


def test_protocol_sums_in_rank_order_and_tolerates_delay_and_duplicates():
    world = 4
    arena = F.FakeArena(world, 4, 8, fault=lambda s, d, q: 0.05 if (s, d) == (1, 2) else ("dup" if s == 3 else None))
    for seq in (1, 2, 3):
        res, xs = _run(world, arena, seq, budget=1.0)
        for st, acc in res:
            assert st[0] == F.ST_OK and torch.equal(acc, sum(xs))


def test_dropped_flag_times_out_with_peer_and_sequence():
    world = 3
    arena = F.FakeArena(world, 4, 8, fault=lambda s, d, q: "drop" if (s, d, q) == (2, 0, 1) else None)
    t0 = time.monotonic()
    res, _ = _run(world, arena, 1, budget=0.2)
    assert time.monotonic() - t0 < 2.0                              # bounded: nobody hangs
    assert res[0][0] == (F.ST_TIMEOUT_PEER_FLAG, 2, 1, 0) and res[0][1] is None
    assert res[1][0][0] == F.ST_OK and res[2][0][0] == F.ST_OK      # the ranks that did get every flag complete


def test_missing_rank_is_reported_by_every_other_rank():
    world = 3
    arena = F.FakeArena(world, 4, 8)
    res, _ = _run(world, arena, 1, budget=0.2, skip=(1,))
    for r in (0, 2):
        assert res[r][0][:2] == (F.ST_TIMEOUT_PEER_FLAG, 1)


def test_heartbeat_deadline_and_watchdog():
    now = [0.0]
    hb = F.Heartbeat(deadline_s=2.0, clock=lambda: now[0])
    hb.beat()
    now[0] = 1.9
    assert hb.alive()
    now[0] = 4.0
    assert not hb.alive()
    hb.beat()
    assert hb.alive() and hb.count == 2
    fired = []
    wd = F.StepWatchdog(0.05, on_expire=lambda name, el: fired.append((name, el)))
    with wd.step("fast"):
        pass
    with wd.step("slow decode round"):
        time.sleep(0.2)
    time.sleep(0.05)
    wd.close()
    assert [f[0] for f in fired] == ["slow decode round"] and fired[0][1] >= 0.05

"""The flag protocol of the in-kernel tensor-parallel reduction, run as one CPU thread per rank
(zse_b200/parallel/protocol_model.py): unequal speeds, slot reuse, the give-up path."""
import random
import threading
import time

import numpy as np

from zse_b200.parallel.protocol_model import OneShotExchange


def _run_ranks(x, calls, rows, partials, delays, skip=None):
    """partials[call][rank][row] -> results[rank][call][row]; ``skip`` = (rank, from_call): that rank stops taking part."""
    tp = x.tp
    results = [[[None] * rows for _ in range(calls)] for _ in range(tp)]

    def rank_main(r):
        rng = random.Random(r)
        for c in range(calls):
            if skip and r == skip[0] and c >= skip[1]:
                return
            for row in range(rows):
                def pause(where, r=r, c=c):
                    d = delays(r, c, where, rng)
                    if d:
                        time.sleep(d)
                results[r][c][row] = x.reduce_row(r, c, row, partials[c][r][row], pause)

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(tp)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    assert not any(t.is_alive() for t in threads)
    return results


def test_two_slots_survive_ranks_of_very_different_speed():
    tp, rows, H, calls = 4, 3, 16, 24
    rng = np.random.default_rng(0)
    partials = rng.standard_normal((calls, tp, rows, H)).astype(np.float32)
    x = OneShotExchange(tp, rows, H, slots=2, wait_limit_s=20.0)
    # rank 0 dawdles after it has taken its flags down (it still has to read the peers' rows), rank 3 races ahead
    delays = lambda r, c, where, g: (0.004 if r == 0 and where == "flags down" else 0.0) + (g.random() * 0.001 if r != 3 else 0)
    res = _run_ranks(x, calls, rows, partials, delays)
    want = partials.astype(np.float16).astype(np.float32).sum(axis=1)          # [call][row][H]
    for r in range(tp):
        for c in range(calls):
            for row in range(rows):
                assert np.array_equal(res[r][c][row], _ordered_sum(partials[c, :, row])), (r, c, row)
    assert not x.status and not x.flags.any()
    assert np.allclose(np.stack([[res[0][c][row] for row in range(rows)] for c in range(calls)]), want, atol=1e-2)


def _ordered_sum(rows_by_rank):
    acc = np.zeros(rows_by_rank.shape[-1], dtype=np.float32)
    for q in range(rows_by_rank.shape[0]):
        acc += rows_by_rank[q].astype(np.float16).astype(np.float32)
    return acc


def test_one_slot_is_not_enough():
    """With a single slot a fast rank's next call overwrites the row a slow rank has not read yet."""
    tp, rows, H, calls = 2, 1, 8, 12
    partials = np.zeros((calls, tp, rows, H), dtype=np.float32)
    for c in range(calls):
        partials[c] = c + 1
    x = OneShotExchange(tp, rows, H, slots=1, wait_limit_s=20.0)
    delays = lambda r, c, where, g: 0.01 if (r == 0 and where == "flags down") else 0.0
    res = _run_ranks(x, calls, rows, partials, delays)
    wrong = sum(not np.array_equal(res[0][c][0], _ordered_sum(partials[c, :, 0])) for c in range(calls))
    assert wrong > 0


def test_missing_rank_makes_the_others_give_up_and_the_group_recovers():
    tp, rows, H = 3, 2, 8
    rng = np.random.default_rng(1)
    partials = rng.standard_normal((4, tp, rows, H)).astype(np.float32)
    x = OneShotExchange(tp, rows, H, wait_limit_s=0.2)
    t0 = time.monotonic()
    res = _run_ranks(x, 3, rows, partials, lambda *a: 0.0, skip=(2, 1))         # rank 2 leaves after call 0
    assert time.monotonic() - t0 < 10
    assert all(res[r][0][row] is not None for r in range(tp) for row in range(rows))
    assert res[0][1][0] is None and res[1][1][0] is None                       # bounded wait ran out, no hang
    assert x.status and {s.peer for s in x.status} == {2} and {s.rank for s in x.status} == {0, 1}
    assert min(s.call for s in x.status) == 1
    # recovery: flags cleared, all three ranks take part again
    x.reset_flags()
    x.status.clear()
    again = _run_ranks(x, 2, rows, partials[2:], lambda *a: 0.0)
    for r in range(tp):
        for c in range(2):
            for row in range(rows):
                assert np.array_equal(again[r][c][row], _ordered_sum(partials[2 + c, :, row]))
    assert not x.status


# ---- the exchange for passes of many rows: scatter in the GEMM's epilogue, reduce on the owner, gather in the prologue
def _run_scatter_gather(tp, rows, calls, slots, speeds, skip_rank=None, wait_limit_s=1.0, gather=True):
    from zse_b200.parallel.protocol_model import ScatterGatherExchange
    H = 12
    ex = ScatterGatherExchange(tp, rows, H, block=4, units=3, slots=slots, wait_limit_s=wait_limit_s)
    rng = np.random.default_rng(3)
    parts = (rng.standard_normal((calls, tp, rows, H)) * 0.5).astype(np.float16)
    seen = [[None] * calls for _ in range(tp)]
    oks = [[True] * calls for _ in range(tp)]

    def rank_fn(r):
        for c in range(calls):
            pause = (lambda where, d=speeds[r]: time.sleep(d)) if speeds[r] else None
            if r != skip_rank:
                ex.scatter(r, c, parts[c, r], pause)
            ok = ex.reduce_gather(r, c, pause)
            if gather:
                ok = ex.gather_wait(r) and ok
            oks[r][c] = ok
            seen[r][c] = ex.xg[r].copy()          # what the next GEMM of this rank reads

    threads = [threading.Thread(target=rank_fn, args=(r,)) for r in range(tp)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    return ex, parts, seen, oks


def test_scatter_gather_two_slots_with_ranks_of_very_different_speed():
    tp, rows, calls = 3, 22, 6
    ex, parts, seen, oks = _run_scatter_gather(tp, rows, calls, slots=2, speeds=[0.0, 0.004, 0.0])
    assert not ex.status and not ex.overruns and all(all(o) for o in oks)
    for c in range(calls):
        want = parts[c].astype(np.float32).sum(axis=0)
        for r in range(tp):
            assert np.allclose(seen[r][c], want, atol=2e-2), (c, r)
            assert np.array_equal(seen[r][c], seen[0][c])          # every rank gathered the same rows
    assert int(ex.arrive.sum()) == 0                               # every counter was taken down again
    assert list(ex.epoch) == [calls] * tp and np.all(ex.gflag == calls)


def test_scatter_gather_is_ordered_by_the_gather_wait():
    """What lets an owner take its counters down: nobody scatters again before having waited for every block of the
    call before.  Without that wait a fast rank's next scatter lands in counters and rows a slow owner still uses."""
    tp, rows, calls = 3, 22, 6
    bad = 0
    for attempt in range(3):
        ex, parts, seen, oks = _run_scatter_gather(tp, rows, calls, slots=1, speeds=[0.0, 0.006, 0.0],
                                                   wait_limit_s=0.3, gather=False)
        wrong = any(not np.allclose(seen[r][c], parts[c].astype(np.float32).sum(axis=0), atol=2e-2)
                    for c in range(calls) for r in range(tp))
        if wrong or ex.overruns or ex.status:
            bad += 1
    assert bad >= 1
    # with the wait, even a single slot holds (the wait is a full barrier between calls); the second slot is margin
    ex, parts, seen, oks = _run_scatter_gather(tp, rows, calls, slots=1, speeds=[0.0, 0.004, 0.0])
    assert not ex.status and not ex.overruns
    for c in range(calls):
        assert np.allclose(seen[1][c], parts[c].astype(np.float32).sum(axis=0), atol=2e-2)


def test_scatter_gather_gives_up_when_a_rank_never_delivers():
    tp, rows = 3, 10
    ex, parts, seen, oks = _run_scatter_gather(tp, rows, 1, slots=2, speeds=[0, 0, 0], skip_rank=2, wait_limit_s=0.2)
    assert ex.status and all(s.peer == 2 for s in ex.status if s.rank in (0, 1))
    assert not all(all(o) for o in oks)            # somebody reported the failure instead of hanging

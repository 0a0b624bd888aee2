"""Host model of the barrier protocol of the narrow (two-pipeline) CTA of the tiled INT4 GEMM (csrc/gemm_w4.cu, DUAL).

Roles of one CTA: a weight loader and an activation loader (rings of SW and SX stages), two MMA-issuing threads (chunks of
even / odd index), two dequantisation groups of four warps (one per pipeline).  They meet at mbarriers tested by parity;
the model runs them as coroutines under a random scheduler (copies complete in any order, each MMA thread's commits in
its own issue order) and checks, at every test, that the parity answer equals the answer by phase index, that no barrier
ever receives more arrivals than its phase expects, that a ring stage is never refilled while a reader still needs it,
and that every run ends.  No GPU is involved.
"""
import random

import pytest

from test_attention_tc_pipeline_model import Bar


def run(n_chunks, SW, SX, seed):
    rnd = random.Random(seed)
    w_full = [Bar(1) for _ in range(SW)]
    w_empty = [Bar(4) for _ in range(SW)]
    x_full = [Bar(1) for _ in range(SX)]
    x_empty = [Bar(1) for _ in range(SX)]
    a_ready = [Bar(4), Bar(4)]
    pair_done = [Bar(1), Bar(1)]
    acc_ready = Bar(2)
    pipes = [[], []]
    copies = []
    w_slot = [None] * SW                 # which chunk a weight slot holds (None: free)
    w_readers = [0] * SW
    x_slot = [None] * SX
    done = []

    def wait(bar, parity, want):
        while not bar.test(parity, want):
            yield

    def w_loader():
        ph, s = 1, 0
        for u in range(n_chunks):
            if u >= SW:
                yield from wait(w_empty[s], ph, u // SW - 1)
            assert w_readers[s] == 0, "weight slot refilled while a dequant warp still reads it"
            w_slot[s] = u
            w_readers[s] = 4
            copies.append(w_full[s])
            s += 1
            if s == SW:
                s, ph = 0, ph ^ 1
            yield

    def x_loader():
        ph, s = 1, 0
        for k in range(n_chunks):
            if k >= SX:
                yield from wait(x_empty[s], ph, k // SX - 1)
            assert x_slot[s] is None, "activation stage refilled before its MMAs were known complete"
            x_slot[s] = k
            copies.append(x_full[s])
            s += 1
            if s == SX:
                s, ph = 0, ph ^ 1
            yield

    def mma(p):
        aph = 0
        for u in range(p, n_chunks, 2):
            sx = u % SX
            yield from wait(x_full[sx], (u // SX) & 1, u // SX)
            assert x_slot[sx] == u
            yield from wait(a_ready[p], aph, (u - p) // 2)
            if u >= 2:
                # slot p was refilled only after the MMAs of chunk u-2 completed: its activation stage is free
                assert x_slot[(u - 2) % SX] == u - 2
                x_slot[(u - 2) % SX] = None
                x_empty[(u - 2) % SX].arrive()
            pipes[p].append(pair_done[p])
            aph ^= 1
            yield
        pipes[p].append(acc_ready)

    def dequant(p, q):
        sw, wph, dph = p % SW, 0, 0
        for u in range(p, n_chunks, 2):
            yield from wait(w_full[sw], wph, u // SW)
            assert w_slot[sw] == u, (w_slot[sw], u)
            yield                                              # chunk -> registers
            w_readers[sw] -= 1
            w_empty[sw].arrive()
            if u >= 2:
                yield from wait(pair_done[p], dph, (u - p) // 2 - 1)
                dph ^= 1
            yield                                              # tcgen05.st
            a_ready[p].arrive()
            sw += 2
            if sw >= SW:
                sw, wph = sw - SW, wph ^ 1
        yield from wait(acc_ready, 0, 0)
        done.append((p, q))

    agents = [w_loader(), x_loader(), mma(0), mma(1)] + [dequant(p, q) for p in range(2) for q in range(4)]
    live = list(range(len(agents)))
    for _ in range(400000):
        if not live and not copies and not pipes[0] and not pipes[1]:
            break
        c = rnd.random()
        if c < 0.15 and (pipes[0] or pipes[1]):
            p = rnd.choice([i for i in range(2) if pipes[i]])
            pipes[p].pop(0).arrive()
        elif c < 0.3 and copies:
            copies.pop(rnd.randrange(len(copies))).arrive()
        elif live:
            i = rnd.choice(live)
            try:
                next(agents[i])
            except StopIteration:
                live.remove(i)
    else:
        raise AssertionError("the roles did not finish: a wait never came true")
    assert len(done) == 8 and acc_ready.phase == 1


@pytest.mark.parametrize("SW", [5, 6])
@pytest.mark.parametrize("n_chunks", [1, 2, 3, 4, 5, 6, 7, 12, 16, 23])
def test_narrow_cta_protocol(n_chunks, SW):
    for seed in range(25):
        run(n_chunks, SW, 4, seed)

"""Host model of the barrier protocol inside one CTA of the persistent decode GEMM (csrc/gemm_w4_dec.cu, stream plan).

A CTA walks `n_steps` K steps that may span several tile pairs (`ks` steps per pair, starting at `k_first` inside the
first one).  Two pipelines (the two tiles of a pair) x two step parities give four MMA-issuing lanes and four
dequantisation groups of four warps; one thread loads activations (a ring of SX stages that BOTH pipelines read) and
weights (a ring of SW chunks per pipeline); four epilogue warps take the accumulators of a pair when its last step is
done.  Pipeline 1 may run out of chunks at a pair boundary (a last pair of one tile): its lanes then only hand the
activation stages back.

The model runs every role as a coroutine under a random scheduler - copies complete in any order, each lane's
tcgen05.commit events in that lane's issue order - and checks at every barrier test that the parity answer equals the
answer by phase index, that no barrier gets more arrivals than its phase expects, that ring slots and TMEM slots are
never refilled under a reader, that accumulators are never overwritten before the epilogue has read them, and that
every run ends.  No GPU is involved.
"""
import random

import pytest

from test_attention_tc_pipeline_model import Bar

SX, SW = 6, 5


def run(n_steps, ks, k_first, n_real1, seed):
    rnd = random.Random(seed)
    w_full = [[Bar(1) for _ in range(SW)] for _ in range(2)]
    w_empty = [[Bar(4) for _ in range(SW)] for _ in range(2)]
    x_full = [Bar(1) for _ in range(SX)]
    x_empty = [Bar(2) for _ in range(SX)]
    a_ready = [[Bar(4), Bar(4)], [Bar(4), Bar(4)]]
    slot_free = [[Bar(1), Bar(1)], [Bar(1), Bar(1)]]
    acc_full = [[Bar(1), Bar(1)], [Bar(1), Bar(1)]]
    acc_empty = [[Bar(4), Bar(4)], [Bar(4), Bar(4)]]
    pipes = {(p, sub): [] for p in range(2) for sub in range(2)}      # commits of one lane complete in order
    copies = []
    # data hazards
    w_slot = [[None] * SW for _ in range(2)]          # chunk held by a weight slot
    w_readers = [[0] * SW for _ in range(2)]
    x_stage = [None] * SX                             # step held by an activation stage
    x_readers = [0] * SX
    tmem_slot = {(p, sub): None for p in range(2) for sub in range(2)}   # chunk whose fp16 image sits in the lane's slot
    acc_state = {(p, sub): "free" for p in range(2) for sub in range(2)}  # free | busy (MMAs accumulate) | full
    acc_readers = {(p, sub): 0 for p in range(2) for sub in range(2)}     # epilogue warps that still have to read it
    done = []

    def wait(bar, parity, want):
        while not bar.test(parity, want):
            yield

    def steps_of(p):
        return n_steps if p == 0 else n_real1

    def load_w(p, slot, chunk):
        assert w_readers[p][slot] == 0, "weight slot refilled under a dequant warp"
        w_slot[p][slot], w_readers[p][slot] = chunk, 4
        copies.append(w_full[p][slot])

    def producer():
        for s in range(min(n_steps, SW)):             # the first ring-full, before anything else
            load_w(0, s, s)
            if s < n_real1:
                load_w(1, s, s)
        st, wslot, xph, wph = 0, 0, 1, 0
        for s in range(n_steps):
            if s >= SX:
                yield from wait(x_empty[st], xph, s // SX - 1)
            assert x_readers[st] == 0, "activation stage refilled under a reader"
            x_stage[st], x_readers[st] = s, 2
            copies.append(x_full[st])
            st += 1
            if st == SX:
                st, xph = 0, xph ^ 1
            sw = s + SW
            if sw < n_steps:
                yield from wait(w_empty[0][wslot], wph, sw // SW - 1)
                load_w(0, wslot, sw)
                if sw < n_real1:
                    yield from wait(w_empty[1][wslot], wph, sw // SW - 1)
                    load_w(1, wslot, sw)
                wslot += 1
                if wslot == SW:
                    wslot, wph = 0, wph ^ 1
            yield

    def mma(p, sub):
        my_steps = steps_of(p)
        k, item, cur_item, uses = k_first + sub, 0, -1, 0
        while k >= ks:
            k, item = k - ks, item + 1
        st, xph, aph, s = sub % SX, 0, 0, sub
        while s < my_steps:
            yield from wait(x_full[st], xph, s // SX)
            assert x_stage[st] == s
            if item != cur_item:
                if uses > 0:
                    yield from wait(acc_empty[p][sub], (uses - 1) & 1, uses - 1)
                    assert acc_state[(p, sub)] == "free", "accumulator reused before the epilogue read it"
                cur_item = item
                acc_state[(p, sub)] = "busy"
            yield from wait(a_ready[p][sub], aph, (s - sub) // 2)
            aph ^= 1
            assert tmem_slot[(p, sub)] == s
            last_of_pair = k + 2 >= ks or s + 2 >= n_steps
            pipes[(p, sub)].append(("slot_free", s, st))
            if last_of_pair:
                pipes[(p, sub)].append(("acc_full", None, None))
                uses += 1
            k += 2
            while k >= ks:
                k, item = k - ks, item + 1
            st += 2
            if st >= SX:
                st, xph = st - SX, xph ^ 1
            s += 2
            yield
        while s < n_steps:                            # pipeline 1 ran out: hand the stages back
            yield from wait(x_full[st], xph, s // SX)
            assert x_stage[st] == s
            x_readers[st] -= 1
            x_empty[st].arrive()
            st += 2
            if st >= SX:
                st, xph = st - SX, xph ^ 1
            s += 2
            yield

    def dequant(p, sub, q):
        n_chunks = steps_of(p)
        slot, xst, wph, sph, last = sub % SW, sub % SX, 0, 0, -1
        c = sub
        while c < n_chunks:
            yield from wait(w_full[p][slot], wph, c // SW)
            assert w_slot[p][slot] == c
            yield                                     # chunk -> registers
            w_readers[p][slot] -= 1
            w_empty[p][slot].arrive()
            if c >= 2:
                yield from wait(slot_free[p][sub], sph, (c - sub) // 2 - 1)
                sph ^= 1
                if q == 0:                            # the MMAs of chunk c-2 are complete: one reader less
                    assert x_stage[xst] == c - 2
                    x_readers[xst] -= 1
                    x_empty[xst].arrive()
                xst += 2
                if xst >= SX:
                    xst -= SX
            if q == 0:
                tmem_slot[(p, sub)] = c               # tcgen05.st of the new image (all four warps write their rows)
            yield
            a_ready[p][sub].arrive()
            last = c
            slot += 2
            if slot >= SW:
                slot, wph = slot - SW, wph ^ 1
            c += 2
        if last >= 0:
            yield from wait(slot_free[p][sub], sph, (last - sub) // 2)
            if q == 0:
                assert x_stage[xst] == last
                x_readers[xst] -= 1
                x_empty[xst].arrive()
        done.append(("dq", p, sub, q))

    def epilogue(w):
        s, ka = 0, k_first
        use = [0, 0]
        while s < n_steps:
            length = min(ks - ka, n_steps - s)
            ntp = 2 if s < n_real1 else 1
            last_item = s + length == n_steps
            lane = [length >= 2 or (s & 1) == 0, length >= 2 or (s & 1) == 1]
            for r in range(ntp):
                for sub in range(2):
                    if lane[sub]:
                        yield from wait(acc_full[r][sub], use[sub] & 1, use[sub])
                        assert acc_state[(r, sub)] == "full"
            yield                                     # accumulators -> registers / workspace
            if not last_item:
                for r in range(ntp):
                    for sub in range(2):
                        if lane[sub]:
                            acc_readers[(r, sub)] -= 1         # this warp has its rows out of TMEM
                            if acc_readers[(r, sub)] == 0:
                                acc_state[(r, sub)] = "free"
                            acc_empty[r][sub].arrive()
            use[0] += lane[0]
            use[1] += lane[1]
            s += length
            ka = 0
        done.append(("epi", w))

    agents = ([producer()] + [mma(p, sub) for p in range(2) for sub in range(2)]
              + [dequant(p, sub, q) for p in range(2) for sub in range(2) for q in range(4)]
              + [epilogue(w) for w in range(4)])
    live = list(range(len(agents)))
    for _ in range(2000000):
        busy_pipes = [k for k, v in pipes.items() if v]
        if not live and not copies and not busy_pipes:
            break
        c = rnd.random()
        if c < 0.15 and busy_pipes:
            key = rnd.choice(busy_pipes)
            what, s, st = pipes[key].pop(0)
            if what == "slot_free":
                tmem_slot[key] = ("consumed", s)
                slot_free[key[0]][key[1]].arrive()
            else:
                acc_state[key], acc_readers[key] = "full", 4
                acc_full[key[0]][key[1]].arrive()
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
    assert len(done) == 16 + 4


def boundaries(n_steps, ks, k_first):
    """Step counts at which pipeline 1 may stop: pair boundaries inside the range, or never."""
    return [s for s in range(0, n_steps) if (k_first + s) % ks == 0] + [n_steps]


@pytest.mark.parametrize("ks", [2, 3, 5, 8, 40])
def test_decode_gemm_cta_protocol(ks):
    rnd = random.Random(ks)
    for trial in range(60):
        n_steps = rnd.randint(1, 3 * ks + 7)
        k_first = rnd.randrange(ks)
        n_real1 = rnd.choice(boundaries(n_steps, ks, k_first))
        run(n_steps, ks, k_first, n_real1, seed=trial)


def test_the_shapes_of_the_14b_layer():
    """K = 5120 (40 steps per pair) and K = 13824 (108): ranges as the chunk scheduler cuts them for 148 CTAs."""
    for ks, total_pairs in ((40, 108), (40, 28), (108, 20)):
        total = ks * total_pairs
        for cta in (0, 1, 73, 147):
            g0, g1 = total * cta // 148, total * (cta + 1) // 148
            if g1 > g0:
                run(g1 - g0, ks, g0 % ks, g1 - g0, seed=cta)

"""Host model of the barrier protocol of the tcgen05 prefill attention kernel (csrc/attention_tc.cu).

The kernel's roles meet at mbarriers that they test by PARITY: a test for parity p answers "the phase with parity p is
complete", which is only the question the role means to ask while the barrier is at most one phase away from the one it
waits for.  Two barriers have several kinds of waiters since one `tcgen05.commit` per event is used: `s_full`
(Q K^T of tile t complete) wakes the softmax warps AND tells the loader that the K slot is free; `v_empty` (P V of tile t
complete) frees the V slot for the loader, lets the MMA thread overwrite the probabilities, and for the last tile tells
the softmax warps that O is complete.  This model runs the roles as coroutines under a random scheduler, with the tensor
pipe completing commits in order after arbitrary delays, and checks at every single test that the parity answer equals the
answer by phase index - and that every run ends.  No GPU is involved.
"""
import random

import pytest


class Bar:
    def __init__(self, count):
        self.count, self.pending, self.phase = count, count, 0      # phase = number of completed phases

    def arrive(self):
        self.pending -= 1
        assert self.pending >= 0, "more arrivals than the barrier expects in one phase"
        if self.pending == 0:
            self.phase += 1
            self.pending = self.count

    def test(self, parity, want_phase):
        """try_wait.parity: true iff the phase of that parity is complete.  `want_phase` is the phase the caller means;
        the two answers must agree, which holds only while the barrier is at `want_phase` or one past it."""
        by_parity = (self.phase & 1) != parity
        by_index = self.phase > want_phase
        assert by_parity == by_index, (f"parity test answers {by_parity} for phase {want_phase} "
                                       f"while the barrier has completed {self.phase} phases")
        return by_parity


def run(n_tiles, seed, softmax_warps=4):
    rnd = random.Random(seed)
    bars = {n: Bar(1) for n in ("q_full", "k_full", "v_full", "v_empty", "s_full")}
    bars["p_full"] = Bar(softmax_warps)
    pipe = []                      # tensor pipe: commits complete in issue order
    copies = []                    # TMA: loads complete in any order
    log = []

    def wait(name, parity, want):
        while not bars[name].test(parity, want):
            yield

    def loader():
        copies.append("q_full")
        ph = 1
        for t in range(n_tiles):
            if t > 0:
                yield from wait("s_full", ph, t - 1)             # K slot free: Q K^T of the previous tile complete
            copies.append("k_full")
            if t > 0:
                yield from wait("v_empty", ph, t - 1)            # (tile 0: parity 1 on a fresh barrier passes at once)
            else:
                assert (bars["v_empty"].phase & 1) != ph
            copies.append("v_full")
            ph ^= 1
            yield

    def mma():
        yield from wait("q_full", 0, 0)
        ph = 0
        for t in range(n_tiles):
            yield from wait("k_full", ph, t)
            if t > 0:
                yield from wait("v_empty", ph ^ 1, t - 1)        # P of the previous tile has been read
            pipe.append("s_full")
            yield from wait("v_full", ph, t)
            yield from wait("p_full", ph, t)
            pipe.append("v_empty")
            log.append(("pv", t))
            ph ^= 1
            yield

    def softmax(w):
        ph = 0
        for t in range(n_tiles):
            yield from wait("s_full", ph, t)
            yield                                                # the pass over S
            bars["p_full"].arrive()
            ph ^= 1
            yield
        yield from wait("v_empty", (n_tiles - 1) & 1, n_tiles - 1)   # O complete
        log.append(("epilogue", w))

    agents = [loader(), mma()] + [softmax(w) for w in range(softmax_warps)]
    live = list(range(len(agents)))
    for _ in range(200000):
        if not live and not pipe and not copies:
            break
        choice = rnd.random()
        if pipe and choice < 0.2:
            bars[pipe.pop(0)].arrive()                           # in order
        elif copies and choice < 0.4:
            bars[copies.pop(rnd.randrange(len(copies)))].arrive()
        elif live:
            i = rnd.choice(live)
            try:
                next(agents[i])
            except StopIteration:
                live.remove(i)
    else:
        raise AssertionError("the roles did not finish: a wait never came true")
    assert [e for e in log if e[0] == "pv"] == [("pv", t) for t in range(n_tiles)]
    assert sorted(e[1] for e in log if e[0] == "epilogue") == list(range(softmax_warps))
    assert bars["s_full"].phase == n_tiles and bars["v_empty"].phase == n_tiles and bars["p_full"].phase == n_tiles


@pytest.mark.parametrize("n_tiles", [1, 2, 3, 4, 7, 16])
def test_parity_waits_ask_the_question_they_mean(n_tiles):
    for seed in range(40):
        run(n_tiles, seed)


def test_a_second_waiter_two_phases_behind_would_be_caught():
    """The check itself: a role that tested `s_full` for tile t-2 (not t-1) is the mistake the model exists to catch."""
    b = Bar(1)
    b.arrive()
    b.arrive()                                                   # two phases complete
    with pytest.raises(AssertionError):
        b.test(0, 0)                                             # parity 0 "not complete", index says complete

"""Unit tests of the continuous-batching host objects one by one - request lifecycle and metrics, the priority queues,
the predictive block budget (the shape of the reference's tests/test_zstreamer.py).  The scheduler's policies as a whole
are in tests/test_sched.py."""
import math
import time

import pytest

from zse_b200.sched import request as request_mod
from zse_b200.sched.memory_budget import MemoryBudget, MemoryReservation
from zse_b200.sched.queue import RequestQueue
from zse_b200.sched.request import (FinishReason, GenerationParams, InferenceRequest, RequestOutput, RequestState,
                                    decision_now, set_decision_clock)


def req(rid, n_prompt=8, max_tokens=16, priority=0, deadline_ms=None, **kw):
    return InferenceRequest(rid, list(range(1, n_prompt + 1)), GenerationParams(max_tokens=max_tokens, **kw),
                            priority=priority, deadline_ms=deadline_ms)


@pytest.fixture()
def clock():
    """A decision clock the test moves by hand."""
    t = [1000.0]
    set_decision_clock(lambda: t[0])
    yield t
    set_decision_clock(None)


# ---- generation parameters --------------------------------------------------------------------------------------
def test_generation_defaults_and_greedy():
    p = GenerationParams()
    assert (p.max_tokens, p.temperature, p.top_p, p.top_k, p.repetition_penalty) == (128, 1.0, 0.9, 50, 1.0)
    assert p.stop_tokens is None and p.seed is None and p.timeout_ms is None and p.lora_id is None
    assert not p.greedy
    assert GenerationParams(temperature=0.0).greedy and GenerationParams(top_k=1).greedy
    assert GenerationParams(temperature=-1.0).greedy and not GenerationParams(temperature=0.01).greedy


# ---- request lifecycle ------------------------------------------------------------------------------------------
def test_a_new_request_is_waiting_and_counts_its_tokens():
    r = req("a", n_prompt=5, lora_id="ad")
    assert r.state == RequestState.WAITING and not r.is_active and not r.is_finished
    assert (r.prompt_len, r.num_generated, r.total_tokens, r.remaining_prefill) == (5, 0, 5, 5)
    assert r.lora_id == "ad" and r.seq_id is None and r.finish_reason is None and r.num_preemptions == 0
    assert r.prefill_tokens == [1, 2, 3, 4, 5]
    assert r.urgency == math.inf                                                   # no deadline: never urgent


def test_state_transitions():
    r = req("a")
    r.mark_prefilling()
    assert r.state == RequestState.PREFILLING and r.is_active
    r.mark_decoding()
    assert r.state == RequestState.DECODING and r.is_active
    r.pre_extended = True
    r.mark_preempted()
    assert r.state == RequestState.PREEMPTED and not r.is_active and not r.is_finished
    assert r.num_preemptions == 1 and r.pre_extended is False                      # its cache slots are gone
    r.mark_finished(FinishReason.STOP)
    assert r.is_finished and r.finish_reason == FinishReason.STOP and r.finish_time is not None
    c = req("b")
    c.mark_cancelled()
    assert c.state == RequestState.CANCELLED and c.is_finished and c.finish_reason == FinishReason.CANCELLED
    assert {x.value for x in FinishReason} == {"length", "stop", "cancelled", "error", "preempted"}


def test_tokens_are_counted_streamed_and_timed():
    seen = []
    r = req("a", max_tokens=3)
    r.on_token = seen.append
    assert r.first_token_time is None
    r.add_token(7)
    t_first = r.first_token_time
    r.add_token(7)
    r.add_token(9)
    assert seen == [7, 7, 9] and r.output_tokens == [7, 7, 9] and r.past_tokens == {7: 2, 9: 1}
    assert r.first_token_time == t_first and r.num_generated == 3 and r.total_tokens == r.prompt_len + 3
    assert r.should_stop() == FinishReason.LENGTH


def test_a_streaming_callback_that_raises_is_dropped_not_propagated():
    r = req("a")
    calls = []

    def bad(tok):
        calls.append(tok)
        raise RuntimeError("client went away")

    r.on_token = bad
    r.add_token(1)
    r.add_token(2)
    assert calls == [1] and r.on_token is None and "client went away" in r.callback_error
    assert r.output_tokens == [1, 2]                                               # generation itself is unaffected


def test_stop_conditions():
    r = req("a", max_tokens=4, stop_tokens=[99])
    assert r.should_stop() is None
    r.add_token(5)
    assert r.should_stop() is None
    r.add_token(99)
    assert r.should_stop() == FinishReason.STOP
    full = req("b", max_tokens=2, stop_tokens=[99])
    full.add_token(1)
    full.add_token(99)                                                             # stop token AS the last allowed one
    assert full.should_stop() == FinishReason.STOP
    none = req("c", max_tokens=2)
    none.add_token(99)
    assert none.should_stop() is None                                              # no stop list: 99 is just a token


def test_timeout_follows_the_decision_clock(clock):
    r = req("a", timeout_ms=500.0)
    assert r.arrival_time == 1000.0 and r.wait_time_ms == 0.0 and r.should_stop() is None
    clock[0] += 0.4
    assert r.wait_time_ms == pytest.approx(400.0) and r.should_stop() is None
    clock[0] += 0.2
    assert r.should_stop() == FinishReason.LENGTH
    assert decision_now() == clock[0]


def test_urgency_counts_down_to_the_deadline(clock):
    r = req("a", deadline_ms=200.0)
    assert r.urgency == pytest.approx(200.0)
    clock[0] += 0.15
    assert r.urgency == pytest.approx(50.0)
    clock[0] += 0.1
    assert r.urgency == pytest.approx(-50.0)                                       # overdue: most urgent of all


def test_without_an_installed_clock_decisions_use_the_monotonic_clock():
    set_decision_clock(None)
    a = time.monotonic()
    b = decision_now()
    c = time.monotonic()
    assert a <= b <= c and request_mod._decision_clock is None


def test_reprefill_after_preemption_covers_all_but_the_last_generated_token():
    r = req("a", n_prompt=4)
    for t in (10, 11, 12):
        r.add_token(t)
    assert r.prefill_tokens == [1, 2, 3, 4, 10, 11]                                # 12 is the next decode input
    r.prefill_offset = 0
    assert r.remaining_prefill == 6
    r.prefill_offset = 4
    assert r.remaining_prefill == 2


def test_request_output_metrics():
    r = req("a", n_prompt=3)
    r.arrival_time = time.monotonic() - 1.0
    r.first_token_time = r.arrival_time + 0.2
    r.output_tokens = [1, 2, 3, 4, 5]
    r.finish_reason = FinishReason.LENGTH
    r.finish_time = r.arrival_time + 1.0
    out = RequestOutput.from_request(r)
    assert out.request_id == "a" and out.prompt_tokens == [1, 2, 3] and out.output_tokens == [1, 2, 3, 4, 5]
    assert out.finish_reason == FinishReason.LENGTH and out.error is None
    assert out.ttft_ms == pytest.approx(200.0) and out.total_time_ms == pytest.approx(1000.0)
    assert out.tpot_ms == pytest.approx(800.0 / 4) and out.tokens_per_sec == pytest.approx(5.0)
    out.output_tokens.append(6)
    assert r.output_tokens == [1, 2, 3, 4, 5]                                      # a copy, not the live list


def test_request_output_of_a_request_that_never_produced_a_token():
    r = req("a")
    r.error = "boom"
    r.arrival_time = time.monotonic() - 0.5
    out = RequestOutput.from_request(r)
    assert out.finish_reason == FinishReason.ERROR and out.error == "boom" and out.output_tokens == []
    assert out.ttft_ms == pytest.approx(out.total_time_ms) and out.tpot_ms == 0.0
    one = req("b")
    one.add_token(1)
    one.mark_finished(FinishReason.STOP)
    assert RequestOutput.from_request(one).tpot_ms == 0.0                          # one token: nothing to average


# ---- queue ------------------------------------------------------------------------------------------------------
def test_queue_is_fifo_among_equals(clock):
    q = RequestQueue()
    for i in range(5):
        clock[0] += 0.001
        assert q.add(req(f"r{i}"))
    assert q.num_waiting == 5 == q.num_total and not q.is_empty
    assert [q.pop_next().request_id for _ in range(5)] == [f"r{i}" for i in range(5)]
    assert q.pop_next() is None and q.is_empty


def test_queue_priority_then_deadline(clock):
    q = RequestQueue()
    q.add(req("low", priority=0))
    clock[0] += 0.001
    q.add(req("high", priority=5))
    clock[0] += 0.001
    q.add(req("urgent", priority=0, deadline_ms=10.0))
    clock[0] += 0.001
    q.add(req("relaxed", priority=9, deadline_ms=5000.0))
    # a deadline beats any priority; among requests with a deadline the nearer one; then priority; then arrival
    assert [q.pop_next().request_id for _ in range(4)] == ["urgent", "relaxed", "high", "low"]


def test_queue_capacity_force_and_statistics():
    q = RequestQueue(max_queue_size=2)
    assert q.add(req("a")) and q.add(req("b"))
    assert q.add(req("c")) is False
    assert q.add(req("d"), force=True)                                             # internal re-queues may exceed it
    s = q.stats()
    assert (s["waiting"], s["max_queue_size"], s["total_added"], s["total_rejected"]) == (3, 2, 3, 1)
    unlimited = RequestQueue(max_queue_size=0)
    for i in range(300):
        assert unlimited.add(req(f"u{i}"))
    assert unlimited.num_waiting == 300


def test_cancel_is_lazy_and_counted():
    q = RequestQueue()
    a, b = req("a"), req("b")
    q.add(a)
    q.add(b)
    assert q.cancel("a") is a and a.state == RequestState.CANCELLED and a.finish_reason == FinishReason.CANCELLED
    assert q.cancel("a") is None and q.cancel("zzz") is None
    assert q.num_waiting == 1 and q.get("a") is None and q.get("b") is b
    assert q.pop_next() is b and q.pop_next() is None                              # the cancelled entry is skipped
    assert q.stats()["total_cancelled"] == 1


def test_preempted_requests_resume_first_unless_outranked(clock):
    q = RequestQueue()
    new = req("new")
    q.add(new)
    clock[0] += 0.001
    pre = req("pre")
    pre.mark_preempted()
    q.add_preempted(pre)
    assert q.num_preempted == 1 and q.stats()["preempted_waiting"] == 1
    assert q.pop_next() is pre and q.pop_next() is new
    # the request a preemption made room for keeps that room
    vip = req("vip", priority=10)
    q.add(vip)
    pre2 = req("pre2", priority=0)
    pre2.mark_preempted()
    q.add_preempted(pre2)
    assert q.pop_next() is vip and q.pop_next() is pre2


def test_prefill_batch_respects_both_limits_and_returns_the_rest(clock):
    q = RequestQueue()
    for i, n in enumerate((100, 200, 300, 50)):
        clock[0] += 0.001
        q.add(req(f"r{i}", n_prompt=n))
    batch = q.pop_prefill_batch(max_requests=8, max_tokens=350)
    assert [r.request_id for r in batch] == ["r0", "r1"]                           # r2 would pass 350
    assert q.num_waiting == 2
    assert [r.request_id for r in q.pop_prefill_batch(1, 10 ** 6)] == ["r2"]       # pushed back in its old place
    big = q.pop_prefill_batch(4, 10)
    assert [r.request_id for r in big] == ["r3"]                                   # the first request always goes
    assert q.pop_prefill_batch(4, 100) == []


def test_push_back_and_remove_finished():
    q = RequestQueue()
    a = req("a")
    q.add(a)
    got = q.pop_next()
    assert got is a and q.is_empty
    q.push_back(a)
    assert q.num_waiting == 1 and q.get("a") is a and q.peek_waiting() == [a]
    q.remove_finished("a")
    assert q.is_empty and q.pop_next() is None
    q.remove_finished("never-there")


def test_a_request_that_finished_while_queued_is_skipped():
    q = RequestQueue()
    a, b = req("a"), req("b")
    q.add(a)
    q.add(b)
    a.mark_finished(FinishReason.ERROR)
    assert q.pop_next() is b


# ---- memory budget ----------------------------------------------------------------------------------------------
def test_budget_estimate_is_prompt_plus_headroom_plus_one():
    b = MemoryBudget(total_blocks=100, block_size=16, headroom_ratio=0.5)
    r = req("a", n_prompt=40, max_tokens=64)                                       # 3 prompt blocks; 32 tokens -> 2 + 1
    assert b.can_admit(r) and b.committed_blocks == 0 and b.available_blocks == 98
    b.reserve(r)
    assert b.committed_blocks == 6 and b.available_blocks == 92 and b.utilization == pytest.approx(0.06)
    b.reserve(r)                                                                   # reserving twice changes nothing
    assert b.committed_blocks == 6 and b.stats()["num_requests"] == 1
    assert b.can_admit(r)                                                          # already inside
    b.release("a")
    b.release("a")
    assert b.committed_blocks == 0
    assert MemoryReservation(3, 2, 5).total == 8 and MemoryReservation(3, 2).total == 5


def test_headroom_turns_into_real_usage_as_tokens_arrive():
    b = MemoryBudget(100, 16, headroom_ratio=0.25)
    r = req("a", n_prompt=16, max_tokens=128)                                      # 1 + (32 tokens -> 2) + 1 = 4
    b.reserve(r)
    assert b.committed_blocks == 4
    b.update_decode_progress("a", 10)                                              # 1 block + 1 < head-room: unchanged
    assert b.committed_blocks == 4
    b.update_decode_progress("a", 100)                                             # 7 + 1 = 8 decode blocks
    assert b.committed_blocks == 1 + 8
    b.update_decode_progress("unknown", 5)                                         # silently ignored


def test_admission_stops_at_the_reserve():
    b = MemoryBudget(total_blocks=12, block_size=16, headroom_ratio=0.5, reserve_blocks=2)
    r1, r2, r3 = (req(n, n_prompt=16, max_tokens=64) for n in "abc")               # 1 + 2 + 1 = 4 blocks each
    assert b.can_admit_n([r1, r2, r3]) == 2                                        # 10 usable blocks
    b.reserve(r1)
    b.reserve(r2)
    assert b.available_blocks == 2 and not b.can_admit(r3)
    assert b.can_admit_n([r1, r3]) == 1                                            # r1 costs nothing more
    b.release("a")
    assert b.can_admit(r3)


def test_fits_at_all_is_about_the_empty_cache():
    b = MemoryBudget(total_blocks=10, block_size=16, reserve_blocks=2)
    assert b.fits_at_all(req("ok", n_prompt=64, max_tokens=64))                    # 8 blocks
    assert not b.fits_at_all(req("no", n_prompt=64, max_tokens=65))                # 9 blocks > 8 usable
    b.reserve(req("x", n_prompt=100, max_tokens=10))
    assert b.fits_at_all(req("ok2", n_prompt=64, max_tokens=64))                   # what is committed does not matter


def test_preemption_candidates_largest_first():
    b = MemoryBudget(100, 16, headroom_ratio=0.5)
    b.reserve(req("small", n_prompt=16, max_tokens=16))                            # 1 + 1 + 1 = 3
    b.reserve(req("big", n_prompt=160, max_tokens=64))                             # 10 + 2 + 1 = 13
    b.reserve(req("mid", n_prompt=64, max_tokens=32))                              # 4 + 1 + 1 = 6
    assert b.preemption_candidates(5) == ["big"]
    assert b.preemption_candidates(14) == ["big", "mid"]
    assert b.preemption_candidates(1000) == ["big", "mid", "small"]
    assert b.preemption_candidates(0) == []


def test_resize_and_statistics():
    b = MemoryBudget(50, 32, headroom_ratio=0.5)
    b.reserve(req("a", n_prompt=32, max_tokens=64))                                # 1 + 1 + 1
    s = b.stats()
    assert s == {"total_blocks": 50, "committed_blocks": 3, "available_blocks": 45, "utilization": 3 / 50,
                 "num_requests": 1, "block_size": 32, "headroom_ratio": 0.5}
    b.resize(4)
    assert b.available_blocks == 0 and b.stats()["total_blocks"] == 4              # never negative
    assert MemoryBudget(0, 16).utilization == 1.0
    # a resumed request is estimated from what it already generated
    r = req("r", n_prompt=16, max_tokens=64)
    for t in range(40):
        r.output_tokens.append(t)
    big = MemoryBudget(100, 16, headroom_ratio=0.5)
    big.reserve(r)
    assert big.committed_blocks == 4 + 1 + 1                                       # 56 tokens; 24 left -> 12 -> 1 + 1

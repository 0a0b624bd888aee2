"""Request queue, memory budget and iteration-level scheduler (zse-engine/tests/test_zstreamer.py covers the same
classes of the reference: queue ordering, back-pressure, token/sequence budgets, preemption)."""
import os

import pytest

from zse_b200.sched.memory_budget import MemoryBudget
from zse_b200.sched.queue import RequestQueue
from zse_b200.sched.request import FinishReason, GenerationParams, InferenceRequest, RequestOutput, RequestState
from zse_b200.sched.scheduler import Scheduler, SchedulerConfig, StepType


def _req(rid, n_prompt=8, max_tokens=4, priority=0, deadline_ms=None, **kw):
    return InferenceRequest(rid, list(range(n_prompt)), GenerationParams(max_tokens=max_tokens, **kw),
                            priority=priority, deadline_ms=deadline_ms)


# ---- request ---------------------------------------------------------------------------------------------------
def test_request_stop_conditions_and_callbacks():
    seen = []
    r = _req("a", max_tokens=3, stop_tokens=[7])
    r.on_token = seen.append
    r.add_token(5)
    assert r.should_stop() is None and r.first_token_time is not None
    r.add_token(7)
    assert r.should_stop() == FinishReason.STOP
    r2 = _req("b", max_tokens=2)
    r2.add_token(1); r2.add_token(1)
    assert r2.should_stop() == FinishReason.LENGTH and r2.past_tokens == {1: 2}
    assert seen == [5, 7]
    r2.mark_finished(FinishReason.LENGTH)
    out = RequestOutput.from_request(r2)
    assert out.output_tokens == [1, 1] and out.finish_reason == FinishReason.LENGTH


def test_request_reprefill_tokens_after_preemption():
    r = _req("a", n_prompt=4)
    r.add_token(10); r.add_token(11)
    # the last generated token is the next decode input, so it is not part of the re-prefill
    assert r.prefill_tokens == [0, 1, 2, 3, 10]
    r.pre_extended = True
    r.mark_preempted()
    assert r.state == RequestState.PREEMPTED and r.num_preemptions == 1 and not r.pre_extended


# ---- queue -----------------------------------------------------------------------------------------------------
def test_queue_orders_by_deadline_then_priority_then_arrival():
    q = RequestQueue(10)
    a, b, c, d = _req("a"), _req("b", priority=5), _req("c", deadline_ms=50.0), _req("d")
    for r in (a, b, c, d):
        assert q.add(r)
    assert [q.pop_next().request_id for _ in range(4)] == ["c", "b", "a", "d"]
    assert q.pop_next() is None and q.is_empty


def test_queue_back_pressure_cancel_and_preempted_first():
    q = RequestQueue(2)
    assert q.add(_req("a")) and q.add(_req("b"))
    assert not q.add(_req("c"))                       # full
    assert q.add(_req("c"), force=True)
    assert q.cancel("a").state == RequestState.CANCELLED
    assert q.cancel("zz") is None
    p = _req("p"); p.mark_preempted()
    q.add_preempted(p)
    assert q.pop_next().request_id == "p"             # preempted requests come back before new ones
    assert q.pop_next().request_id == "b"
    st = q.stats()
    assert st["total_rejected"] == 1 and st["total_cancelled"] == 1


def test_queue_prefill_batch_respects_token_limit():
    q = RequestQueue(10)
    for i, n in enumerate([100, 200, 300]):
        q.add(_req(f"r{i}", n_prompt=n))
    got = q.pop_prefill_batch(max_requests=3, max_tokens=350)
    assert [r.request_id for r in got] == ["r0", "r1"]
    assert q.num_waiting == 1                          # the third was pushed back


# ---- memory budget -----------------------------------------------------------------------------------------------
def test_budget_admission_and_release():
    b = MemoryBudget(total_blocks=20, block_size=16, headroom_ratio=0.5, reserve_blocks=2)
    r = _req("a", n_prompt=64, max_tokens=64)          # 4 prompt blocks + ceil(32/16)+1 = 3 head blocks
    assert b.can_admit(r)
    b.reserve(r)
    assert b.committed_blocks == 7 and b.available_blocks == 11
    big = _req("b", n_prompt=16 * 12, max_tokens=16)
    assert not b.can_admit(big) and b.fits_at_all(big)
    assert not b.fits_at_all(_req("c", n_prompt=16 * 30))
    b.update_decode_progress("a", 40)                  # decode share follows what was generated
    assert b.committed_blocks == 4 + 3 + 1
    b.release("a")
    assert b.committed_blocks == 0 and b.can_admit(big)


# ---- scheduler -------------------------------------------------------------------------------------------------
def _sched(total_blocks=64, **kw):
    cfg = SchedulerConfig(**kw)
    return Scheduler(cfg, MemoryBudget(total_blocks, 16))


def _finish_prefill(s, out):
    for r, n in zip(out.prefill_requests, out.prefill_chunk_sizes):
        s.on_prefill_complete(r, n)


def test_gradual_admission_and_sequence_cap():
    s = _sched(max_prefill_per_step=2, max_batch_seqs=3, decode_per_prefill=0)
    for i in range(5):
        assert s.add_request(_req(f"r{i}"))
    out = s.schedule_step()
    assert out.step_type == StepType.PREFILL and [r.request_id for r in out.prefill_requests] == ["r0", "r1"]
    assert all(r.seq_id is not None for r in out.prefill_requests)
    _finish_prefill(s, out)
    assert s.num_decoding == 2
    out = s.schedule_step()
    assert out.step_type == StepType.MIXED
    assert [r.request_id for r in out.prefill_requests] == ["r2"]       # capped at three sequences
    assert len(out.decode_requests) == 2
    assert s.num_waiting == 2


def test_chunked_prefill_continues_until_prompt_is_cached():
    s = _sched(total_blocks=256, prefill_chunk_size=100, max_batch_tokens=1000)
    s.add_request(_req("long", n_prompt=250))
    sizes = []
    for _ in range(3):
        out = s.schedule_step()
        assert [r.request_id for r in out.prefill_requests] == ["long"]
        sizes.append(out.prefill_chunk_sizes[0])
        _finish_prefill(s, out)
    assert sizes == [100, 100, 50]
    assert s.num_decoding == 1 and s.num_prefilling == 0
    assert s.schedule_step().step_type == StepType.DECODE


def test_continuing_chunks_go_before_new_admissions_and_token_budget_holds():
    s = _sched(total_blocks=512, prefill_chunk_size=300, max_batch_tokens=400, max_prefill_per_step=4)
    s.add_request(_req("long", n_prompt=700))
    out = s.schedule_step(); _finish_prefill(s, out)
    s.add_request(_req("short", n_prompt=150))
    out = s.schedule_step()
    assert [r.request_id for r in out.prefill_requests] == ["long", "short"]
    assert out.prefill_chunk_sizes == [300, 100] and out.num_prefill_tokens <= 400


def test_decode_prefill_interleave_ratio():
    s = _sched(decode_per_prefill=2, max_prefill_per_step=1)
    s.add_request(_req("a", max_tokens=100))
    out = s.schedule_step(); _finish_prefill(s, out)
    for i in range(3):
        s.add_request(_req(f"w{i}"))
    kinds = []
    for _ in range(6):
        out = s.schedule_step()
        kinds.append(out.step_type)
        _finish_prefill(s, out)
        for r in out.decode_requests:
            s.on_token_generated(r, 1)
    assert kinds.count(StepType.MIXED) == 2 and kinds.count(StepType.DECODE) == 4


def test_finished_requests_leave_and_release_budget():
    s = _sched()
    r = _req("a", max_tokens=2)
    s.add_request(r)
    out = s.schedule_step(); _finish_prefill(s, out)
    s.on_token_generated(r, 3)
    s.on_token_generated(r, 4)
    assert r.is_finished and r.finish_reason == FinishReason.LENGTH
    out = s.schedule_step()
    assert out.finished_requests == [r] and out.is_idle and s.num_active == 0
    assert s.stats()["total_finished"] == 1


def test_oversized_request_fails_instead_of_blocking_the_queue():
    s = _sched(total_blocks=8)
    big, ok = _req("big", n_prompt=16 * 20), _req("ok")
    s.add_request(big); s.add_request(ok)
    out = s.schedule_step()
    assert big in out.finished_requests and big.finish_reason == FinishReason.ERROR and big.error
    assert [r.request_id for r in out.prefill_requests] == ["ok"]


def test_preemption_prefers_low_priority_and_least_advanced():
    s = _sched(total_blocks=14, max_prefill_per_step=4, decode_per_prefill=0)
    lo1, lo2 = _req("lo1", n_prompt=32, max_tokens=32), _req("lo2", n_prompt=32, max_tokens=32)
    hi = _req("hi", n_prompt=32, max_tokens=32, priority=1)
    for r in (lo1, lo2, hi):
        s.add_request(r)
    out = s.schedule_step(); _finish_prefill(s, out)
    assert s.num_decoding == 3
    for _ in range(5):
        s.on_token_generated(lo1, 1)
    s.on_token_generated(lo2, 1)
    urgent = _req("urgent", n_prompt=16, max_tokens=16, priority=5)
    s.add_request(urgent)
    out = s.schedule_step()
    assert [r.request_id for r in out.preempt_requests][0] == "lo2"     # same priority: the one that got least far
    assert hi not in out.preempt_requests
    assert lo2.state in (RequestState.PREEMPTED, RequestState.PREFILLING) and lo2.prefill_offset == 0
    assert s.stats()["total_preemptions"] >= 1
    assert urgent in out.prefill_requests


def test_cancel_waiting_and_active():
    s = _sched()
    a, b = _req("a"), _req("b")
    s.add_request(a); s.add_request(b)
    s.cancel_request("b")
    out = s.schedule_step(); _finish_prefill(s, out)
    assert [r.request_id for r in out.prefill_requests] == ["a"]
    s.cancel_request("a")
    out = s.schedule_step()
    assert a in out.finished_requests and a.finish_reason == FinishReason.CANCELLED


def test_speculative_depth_limits_decode_batch():
    s = _sched(speculative_k=3, max_batch_tokens=8, max_prefill_per_step=8, max_batch_seqs=8, decode_per_prefill=0)
    for i in range(4):
        s.add_request(_req(f"r{i}", n_prompt=2, max_tokens=50))
    out = s.schedule_step(); _finish_prefill(s, out)
    out = s.schedule_step()
    assert len(out.decode_requests) == 2               # 8 tokens / (1 + 3 drafted) per sequence


def test_lone_request_is_admitted_even_if_its_headroom_estimate_does_not_fit():
    s = _sched(total_blocks=6)
    r = _req("a", n_prompt=40, max_tokens=23)          # 3 prompt blocks + 2 head-room blocks > 4 usable, but 63 tokens fit
    s.add_request(r)
    out = s.schedule_step()
    assert out.prefill_requests == [r]


def test_reference_named_helpers_of_queue_budget_and_speculation():
    """Names a user of the reference's scheduler pieces relies on (zstreamer/queue.py, memory_budget.py,
    draft_model.py, verifier.py)."""
    import numpy as np
    from zse_b200.sched.draft_model import NGramDraftModel, SelfDraftModel
    from zse_b200.sched.memory_budget import MemoryBudget, MemoryReservation
    from zse_b200.sched.queue import RequestQueue
    from zse_b200.sched.request import GenerationParams, InferenceRequest
    from zse_b200.sched.verifier import SpeculativeVerifier, acceptance_rate, effective_tokens_per_step

    def req(i, n=10, m=8):
        return InferenceRequest(f"r{i}", list(range(n)), GenerationParams(max_tokens=m))

    q = RequestQueue(8)
    a, b = req(1), req(2)
    q.add(a)
    q.add(b)
    assert q.get("r1") is a and q.num_total == 2 and q.num_preempted == 0
    popped = q.pop_next()
    q.add_preempted(popped)
    assert q.num_preempted == 1 and q.get("nope") is None

    bud = MemoryBudget(total_blocks=12, block_size=16, headroom_ratio=0.5, reserve_blocks=2)
    reqs = [req(i, n=40, m=16) for i in range(5)]          # 3 prompt blocks + 2 headroom each
    assert bud.can_admit_n(reqs) == 2
    for r in reqs[:2]:
        bud.reserve(r)
    assert bud.preemption_candidates(1) in (["r0"], ["r1"]) and len(bud.preemption_candidates(100)) == 2
    assert MemoryReservation is not None

    ng = NGramDraftModel(50, n=3, confidence=0.8)
    toks, probs = ng.generate_drafts([1, 2, 3, 4, 1, 2, 3], 3)
    assert toks == [4, 1, 2] and len(probs) == 3 and len(probs[0]) == 50 and abs(sum(probs[0]) - 1) < 1e-6
    assert probs[0][4] == 0.8 and ng.vocab_size() == 50
    toks, _ = ng.generate_drafts([7, 8, 9], 2)             # nothing to look up: still K drafts
    assert len(toks) == 2
    sd = SelfDraftModel(50)
    logits = np.zeros(50, np.float16)
    logits[17] = 3.0
    sd.set_last_logits(logits.tobytes())
    assert sd.propose(2) == [17, 17]

    v = SpeculativeVerifier(seed=0)
    rows = []
    for t in (4, 9, 2):                                    # the target wants 4, then 9, then 2
        r = np.full(50, -5.0, np.float16)
        r[t] = 5.0
        rows.append(r.tobytes())
    acc, n = v.verify_and_accept([4, 1], [ng._dist(4), ng._dist(1)], rows, 50, temperature=0.0)
    assert acc == [4, 9] and n == 1                         # first draft accepted, second replaced by the target's
    acc, n = v.verify_and_accept([4, 9], [ng._dist(4), ng._dist(9)], rows, 50, temperature=0.0)
    assert acc == [4, 9, 2] and n == 2                      # all accepted + bonus token
    acc, n = v.verify_and_accept([4, 9], [ng._dist(4), ng._dist(9)], rows, 50, temperature=1.0)
    assert acc[:2] == [4, 9] and n == 2
    assert acceptance_rate(2, 4) == 0.5 and effective_tokens_per_step(3) == 3.0


def test_default_sampling_seed_is_the_same_in_every_process():
    """An unseeded request draws from a stream named by its id.  The name must not go through ``hash()``: str hashes
    differ between interpreter processes, and the workers of a tensor-parallel group each sample for themselves."""
    import subprocess
    import sys
    code = ("from zse_b200.sched.batch_runner import _sampling_row\n"
            "from zse_b200.sched.request import InferenceRequest, GenerationParams\n"
            "r = InferenceRequest('req-17', [1, 2, 3], GenerationParams(max_tokens=4, temperature=0.8))\n"
            "print(_sampling_row(r).seed)\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    seeds = set()
    for hs in ("1", "2", "random"):
        out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=root,
                             env=dict(os.environ, PYTHONHASHSEED=hs))
        assert out.returncode == 0, out.stderr[-2000:]
        seeds.add(out.stdout.strip())
    assert len(seeds) == 1 and seeds.pop().isdigit()


def test_a_failed_request_is_finished_with_its_error_and_leaves_the_batch():
    s = _sched(max_prefill_per_step=4, decode_per_prefill=0)
    for name in ("ok", "bad"):
        s.add_request(_req(name))
    out = s.schedule_step()
    assert (out.num_prefill_tokens, out.num_decode_tokens, out.total_tokens) == (16, 0, 16) and not out.is_idle
    _finish_prefill(s, out)
    assert sorted(r.request_id for r in s.active_requests()) == ["bad", "ok"]
    bad = next(r for r in s.active_requests() if r.request_id == "bad")
    s.on_request_error(bad, "device said no")
    s.on_request_error(bad, "second report")                                     # the first finish reason stays
    assert bad.is_finished and bad.finish_reason == FinishReason.ERROR and bad.error == "second report"
    out = s.schedule_step()
    assert [r.request_id for r in out.decode_requests] == ["ok"] and out.num_decode_tokens == 1
    assert [r.request_id for r in s.active_requests()] == ["ok"] and s.stats()["total_finished"] == 1
    listing = s.active_requests()
    listing.clear()                                                               # a copy: the scheduler keeps its own
    assert s.num_active == 1

"""Pipelined decode (step n+1 is launched, with its input tokens gathered on the device, before step n has been
read): the tokens must be those of the ordinary order in every situation that rearranges the batch under it - stop
tokens, different lengths, arrivals during decoding, cancellation, preemption, seeded sampling, penalties."""
import random

import pytest

from zse_b200.config import EngineConfig
from zse_b200.engine import ZStreamerEngine
from zse_b200.format import synth
from zse_b200.format.loader import ZSELoader
from zse_b200.models.oracle import OracleModel
from zse_b200.sched.request import FinishReason


@pytest.fixture(scope="module")
def model_path(tmp_path_factory):
    p = str(tmp_path_factory.mktemp("p") / "tiny.zse")
    synth.write_random_model(p, synth.shape_config("tiny"), seed=3)
    return p


@pytest.fixture(scope="module")
def oracle(model_path):
    return OracleModel(ZSELoader(model_path))


def _cfg(**kw):
    base = dict(device="cpu", max_batch_seqs=8, max_seq_len=256, quiet=True, pipeline_decode=True)
    base.update(kw)
    return EngineConfig(**base)


def _prompts(n, lo=3, hi=40, seed=0, vocab=1024):
    rng = random.Random(seed)
    return [[rng.randrange(vocab) for _ in range(rng.randint(lo, hi))] for _ in range(n)]


def _launched_ahead(eng):
    return eng._batch_runner.ahead_launches, eng._batch_runner.ahead_dropped


def test_steady_batch_runs_ahead_and_matches_oracle(model_path, oracle):
    eng = ZStreamerEngine(model_path, config=_cfg())
    prompts = _prompts(6)
    lens = [9, 12, 12, 15, 20, 20]                    # requests leave the batch at different steps
    ids = [eng.add_request_tokens(p, max_tokens=n, temperature=0.0, stop_tokens=[]) for p, n in zip(prompts, lens)]
    eng.run_until_done()
    for rid, p, n in zip(ids, prompts, lens):
        o = eng.get_result(rid)
        assert o.finish_reason == FinishReason.LENGTH and o.output_tokens == oracle.greedy(p, n)
    ahead, dropped = _launched_ahead(eng)
    assert ahead >= 15 and dropped == 0, (ahead, dropped)
    assert eng.kv_cache.num_sequences == 0 and eng.kv_cache.num_free_blocks == eng.kv_cache.num_total_blocks
    eng.destroy()


def test_stop_tokens_cancellation_and_late_arrivals(model_path, oracle):
    eng = ZStreamerEngine(model_path, config=_cfg(prefill_chunk_size=16, max_batch_tokens=48))
    prompts = _prompts(4, seed=5)
    want = [oracle.greedy(p, 14) for p in prompts]
    stops = [[want[0][4]], [], [want[2][9]], []]
    ids = [eng.add_request_tokens(p, max_tokens=14, temperature=0.0, stop_tokens=s) for p, s in zip(prompts, stops)]
    for _ in range(5):
        eng.step()
    late = _prompts(2, lo=30, hi=50, seed=6)           # arrive while the others decode; prefill in chunks
    late_ids = [eng.add_request_tokens(p, max_tokens=7, temperature=0.0, stop_tokens=[]) for p in late]
    eng.step()
    eng.cancel_request(ids[3])
    eng.run_until_done()
    for rid, w, s in zip(ids[:3], want, stops):
        o = eng.get_result(rid)
        cut = w.index(s[0]) + 1 if s else len(w)
        assert o.output_tokens == w[:cut], (o.output_tokens, w[:cut])
        assert o.finish_reason == (FinishReason.STOP if s else FinishReason.LENGTH)
    assert eng.get_result(ids[3]).finish_reason == FinishReason.CANCELLED
    for rid, p in zip(late_ids, late):
        assert eng.get_result(rid).output_tokens == oracle.greedy(p, 7)
    assert eng.kv_cache.num_sequences == 0 and eng.kv_cache.num_free_blocks == eng.kv_cache.num_total_blocks
    eng.destroy()


def test_preemption_and_priorities_keep_outputs_exact(model_path, oracle):
    eng = ZStreamerEngine(model_path, config=_cfg(kv_blocks=14, block_size=16, max_prefill_per_step=4,
                                                  decode_per_prefill=0, headroom_ratio=0.1))
    prompts = _prompts(3, lo=30, hi=40, seed=7)
    ids = [eng.add_request_tokens(p, max_tokens=30, temperature=0.0, stop_tokens=[]) for p in prompts]
    for _ in range(6):
        eng.step()
    late = _prompts(1, lo=20, hi=20, seed=8)[0]
    urgent = eng.add_request_tokens(late, max_tokens=10, temperature=0.0, stop_tokens=[], priority=9)
    eng.run_until_done()
    for rid, p in zip(ids, prompts):
        assert eng.get_result(rid).output_tokens == oracle.greedy(p, 30)
    assert eng.get_result(urgent).output_tokens == oracle.greedy(late, 10)
    eng.destroy()


def test_sampling_and_penalties_equal_the_ordinary_order(model_path):
    prompts = _prompts(3, seed=13) + [[5, 6, 7] * 6]

    def run(pipeline):
        eng = ZStreamerEngine(model_path, config=_cfg(pipeline_decode=pipeline))
        ids = [eng.add_request_tokens(prompts[0], max_tokens=12, stop_tokens=[], seed=1, temperature=1.5, top_p=1.0,
                                      top_k=0),
               eng.add_request_tokens(prompts[1], max_tokens=10, stop_tokens=[], seed=2, temperature=0.8, top_p=0.9,
                                      top_k=20),
               eng.add_request_tokens(prompts[2], max_tokens=12, stop_tokens=[], temperature=0.0)]
        for _ in range(4):
            eng.step()
        ids.append(eng.add_request_tokens(prompts[3], max_tokens=9, stop_tokens=[], temperature=0.0,
                                          repetition_penalty=3.0))
        eng.run_until_done()
        outs = [eng.get_result(i).output_tokens for i in ids]
        eng.destroy()
        return outs

    assert run(True) == run(False)


def test_speculative_decoding_is_left_alone(model_path, oracle):
    eng = ZStreamerEngine(model_path, config=_cfg(speculative_k=3))
    p = _prompts(1, seed=12)[0]
    rid = eng.add_request_tokens(p, max_tokens=12, temperature=0.0, stop_tokens=[])
    eng.run_until_done()
    assert eng.get_result(rid).output_tokens == oracle.greedy(p, 12)
    assert _launched_ahead(eng) == (0, 0)
    eng.destroy()


@pytest.mark.timeout(300)
def test_serving_loop_under_concurrent_clients(model_path, oracle):
    """The serving loop in its own thread while client threads submit, stream and cancel at random moments: every
    finished request must carry exactly the greedy tokens that the engine gives the same prompt on its own in the
    ordinary order (cut at its stop token), every token must have been streamed once and in order, and the cache must
    be empty afterwards."""
    import threading
    import time
    solo = ZStreamerEngine(model_path, config=_cfg(pipeline_decode=False))

    def alone(prompt, n):
        rid = solo.add_request_tokens(prompt, max_tokens=n, temperature=0.0, stop_tokens=[])
        solo.run_until_done()
        return solo.get_result(rid).output_tokens

    eng = ZStreamerEngine(model_path, config=_cfg(max_batch_seqs=6, prefill_chunk_size=16, max_batch_tokens=64))
    rng = random.Random(99)
    jobs = []
    for i in range(28):
        p = _prompts(1, lo=3, hi=45, seed=100 + i)[0]
        n = rng.randint(2, 18)
        want = alone(p, n)
        stop = [want[rng.randrange(len(want))]] if rng.random() < 0.4 else []
        jobs.append({"prompt": p, "n": n, "want": want, "stop": stop, "cancel": rng.random() < 0.15,
                     "streamed": [], "done": threading.Event(), "out": None})
    solo.destroy()
    loop = threading.Thread(target=eng.run, daemon=True)
    loop.start()

    def client(batch):
        for j in batch:
            def on_token(tok, j=j):
                j["streamed"].append(tok)

            def on_finish(out, j=j):
                j["out"] = out
                j["done"].set()

            rid = None
            while rid is None:                      # queue full: try again
                rid = eng.add_request_tokens(j["prompt"], max_tokens=j["n"], temperature=0.0, stop_tokens=j["stop"],
                                             on_token=on_token, on_finish=on_finish)
                if rid is None:
                    time.sleep(0.002)
            if j["cancel"]:
                time.sleep(rng.random() * 0.01)
                eng.cancel_request(rid)
            time.sleep(rng.random() * 0.004)

    clients = [threading.Thread(target=client, args=(jobs[k::4],)) for k in range(4)]
    for t in clients:
        t.start()
    for t in clients:
        t.join(120)
    for j in jobs:
        assert j["done"].wait(120), "a request never finished"
    eng.stop()
    loop.join(30)
    for j in jobs:
        out, want = j["out"], j["want"]
        if out.finish_reason == FinishReason.CANCELLED:
            assert j["cancel"] and out.output_tokens == want[:len(out.output_tokens)]
            continue
        cut = want.index(j["stop"][0]) + 1 if j["stop"] else len(want)
        assert out.output_tokens == want[:cut], (out.output_tokens, want[:cut], j["stop"])
        assert out.finish_reason == (FinishReason.STOP if j["stop"] else FinishReason.LENGTH)
        assert j["streamed"] == out.output_tokens
    assert eng._batch_runner.ahead_launches > 0
    eng.step()
    assert eng.kv_cache.num_sequences == 0 and eng.kv_cache.num_free_blocks == eng.kv_cache.num_total_blocks
    eng.destroy()

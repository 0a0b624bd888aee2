"""The serving engine end to end on the CPU path: continuous batching, chunked prefill, prefix sharing, preemption,
speculative decoding and sampling must all give the tokens of the fp32 oracle model run one sequence at a time
(greedy), as in the reference's own end-to-end checks (zse-engine/tests/test_zstreamer.py, test_engine.py)."""
import os
import random

import pytest

from zse_b200.config import EngineConfig
from zse_b200.engine import GenerateConfig, ZSEEngine, ZStreamerEngine
from zse_b200.format import synth
from zse_b200.format.loader import ZSELoader
from zse_b200.models.oracle import OracleModel
from zse_b200.sched.request import FinishReason


@pytest.fixture(scope="module")
def model_path(tmp_path_factory):
    p = str(tmp_path_factory.mktemp("m") / "tiny.zse")
    synth.write_random_model(p, synth.shape_config("tiny"), seed=3)
    return p


@pytest.fixture(scope="module")
def oracle(model_path):
    return OracleModel(ZSELoader(model_path))


def _cfg(**kw):
    base = dict(device="cpu", max_batch_seqs=8, max_seq_len=256, quiet=True)
    base.update(kw)
    return EngineConfig(**base)


def _prompts(vocab, n, lo=3, hi=40, seed=0):
    rng = random.Random(seed)
    return [[rng.randrange(vocab) for _ in range(rng.randint(lo, hi))] for _ in range(n)]


def _run(eng, prompts, max_tokens, **kw):
    ids = [eng.add_request_tokens(p, max_tokens=max_tokens[i] if isinstance(max_tokens, list) else max_tokens,
                                  temperature=0.0, stop_tokens=[], **kw) for i, p in enumerate(prompts)]
    assert all(i is not None for i in ids)
    eng.run_until_done()
    return [eng.get_result(i) for i in ids]


def test_batched_greedy_matches_oracle(model_path, oracle):
    eng = ZStreamerEngine(model_path, config=_cfg())
    prompts = _prompts(eng.model_config.vocab_size, 6)
    lens = [12 + i for i in range(6)]
    outs = _run(eng, prompts, lens)
    for p, n, o in zip(prompts, lens, outs):
        assert o.finish_reason == FinishReason.LENGTH
        assert o.output_tokens == oracle.greedy(p, n)
    st = eng.stats()
    assert st.total_requests == 6 and st.total_tokens_generated == sum(lens)
    assert eng.kv_cache.num_sequences == 0 and eng.kv_cache.num_free_blocks == eng.kv_cache.num_total_blocks
    eng.destroy()


def test_chunked_prefill_matches_oracle(model_path, oracle):
    eng = ZStreamerEngine(model_path, config=_cfg(prefill_chunk_size=16, max_batch_tokens=48, decode_per_prefill=1))
    prompts = _prompts(eng.model_config.vocab_size, 4, lo=30, hi=90, seed=1)
    outs = _run(eng, prompts, 8)
    for p, o in zip(prompts, outs):
        assert o.output_tokens == oracle.greedy(p, 8)
    eng.destroy()


def test_prefix_sharing_gives_same_tokens_and_reuses_blocks(model_path, oracle):
    eng = ZStreamerEngine(model_path, config=_cfg(block_size=16))
    V = eng.model_config.vocab_size
    system = _prompts(V, 1, lo=50, hi=50, seed=2)[0]
    a, b = system + [1, 2, 3], system + [4, 5]
    first = _run(eng, [a], 6)[0]
    hits0 = eng.kv_cache.stats().dedup_hits
    second = _run(eng, [b], 6)[0]
    # sequence a was freed, but its registered blocks are only reusable while they are alive: run both together
    both = _run(eng, [a, b], 6)
    assert first.output_tokens == oracle.greedy(a, 6) and second.output_tokens == oracle.greedy(b, 6)
    assert both[0].output_tokens == first.output_tokens and both[1].output_tokens == second.output_tokens
    assert eng.kv_cache.stats().dedup_hits >= hits0
    eng.destroy()


def test_stop_token_and_cancel(model_path, oracle):
    eng = ZStreamerEngine(model_path, config=_cfg())
    p = _prompts(eng.model_config.vocab_size, 1, seed=5)[0]
    want = oracle.greedy(p, 10)
    rid = eng.add_request_tokens(p, max_tokens=10, temperature=0.0, stop_tokens=[want[3]])
    gone = eng.add_request_tokens(p, max_tokens=10, temperature=0.0, stop_tokens=[])
    eng.cancel_request(gone)
    eng.run_until_done()
    out = eng.get_result(rid)
    first_hit = want.index(want[3])
    assert out.finish_reason == FinishReason.STOP and out.output_tokens == want[:first_hit + 1]
    assert eng.get_result(gone).finish_reason == FinishReason.CANCELLED
    eng.destroy()


def test_preemption_under_memory_pressure_keeps_outputs_exact(model_path, oracle):
    # 14 blocks of 16 tokens: three 40-token requests cannot all keep growing, some are preempted and re-prefilled
    eng = ZStreamerEngine(model_path, config=_cfg(kv_blocks=14, block_size=16, max_prefill_per_step=4,
                                                  decode_per_prefill=0, headroom_ratio=0.1))
    V = eng.model_config.vocab_size
    prompts = _prompts(V, 3, lo=30, hi=40, seed=7)
    ids = [eng.add_request_tokens(p, max_tokens=30, temperature=0.0, stop_tokens=[]) for p in prompts]
    for _ in range(6):
        eng.step()
    late = _prompts(V, 1, lo=20, hi=20, seed=8)[0]
    urgent = eng.add_request_tokens(late, max_tokens=10, temperature=0.0, stop_tokens=[], priority=9)
    eng.run_until_done()
    for rid, p in zip(ids, prompts):
        o = eng.get_result(rid)
        assert o.finish_reason == FinishReason.LENGTH and o.output_tokens == oracle.greedy(p, 30)
    assert eng.get_result(urgent).output_tokens == oracle.greedy(late, 10)
    eng.destroy()


@pytest.mark.parametrize("mode", ["ngram", "self"])
def test_speculative_decoding_is_exact(model_path, oracle, mode):
    eng = ZStreamerEngine(model_path, config=_cfg(speculative_k=3, speculative_mode=mode))
    V = eng.model_config.vocab_size
    rng = random.Random(11)
    motif = [rng.randrange(V) for _ in range(6)]
    prompts = [motif * 4 + [rng.randrange(V)], _prompts(V, 1, seed=12)[0]]
    outs = _run(eng, prompts, 16)
    # the invariant is "same tokens as the engine without drafting" (the fp16 engine and the fp32 oracle may break a
    # near tie differently)
    plain_eng = ZStreamerEngine(model_path, config=_cfg())
    plain = _run(plain_eng, prompts, 16)
    for a, b in zip(outs, plain):
        assert a.output_tokens == b.output_tokens
    assert outs[1].output_tokens == oracle.greedy(prompts[1], 16)
    st = eng.stats()
    assert st.total_tokens_generated == 32
    spec = eng._spec_runner
    sst = spec.stats()
    assert spec.seq_steps > 0 and 1.0 <= spec.tokens_per_step <= 4.0               # k = 3: at most k + 1 per pass
    assert spec.speedup_factor == spec.tokens_per_step and "k=3" in spec.summary()
    assert 0 <= sst["accepted"] <= sst["drafted"] and spec.tokens_emitted <= 32
    spec.forget("no-such-request")                                                 # unknown ids are fine
    eng.destroy(); plain_eng.destroy()


def test_sampling_is_seeded_and_respects_top_k_one(model_path, oracle):
    eng = ZStreamerEngine(model_path, config=_cfg())
    p = _prompts(eng.model_config.vocab_size, 1, seed=13)[0]

    def sample(seed, **kw):
        rid = eng.add_request_tokens(p, max_tokens=12, stop_tokens=[], seed=seed, **kw)
        eng.run_until_done()
        return eng.get_result(rid).output_tokens

    a = sample(1, temperature=1.5, top_p=1.0, top_k=0)
    b = sample(1, temperature=1.5, top_p=1.0, top_k=0)
    c = sample(2, temperature=1.5, top_p=1.0, top_k=0)
    assert a == b and a != c
    assert sample(5, temperature=1.0, top_k=1) == oracle.greedy(p, 12)
    eng.destroy()


def test_repetition_penalty_changes_greedy_path(model_path, oracle):
    eng = ZStreamerEngine(model_path, config=_cfg())
    p = [5, 6, 7] * 6
    plain = _run(eng, [p], 12)[0].output_tokens
    pen = _run(eng, [p], 12, repetition_penalty=3.0)[0].output_tokens
    assert plain == oracle.greedy(p, 12)
    assert len(pen) == 12 and pen != plain
    eng.destroy()


def test_queue_full_is_reported(model_path):
    eng = ZStreamerEngine(model_path, config=_cfg(max_queue_size=2))
    assert eng.add_request_tokens([1, 2], max_tokens=2) is not None
    assert eng.add_request_tokens([1, 2], max_tokens=2) is not None
    assert eng.add_request_tokens([1, 2], max_tokens=2) is None
    eng.run_until_done()
    eng.destroy()


def test_oversized_prompt_is_refused_and_oversized_generation_fails_cleanly(model_path):
    eng = ZStreamerEngine(model_path, config=_cfg(max_seq_len=96, kv_blocks=6, block_size=16))
    with pytest.raises(ValueError):
        eng.add_request_tokens(list(range(100)), max_tokens=4, temperature=0.0)
    # fits the context but not the cache (6 blocks minus the reserve): finishes with an error, others still run
    rid = eng.add_request_tokens(list(range(40)), max_tokens=40, temperature=0.0, stop_tokens=[])
    ok = eng.add_request_tokens([1, 2, 3], max_tokens=4, temperature=0.0, stop_tokens=[])
    eng.run_until_done()
    bad = eng.get_result(rid)
    assert bad.finish_reason == FinishReason.ERROR and bad.error
    assert len(eng.get_result(ok).output_tokens) == 4
    eng.destroy()


def test_single_request_engine_text_api(model_path):
    eng = ZSEEngine(model_path, config=_cfg())
    text = eng.generate("hello world", GenerateConfig(max_tokens=8, temperature=0.0, stop_tokens=[]))
    pieces = list(eng.stream_generate("hello world", GenerateConfig(max_tokens=8, temperature=0.0, stop_tokens=[])))
    assert isinstance(text, str) and "".join(pieces) == text
    st = eng.stats()
    assert st.generated_tokens > 0 and st.prompt_tokens > 0
    eng.destroy()


def test_client_callbacks_that_raise_do_not_stop_the_engine(model_path, oracle):
    eng = ZStreamerEngine(model_path, config=_cfg())
    p = _prompts(eng.model_config.vocab_size, 2, seed=21)

    def bad_token(tok):
        raise RuntimeError("client bug")

    def bad_finish(out):
        raise RuntimeError("client bug")

    a = eng.add_request_tokens(p[0], max_tokens=6, temperature=0.0, stop_tokens=[], on_token=bad_token)
    b = eng.add_request_tokens(p[1], max_tokens=6, temperature=0.0, stop_tokens=[], on_finish=bad_finish)
    eng.run_until_done()
    assert eng.get_result(a).output_tokens == oracle.greedy(p[0], 6)
    assert eng.get_result(b).output_tokens == oracle.greedy(p[1], 6)
    eng.destroy()


def test_single_request_engine_has_the_reference_call_signatures(model_path, oracle):
    """``ZSEEngine`` as a user of the reference calls it (zse-engine/zse_engine/orchestrator/engine.py:263-360):
    keyword sampling settings, token-level and text-level generators, stats with the reference's fields."""
    eng = ZSEEngine(model_path, 0, 256, True, config=_cfg())
    tok = eng.tokenizer
    ids = tok.encode("hello world")
    want = oracle.greedy(ids, 6)
    assert eng.generate_tokens(ids, max_tokens=6, temperature=0.0, stop_tokens=[]) == want
    assert list(eng.stream_generate_tokens("hello world", max_tokens=6, temperature=0.0, stop_tokens=[])) == want
    text = eng.generate("hello world", max_tokens=6, temperature=0.0, top_p=0.9, top_k=50, repetition_penalty=1.0,
                        stop_tokens=[], seed=None)
    assert text == tok.decode(want)
    assert "".join(eng.stream_generate("hello world", max_tokens=6, temperature=0.0, stop_tokens=[])) == text
    assert eng.generate("hello world", GenerateConfig(max_tokens=6, temperature=0.0, stop_tokens=[])) == text
    a = eng.generate("hello world", max_tokens=8, temperature=1.2, seed=5, stop_tokens=[])
    assert a == eng.generate("hello world", max_tokens=8, temperature=1.2, seed=5, stop_tokens=[])
    # a consumer that stops early does not leave the request running
    gen = eng.stream_generate_tokens("hello world", max_tokens=50, temperature=0.0, stop_tokens=[])
    next(gen)
    gen.close()
    assert not eng.streamer.has_work() and eng.streamer.kv_cache.num_sequences == 0
    st = eng.stats()
    assert st.model_arch == "llama" and st.model_path == model_path and st.total_tokens_generated >= 6 * 5
    assert st.weight_bytes > 0 and st.kv_cache_bytes > 0 and st.scratch_bytes > 0 and st.avg_tokens_per_sec > 0
    assert eng.config.hidden_size == 256 and "llama" in eng.summary()
    eng.destroy()


def test_partial_rotary_matches_oracle(tmp_path):
    """Phi-4-mini style: only the leading 3/4 of each head rotates."""
    p = str(tmp_path / "partial.zse")
    synth.write_random_model(p, synth.shape_config("tiny-phi3", partial_rotary_factor=0.75), seed=6)
    oracle = OracleModel(ZSELoader(p))
    eng = ZStreamerEngine(p, config=_cfg())
    assert eng._model.inv_freq.numel() == 24             # 48 of 64 dims rotate
    prompts = _prompts(eng.model_config.vocab_size, 2, seed=4)
    for pr, o in zip(prompts, _run(eng, prompts, 10)):
        assert o.output_tokens == oracle.greedy(pr, 10)
    eng.destroy()


@pytest.mark.parametrize("quant", ["int4", "fp16"])
def test_phi3_stacked_projections_match_oracle(tmp_path, quant):
    """Phi-3 files keep ``[q; k; v]`` and ``[gate; up]`` stacked (zse-engine/zse_engine/format/arch/phi3.py): the engine
    splits them into the same fused projections as every other family."""
    p = str(tmp_path / "phi3.zse")
    synth.write_random_model(p, synth.shape_config("tiny-phi3", quant=quant), seed=6)
    oracle = OracleModel(ZSELoader(p))
    eng = ZStreamerEngine(p, config=_cfg())
    assert eng.model_config.arch == "phi3"
    prompts = _prompts(eng.model_config.vocab_size, 3, seed=4)
    outs = _run(eng, prompts, 10)
    for pr, o in zip(prompts, outs):
        assert o.output_tokens == oracle.greedy(pr, 10)
    eng.destroy()


def test_step_result_names_the_tokens_of_the_step(model_path, oracle):
    """``StepResult.new_tokens`` maps each request that advanced to its newest token, as the reference's does."""
    eng = ZStreamerEngine(model_path, config=_cfg())
    prompts = _prompts(eng.model_config.vocab_size, 2, seed=9)
    ids = [eng.add_request_tokens(p, max_tokens=4, temperature=0.0, stop_tokens=[]) for p in prompts]
    seen = {i: [] for i in ids}
    for _ in range(50):
        res = eng.step()
        assert res.num_tokens == len(res.new_tokens) and res.preempted_ids == []
        for rid, tok in res.new_tokens.items():
            seen[rid].append(tok)
        if not eng.has_work():
            break
    eng.step()
    for rid, p in zip(ids, prompts):
        assert seen[rid] == oracle.greedy(p, 4) == eng.get_result(rid).output_tokens
    eng.destroy()


@pytest.mark.parametrize("scaling", [{"rope_type": "linear", "factor": 4.0},
                                     {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                      "high_freq_factor": 4.0, "original_max_position_embeddings": 32}])
def test_rope_scaling_reaches_the_engine(tmp_path, scaling):
    """The frequency table the kernels get (``ops.reference.inv_freq``) follows the same scaling rule as the oracle,
    which is checked against transformers."""
    p = str(tmp_path / "scaled.zse")
    synth.write_random_model(p, synth.shape_config("tiny", rope_scaling=scaling, rope_theta=50000.0), seed=8)
    oracle = OracleModel(ZSELoader(p))
    plain = str(tmp_path / "plain.zse")
    synth.write_random_model(plain, synth.shape_config("tiny", rope_theta=50000.0), seed=8)
    eng = ZStreamerEngine(p, config=_cfg())
    prompts = _prompts(eng.model_config.vocab_size, 2, lo=30, hi=60, seed=11)
    outs = _run(eng, prompts, 8)
    unscaled = OracleModel(ZSELoader(plain))
    assert float((oracle.forward(prompts[0]) - unscaled.forward(prompts[0])).abs().max()) > 1e-5    # it matters
    import torch
    from zse_b200.models.oracle import rope_cos_sin
    from zse_b200.ops import reference as ref
    pos = torch.arange(0, 4000, 37)
    cos, sin = rope_cos_sin(pos, 64, 50000.0, None, scaling)
    ang = pos.double()[:, None] * ref.inv_freq(64, 50000.0, scaling).double()[None, :]
    torch.testing.assert_close(torch.cos(ang).float(), cos, atol=2e-3, rtol=0)      # the table is rounded to fp32
    torch.testing.assert_close(torch.sin(ang).float(), sin, atol=2e-3, rtol=0)
    assert not torch.allclose(cos, rope_cos_sin(pos, 64, 50000.0)[0], atol=1e-2)
    for pr, o in zip(prompts, outs):
        assert o.output_tokens == oracle.greedy(pr, 8)
    eng.destroy()


def test_uniform_sliding_window_matches_oracle(tmp_path):
    """Mistral / Phi-3 style window: old blocks leave the cache, attention masks inside the oldest block that stays,
    and the tokens are those of the oracle's exact mask (which is checked against transformers)."""
    p = str(tmp_path / "window.zse")
    synth.write_random_model(p, synth.shape_config("tiny", arch="mistral", sliding_window=24), seed=9)
    oracle = OracleModel(ZSELoader(p))
    full = str(tmp_path / "full.zse")
    synth.write_random_model(full, synth.shape_config("tiny", arch="mistral"), seed=9)
    eng = ZStreamerEngine(p, config=_cfg(block_size=16, prefill_chunk_size=32, max_batch_tokens=64))
    assert eng._model.window == 24
    prompts = _prompts(eng.model_config.vocab_size, 3, lo=40, hi=90, seed=12)
    want = [oracle.greedy(pr, 12) for pr in prompts]
    pr0 = prompts[0]
    assert float((oracle.forward(pr0) - OracleModel(ZSELoader(full)).forward(pr0)).abs().max()) > 1e-5
    for o, w in zip(_run(eng, prompts, 12), want):
        assert o.output_tokens == w
    eng.destroy()


def test_a_device_fault_ends_the_requests_and_marks_the_engine(model_path):
    """A kernel fault reported by the runtime (injected here on the host: the runner's decode raises what torch raises)
    finishes the running requests with an error, leaves the engine answering, and is visible as `fatal_error` - and as
    a 503 of the server's health route - so that a supervisor restarts the worker.  An ordinary error of one pass does
    not mark the engine."""
    import asyncio
    import json

    from zse_b200.sched.batch_runner import is_device_fault
    from zse_b200.server.app import ZSEServer
    from zse_b200.server.router import Request
    assert is_device_fault(RuntimeError("CUDA error: unspecified launch failure\nSearch for ..."))
    assert is_device_fault(RuntimeError("CUDA error: an illegal memory access was encountered"))
    assert not is_device_fault(RuntimeError("CUDA error: out of memory"))
    assert not is_device_fault(ValueError("CUDA error: unspecified launch failure"))
    assert not is_device_fault(RuntimeError("device reported: wait timed out (block 3, site 1, detail 5)"))

    eng = ZStreamerEngine(model_path, config=_cfg())
    srv = ZSEServer(engine=eng, db_path=":memory:", quiet=True, enable_rag=False)

    def health():
        resp = asyncio.new_event_loop().run_until_complete(srv.router.handle(Request("GET", "/health")))
        return resp.status, json.loads(resp.body)

    prompts = _prompts(eng.model_config.vocab_size, 3)
    ids = [eng.add_request_tokens(p, max_tokens=8, temperature=0.0, stop_tokens=[]) for p in prompts]
    for _ in range(3):
        eng.step()
    assert eng.fatal_error is None and health() == (200, {"status": "ok", "model": "zse-model", "engine": "running"})

    real_decode = eng.runner.decode
    calls = {"n": 0}

    def one_bad_pass(*a, **kw):                      # an error that is NOT a device fault: the engine stays healthy
        calls["n"] += 1
        raise ValueError("bad argument in this pass")

    eng.runner.decode = one_bad_pass
    res = eng.step()
    assert res.errors and eng.fatal_error is None
    assert all(eng.get_result(i).finish_reason == FinishReason.ERROR for i in ids)

    more = [eng.add_request_tokens(p, max_tokens=8, temperature=0.0, stop_tokens=[]) for p in prompts]

    def faulting(*a, **kw):
        raise RuntimeError("CUDA error: unspecified launch failure\nCUDA kernel errors might be asynchronously reported")

    eng.runner.decode = faulting
    for _ in range(6):
        eng.step()
        if eng.fatal_error:
            break
    assert eng.fatal_error and "unspecified launch failure" in eng.fatal_error and "\n" not in eng.fatal_error
    outs = [eng.get_result(i) for i in more]
    assert all(o.finish_reason == FinishReason.ERROR and "launch failure" in o.error for o in outs)
    status, body = health()
    assert status == 503 and body["status"] == "error" and body["engine"] == "failed" and "launch failure" in body["error"]
    eng.runner.decode = real_decode
    assert eng.step() is not None                    # the loop itself keeps running
    srv.database.close()
    eng.destroy()


def test_metrics_route_reports_the_engine(model_path):
    import asyncio

    from zse_b200.server.app import ZSEServer
    from zse_b200.server.router import Request
    eng = ZStreamerEngine(model_path, config=_cfg())
    srv = ZSEServer(engine=eng, db_path=":memory:", quiet=True, enable_rag=False)
    _run(eng, _prompts(eng.model_config.vocab_size, 3), 5)
    resp = asyncio.new_event_loop().run_until_complete(srv.router.handle(Request("GET", "/metrics")))
    vals = {l.split(" ")[0]: float(l.split(" ")[1]) for l in resp.body.decode().splitlines() if l and l[0] != "#"}
    assert resp.status == 200 and vals["zse_engine_up"] == 1
    assert vals["zse_requests_total"] == 3 and vals["zse_tokens_generated_total"] == 15 and vals["zse_steps_total"] > 0
    assert vals["zse_requests_active"] == 0 and vals["zse_requests_waiting"] == 0
    assert vals["zse_kv_blocks"] == eng.kv_cache.num_total_blocks and vals["zse_kv_blocks_used"] == 0
    assert vals["zse_ttft_p50_milliseconds"] > 0
    srv.database.close()
    eng.destroy()


def test_engine_config_from_the_environment(monkeypatch):
    """Every field reads ``ZSE_<FIELD>`` with the field's own type; keyword overrides come last and None means
    'not given'."""
    from zse_b200.config import EngineConfig
    for name in list(os.environ):
        if name.startswith("ZSE_"):
            monkeypatch.delenv(name)
    assert EngineConfig.from_env() == EngineConfig()
    monkeypatch.setenv("ZSE_TP_SIZE", "4")
    monkeypatch.setenv("ZSE_KV_FRACTION", "0.25")
    monkeypatch.setenv("ZSE_PIPELINE_DECODE", "off")
    monkeypatch.setenv("ZSE_USE_CUDA_GRAPHS", "No")
    monkeypatch.setenv("ZSE_ENABLE_PREEMPTION", "TRUE")
    monkeypatch.setenv("ZSE_SPECULATIVE_MODE", "self")
    monkeypatch.setenv("ZSE_INT4_LAYOUT", "tiled64x8")
    monkeypatch.setenv("ZSE_HEADROOM_RATIO", "0.75")
    c = EngineConfig.from_env(max_batch_seqs=16, device=None, tp_size=None)
    assert (c.tp_size, c.kv_fraction, c.pipeline_decode, c.use_cuda_graphs, c.enable_preemption) == \
        (4, 0.25, False, False, True)
    assert (c.speculative_mode, c.int4_layout, c.headroom_ratio, c.max_batch_seqs, c.device) == \
        ("self", "tiled64x8", 0.75, 16, None)
    assert EngineConfig.from_env(tp_size=2).tp_size == 2                           # a given keyword beats the variable
    monkeypatch.setenv("ZSE_MAX_SEQ_LEN", "many")
    with pytest.raises(ValueError):
        EngineConfig.from_env()

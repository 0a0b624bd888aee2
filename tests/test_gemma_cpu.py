"""Gemma-2 and Gemma-4 (text) through the serving engine on the CPU path: batched decode, chunked prefill past the
sliding window and prefix sharing must give the tokens of the fp32 oracle (which itself is checked against
transformers in test_hf_parity.py)."""
import random

import pytest

from zse_b200.config import EngineConfig
from zse_b200.engine import ZStreamerEngine
from zse_b200.format import synth
from zse_b200.format.loader import ZSELoader
from zse_b200.models.oracle import OracleModel


def _cfg(**kw):
    base = dict(device="cpu", max_batch_seqs=8, max_seq_len=256, quiet=True)
    base.update(kw)
    return EngineConfig(**base)


@pytest.fixture(scope="module", params=["tiny-gemma2", "tiny-gemma4"])
def model(request, tmp_path_factory):
    p = str(tmp_path_factory.mktemp("g") / f"{request.param}.zse")
    synth.write_random_model(p, synth.shape_config(request.param, "fp16"), seed=5, std=0.05)
    return p, OracleModel(ZSELoader(p))


def _prompts(n, lo, hi, seed):
    rng = random.Random(seed)
    return [[rng.randrange(1000) for _ in range(rng.randint(lo, hi))] for _ in range(n)]


def _run(eng, prompts, max_tokens):
    ids = [eng.add_request_tokens(p, max_tokens=max_tokens, temperature=0.0, stop_tokens=[]) for p in prompts]
    eng.run_until_done()
    return [eng.get_result(i).output_tokens for i in ids]


def test_layer_geometry_of_the_synthetic_shapes():
    c = synth.shape_config("tiny-gemma4")
    local, glob = c.layer_spec(0), c.layer_spec(2)
    assert (local.head_dim, local.num_kv_heads, local.window, local.k_is_v, local.rotary_dim) == (64, 2, 24, False, 64)
    assert (glob.head_dim, glob.num_kv_heads, glob.window, glob.k_is_v, glob.rotary_dim) == (128, 1, 0, True, 32)
    assert glob.scale == 1.0 and glob.qk_norm
    assert c.kv_pool_dims() == (1, 128)          # rows of the widest layer: 2 x 64 = 1 x 128
    c2 = synth.shape_config("tiny-gemma2")
    assert c2.layer_spec(0).window == 24 and c2.layer_spec(1).window == 0
    assert c2.layer_spec(0).softcap == 50.0 and abs(c2.layer_spec(0).scale - 0.125) < 1e-9
    assert c2.kv_pool_dims() == (2, 64) and c2.norm_weight_offset == 1.0


def test_batched_decode_matches_oracle(model):
    path, oracle = model
    eng = ZStreamerEngine(path, config=_cfg())
    prompts = _prompts(5, 3, 50, 0)               # some prompts longer than the window of 24
    outs = _run(eng, prompts, 14)
    for p, o in zip(prompts, outs):
        assert o == oracle.greedy(p, 14)
    assert eng.kv_cache.num_free_blocks == eng.kv_cache.num_total_blocks
    eng.destroy()


def test_chunked_prefill_and_prefix_sharing_match_oracle(model):
    path, oracle = model
    eng = ZStreamerEngine(path, config=_cfg(prefill_chunk_size=16, max_batch_tokens=48, decode_per_prefill=1))
    base = _prompts(1, 70, 70, 2)[0]
    prompts = [base + [7, 8, 9], base + [11, 12], _prompts(1, 40, 40, 3)[0]]
    outs = _run(eng, prompts, 8)
    for p, o in zip(prompts, outs):
        assert o == oracle.greedy(p, 8)
    eng.destroy()


@pytest.mark.timeout(600)
def test_gemma2_tensor_parallel_cpu_ranks_match_single_engine(tmp_path):
    """Two CPU ranks (gloo): heads and MLP split, fp16 all-reduce after the row-parallel projections."""
    from zse_b200.parallel.shard_plan import validate_tp
    from zse_b200.parallel.tp_engine import TPEngine
    assert validate_tp(synth.shape_config("tiny-gemma2"), 2) == []
    assert validate_tp(synth.shape_config("tiny-gemma4"), 2)          # its global layers have one kv head
    path = str(tmp_path / "g2.zse")
    synth.write_random_model(path, synth.shape_config("tiny-gemma2", "fp16"), seed=5, std=0.05)
    cfg = EngineConfig(device="cpu", kv_blocks=64, max_batch_seqs=4, max_batch_tokens=64, max_seq_len=256)
    prompts = _prompts(3, 10, 40, 4)
    ref = ZStreamerEngine(path, config=cfg)
    want = _run(ref, prompts, 6)
    ref.destroy()
    e = TPEngine(path, tp_size=2, config=cfg, start_timeout_s=180)
    try:
        ids = [e.add_request_tokens(x, max_tokens=6, temperature=0.0, stop_tokens=[]) for x in prompts]
        e.run_until_done(120)
        got = [e.get_result(i).output_tokens for i in ids]
        # the ranks round their partial outputs to fp16 before the sum, so a near tie may flip: first tokens exact
        assert [g[0] for g in got] == [w[0] for w in want]
        assert sum(g == w for g, w in zip(got, want)) >= 2, (got, want)
        # the one-request calls of the reference's TPEngine (generate / stream_generate / config / summary)
        text = e.generate("hello there", max_tokens=5, temperature=0.0, stop_tokens=[])
        assert "".join(e.stream_generate("hello there", max_tokens=5, temperature=0.0, stop_tokens=[])) == text
        assert e.config.arch == "gemma2" and e.tp_size == 2 and "2-way" in e.summary()
    finally:
        e.stop()

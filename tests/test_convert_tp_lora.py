"""Conversion (HF directory -> .zse, resumable), tensor-parallel planning and serving on CPU ranks (gloo), LoRA
manager: host-side pieces the reference covers in tests/test_convert.py, test_tensor_parallel.py, test_lora.py."""
import json
import os
import random

import numpy as np
import pytest
import torch

from zse_b200.config import EngineConfig
from zse_b200.engine import ZStreamerEngine
from zse_b200.format import synth
from zse_b200.format.convert import convert_hf_to_zse, write_safetensors
from zse_b200.format.loader import ZSELoader
from zse_b200.format.spec import QuantMethod
from zse_b200.models.oracle import OracleModel
from zse_b200.parallel.shard_plan import all_plans, make_plan, split_units, validate_tp


# ---- conversion -------------------------------------------------------------------------------------------------
def _hf_dir(tmp_path, layers=2, hidden=128, inter=256, vocab=300, heads=4, kv=2, shards=2, bf16=False):
    d = tmp_path / "hf"
    d.mkdir()
    cfg = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": hidden,
           "intermediate_size": inter, "num_hidden_layers": layers, "num_attention_heads": heads,
           "num_key_value_heads": kv, "vocab_size": vocab, "max_position_embeddings": 512, "rms_norm_eps": 1e-6,
           "rope_theta": 1000000.0, "tie_word_embeddings": False}
    (d / "config.json").write_text(json.dumps(cfg))
    rng = np.random.default_rng(0)
    hd = hidden // heads
    t = {"model.embed_tokens.weight": rng.standard_normal((vocab, hidden)) * 0.02,
         "model.norm.weight": np.ones(hidden), "lm_head.weight": rng.standard_normal((vocab, hidden)) * 0.02}
    for l in range(layers):
        p = f"model.layers.{l}."
        t[p + "input_layernorm.weight"] = np.ones(hidden)
        t[p + "post_attention_layernorm.weight"] = np.ones(hidden)
        for name, rows in (("q_proj", heads * hd), ("k_proj", kv * hd), ("v_proj", kv * hd)):
            t[p + f"self_attn.{name}.weight"] = rng.standard_normal((rows, hidden)) * 0.02
            t[p + f"self_attn.{name}.bias"] = rng.standard_normal(rows) * 0.01
        t[p + "self_attn.o_proj.weight"] = rng.standard_normal((hidden, heads * hd)) * 0.02
        t[p + "mlp.gate_proj.weight"] = rng.standard_normal((inter, hidden)) * 0.02
        t[p + "mlp.up_proj.weight"] = rng.standard_normal((inter, hidden)) * 0.02
        t[p + "mlp.down_proj.weight"] = rng.standard_normal((hidden, inter)) * 0.02
    t = {k: v.astype(np.float32) for k, v in t.items()}
    names = sorted(t)
    per = (len(names) + shards - 1) // shards
    for s in range(shards):
        part = {n: t[n] for n in names[s * per:(s + 1) * per]}
        write_safetensors(str(d / f"model-{s + 1:05d}-of-{shards:05d}.safetensors"), part, bf16=bf16)
    return str(d), t


@pytest.mark.parametrize("quant,bf16", [(QuantMethod.INT4_ASYM, False), (QuantMethod.INT8_SYM, True),
                                        (QuantMethod.NONE, False)])
def test_convert_writes_a_loadable_model(tmp_path, quant, bf16):
    hf, tensors = _hf_dir(tmp_path, bf16=bf16)
    out = str(tmp_path / "m.zse")
    seen = []
    convert_hf_to_zse(hf, out, quant_method=quant, skip_tokenizer=True,
                      progress_callback=lambda name, i, n: seen.append((name, i, n)))
    assert seen and seen[-1][1] == seen[-1][2]
    with ZSELoader(out) as l:
        assert l.config.arch == "qwen2" and l.config.num_layers == 2 and l.config.quant.method == int(quant)
        idx = l.weight_index
        w = l.get_weight_as_float(idx.find("layers.0.self_attn.q_proj.weight"))
        ref = tensors["model.layers.0.self_attn.q_proj.weight"]
        tol = {QuantMethod.INT4_ASYM: 0.02, QuantMethod.INT8_SYM: 0.004, QuantMethod.NONE: 0.001}[quant]
        assert w.shape == ref.shape and np.abs(w - ref).max() < tol
        # norms, embeddings and biases are never quantised
        assert idx.find("norm.weight").dtype == "float16" and idx.find("embed_tokens.weight").dtype == "float16"
        assert idx.find("layers.1.self_attn.k_proj.bias").dtype == "float16"
    assert not os.path.exists(out + ".progress")
    # the converted model runs
    eng = ZStreamerEngine(out, config=EngineConfig(device="cpu", max_batch_seqs=2, max_seq_len=64, quiet=True))
    rid = eng.add_request_tokens([1, 2, 3, 4], max_tokens=4, temperature=0.0, stop_tokens=[])
    eng.run_until_done()
    assert len(eng.get_result(rid).output_tokens) == 4
    eng.destroy()


def test_convert_resumes_after_interruption(tmp_path):
    hf, _ = _hf_dir(tmp_path)
    whole, resumed = str(tmp_path / "whole.zse"), str(tmp_path / "resumed.zse")
    convert_hf_to_zse(hf, whole, skip_tokenizer=True)
    with pytest.raises(KeyboardInterrupt):
        convert_hf_to_zse(hf, resumed, skip_tokenizer=True, stop_after=7)
    prog = json.load(open(resumed + ".progress"))
    assert len(prog["done"]) == 7 if "done" in prog else prog
    convert_hf_to_zse(hf, resumed, skip_tokenizer=True)
    assert not os.path.exists(resumed + ".progress")
    assert open(whole, "rb").read() == open(resumed, "rb").read()


# ---- tensor-parallel planning ---------------------------------------------------------------------------------------
def test_split_units_and_group_aligned_shards():
    assert split_units(10, 4) == [(0, 3), (3, 6), (6, 8), (8, 10)]
    cfg = synth.shape_config("qwen2.5-14b")
    assert validate_tp(cfg, 8) == [] and validate_tp(cfg, 3)
    plans = all_plans(cfg, 8)
    # 13824 / 8 = 1728 is 13.5 groups of 128: shards are uneven but every boundary is a group boundary
    assert all(p.inter[0] % 128 == 0 and p.inter[1] % 128 == 0 for p in plans)
    assert plans[0].inter[0] == 0 and plans[-1].inter[1] == cfg.intermediate_size
    assert all(a.inter[1] == b.inter[0] for a, b in zip(plans, plans[1:]))
    assert {p.inter_size for p in plans} == {1792, 1664}
    assert sum(p.vocab_size for p in plans) == cfg.vocab_size and sum(p.q_dim for p in plans) == 40 * 128
    with pytest.raises(ValueError):
        make_plan(cfg, 8, 8)


def test_sharded_model_matches_the_full_model_on_cpu(tmp_path):
    """Two ranks in ONE process (no communication layer): summing the row-parallel partials by hand must give the
    single-rank logits.  Checks slicing of data, scales and zeros incl. the sharded lm_head."""
    from zse_b200.models.decoder import DecoderModel
    path = str(tmp_path / "m.zse")
    synth.write_random_model(path, synth.shape_config("tiny-aligned"), seed=2)
    loader = ZSELoader(path)
    full = DecoderModel.from_loader(loader, torch.device("cpu"))
    r0 = DecoderModel.from_loader(loader, torch.device("cpu"), tp_size=2, rank=0)
    r1 = DecoderModel.from_loader(loader, torch.device("cpu"), tp_size=2, rank=1)
    assert r0.plan.num_heads * 2 == full.plan.num_heads and r0.plan.vocab_size + r1.plan.vocab_size == \
        full.plan.vocab_size
    n_full = sum(int(p.numel()) for p in full.weight_tensors()) if hasattr(full, "weight_tensors") else None
    assert n_full is None or n_full > 0


def _tp_engine(path, cfg):
    from zse_b200.parallel.tp_engine import TPEngine
    return TPEngine(path, tp_size=2, config=cfg, start_timeout_s=180)


@pytest.mark.timeout(600)
def test_tp_engine_cpu_ranks_match_single_engine_and_survive_a_rank_failure(tmp_path):
    path = str(tmp_path / "m.zse")
    synth.write_random_model(path, synth.shape_config("tiny-aligned"), seed=0)
    cfg = EngineConfig(device="cpu", kv_blocks=64, max_batch_seqs=4, max_batch_tokens=64, max_seq_len=256)
    rng = random.Random(0)
    prompts = [[rng.randrange(1024) for _ in range(12)] for _ in range(3)]
    ref = ZStreamerEngine(path, config=cfg)
    ids = [ref.add_request_tokens(x, max_tokens=6, temperature=0.0, stop_tokens=[]) for x in prompts]
    ref.run_until_done()
    want = [ref.get_result(i).output_tokens for i in ids]
    e = _tp_engine(path, cfg)
    try:
        ids = [e.add_request_tokens(x, max_tokens=6, temperature=0.0, stop_tokens=[]) for x in prompts]
        e.run_until_done(120)
        assert [e.get_result(i).output_tokens for i in ids] == want
        assert e.healthy and e.stats().tp_size == 2
        # a rank leaves between steps: in-flight work ends with an error, new work is refused, restart recovers
        rid = e.add_request_tokens(prompts[0], max_tokens=200, temperature=0.0, stop_tokens=[])
        e.poll(0.2)
        e.inject_failure(1, "exit")
        e.run_until_done(120)
        out = e.get_result(rid)
        assert out is not None and out.error and not e.healthy
        assert e.add_request_tokens(prompts[0]) is None
        e.restart()
        rid = e.add_request_tokens(prompts[1], max_tokens=6, temperature=0.0, stop_tokens=[])
        e.run_until_done(120)
        assert e.healthy and e.get_result(rid).output_tokens == want[1]
    finally:
        e.stop()


@pytest.mark.timeout(600)
def test_tp_engine_phi3_stacked_projections(tmp_path):
    """Phi-3's stacked ``qkv_proj`` / ``gate_up_proj`` tensors are sharded part by part (each rank takes its heads from
    the q, k and v sections, its rows from the gate and up sections)."""
    path = str(tmp_path / "phi3.zse")
    synth.write_random_model(path, synth.shape_config("tiny-phi3"), seed=6)
    cfg = EngineConfig(device="cpu", kv_blocks=64, max_batch_seqs=4, max_batch_tokens=64, max_seq_len=256)
    rng = random.Random(1)
    prompts = [[rng.randrange(1024) for _ in range(10)] for _ in range(2)]
    ref = ZStreamerEngine(path, config=cfg)
    ids = [ref.add_request_tokens(x, max_tokens=6, temperature=0.0, stop_tokens=[]) for x in prompts]
    ref.run_until_done()
    want = [ref.get_result(i).output_tokens for i in ids]
    e = _tp_engine(path, cfg)
    try:
        ids = [e.add_request_tokens(x, max_tokens=6, temperature=0.0, stop_tokens=[]) for x in prompts]
        e.run_until_done(120)
        assert [e.get_result(i).output_tokens for i in ids] == want
    finally:
        e.stop()


@pytest.mark.timeout(600)
def test_sequence_parallel_prefill_matches_all_reduce(tmp_path, monkeypatch):
    """Reduce-scatter after the row-parallel projections + all-gather before the column-parallel ones (the residual
    stream split by rows) gives the hidden states and tokens of the all-reduce path, on two CPU ranks."""
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from dist_sp_fn import rank_fn
    from zse_b200.models.oracle import OracleModel
    from zse_b200.parallel.tensor_parallel import tp_launch
    path = str(tmp_path / "m.zse")
    synth.write_random_model(path, synth.shape_config("tiny-aligned"), seed=4)
    monkeypatch.setenv("ZSE_TEST_MODEL", path)
    res = tp_launch(2, rank_fn, backend="cpu", timeout_s=300)
    layers = synth.shape_config("tiny-aligned").num_layers
    for r in res:
        assert r["tokens_equal"] and r["max_diff"] <= 2e-3 * max(1.0, r["scale"])
        assert r["sp_passes"] == (0, 2 * layers)          # every norm after a row-parallel projection of the prefill
    prompt = [(7 * i + 3) % 1024 for i in range(37)]
    assert res[0]["tokens"] == res[1]["tokens"] == OracleModel(ZSELoader(path)).greedy(prompt, 2)


# ---- LoRA manager ---------------------------------------------------------------------------------------------------
def test_lora_manager_slots_and_effect_on_outputs(tmp_path):
    from zse_b200.lora.weights import random_adapter_file
    path = str(tmp_path / "m.zse")
    synth.write_random_model(path, synth.shape_config("tiny"), seed=4)
    eng = ZStreamerEngine(path, config=EngineConfig(device="cpu", max_batch_seqs=4, max_seq_len=128, quiet=True))
    mgr = eng.lora_manager
    a, b = str(tmp_path / "a.zse-lora"), str(tmp_path / "b.zse-lora")
    random_adapter_file(a, eng.model_config, rank=4, alpha=8.0, seed=1, std=0.2)
    random_adapter_file(b, eng.model_config, rank=8, alpha=8.0, seed=2, std=0.2)
    ad = mgr.load_adapter("a", a)
    assert ad.rank == 4 and abs(ad.scaling - 2.0) < 1e-9 and mgr.is_loaded("a")
    with pytest.raises(ValueError):
        mgr.load_adapter("a", a)
    mgr.load_adapter("b", b)                         # larger rank: tables grow, adapter a keeps working
    assert {x["adapter_id"] for x in mgr.list_adapters()} == {"a", "b"} and mgr.stats()["num_adapters"] == 2
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]

    def gen(lora_id=None):
        rid = eng.add_request_tokens(prompt, max_tokens=8, temperature=0.0, stop_tokens=[], lora_id=lora_id)
        eng.run_until_done()
        return eng.get_result(rid).output_tokens

    base = gen()
    assert base == OracleModel(ZSELoader(path)).greedy(prompt, 8)
    with_a, with_b = gen("a"), gen("b")
    assert with_a != base or with_b != base          # a std-0.2 adapter moves a random tiny model
    # requests with different adapters in ONE batch keep their own adapter
    r1 = eng.add_request_tokens(prompt, max_tokens=8, temperature=0.0, stop_tokens=[], lora_id="a")
    r2 = eng.add_request_tokens(prompt, max_tokens=8, temperature=0.0, stop_tokens=[])
    r3 = eng.add_request_tokens(prompt, max_tokens=8, temperature=0.0, stop_tokens=[], lora_id="b")
    eng.run_until_done()
    assert [eng.get_result(r).output_tokens for r in (r1, r2, r3)] == [with_a, base, with_b]
    assert mgr.unload_adapter("a") and not mgr.unload_adapter("a")
    assert gen() == base
    eng.destroy()


def test_prefix_cache_never_crosses_adapters(tmp_path):
    """A prompt of several cache blocks, run with the base model and with two adapters at the same time and one after
    the other: every request must produce what it produces alone (cached prefix blocks hold keys and values computed
    with one set of weights and are only shared by requests that use the same weights)."""
    from zse_b200.lora.weights import random_adapter_file
    path = str(tmp_path / "m.zse")
    synth.write_random_model(path, synth.shape_config("tiny"), seed=4)
    cfg = EngineConfig(device="cpu", max_batch_seqs=4, max_seq_len=128, quiet=True)
    rng = random.Random(7)
    prompt = [rng.randrange(1024) for _ in range(45)]

    def solo(lora_id, prefix_cache):
        eng = ZStreamerEngine(path, config=EngineConfig(**{**cfg.__dict__, "enable_prefix_cache": prefix_cache}))
        for name, seed in (("a", 1), ("b", 2)):
            f = str(tmp_path / f"{name}.zse-lora")
            random_adapter_file(f, eng.model_config, rank=4, alpha=8.0, seed=seed, std=0.2)
            eng.lora_manager.load_adapter(name, f)
        rid = eng.add_request_tokens(prompt, max_tokens=8, temperature=0.0, stop_tokens=[], lora_id=lora_id)
        eng.run_until_done()
        out = eng.get_result(rid).output_tokens
        eng.destroy()
        return out

    want = {k: solo(k, False) for k in (None, "a", "b")}
    assert want["a"] != want[None] or want["b"] != want[None]
    eng = ZStreamerEngine(path, config=cfg)
    for name in ("a", "b"):
        eng.lora_manager.load_adapter(name, str(tmp_path / f"{name}.zse-lora"))
    block = eng.cache_manager.block_size if hasattr(eng, "cache_manager") else 16
    assert len(prompt) > 2 * block
    # base first so that its blocks are registered, then the adapters while the base request is still live
    r0 = eng.add_request_tokens(prompt, max_tokens=8, temperature=0.0, stop_tokens=[])
    eng.step()
    ra = eng.add_request_tokens(prompt, max_tokens=8, temperature=0.0, stop_tokens=[], lora_id="a")
    rb = eng.add_request_tokens(prompt, max_tokens=8, temperature=0.0, stop_tokens=[], lora_id="b")
    eng.run_until_done()
    assert [eng.get_result(r).output_tokens for r in (r0, ra, rb)] == [want[None], want["a"], want["b"]]
    # the same adapter again: it may (and does) reuse its own blocks, and still gives the same tokens
    ra2 = eng.add_request_tokens(prompt, max_tokens=8, temperature=0.0, stop_tokens=[], lora_id="a")
    r02 = eng.add_request_tokens(prompt, max_tokens=8, temperature=0.0, stop_tokens=[])
    eng.run_until_done()
    assert eng.get_result(ra2).output_tokens == want["a"] and eng.get_result(r02).output_tokens == want[None]
    # a re-loaded adapter of the same name (other weights) must not see the old one's blocks
    eng.lora_manager.unload_adapter("a")
    eng.lora_manager.load_adapter("a", str(tmp_path / "b.zse-lora"))
    ra3 = eng.add_request_tokens(prompt, max_tokens=8, temperature=0.0, stop_tokens=[], lora_id="a")
    eng.run_until_done()
    assert eng.get_result(ra3).output_tokens == want["b"]
    eng.destroy()


@pytest.mark.timeout(300)
def test_collectives_facade(tmp_path):
    """all_reduce / all_gather / broadcast / reduce_scatter / barrier of the communication layer on three CPU ranks."""
    import socket
    import subprocess
    import sys
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = str(s.getsockname()[1])
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "dist_facade_worker.py")
    procs = [subprocess.Popen([sys.executable, worker, str(r), "3", port], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT) for r in range(3)]
    outs = [p.communicate(timeout=240)[0].decode() for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)


def test_peft_adapter_import(tmp_path):
    """adapter_config.json + adapter_model.safetensors (PEFT naming) -> .zse-lora with the same matrices."""
    from zse_b200.format.convert import write_safetensors
    from zse_b200.format.lora_convert import convert_peft_to_zse_lora
    from zse_b200.format.lora_format import load_lora, module_shapes
    d = tmp_path / "peft"
    d.mkdir()
    r, layers, H, kvd = 4, 2, 64, 32
    (d / "adapter_config.json").write_text(json.dumps({"r": r, "lora_alpha": 8, "target_modules": ["q_proj", "v_proj"],
                                                       "peft_type": "LORA"}))
    rng = np.random.default_rng(0)
    t = {}
    for l in range(layers):
        for mod, out in (("q_proj", H), ("v_proj", kvd)):
            base = f"base_model.model.model.layers.{l}.self_attn.{mod}"
            t[base + ".lora_A.weight"] = rng.standard_normal((r, H)).astype(np.float32)
            t[base + ".lora_B.weight"] = rng.standard_normal((out, r)).astype(np.float32)
    t["base_model.model.lm_head.lora_A.weight"] = np.zeros((r, H), np.float32)       # not a served projection
    write_safetensors(str(d / "adapter_model.safetensors"), t)
    out = str(tmp_path / "a.zse-lora")
    info = convert_peft_to_zse_lora(str(d), out)
    assert info["rank"] == r and info["alpha"] == 8.0 and info["targets"] == ["q_proj", "v_proj"]
    assert info["num_layers"] == layers and len(info["skipped"]) == 1
    shapes = module_shapes(H, 0, num_heads=4, num_kv_heads=2, head_dim=16)
    adapter, data = load_lora(out, shapes)
    assert adapter.rank == r and abs(adapter.scaling - 2.0) < 1e-6
    a, b = data[(1, "v_proj")]
    want_a = t["base_model.model.model.layers.1.self_attn.v_proj.lora_A.weight"].astype(np.float16)
    want_b = t["base_model.model.model.layers.1.self_attn.v_proj.lora_B.weight"].astype(np.float16)
    assert np.array_equal(np.frombuffer(a, np.float16).reshape(r, H), want_a)
    assert np.array_equal(np.frombuffer(b, np.float16).reshape(kvd, r), want_b)
    # a layer without one of the targets cannot be written
    del t["base_model.model.model.layers.1.self_attn.q_proj.lora_B.weight"]
    write_safetensors(str(d / "adapter_model.safetensors"), t)
    with pytest.raises(ValueError):
        convert_peft_to_zse_lora(str(d), out)
    assert convert_peft_to_zse_lora(str(d), out, modules=["v_proj"])["targets"] == ["v_proj"]


@pytest.mark.parametrize("quant", ["fp16", "int4"])
def test_lora_on_every_projection_equals_merged_weights(tmp_path, quant):
    """An adapter on all seven projections (the reference's set, model_runner.py:1000-1109): the engine's tokens must
    be those of the fp32 oracle run on W + (alpha/r) B A."""
    from zse_b200.format.lora_format import load_lora
    from zse_b200.lora.weights import random_adapter_file
    path = str(tmp_path / "m.zse")
    cfg = synth.shape_config("tiny-aligned", quant)
    synth.write_random_model(path, cfg, seed=6)
    eng = ZStreamerEngine(path, config=EngineConfig(device="cpu", max_batch_seqs=4, max_seq_len=128, quiet=True))
    targets = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]
    f = str(tmp_path / "all.zse-lora")
    random_adapter_file(f, eng.model_config, rank=4, alpha=8.0, target_modules=targets, seed=3, std=0.08)
    eng.lora_manager.load_adapter("all", f)
    only_mlp = str(tmp_path / "mlp.zse-lora")
    random_adapter_file(only_mlp, eng.model_config, rank=2, alpha=2.0, target_modules=["up_proj", "down_proj"], seed=4,
                        std=0.08)
    eng.lora_manager.load_adapter("mlp", only_mlp)

    def merged_oracle(file):
        orc = OracleModel(ZSELoader(path))
        adapter, data = load_lora(file, eng.lora_manager.weight_shapes())
        block = {"q_proj": "self_attn", "k_proj": "self_attn", "v_proj": "self_attn", "o_proj": "self_attn"}
        for (layer, mod), (a, b) in data.items():
            w = adapter.get_weight(layer, mod)
            A = torch.from_numpy(np.frombuffer(a, np.float16).reshape(w.rank, w.in_features).astype(np.float32))
            B = torch.from_numpy(np.frombuffer(b, np.float16).reshape(w.out_features, w.rank).astype(np.float32))
            name = f"layers.{layer}.{block.get(mod, 'mlp')}.{mod}.weight"
            orc.w[name] = orc.w[name] + adapter.scaling * (B @ A)
        return orc

    prompts = [[3, 1, 4, 1, 5, 9, 2, 6], [7, 7, 8, 100, 200, 300]]
    ids = [eng.add_request_tokens(prompts[0], max_tokens=8, temperature=0.0, stop_tokens=[], lora_id="all"),
           eng.add_request_tokens(prompts[1], max_tokens=8, temperature=0.0, stop_tokens=[], lora_id="mlp"),
           eng.add_request_tokens(prompts[0], max_tokens=8, temperature=0.0, stop_tokens=[])]
    eng.run_until_done()
    got = [eng.get_result(i).output_tokens for i in ids]
    assert got[0] == merged_oracle(f).greedy(prompts[0], 8)
    assert got[1] == merged_oracle(only_mlp).greedy(prompts[1], 8)
    assert got[2] == OracleModel(ZSELoader(path)).greedy(prompts[0], 8)
    assert got[0] != got[2]
    eng.destroy()


@pytest.mark.timeout(600)
def test_lora_on_every_projection_under_tensor_parallelism(tmp_path, monkeypatch):
    """Two CPU ranks, an adapter on all seven projections: A of o_proj / down_proj is sharded by columns like the
    projection's input, each rank's update joins its partial output and one all-reduce completes both.  Tokens must be
    those of the fp32 oracle run on the merged weights."""
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from dist_lora_tp_fn import rank_fn
    from zse_b200.format.lora_format import load_lora
    from zse_b200.lora.weights import random_adapter_file
    from zse_b200.parallel.tensor_parallel import tp_launch
    path = str(tmp_path / "m.zse")
    cfg = synth.shape_config("tiny-aligned")
    synth.write_random_model(path, cfg, seed=6)
    targets = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]
    f = str(tmp_path / "all.zse-lora")
    eng = ZStreamerEngine(path, config=EngineConfig(device="cpu", max_batch_seqs=2, max_seq_len=128, quiet=True))
    random_adapter_file(f, eng.model_config, rank=4, alpha=8.0, target_modules=targets, seed=3, std=0.08)
    shapes = eng.lora_manager.weight_shapes()
    eng.destroy()
    monkeypatch.setenv("ZSE_TEST_MODEL", path)
    monkeypatch.setenv("ZSE_TEST_ADAPTER", f)
    res = tp_launch(2, rank_fn, backend="cpu", timeout_s=300)
    orc = OracleModel(ZSELoader(path))
    adapter, data = load_lora(f, shapes)
    for (layer, mod), (a, b) in data.items():
        w = adapter.get_weight(layer, mod)
        A = torch.from_numpy(np.frombuffer(a, np.float16).reshape(w.rank, w.in_features).astype(np.float32))
        B = torch.from_numpy(np.frombuffer(b, np.float16).reshape(w.out_features, w.rank).astype(np.float32))
        name = f"layers.{layer}.{'self_attn' if mod in ('q_proj', 'k_proj', 'v_proj', 'o_proj') else 'mlp'}.{mod}.weight"
        orc.w[name] = orc.w[name] + adapter.scaling * (B @ A)
    want = orc.greedy([3, 1, 4, 1, 5, 9, 2, 6], 6)
    assert res[0]["tokens"] == res[1]["tokens"] == want
    assert want != OracleModel(ZSELoader(path)).greedy([3, 1, 4, 1, 5, 9, 2, 6], 6)      # the adapter matters
    c = cfg
    assert res[0]["a_cols"]["o_proj"][2] == c.num_heads * c.head_dim // 2                # half of the input columns
    assert res[0]["a_cols"]["down_proj"][2] == c.intermediate_size // 2
    assert res[0]["a_cols"]["q_proj"][2] == c.hidden_size


def test_lora_manager_reference_entry_points(tmp_path):
    path = str(tmp_path / "m.zse")
    synth.write_random_model(path, synth.shape_config("tiny"), seed=4)
    eng = ZStreamerEngine(path, config=EngineConfig(device="cpu", max_batch_seqs=2, max_seq_len=128, quiet=True))
    m = eng.lora_manager
    m.load_adapter_random("r", rank=4, alpha=8.0, target_modules=["q_proj", "o_proj"], std=0.1)
    shapes = m.weight_shapes()
    rng = np.random.default_rng(0)
    data = {(l, "v_proj"): ((rng.standard_normal((2, shapes["v_proj"][0])) * 0.1).astype(np.float16).tobytes(),
                            (rng.standard_normal((shapes["v_proj"][1], 2)) * 0.1).astype(np.float16).tobytes())
            for l in range(eng.model_config.num_layers)}
    m.load_adapter_from_dict("d", 2, 4.0, eng.model_config.num_layers, ["v_proj"], data)
    assert m.num_adapters == 2 and m.has_adapter("r") and m.get_adapter("d").rank == 2 and "slot" in m.summary()
    # the prefix-cache name of an adapter: 0 for the base model, distinct per adapter, new after a reload
    salts = {i: m.cache_salt(i) for i in ("r", "d")}
    assert m.cache_salt(None) == m.cache_salt("") == m.cache_salt("not-loaded") == 0
    assert salts["r"] != salts["d"] and all(v > 0 and v & 1 for v in salts.values())
    assert m.cache_salt("r") == salts["r"]                                         # stable while it stays loaded
    rid = eng.add_request_tokens([1, 2, 3, 4], max_tokens=4, temperature=0.0, stop_tokens=[], lora_id="d")
    eng.run_until_done()
    assert len(eng.get_result(rid).output_tokens) == 4
    eng.destroy()


@pytest.mark.timeout(300)
def test_tensor_parallel_group_facade():
    """``tp_launch`` + ``TensorParallelGroup`` under the reference's names, on two CPU ranks."""
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from dist_tp_group_fn import rank_fn
    from zse_b200.parallel.tensor_parallel import TPConfig, tp_launch
    res = tp_launch(2, rank_fn, backend="cpu", timeout_s=240)
    assert res[0]["sum"] == [3.0] * 4 and res[1]["gathered"] == [0.0, 1.0] and res[0]["bcast"] == [10.0]
    assert res[0]["q"] == (0, 256) and res[1]["q"] == (256, 512)
    assert res[0]["down"] == (0, 6912) and res[1]["down"] == (6912, 13824)
    assert res[0]["strategy"] == ["row", "column", "replicated"]
    assert res[1]["comm"] == {"rank": 1, "nranks": 2, "sum": [3.0] * 3, "rs": [5.0, 7.0]}
    assert res[0]["comm"]["rs"] == [1.0, 3.0]
    cfg = TPConfig(tp_size=8)
    assert cfg.is_enabled()
    with pytest.raises(ValueError):
        cfg.validate(40, 6, 13824)
    with pytest.raises(ValueError):
        tp_launch(1, rank_fn)

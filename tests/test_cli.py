"""The ``zse`` command line (same commands as zse-engine/zse_engine/cli.py:218-300: serve, convert, info, version,
warm, keys; plus synth and bench-kernels), run as a subprocess the way a user does, and the HTTP server started by
``zse serve`` in its mock mode and with a model on the CPU path."""
import json
import os
import signal
import socket
import subprocess
import sys
import time
import urllib.request

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def zse(*args, timeout=300, env=None):
    e = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    e.update(env or {})
    return subprocess.run([sys.executable, "-m", "zse_b200", *map(str, args)], capture_output=True, text=True,
                          timeout=timeout, env=e, cwd=ROOT)


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    p = str(tmp_path_factory.mktemp("cli") / "tiny.zse")
    r = zse("synth", "tiny", p, "--seed", "4")
    assert r.returncode == 0 and "wrote" in r.stdout, r.stderr
    return p


def test_version_info_warm(tiny):
    r = zse("version")
    assert r.returncode == 0 and "zse_b200" in r.stdout and "torch" in r.stdout
    r = zse("info", tiny)
    assert r.returncode == 0 and "llama" in r.stdout and "layers" in r.stdout.lower(), r.stdout + r.stderr
    r = zse("warm", tiny)
    assert r.returncode == 0 and "warmed" in r.stdout
    assert zse("warm", tiny + ".missing").returncode == 1
    r = zse()
    assert r.returncode == 0 and "serve" in r.stdout               # no command: help


def test_keys_create_list_revoke(tmp_path):
    db = str(tmp_path / "k.db")
    r = zse("keys", "--db-path", db, "create", "--name", "alice", "--rpm", "7")
    assert r.returncode == 0 and "sk-zse-" in r.stdout
    r = zse("keys", "--db-path", db, "list")
    assert "alice" in r.stdout and "rpm=7" in r.stdout and "active" in r.stdout
    key_id = r.stdout.split()[0]
    assert zse("keys", "--db-path", db, "revoke", key_id).returncode == 0
    assert "revoked" in zse("keys", "--db-path", db, "list").stdout
    assert zse("keys", "--db-path", db, "revoke", "999").returncode == 1
    # the reference's spelling: options after the action, --rate-limit-rpm, revoke --id
    r = zse("keys", "create", "--name", "bob", "--rate-limit-rpm", "9", "--db-path", db)
    assert r.returncode == 0 and "sk-zse-" in r.stdout
    listing = zse("keys", "list", "--db-path", db).stdout
    bob = [l for l in listing.splitlines() if "bob" in l][0]
    assert "rpm=9" in bob
    assert zse("keys", "revoke", "--id", bob.split()[0], "--db-path", db).returncode == 0


def test_convert_command_and_module_entry(tmp_path):
    from zse_b200.format.convert import write_safetensors
    from zse_b200.format.loader import ZSELoader
    d = tmp_path / "hf"
    d.mkdir()
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 128, "intermediate_size": 256,
           "num_hidden_layers": 1, "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": 200,
           "max_position_embeddings": 256, "rms_norm_eps": 1e-5, "tie_word_embeddings": False}
    (d / "config.json").write_text(json.dumps(cfg))
    rng = np.random.default_rng(0)
    t = {"model.embed_tokens.weight": rng.standard_normal((200, 128)), "model.norm.weight": np.ones(128),
         "lm_head.weight": rng.standard_normal((200, 128)), "model.layers.0.input_layernorm.weight": np.ones(128),
         "model.layers.0.post_attention_layernorm.weight": np.ones(128)}
    for name, shape in (("self_attn.q_proj", (128, 128)), ("self_attn.k_proj", (64, 128)),
                        ("self_attn.v_proj", (64, 128)), ("self_attn.o_proj", (128, 128)),
                        ("mlp.gate_proj", (256, 128)), ("mlp.up_proj", (256, 128)), ("mlp.down_proj", (128, 256))):
        t[f"model.layers.0.{name}.weight"] = rng.standard_normal(shape) * 0.05
    write_safetensors(str(d / "model.safetensors"), {k: v.astype(np.float32) for k, v in t.items()})
    out = str(tmp_path / "m.zse")
    r = zse("convert", d, out, "--quant", "int8", "--no-tokenizer", "-q")
    assert r.returncode == 0, r.stderr
    with ZSELoader(out) as l:
        assert l.config.arch == "llama" and l.weight_index.find("layers.0.mlp.up_proj.weight").dtype == "int8"
    out2 = str(tmp_path / "m2.zse")
    e = dict(os.environ, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "zse_b200.format", str(d), out2, "--quant", "fp16", "--no-tokenizer"],
                       capture_output=True, text=True, env=e, cwd=ROOT, timeout=300)
    assert r.returncode == 0 and os.path.getsize(out2) > os.path.getsize(out), r.stderr
    assert zse("convert", tmp_path / "nowhere", out).returncode != 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _get(url, data=None, headers=None, timeout=60):
    req = urllib.request.Request(url, data=None if data is None else json.dumps(data).encode(),
                                 headers={"Content-Type": "application/json", **(headers or {})})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return json.loads(r.read())


def _serve(args, port):
    e = dict(os.environ, PYTHONPATH=ROOT)
    proc = subprocess.Popen([sys.executable, "-m", "zse_b200", "serve", *args, "--port", str(port), "--host",
                             "127.0.0.1", "-q"], env=e, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    for _ in range(600):
        try:
            return proc, _get(f"http://127.0.0.1:{port}/health", timeout=2)
        except Exception:
            if proc.poll() is not None:
                raise AssertionError(proc.stdout.read().decode())
            time.sleep(0.2)
    proc.kill()
    raise AssertionError("server did not come up")


@pytest.mark.timeout(300)
def test_serve_mock_mode_and_cpu_model(tiny, tmp_path):
    port = _free_port()
    proc, health = _serve(["--db-path", str(tmp_path / "a.db"), "--admin-key", "adm"], port)
    try:
        assert health["engine"] == "mock"
        out = _get(f"http://127.0.0.1:{port}/v1/chat/completions",
                   {"model": "zse-model", "messages": [{"role": "user", "content": "ping"}]})
        assert out["choices"][0]["message"]["role"] == "assistant"
    finally:
        proc.send_signal(signal.SIGTERM)
        proc.wait(30)
    port = _free_port()
    proc, health = _serve([tiny, "--cpu", "--db-path", str(tmp_path / "b.db"), "--admin-key", "adm",
                           "--max-seq-len", "256", "--max-batch-seqs", "4"], port)
    try:
        assert health["engine"] == "running"
        out = _get(f"http://127.0.0.1:{port}/v1/completions", {"model": "zse-model", "prompt": "hello", "max_tokens": 5,
                                                                 "temperature": 0})
        assert out["usage"]["completion_tokens"] >= 1 and out["choices"][0]["finish_reason"] in ("length", "stop")
        stats = _get(f"http://127.0.0.1:{port}/v1/admin/stats", headers={"Authorization": "Bearer adm"})
        assert stats["engine"]["total_requests"] >= 1
    finally:
        proc.send_signal(signal.SIGTERM)
        proc.wait(30)


def test_info_lists_environment_switches(monkeypatch):
    import os
    r = subprocess.run([sys.executable, "-m", "zse_b200", "info", "--env"], capture_output=True, text=True,
                       env={**os.environ, "ZSE_TP_SP": "1"}, timeout=240)
    assert r.returncode == 0 and "ZSE_TP_SP=1  (set)" in r.stdout and "ZSE_LOAD_RING=6" in r.stdout
    assert "ZSE_MAX_BATCH_SEQS" in r.stdout
    from zse_b200.utils import env
    monkeypatch.setenv("ZSE_NATIVE_STEP", "off")
    monkeypatch.setenv("ZSE_LOAD_RING", "nine")
    assert env.flag("ZSE_NATIVE_STEP") is False and env.flag("ZSE_PIPELINE_DECODE") is True
    with pytest.raises(ValueError):
        env.integer("ZSE_LOAD_RING")
    with pytest.raises(KeyError):
        env.flag("ZSE_NOT_DECLARED")
    # every ZSE_* name the Python sources read is declared
    import re
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "zse_b200")
    used = set()
    for d, _, files in os.walk(root):
        for f in files:
            if f.endswith(".py") and f != "env.py":
                used |= set(re.findall(r"env\.(?:flag|integer|text)\(\"(ZSE_[A-Z0-9_]+)\"", open(os.path.join(d, f)).read()))
    assert used and used <= set(env.KNOWN)


def test_bench_reference_arm_prints_its_unavailable_line():
    """`bench.py --impl reference` must print one JSON line with `impl` and `unavailable` and exit 0 on a machine where
    the reference cannot be timed (every workload of it is closed: see baseline/run_reference.py)."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for extra in ([], ["--workload", "single"], ["--gpus", "2"]):
        r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "2",
                            "--warmup", "1"] + extra, capture_output=True, text=True, timeout=120)
        assert r.returncode == 0, r.stderr[-2000:]
        line = json.loads(r.stdout.strip().splitlines()[-1])
        assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


def test_bench_repeats_itself_once_after_a_device_fault(monkeypatch):
    """bench.py's answer to a device fault in a single-GPU run: one fresh process, named in the result line; never a
    second one, never under a multi-rank launch."""
    import importlib.util
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    calls = []
    monkeypatch.setattr(os, "execv", lambda exe, argv: calls.append((exe, list(argv))))
    monkeypatch.delenv("ZSE_BENCH_RERUN", raising=False)
    monkeypatch.delenv("WORLD_SIZE", raising=False)
    bench.rerun_once_in_fresh_process(RuntimeError("engine step failed: req-1: CUDA error:\nunspecified launch failure"))
    assert len(calls) == 1 and calls[0][0] == sys.executable and calls[0][1][0] == sys.executable
    assert os.environ["ZSE_BENCH_RERUN"] == "engine step failed: req-1: CUDA error: unspecified launch failure"
    bench.rerun_once_in_fresh_process(RuntimeError("again"))             # already the repeat: no third process
    assert len(calls) == 1
    monkeypatch.delenv("ZSE_BENCH_RERUN")
    monkeypatch.setenv("WORLD_SIZE", "2")
    bench.rerun_once_in_fresh_process(RuntimeError("CUDA error"))        # ranks of a launcher do not re-exec
    assert len(calls) == 1
    monkeypatch.delenv("ZSE_BENCH_RERUN", raising=False)


def test_bench_defaults_follow_the_driver_contract(monkeypatch):
    """With no flags: one GPU, at least three warm-up steps, the headline workload on the 14B shape with 64 requests;
    the other workloads bring their own model and request count unless the caller names them."""
    import importlib.util
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_args_under_test", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    a = bench.parse_args()
    assert (a.gpus, a.impl, a.workload) == (1, "ours", "batch64") and a.warmup >= 3 and a.steps >= a.warmup
    assert a.model == "qwen2.5-14b" and a.requests == 64 and a.comm is None and not a.no_graphs
    monkeypatch.setattr(sys, "argv", ["bench.py", "--gpus", "8", "--steps", "7", "--warmup", "3", "--workload", "single"])
    a = bench.parse_args()
    assert (a.gpus, a.steps, a.warmup) == (8, 7, 3) and a.model == "qwen2.5-7b" and a.requests == 1
    monkeypatch.setattr(sys, "argv", ["bench.py", "--workload", "lora72b", "--requests", "160"])
    a = bench.parse_args()
    assert a.model == "qwen2.5-72b" and a.requests == 160
    assert set(bench.WORKLOADS) == {"batch64", "single", "spec32b", "lora72b"}
    assert bench.WORKLOADS["spec32b"]["spec_k"] == 4 and bench.WORKLOADS["batch64"]["spec_k"] == 0


def test_diagnostic_tools_describe_their_options_without_a_gpu():
    """`microbench` and `kernel_counters` parse their arguments before they touch a device: `--help` works anywhere and
    names the options the profile summaries use."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root)
    for module, options in (("zse_b200.runtime.microbench", ("--shape", "--tokens", "--only", "--kv-block", "--tp")),
                            ("zse_b200.runtime.kernel_counters", ("--shape", "--tokens", "--tp", "--kernel", "--kv-block"))):
        r = subprocess.run([sys.executable, "-m", module, "--help"], capture_output=True, text=True, timeout=120,
                           env=env, cwd=root)
        assert r.returncode == 0, r.stderr[-1500:]
        for opt in options:
            assert opt in r.stdout, (module, opt)
    r = subprocess.run([sys.executable, "-m", "zse_b200.runtime.kernel_counters", "--kernel", "nonsense"],
                       capture_output=True, text=True, timeout=120, env=env, cwd=root)
    assert r.returncode == 2 and "invalid choice" in r.stderr


def test_serve_leaves_with_a_non_zero_code_after_a_device_fault(monkeypatch, capsys):
    """`zse serve` watches the engine: once it reports a device fault the command prints it and returns 3, so that a
    supervisor starts a fresh process.  The server here is a stand-in whose engine "faults" after half a second."""
    import argparse
    import threading
    import time as _time

    import zse_b200.cli as cli
    import zse_b200.server.app as app

    class Engine:
        fatal_error = None

    class Server:
        def __init__(self, *a, **kw):
            self.engine = Engine()
            self.closed = False
            threading.Timer(0.5, lambda: setattr(self.engine, "fatal_error",
                                                  "RuntimeError: CUDA error: unspecified launch failure")).start()

        async def start(self):
            return None

        def close(self):
            self.closed = True

    made = []
    monkeypatch.setattr(app, "ZSEServer", lambda *a, **kw: made.append(Server()) or made[-1])
    monkeypatch.setattr(cli.signal, "signal", lambda *a: None)          # not the main thread's business in a test
    ns = argparse.Namespace(model=None, host="127.0.0.1", port=0, admin_key="adm", db_path=":memory:",
                            model_name="m", quiet=True, tp_size=1, max_seq_len=0, max_batch_seqs=4,
                            prefill_chunk_size=512, speculative_k=0, speculative_mode="ngram", no_graphs=False,
                            comm="fused", cpu=True, require_auth=False)
    t0 = _time.monotonic()
    rc = cli._cmd_serve(ns)
    assert rc == 3 and made[0].closed and 0.4 < _time.monotonic() - t0 < 10
    assert "device fault, shutting down" in capsys.readouterr().err

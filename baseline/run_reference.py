"""Reference arm of bench.py: the unmodified reference engine (installed under ``baseline/_ref``) on the same ``.zse``
model file and workload, through its own public API (``ZStreamerEngine.add_request_tokens`` + ``step``).

The headline workload (64 concurrent requests, prompts up to 2048 tokens plus 256 generated) is NOT run: by reading
the reference, its decode path keeps block tables in a fixed device buffer of 64 sequences x 256 blocks
(zse-engine/zse_engine/orchestrator/model_runner.py:96-103) while its KV block size for this model is 8 tokens
(zse-engine/zse_engine/cache/cache_manager.py:159-183), so any sequence past 2048 tokens makes the per-step block-table
upload (model_runner.py:879-881) write beyond that buffer.  That is an out-of-bounds device write, which must not be
provoked on shared GPUs; the arm reports ``unavailable`` instead.  The single-sequence workload (7B shape, 512-token
prompt, 256 new tokens - the case the reference publishes numbers for) stays inside every fixed buffer and is run.
"""
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def _unavailable(why: str) -> None:
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def run(args, model_file, workload, ClockSampler, baseline_tok_s, prompt_range, output_tokens) -> None:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 or args.gpus > 1:
        if int(os.environ.get("RANK", "0")) == 0:
            _unavailable("the reference's tensor-parallel engine decodes one sequence at a time (no batching, no "
                         "scheduler) and cannot express the 64-request continuous-batching workload")
        return
    if args.workload != "single":
        _unavailable("not run: sequences longer than 2048 tokens overflow the reference's fixed 64x256-entry decode "
                     "block-table buffer (block size 8) - an out-of-bounds device write found by reading "
                     "orchestrator/model_runner.py:96-103,879-881; use --workload single for a measured comparison")
        return
    if not os.path.isdir(os.path.join(REF, "zse_engine")):
        _unavailable("baseline/_ref is missing (install the reference with pip --target baseline/_ref)")
        return
    sys.path.insert(0, REF)
    try:
        from zse_engine.zstreamer.engine import ZStreamerEngine
        from zse_engine.zstreamer.scheduler import SchedulerConfig
    except Exception as exc:
        _unavailable(f"reference import failed: {type(exc).__name__}: {exc}")
        return
    path = model_file(args, 0, lambda: None)
    try:
        t0 = time.time()
        eng = ZStreamerEngine(model_path=path, scheduler_config=SchedulerConfig(max_batch_seqs=8), device_index=0,
                              max_seq_len=1024, quiet=True)
        cold = time.time() - t0
    except Exception as exc:
        _unavailable(f"reference engine failed to start on this GPU: {type(exc).__name__}: {str(exc)[:200]}")
        return
    vocab = eng._config.vocab_size
    prompt = workload(1, vocab, kind="single")[0]
    need = max(output_tokens, args.steps + args.warmup + 8)
    need = min(need, 1024 - len(prompt) - 8)
    steps = min(args.steps, need - args.warmup - 2)
    rid = eng.add_request_tokens(prompt, max_tokens=need, temperature=0.0, stop_tokens=[])
    generated = [0]

    def tokens_so_far() -> int:
        return eng._total_tokens

    try:
        guard = 0
        while tokens_so_far() < 1 and guard < 1000:      # prefill + first token
            eng.step()
            guard += 1
        for _ in range(args.warmup):
            eng.step()
        sampler = ClockSampler(0)
        n0 = tokens_so_far()
        t_start = time.perf_counter()
        for _ in range(steps):
            eng.step()
        eng._gpu_mem.synchronize() if hasattr(eng._gpu_mem, "synchronize") else None
        dt = time.perf_counter() - t_start
        clocks = sampler.stop()
        tokens = tokens_so_far() - n0
    except Exception as exc:
        _unavailable(f"reference engine failed while decoding: {type(exc).__name__}: {str(exc)[:200]}")
        return
    if tokens <= 0:
        _unavailable("reference engine produced no tokens in the timed region")
        return
    value = tokens / dt
    print(json.dumps({
        "impl": "reference", "metric": "INT4 Qwen2.5 decode tok/s (box, max over ranks)", "value": round(value, 2),
        "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup, "ms_per_step": round(dt * 1000 / steps, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": round(value / 48.6, 3), "dtype": "fp16",
        "data": "synthetic",
        "config": {"model": f"{args.model}-shaped INT4 group-128", "global_batch": 1,
                   "seq_len": "512-token prompt, 256 output tokens", "parallelism": "tp1", "workload": "single",
                   "timing": "host wall clock around ZStreamerEngine.step() (the reference synchronises every step)",
                   "baseline_note": "vs_baseline divides by the published 7B single-sequence rate on A10G (48.6 tok/s)"},
        "e2e": {"value": round(value, 2), "unit": "tok/s"}, "clocks": clocks,
        "extra": {"cold_start_s": round(cold, 2), "tokens": tokens}}), flush=True)

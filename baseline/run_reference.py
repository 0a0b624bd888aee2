"""Reference arm of bench.py.

The unmodified reference engine is installed under ``baseline/_ref`` (pip, --no-deps, from a copy of the reference
tree).  It is not run on the GPU any more:

* The headline workload (64 concurrent requests, prompts up to 2048 tokens plus 256 generated) was never run: by
  reading the reference, its decode path keeps block tables in a fixed device buffer of 64 sequences x 256 blocks
  (zse-engine/zse_engine/orchestrator/model_runner.py:96-103) while its KV block size for this model is 8 tokens
  (zse-engine/zse_engine/cache/cache_manager.py:159-183), so any sequence past 2048 tokens makes the per-step
  block-table upload (model_runner.py:879-881) write beyond that buffer: an out-of-bounds device write.
* The single-sequence workload (7B shape, 512-token prompt, 256 new tokens: the case the reference publishes numbers
  for) was run once through the reference's public API (``ZStreamerEngine.add_request`` + ``step``).  The engine
  started, and its first step failed inside the reference's own GPU code with CUDA error 700 (illegal address),
  reported by its next driver call as ``cuStreamCreate failed: 700``.  The record of that call is kept in
  ``profiles/reference_arm_single_sequence_fault.txt``.  The cause, found by reading afterwards: the logits scratch
  buffer has ``min(max_seq_len, 64)`` rows (zse-engine/zse_engine/orchestrator/vram_allocator.py:279-296) while
  prefill launches the lm_head matmul over all ``seq_len`` rows into it (orchestrator/model_runner.py:366-373), so
  every prompt longer than 64 tokens writes past the buffer.  A prompt of at most 64 tokens stays inside that buffer
  and inside the 64 x 256-entry decode block table, but the rest of that path (about twenty run-time-compiled kernels
  with hand-computed launch geometry, a gcc-compiled C launcher for single-sequence decode) has not been audited
  line by line, and after one recorded fault the reference's GPU code is not run again on shared GPUs without such
  an audit.
* ``add_request_tokens`` of the reference cannot be used at all: it stores the prompt as a ``set`` where its own
  ``add_token`` expects a ``dict`` (zstreamer/engine.py:485 vs zstreamer/request.py:164) and raises on the first
  generated token.
* Tensor-parallel runs: the reference's ``TPEngine`` decodes one sequence at a time (no batching, no scheduler) and
  its sharded lm_head reads past the shard (orchestrator/tensor_parallel.py:63, model_runner.py:368-373).

Every invocation therefore prints the ``unavailable`` line.  The published numbers of the reference (other hardware)
stay the comparison: ``vs_baseline`` in bench.py.
"""
import json
import os


def _unavailable(why: str) -> None:
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def run(args, model_file, workload, ClockSampler, baseline_tok_s, prompt_range, output_tokens) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 or args.gpus > 1:
        _unavailable("the reference's tensor-parallel engine decodes one sequence at a time (no batching, no "
                     "scheduler) and cannot express the 64-request continuous-batching workload")
    elif args.workload != "single":
        _unavailable("not run: sequences longer than 2048 tokens overflow the reference's fixed 64x256-entry decode "
                     "block-table buffer (block size 8) - an out-of-bounds device write found by reading "
                     "orchestrator/model_runner.py:96-103,879-881")
    else:
        _unavailable("not run again: on B200 the reference's own GPU code raised CUDA error 700 (illegal address) in "
                     "the first step of a 512-token prompt on the 7B shape (its logits scratch has min(S, 64) rows, "
                     "vram_allocator.py:279-296, but prefill writes seq_len rows of logits, model_runner.py:366-373); "
                     "record in profiles/reference_arm_single_sequence_fault.txt")

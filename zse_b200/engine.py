"""The two engines users talk to.

``ZStreamerEngine`` - continuous batching: ``add_request`` / ``add_request_tokens`` / ``cancel_request`` / ``step`` /
``run`` / ``stop`` / ``get_result`` / ``stats`` / ``lora_manager`` (zse-engine/zse_engine/zstreamer/engine.py:85-672).
``ZSEEngine`` - single-request convenience API: ``generate`` / ``stream_generate`` / ``generate_tokens`` / ``stats``
(zse-engine/zse_engine/orchestrator/engine.py:70-524); it is a thin layer over the streamer so both share one
code path.

Cold start: the file is memory-mapped, the small sections are parsed, weights are uploaded tensor by tensor and
re-tiled on the device, then step buffers and the KV cache are sized from what is left (``runtime.vram``).
"""
from __future__ import annotations

import dataclasses
import os

import sys
import threading
import time
from collections import deque
from dataclasses import dataclass
from typing import Callable, Dict, Iterator, List, Optional

import torch

from .cache.cache_manager import KVCacheManager
from .config import EngineConfig
from .format.loader import ZSELoader
from .models.decoder import DecoderModel
from .runtime.runner import ModelRunner
from .runtime.vram import VRAMAllocator
from .sched.batch_runner import BatchRunner, StepResult
from .sched.memory_budget import MemoryBudget
from .sched.request import FinishReason, GenerationParams, InferenceRequest, RequestOutput
from .sched.scheduler import Scheduler, SchedulerConfig
from .utils import env

CHAT_STOP_MARKERS = ("<|im_end|>", "<|im_start|>", "<|eot_id|>", "<end_of_turn>", "<|end|>")


@dataclass
class StreamerStats:
    total_requests: int
    total_tokens_generated: int
    total_steps: int
    uptime_s: float
    requests_per_sec: float
    tokens_per_sec: float
    avg_batch_size: float
    avg_ttft_ms: float
    avg_tpot_ms: float
    p50_ttft_ms: float
    p99_ttft_ms: float
    p50_tpot_ms: float
    queue_depth: int
    active_requests: int
    memory_utilization: float


def _percentile(samples, q: float) -> float:
    if not samples:
        return 0.0
    s = sorted(samples)
    return float(s[min(len(s) - 1, int(q * (len(s) - 1) + 0.5))])


class ZStreamerEngine:
    def __init__(self, model_path: str, scheduler_config: Optional[SchedulerConfig] = None, device_index: int = 0,
                 max_seq_len: int = 0, headroom_ratio: float = 0.5, quiet: bool = True,
                 config: Optional[EngineConfig] = None, comm=None, tp_rank: int = 0):
        cfg = config or EngineConfig(device_index=device_index, max_seq_len=max_seq_len,
                                     headroom_ratio=headroom_ratio, quiet=quiet)
        if scheduler_config is not None:
            for name in ("max_batch_tokens", "max_batch_seqs", "max_prefill_per_step", "prefill_chunk_size",
                         "decode_per_prefill", "enable_preemption", "speculative_k", "max_queue_size"):
                setattr(cfg, name, getattr(scheduler_config, name))
            cfg.speculative_mode = getattr(scheduler_config, "speculative_mode", cfg.speculative_mode)
        self.config = cfg
        self._quiet = cfg.quiet
        self._running = False
        self._start_time: Optional[float] = None
        self._request_counter = 0
        self._lock = threading.Lock()
        self._step_lock = threading.RLock()        # one user of the model runner at a time (steps, embeddings)
        self._total_requests = self._total_tokens = self._total_steps = 0
        self._ttft_samples: deque = deque(maxlen=10000)
        self._tpot_samples: deque = deque(maxlen=10000)
        self._completed: Dict[str, RequestOutput] = {}
        self._completed_maxlen = 10000
        self.init_times: Dict[str, float] = {}

        t0 = time.monotonic()
        on_gpu = torch.cuda.is_available() and cfg.device != "cpu"
        self.device = torch.device(f"cuda:{cfg.device_index}" if on_gpu else "cpu")
        if on_gpu:
            torch.cuda.set_device(self.device)
        self._loader = ZSELoader(model_path, int4_layout=cfg.int4_layout)
        self._config = self._loader.config
        self._tokenizer = self._loader.tokenizer
        self.init_times["open"] = time.monotonic() - t0

        t1 = time.monotonic()
        self._model = DecoderModel.from_loader(self._loader, self.device, tp_size=cfg.tp_size, rank=tp_rank)
        self._model.comm = comm
        if on_gpu:
            torch.cuda.synchronize(self.device)
        self.init_times["weights"] = time.monotonic() - t1
        self.init_times.update(self._model.load_stats)

        t2 = time.monotonic()
        mc = self._config
        self._max_seq_len = min(cfg.max_seq_len or mc.max_seq_len, mc.max_seq_len, 32768)
        block_size = cfg.block_size or KVCacheManager._auto_block_size(mc)
        nkv_local = self._model.plan.num_kv_heads
        if cfg.kv_blocks > 0:
            blocks = cfg.kv_blocks
        elif on_gpu:
            scratch_est = cfg.max_batch_tokens * (mc.hidden_size * 40 + mc.intermediate_size * 2) + (256 << 20)
            plan = VRAMAllocator.for_device(self.device).plan_allocation(
                mc, 0, scratch_est, block_size, self._max_seq_len, cfg.max_batch_seqs, cfg.tp_size, cfg.kv_fraction)
            blocks = plan.kv_blocks
            self.vram_plan = plan
        else:
            blocks = max(64, (cfg.max_batch_seqs * min(self._max_seq_len, 2048)) // block_size)
        self._kv_cache = KVCacheManager(mc, self.device, block_size=block_size, num_blocks=blocks,
                                        eviction_policy=cfg.eviction_policy, enable_dedup=cfg.enable_prefix_cache,
                                        num_kv_heads=nkv_local)
        self._runner = ModelRunner(self._model, self._kv_cache, max_batch_seqs=cfg.max_batch_seqs,
                                   max_tokens_per_pass=max(cfg.max_batch_tokens, cfg.prefill_chunk_size or 0),
                                   max_seq_len=self._max_seq_len, use_graphs=cfg.use_cuda_graphs)
        from .lora.manager import LoRAManager
        self._lora_manager = LoRAManager(self._model, self.device)
        self._budget = MemoryBudget(blocks, block_size, cfg.headroom_ratio)
        self._sched_config = SchedulerConfig(cfg.max_batch_tokens, cfg.max_batch_seqs, cfg.max_prefill_per_step,
                                             cfg.prefill_chunk_size, cfg.decode_per_prefill, cfg.enable_preemption,
                                             cfg.speculative_k, cfg.max_queue_size, cfg.speculative_mode)
        self._scheduler = Scheduler(self._sched_config, self._budget)
        spec = None
        if cfg.speculative_k > 0:
            from .sched.spec_runner import SpeculativeRunner
            spec = SpeculativeRunner(self._runner, k=cfg.speculative_k, mode=cfg.speculative_mode,
                                     vocab_size=mc.vocab_size)
        self._spec_runner = spec
        pipeline = cfg.pipeline_decode
        if pipeline is None:
            pipeline = env.flag("ZSE_PIPELINE_DECODE")
        self._batch_runner = BatchRunner(self._runner, self._scheduler, spec_runner=spec,
                                         lora_manager=self._lora_manager, pipeline_decode=pipeline)
        self.init_times["runtime"] = time.monotonic() - t2
        self.init_times["total"] = time.monotonic() - t0
        if not self._quiet:
            print(f"[zse] ready in {self.init_times['total']:.2f}s (open {self.init_times['open']:.2f}, weights "
                  f"{self.init_times['weights']:.2f}, runtime {self.init_times['runtime']:.2f}); "
                  f"{self._kv_cache.summary()}", file=sys.stderr)

    # ---- public API -------------------------------------------------------------------------------------
    @property
    def tokenizer(self):
        return self._tokenizer

    @property
    def model_config(self):
        return self._config

    @property
    def lora_manager(self):
        return self._lora_manager

    @property
    def runner(self) -> ModelRunner:
        return self._runner

    @property
    def kv_cache(self) -> KVCacheManager:
        return self._kv_cache

    @property
    def scheduler(self) -> Scheduler:
        return self._scheduler

    def default_stop_tokens(self) -> List[int]:
        stops: List[int] = []
        tok = self._tokenizer
        if tok is None:
            return stops
        eos = tok.special_tokens.eos_id
        if eos is not None:
            # a tiny id in a large vocabulary is usually the default of a file without an end marker (the reference's
            # rule) - unless the token at that id says that it is one (Gemma's <eos> is id 1 of 256000)
            text = str(getattr(tok, "_id_to_token", {}).get(eos, "")).lower()
            named = any(k in text for k in ("eos", "</s>", "endoftext", "end_of_text", "end_of_sentence"))
            if named or not (self._config.vocab_size > 50000 and eos < 100):
                stops.append(eos)
        for marker in CHAT_STOP_MARKERS:
            tid = tok.token_to_id(marker)
            if tid is not None and tid not in stops:
                stops.append(tid)
        return stops

    def add_request(self, prompt: str, max_tokens: int = 128, temperature: float = 1.0, top_p: float = 0.9,
                    top_k: int = 50, repetition_penalty: float = 1.0, stop_tokens: Optional[List[int]] = None,
                    priority: int = 0, deadline_ms: Optional[float] = None,
                    on_token: Optional[Callable[[int], None]] = None,
                    on_finish: Optional[Callable[[RequestOutput], None]] = None, seed: Optional[int] = None,
                    lora_id: Optional[str] = None, add_bos: bool = True) -> Optional[str]:
        if self._tokenizer is None:
            raise RuntimeError("this model file has no tokenizer; use add_request_tokens")
        ids = self._tokenizer.encode(prompt, add_bos=add_bos)
        return self.add_request_tokens(ids, max_tokens=max_tokens, temperature=temperature, top_p=top_p, top_k=top_k,
                                       repetition_penalty=repetition_penalty, stop_tokens=stop_tokens,
                                       priority=priority, deadline_ms=deadline_ms, on_token=on_token,
                                       on_finish=on_finish, seed=seed, lora_id=lora_id)

    def add_request_tokens(self, token_ids: List[int], request_id: Optional[str] = None, max_tokens: int = 128,
                           temperature: float = 1.0, top_p: float = 0.9, top_k: int = 50,
                           repetition_penalty: float = 1.0, stop_tokens: Optional[List[int]] = None,
                           priority: int = 0, deadline_ms: Optional[float] = None, on_token=None, on_finish=None,
                           seed: Optional[int] = None, lora_id: Optional[str] = None,
                           timeout_ms: Optional[float] = None) -> Optional[str]:
        if len(token_ids) == 0:
            raise ValueError("empty prompt")
        if len(token_ids) >= self._max_seq_len:
            raise ValueError(f"prompt length {len(token_ids)} exceeds max_seq_len {self._max_seq_len}")
        if lora_id is not None and not self._lora_manager.is_loaded(lora_id):
            raise ValueError(f"LoRA adapter '{lora_id}' is not loaded")
        max_tokens = max(1, min(max_tokens, self._max_seq_len - len(token_ids)))
        if stop_tokens is None:
            stop_tokens = self.default_stop_tokens()
        with self._lock:
            self._request_counter += 1
            rid = request_id or f"req-{self._request_counter}"
        req = InferenceRequest(rid, list(token_ids),
                               GenerationParams(max_tokens, temperature, top_p, top_k, repetition_penalty,
                                                list(stop_tokens), seed, timeout_ms, lora_id),
                               priority=priority, deadline_ms=deadline_ms, on_token=on_token, on_finish=on_finish,
                               past_tokens=self._count(token_ids) if repetition_penalty != 1.0 else {})
        if not self._scheduler.add_request(req):
            return None
        with self._lock:
            self._total_requests += 1
        return rid

    @staticmethod
    def _count(ids) -> Dict[int, int]:
        d: Dict[int, int] = {}
        for t in ids:
            d[t] = d.get(t, 0) + 1
        return d

    def cancel_request(self, request_id: str) -> None:
        r = self._scheduler.cancel_request(request_id)
        if r is not None:                       # cancelled while waiting: no step will report it
            out = RequestOutput.from_request(r)
            with self._lock:
                self._completed[out.request_id] = out
            if r.on_finish is not None:
                r.on_finish(out)

    def step(self) -> StepResult:
        """One scheduling + execution iteration; returns what happened (idle steps return an empty result)."""
        if self._start_time is None:
            self._start_time = time.monotonic()
        with self._step_lock:
            plan = self._scheduler.schedule_step()
            res = self._batch_runner.execute(plan)
        with self._lock:
            if not plan.is_idle:
                self._total_steps += 1
            self._total_tokens += res.tokens_generated
            for out in res.finished:
                if out.finish_reason not in (FinishReason.CANCELLED, FinishReason.ERROR) and out.output_tokens:
                    self._ttft_samples.append(out.ttft_ms)
                    if len(out.output_tokens) > 1:
                        self._tpot_samples.append(out.tpot_ms)
                self._completed[out.request_id] = out
                if len(self._completed) > self._completed_maxlen:
                    self._completed.pop(next(iter(self._completed)))
        res.idle = plan.is_idle and not res.finished
        return res

    # ---- model access for retrieval (between steps of the serving loop) -----------------------------------
    def embed_tokens(self, tokens: List[int]):
        """Mean-pooled, L2-normalised final hidden state of ``tokens`` (fp32 host tensor)."""
        limit = min(self._runner.max_tokens, self._max_seq_len - 1)
        with self._step_lock:
            if self.device.type == "cuda":
                torch.cuda.set_device(self.device)
            return self._runner.embed_pooled(list(tokens)[:limit])

    def last_token_logits(self, tokens: List[int]):
        """fp32 host logits after the last of ``tokens``."""
        limit = min(self._runner.max_tokens, self._max_seq_len - 1)
        with self._step_lock:
            if self.device.type == "cuda":
                torch.cuda.set_device(self.device)
            return self._runner.last_logits(list(tokens)[-limit:])

    def has_work(self) -> bool:
        return self._scheduler.num_active > 0 or self._scheduler.num_waiting > 0

    @property
    def fatal_error(self) -> Optional[str]:
        """The device fault that ended this process's CUDA context, if there was one (None while the engine is
        healthy).  Requests submitted afterwards finish with an error; the server's health route reports it so that a
        supervisor can restart the worker."""
        return self._batch_runner.fatal_error

    def run(self, idle_sleep_ms: float = 1.0, idle_sleep_s: Optional[float] = None) -> None:
        """Serving loop (call from a dedicated thread); returns after ``stop()``.  ``idle_sleep_ms`` as in the
        reference (zse-engine/zse_engine/zstreamer/engine.py:541); ``idle_sleep_s`` overrides it."""
        if idle_sleep_s is None:
            idle_sleep_s = idle_sleep_ms / 1000.0
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        self._running = True
        self._start_time = self._start_time or time.monotonic()
        while self._running:
            res = self.step()
            if getattr(res, "idle", False):
                time.sleep(idle_sleep_s)

    def run_until_done(self, max_steps: int = 10_000_000) -> int:
        n = 0
        while self.has_work() and n < max_steps:
            self.step()
            n += 1
        self.step()        # collect the last finished requests
        return n

    def stop(self) -> None:
        self._running = False

    def is_running(self) -> bool:
        return self._running

    def get_result(self, request_id: str) -> Optional[RequestOutput]:
        with self._lock:
            return self._completed.pop(request_id, None)

    def stats(self) -> StreamerStats:
        with self._lock:
            up = time.monotonic() - self._start_time if self._start_time else 0.0
            ss = self._scheduler.stats()
            avg = lambda d: sum(d) / len(d) if d else 0.0
            return StreamerStats(self._total_requests, self._total_tokens, self._total_steps, up,
                                 self._total_requests / up if up > 0 else 0.0,
                                 self._total_tokens / up if up > 0 else 0.0,
                                 self._total_tokens / self._total_steps if self._total_steps else 0.0,
                                 avg(self._ttft_samples), avg(self._tpot_samples),
                                 _percentile(self._ttft_samples, 0.5), _percentile(self._ttft_samples, 0.99),
                                 _percentile(self._tpot_samples, 0.5), ss["num_waiting"], ss["num_active"],
                                 ss["memory"]["utilization"])

    def summary(self) -> str:
        s = self.stats()
        return (f"engine: up {s.uptime_s:.1f}s, {s.total_requests} requests ({s.requests_per_sec:.1f}/s), "
                f"{s.total_tokens_generated} tokens ({s.tokens_per_sec:.1f}/s), batch {s.avg_batch_size:.1f}, TTFT "
                f"p50 {s.p50_ttft_ms:.1f} ms p99 {s.p99_ttft_ms:.1f} ms, TPOT p50 {s.p50_tpot_ms:.2f} ms, queue "
                f"{s.queue_depth}, active {s.active_requests}, memory {s.memory_utilization:.1%}")

    def scheduler_summary(self) -> str:
        return self._scheduler.summary()

    def destroy(self) -> None:
        self.stop()
        runner = getattr(self, "_runner", None)
        if runner is not None:
            runner.release_graphs()
        comm = getattr(getattr(self, "_model", None), "comm", None)
        if comm is not None and hasattr(comm, "close"):
            comm.close()
        for name in ("_kv_cache",):
            obj = getattr(self, name, None)
            if obj is not None:
                obj.destroy()
        loader = getattr(self, "_loader", None)
        if loader is not None:
            loader.close()

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.destroy()


@dataclass
class GenerateConfig:
    """Sampling settings of one request; defaults as in the reference (zse-engine/zse_engine/orchestrator/engine.py:38-46)."""
    max_tokens: int = 128
    temperature: float = 1.0
    top_p: float = 0.9
    top_k: int = 50
    repetition_penalty: float = 1.0
    stop_tokens: Optional[List[int]] = None
    seed: Optional[int] = None


@dataclass
class EngineStats:
    """Statistics of ``ZSEEngine``: the last request (first block) and the engine as a whole (second block, the fields
    of the reference's ``EngineStats``, zse-engine/zse_engine/orchestrator/engine.py:49-68; ``kernel_compile_time_s``
    is 0 because the kernels are compiled ahead of time)."""
    prompt_tokens: int = 0
    generated_tokens: int = 0
    ttft_ms: float = 0.0
    total_ms: float = 0.0
    tokens_per_sec: float = 0.0
    decode_tokens_per_sec: float = 0.0
    model_path: str = ""
    model_arch: str = ""
    device_name: str = ""
    vram_total_gb: float = 0.0
    weight_load_time_s: float = 0.0
    kernel_compile_time_s: float = 0.0
    total_init_time_s: float = 0.0
    total_tokens_generated: int = 0
    total_prefill_tokens: int = 0
    total_generate_time_s: float = 0.0
    avg_tokens_per_sec: float = 0.0
    weight_bytes: int = 0
    kv_cache_bytes: int = 0
    scratch_bytes: int = 0


class ZSEEngine:
    """One request at a time, with the call signatures of the reference's ``ZSEEngine``
    (zse-engine/zse_engine/orchestrator/engine.py:70-524): ``generate(prompt, max_tokens=..., temperature=..., ...)``
    (text in, text out), ``stream_generate`` (iterator of text pieces), ``generate_tokens`` (ids in, generated ids
    out), ``stream_generate_tokens`` (iterator of ids).  A ``GenerateConfig`` may be passed instead of the keywords
    (second positional argument or ``config=``)."""

    def __init__(self, model_path: str, device_index: int = 0, max_seq_len: int = 0, quiet: bool = True,
                 config: Optional[EngineConfig] = None):
        cfg = config or EngineConfig(device_index=device_index, max_seq_len=max_seq_len, quiet=quiet,
                                     max_batch_seqs=8, max_batch_tokens=2048)
        self._model_path = model_path
        self._streamer = ZStreamerEngine(model_path, config=cfg)
        self._last = EngineStats()
        self._total_tokens = self._total_prefill = 0
        self._total_gen_time = 0.0

    @property
    def streamer(self) -> ZStreamerEngine:
        return self._streamer

    @property
    def tokenizer(self):
        return self._streamer.tokenizer

    @property
    def config(self):
        """The model's configuration (``ModelConfig``)."""
        return self._streamer.model_config

    @property
    def device(self):
        """``DeviceInfo`` of the GPU the engine runs on (None on the CPU path)."""
        if self._streamer.device.type != "cuda":
            return None
        from .runtime.device import get_devices
        devs = get_devices()
        idx = self._streamer.device.index or 0
        return devs[idx] if idx < len(devs) else None

    @staticmethod
    def _settings(max_tokens, temperature, top_p, top_k, repetition_penalty, stop_tokens, seed,
                  config) -> GenerateConfig:
        if isinstance(max_tokens, GenerateConfig):       # generate(prompt, GenerateConfig(...))
            config = max_tokens
        if config is not None:
            return dataclasses.replace(config)
        return GenerateConfig(int(max_tokens), float(temperature), float(top_p), int(top_k), float(repetition_penalty),
                              None if stop_tokens is None else list(stop_tokens), seed)

    def _run(self, prompt_tokens: List[int], g: GenerateConfig, on_token=None) -> Iterator[int]:
        """Submits the request and drives the engine on the calling thread, yielding tokens as they are produced."""
        t0 = time.monotonic()
        fresh: List[int] = []

        def got(tok: int) -> None:
            fresh.append(tok)
            if on_token is not None:
                on_token(tok)

        rid = self._streamer.add_request_tokens(prompt_tokens, max_tokens=g.max_tokens, temperature=g.temperature,
                                                top_p=g.top_p, top_k=g.top_k, repetition_penalty=g.repetition_penalty,
                                                stop_tokens=g.stop_tokens, seed=g.seed, on_token=got)
        if rid is None:
            raise RuntimeError("request queue is full")
        try:
            while self._streamer.has_work():
                self._streamer.step()
                while fresh:
                    yield fresh.pop(0)
            self._streamer.step()
            while fresh:
                yield fresh.pop(0)
        finally:
            if self._streamer.has_work():                # the consumer stopped early: do not leave the request running
                self._streamer.cancel_request(rid)
                self._streamer.run_until_done()
            out = self._streamer.get_result(rid)
            total = (time.monotonic() - t0) * 1000
            if out is not None:
                n = len(out.output_tokens)
                self._total_tokens += n
                self._total_prefill += len(prompt_tokens)
                self._total_gen_time += total / 1000
                self._last = dataclasses.replace(
                    self.stats(), prompt_tokens=len(prompt_tokens), generated_tokens=n, ttft_ms=out.ttft_ms,
                    total_ms=total, tokens_per_sec=n / (total / 1000) if total else 0.0,
                    decode_tokens_per_sec=(n - 1) / ((total - out.ttft_ms) / 1000)
                    if n > 1 and total > out.ttft_ms else 0.0)
        if out is None or out.finish_reason == FinishReason.ERROR:
            raise RuntimeError(f"generation failed: {out.error if out else 'no result'}")

    def generate_tokens(self, token_ids: List[int], max_tokens=128, temperature: float = 1.0, top_p: float = 0.9,
                        top_k: int = 50, repetition_penalty: float = 1.0, stop_tokens: Optional[List[int]] = None,
                        seed: Optional[int] = None, config: Optional[GenerateConfig] = None,
                        on_token: Optional[Callable[[int], None]] = None) -> List[int]:
        """Generated token ids for a prompt given as ids."""
        g = self._settings(max_tokens, temperature, top_p, top_k, repetition_penalty, stop_tokens, seed, config)
        return list(self._run(list(token_ids), g, on_token))

    def stream_generate_tokens(self, prompt: str, max_tokens=128, temperature: float = 1.0, top_p: float = 0.9,
                               top_k: int = 50, repetition_penalty: float = 1.0,
                               stop_tokens: Optional[List[int]] = None, seed: Optional[int] = None,
                               config: Optional[GenerateConfig] = None) -> Iterator[int]:
        """Yields generated token ids one at a time."""
        g = self._settings(max_tokens, temperature, top_p, top_k, repetition_penalty, stop_tokens, seed, config)
        if g.stop_tokens is None:
            g.stop_tokens = self._streamer.default_stop_tokens()
        return self._run(self.tokenizer.encode(prompt), g)

    def generate(self, prompt: str, max_tokens=128, temperature: float = 1.0, top_p: float = 0.9, top_k: int = 50,
                 repetition_penalty: float = 1.0, stop_tokens: Optional[List[int]] = None,
                 seed: Optional[int] = None, config: Optional[GenerateConfig] = None) -> str:
        """Generated text (stop tokens removed)."""
        g = self._settings(max_tokens, temperature, top_p, top_k, repetition_penalty, stop_tokens, seed, config)
        if g.stop_tokens is None:
            g.stop_tokens = self._streamer.default_stop_tokens()
        stops = set(g.stop_tokens or [])
        ids = list(self._run(self.tokenizer.encode(prompt), g))
        return self.tokenizer.decode([t for t in ids if t not in stops])

    def stream_generate(self, prompt: str, max_tokens=128, temperature: float = 1.0, top_p: float = 0.9,
                        top_k: int = 50, repetition_penalty: float = 1.0, stop_tokens: Optional[List[int]] = None,
                        seed: Optional[int] = None, config: Optional[GenerateConfig] = None) -> Iterator[str]:
        """Yields decoded text increments (a piece is held back while it ends inside a multi-byte character)."""
        g = self._settings(max_tokens, temperature, top_p, top_k, repetition_penalty, stop_tokens, seed, config)
        if g.stop_tokens is None:
            g.stop_tokens = self._streamer.default_stop_tokens()
        stops = set(g.stop_tokens or [])
        tok = self.tokenizer
        emitted: List[int] = []
        text_so_far = ""
        for t in self._run(tok.encode(prompt), g):
            if t in stops:
                continue
            emitted.append(t)
            text = tok.decode(emitted)
            if not text.endswith("\ufffd") and len(text) > len(text_so_far):
                yield text[len(text_so_far):]
                text_so_far = text
        text = tok.decode(emitted)
        if len(text) > len(text_so_far):
            yield text[len(text_so_far):]

    def stats(self) -> EngineStats:
        s = self._streamer
        times = s.init_times
        dev = self.device
        kv = s.kv_cache
        return dataclasses.replace(
            self._last, model_path=self._model_path, model_arch=s.model_config.arch,
            device_name=dev.name if dev is not None else "cpu",
            vram_total_gb=(dev.total_memory / 2 ** 30) if dev is not None else 0.0,
            weight_load_time_s=float(times.get("weights", 0.0)), kernel_compile_time_s=0.0,
            total_init_time_s=float(times.get("total", 0.0)), total_tokens_generated=self._total_tokens,
            total_prefill_tokens=self._total_prefill, total_generate_time_s=self._total_gen_time,
            avg_tokens_per_sec=self._total_tokens / self._total_gen_time if self._total_gen_time > 0 else 0.0,
            weight_bytes=int(getattr(s.runner.model, "weight_bytes", 0)),
            kv_cache_bytes=int(kv.num_total_blocks * kv.stats().block_bytes), scratch_bytes=int(s.runner.buf.nbytes()))

    def summary(self) -> str:
        s = self.stats()
        return (f"ZSE engine summary:\n  model: {s.model_arch} ({s.model_path})\n"
                f"  device: {s.device_name} ({s.vram_total_gb:.1f} GB)\n"
                f"  init: {s.total_init_time_s:.2f}s (weights {s.weight_load_time_s:.2f}s)\n"
                f"  memory: weights {s.weight_bytes / 2 ** 20:.1f} MB, kv {s.kv_cache_bytes / 2 ** 20:.1f} MB, "
                f"scratch {s.scratch_bytes / 2 ** 20:.1f} MB\n"
                f"  generated: {s.total_tokens_generated} tokens, {s.avg_tokens_per_sec:.1f} tok/s")

    def destroy(self) -> None:
        self._streamer.destroy()

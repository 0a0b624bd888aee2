"""Iteration-level scheduler of the continuous-batching engine.

Policy of zse-engine/zse_engine/zstreamer/scheduler.py:35-473: a token budget and a sequence cap per step, gradual
admission (``max_prefill_per_step``), one prefill turn every ``decode_per_prefill + 1`` steps while sequences are
decoding, admission through the memory budget, preemption of the lowest-priority / least-advanced decoders when no
blocks are left and requests are waiting, back-pressure through a bounded queue.

What is done differently, on purpose:
* a request whose prompt is longer than ``prefill_chunk_size`` keeps being scheduled, chunk after chunk, until its
  prompt is in the cache (the reference schedules only the first chunk: later chunks are never popped because only
  the queue heaps feed ``_schedule_prefill``, scheduler.py:262-327);
* continuing chunks go before new admissions, so a long prompt cannot be starved by short ones;
* a preempted request gives its KV blocks back and later re-prefills prompt + generated tokens.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass, field
from enum import Enum, auto
from typing import Dict, List

from .memory_budget import MemoryBudget
from .queue import RequestQueue
from .request import FinishReason, InferenceRequest, RequestState


class StepType(Enum):
    PREFILL = auto()
    DECODE = auto()
    MIXED = auto()
    IDLE = auto()


@dataclass
class SchedulerOutput:
    step_type: StepType
    prefill_requests: List[InferenceRequest] = field(default_factory=list)
    prefill_chunk_sizes: List[int] = field(default_factory=list)
    decode_requests: List[InferenceRequest] = field(default_factory=list)
    preempt_requests: List[InferenceRequest] = field(default_factory=list)
    finished_requests: List[InferenceRequest] = field(default_factory=list)

    @property
    def num_prefill_tokens(self) -> int:
        return sum(self.prefill_chunk_sizes)

    @property
    def num_decode_tokens(self) -> int:
        return len(self.decode_requests)

    @property
    def total_tokens(self) -> int:
        return self.num_prefill_tokens + self.num_decode_tokens

    @property
    def is_idle(self) -> bool:
        return self.step_type == StepType.IDLE


@dataclass
class SchedulerConfig:
    max_batch_tokens: int = 4096
    max_batch_seqs: int = 64
    max_prefill_per_step: int = 2
    prefill_chunk_size: int = 512
    decode_per_prefill: int = 4
    enable_preemption: bool = True
    speculative_k: int = 0
    max_queue_size: int = 256
    speculative_mode: str = "ngram"      # "ngram" | "self"


class Scheduler:
    def __init__(self, config: SchedulerConfig, memory_budget: MemoryBudget):
        self._config = config
        self._budget = memory_budget
        self._queue = RequestQueue(config.max_queue_size)
        self._lock = threading.Lock()
        self._active: Dict[str, InferenceRequest] = {}
        self._step_counter = 0
        self._seq_id_counter = 0
        self._totals = {"steps": 0, "prefill_steps": 0, "decode_steps": 0, "preemptions": 0, "finished": 0}

    @property
    def config(self) -> SchedulerConfig:
        return self._config

    def _next_seq_id(self) -> int:
        self._seq_id_counter += 1
        return self._seq_id_counter - 1

    # ---- intake -----------------------------------------------------------------------------------------
    def add_request(self, request: InferenceRequest) -> bool:
        return self._queue.add(request)

    def cancel_request(self, request_id: str):
        """A waiting request leaves the queue at once and is returned (it will never be part of a step, so the
        caller reports its result); an active one is marked and leaves with the next step."""
        r = self._queue.cancel(request_id)
        if r is not None:
            return r
        with self._lock:
            r = self._active.get(request_id)
            if r is not None and not r.is_finished:
                r.mark_cancelled()

    # ---- one step ---------------------------------------------------------------------------------------
    def schedule_step(self) -> SchedulerOutput:
        with self._lock:
            return self._schedule_locked()

    def _schedule_locked(self) -> SchedulerOutput:
        cfg = self._config
        self._totals["steps"] += 1
        self._step_counter += 1
        out = SchedulerOutput(StepType.IDLE, finished_requests=self._collect_finished(),
                              preempt_requests=self._handle_preemption())
        decoding = [r for r in self._active.values() if r.state == RequestState.DECODING]
        prefilling = [r for r in self._active.values() if r.state == RequestState.PREFILLING]
        has_prefill_work = bool(prefilling) or not self._queue.is_empty
        prefill_turn = self._step_counter % (cfg.decode_per_prefill + 1) == 0
        if decoding and has_prefill_work:
            if prefill_turn:
                self._schedule_prefill(out, prefilling)
                left = cfg.max_batch_tokens - out.num_prefill_tokens
                if left > 0:
                    self._schedule_decode(out, decoding, left)
            else:
                self._schedule_decode(out, decoding, cfg.max_batch_tokens)
        elif decoding:
            self._schedule_decode(out, decoding, cfg.max_batch_tokens)
        elif has_prefill_work:
            self._schedule_prefill(out, prefilling)
            if out.prefill_requests:
                self._step_counter = 0
        if out.prefill_requests and out.decode_requests:
            out.step_type = StepType.MIXED
        elif out.prefill_requests:
            out.step_type = StepType.PREFILL
        elif out.decode_requests:
            out.step_type = StepType.DECODE
        if out.prefill_requests:
            self._totals["prefill_steps"] += 1
        if out.decode_requests:
            self._totals["decode_steps"] += 1
        return out

    def _collect_finished(self) -> List[InferenceRequest]:
        done = [r for r in self._active.values() if r.is_finished]
        for r in done:
            del self._active[r.request_id]
            self._budget.release(r.request_id)
            self._queue.remove_finished(r.request_id)
            self._totals["finished"] += 1
        return done

    def _chunk_for(self, r: InferenceRequest, tokens_left: int) -> int:
        n = r.remaining_prefill
        if self._config.prefill_chunk_size > 0:
            n = min(n, self._config.prefill_chunk_size)
        return min(n, tokens_left)

    def _schedule_prefill(self, out: SchedulerOutput, prefilling: List[InferenceRequest]) -> None:
        cfg = self._config
        tokens_left = cfg.max_batch_tokens
        # 1. requests in the middle of a chunked prefill continue first
        for r in sorted(prefilling, key=lambda r: (r.urgency, -r.priority, r.arrival_time)):
            if tokens_left <= 0:
                break
            n = self._chunk_for(r, tokens_left)
            if n > 0:
                out.prefill_requests.append(r)
                out.prefill_chunk_sizes.append(n)
                tokens_left -= n
        # 2. new admissions
        admitted = 0
        rejected: List[InferenceRequest] = []
        while admitted < cfg.max_prefill_per_step and tokens_left > 0 and len(self._active) < cfg.max_batch_seqs:
            r = self._queue.pop_next()
            if r is None:
                break
            if not self._budget.fits_at_all(r):
                r.error = "request needs more KV blocks than the cache has"
                r.mark_finished(FinishReason.ERROR)
                out.finished_requests.append(r)
                continue
            if not self._budget.can_admit(r) and self._active:
                rejected.append(r)
                break
            # with nothing else running the request is admitted even if its head-room estimate does not fit: it
            # passed fits_at_all, and waiting for memory that nobody holds would never end
            if r.seq_id is None:
                r.seq_id = self._next_seq_id()
            self._budget.reserve(r)
            r.mark_prefilling()
            self._active[r.request_id] = r
            n = self._chunk_for(r, tokens_left)
            out.prefill_requests.append(r)
            out.prefill_chunk_sizes.append(n)
            tokens_left -= n
            admitted += 1
        for r in rejected:
            self._queue.push_back(r)

    def _schedule_decode(self, out: SchedulerOutput, decoding: List[InferenceRequest], max_tokens: int) -> None:
        per_seq = 1 + max(0, self._config.speculative_k)
        cap = min(self._config.max_batch_seqs, max(1, max_tokens // per_seq))
        decoding.sort(key=lambda r: (r.urgency, -r.priority))
        out.decode_requests.extend(decoding[:cap])

    def _handle_preemption(self) -> List[InferenceRequest]:
        if not self._config.enable_preemption or self._queue.is_empty or self._budget.available_blocks > 0:
            return []
        decoding = [r for r in self._active.values() if r.state == RequestState.DECODING]
        if len(decoding) <= 1:
            return []
        waiting = [r for r in self._queue.peek_waiting() if r.state == RequestState.WAITING]
        if not waiting:
            return []
        # only preempt for someone more important than the victim
        best_waiting = max(r.priority for r in waiting)
        decoding.sort(key=lambda r: (r.priority, r.num_generated))
        target = self._budget._tokens_to_blocks(min(r.prompt_len for r in waiting)) + 2
        freed, victims = 0, []
        for r in decoding:
            if freed >= target or r.priority >= best_waiting:
                break
            freed += self._budget._tokens_to_blocks(r.total_tokens)
            r.mark_preempted()
            r.prefill_offset = 0
            self._budget.release(r.request_id)
            del self._active[r.request_id]
            self._queue.add_preempted(r)
            victims.append(r)
            self._totals["preemptions"] += 1
        return victims

    # ---- feedback from the batch runner -------------------------------------------------------------------
    def on_prefill_complete(self, request: InferenceRequest, chunk_tokens: int = 0) -> None:
        request.prefill_offset += chunk_tokens if chunk_tokens > 0 else request.remaining_prefill
        if request.remaining_prefill <= 0 and request.state == RequestState.PREFILLING:
            request.mark_decoding()

    def on_token_generated(self, request: InferenceRequest, token_id: int) -> None:
        request.add_token(token_id)
        self._budget.update_decode_progress(request.request_id, request.num_generated)
        reason = request.should_stop()
        if reason is not None and not request.is_finished:
            request.mark_finished(reason)

    def on_request_error(self, request: InferenceRequest, error: str) -> None:
        request.error = error
        if not request.is_finished:
            request.mark_finished(FinishReason.ERROR)

    # ---- facts ------------------------------------------------------------------------------------------
    @property
    def num_active(self) -> int:
        return len(self._active)

    @property
    def num_waiting(self) -> int:
        return self._queue.num_waiting

    @property
    def num_decoding(self) -> int:
        return sum(1 for r in self._active.values() if r.state == RequestState.DECODING)

    @property
    def num_prefilling(self) -> int:
        return sum(1 for r in self._active.values() if r.state == RequestState.PREFILLING)

    def active_requests(self) -> List[InferenceRequest]:
        with self._lock:
            return list(self._active.values())

    def stats(self) -> dict:
        return {"total_steps": self._totals["steps"], "prefill_steps": self._totals["prefill_steps"],
                "decode_steps": self._totals["decode_steps"], "total_preemptions": self._totals["preemptions"],
                "total_finished": self._totals["finished"], "num_active": self.num_active,
                "num_decoding": self.num_decoding, "num_prefilling": self.num_prefilling,
                "num_waiting": self.num_waiting, "queue": self._queue.stats(), "memory": self._budget.stats()}

    def summary(self) -> str:
        s = self.stats()
        return (f"scheduler: active {s['num_active']} (prefill {s['num_prefilling']}, decode {s['num_decoding']}), "
                f"waiting {s['num_waiting']}, steps {s['total_steps']} (prefill {s['prefill_steps']}, decode "
                f"{s['decode_steps']}), preemptions {s['total_preemptions']}, finished {s['total_finished']}, "
                f"memory {s['memory']['utilization']:.1%} committed")

"""Executes one scheduler decision on the model runner.

Role of zse-engine/zse_engine/zstreamer/batch_runner.py:33-371 with these differences: all chunks scheduled for a
step run as ONE packed pass (the reference runs one ``prefill`` per request); decode is one batched pass for every
sequence whatever its adapter (per-token adapter routing instead of grouping by ``lora_id``); tokens are chosen on
the device; speculative decoding is wired in (the reference builds ``BatchRunner(spec_runner=None)``).
"""
from __future__ import annotations

import zlib

import threading
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from ..runtime.runner import ModelRunner, SamplingRow
from .request import FinishReason, InferenceRequest, RequestOutput, RequestState
from .scheduler import Scheduler, SchedulerOutput


@dataclass
class StepResult:
    num_prefill_tokens: int = 0
    num_decode_tokens: int = 0
    tokens_generated: int = 0
    finished: List[RequestOutput] = field(default_factory=list)
    errors: List[str] = field(default_factory=list)
    # the reference's fields (zse-engine/zse_engine/zstreamer/batch_runner.py:34-47): the latest token of each request
    # that produced one in this step (speculative steps may produce several; the last is kept), and who was preempted
    new_tokens: Dict[str, int] = field(default_factory=dict)
    preempted_ids: List[str] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return len(self.new_tokens)


def _sampling_row(r: InferenceRequest, ahead: int = 0) -> SamplingRow:
    """``ahead`` = tokens of the request that are still on their way when the row is staged (pipelined decode)."""
    p = r.params
    if p.greedy:
        return SamplingRow()
    # an unseeded request draws from a stream named by its id: crc32, not hash(), because str hashes differ between the
    # worker processes of a tensor-parallel group and every rank must sample the same token
    base = p.seed if p.seed is not None else (zlib.crc32(str(r.request_id).encode("utf-8")) & 0x7FFFFFFF)
    # one random stream per request, indexed by the token's position in the output: a seeded request gives the same
    # tokens whatever else is in the batch, and a replayed CUDA graph (whose scalar arguments are frozen) still draws
    # fresh numbers because the per-row seed is staged from the host every step
    z = (int(base) + (r.num_generated + ahead + 1) * 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    return SamplingRow(float(p.temperature), int(p.top_k), float(p.top_p), int((z ^ (z >> 31)) & 0x7FFFFFFFFFFFFFFF))


@dataclass
class _InFlight:
    """A decode step that was launched before the step ahead of it had been read (pipelined decode)."""
    requests: List[InferenceRequest]          # row i of the launch belongs to requests[i]
    generated: List[int]                      # num_generated of each request when the step was launched
    pending: object                           # callable: waits for the step's tokens


def is_device_fault(exc: BaseException) -> bool:
    """Errors after which the device context of the process cannot be used again (a kernel fault reported by the CUDA
    runtime), as opposed to errors of one request or one pass (a bad argument, a bounded wait that ran out)."""
    text = str(exc)
    return isinstance(exc, RuntimeError) and "CUDA error" in text and any(
        w in text for w in ("launch failure", "illegal memory access", "illegal instruction", "misaligned address",
                            "device-side assert", "unspecified"))


class BatchRunner:
    def __init__(self, runner: ModelRunner, scheduler: Scheduler, spec_runner=None, lora_manager=None,
                 pipeline_decode: bool = False):
        self.fatal_error: Optional[str] = None   # set by the first device fault; the engine must then be restarted
        self._pipeline = bool(pipeline_decode)
        self._inflight: Optional[_InFlight] = None
        self.ahead_launches = 0          # decode steps launched before the step ahead of them had been read
        self.ahead_dropped = 0           # ... of which the result had to be thrown away
        self._runner = runner
        self._cache = runner.cache
        self._sched = scheduler
        self._spec = spec_runner
        self._lora = lora_manager
        self._finalized: set = set()
        self._lock = threading.Lock()

    # ---- entry ----------------------------------------------------------------------------------------
    def execute(self, plan: SchedulerOutput) -> StepResult:
        res = StepResult()
        if self._inflight is not None and (plan.preempt_requests or plan.prefill_requests
                                           or not plan.decode_requests):
            self._drop_inflight()          # the batch is being rearranged: take the next step the ordinary way
        for r in plan.preempt_requests:
            self._release_kv(r)
            res.preempted_ids.append(r.request_id)
        for r in plan.finished_requests:
            self._finalize(r, res)
        if plan.prefill_requests:
            self._run_prefill(plan, res)
        if plan.decode_requests:
            live = [r for r in plan.decode_requests if not r.is_finished]
            if live:
                if self._spec is not None and self._spec.k > 0:
                    self._run_speculative(live, res)
                else:
                    self._run_decode(live, res)
        for r in plan.prefill_requests + plan.decode_requests:
            if r.is_finished:
                self._finalize(r, res)
        return res

    # ---- helpers ----------------------------------------------------------------------------------------
    def _cache_salt(self, r: InferenceRequest) -> int:
        """Prefix-cache salt of a request: 0 for the base model, the adapter's value otherwise."""
        if self._lora is None or r.lora_id is None:
            return 0
        return self._lora.cache_salt(r.lora_id)

    def _adapter_slot(self, r: InferenceRequest) -> int:
        if self._lora is None or r.lora_id is None:
            return -1
        return self._lora.slot_of(r.lora_id)

    def _resolve_lora(self, r: InferenceRequest):
        """The adapter record a request asks for, or None (no manager, no ``lora_id``, or not loaded): the reference's
        helper (zse-engine/zse_engine/zstreamer/batch_runner.py); the passes themselves use ``_adapter_slot``."""
        if self._lora is None or r.lora_id is None:
            return None
        return self._lora.get_adapter(r.lora_id)

    def _release_kv(self, r: InferenceRequest) -> None:
        if r.seq_id is not None and self._cache.has_sequence(r.seq_id):
            self._cache.free_sequence(r.seq_id)

    def _finalize(self, r: InferenceRequest, res: StepResult) -> None:
        with self._lock:
            if r.request_id in self._finalized:
                return
            self._finalized.add(r.request_id)
            if len(self._finalized) > 100_000:
                self._finalized.clear()
        self._release_kv(r)
        if self._spec is not None:
            self._spec.forget(r.request_id)
        out = RequestOutput.from_request(r)
        res.finished.append(out)
        if r.on_finish is not None:
            try:
                r.on_finish(out)
            except Exception as exc:   # a client callback must not take the engine down
                res.errors.append(f"{r.request_id}: on_finish raised {exc!r}")

    def _fail(self, r: InferenceRequest, exc: Exception, res: StepResult) -> None:
        self._sched.on_request_error(r, f"{type(exc).__name__}: {exc}")
        res.errors.append(f"{r.request_id}: {exc}")
        if self.fatal_error is None and is_device_fault(exc):
            # the CUDA context of this process is gone: every later launch fails the same way.  The engine keeps
            # answering (requests finish with an error), says so through `fatal_error`, and has to be restarted
            self.fatal_error = " ".join(f"{type(exc).__name__}: {exc}".split())[:300]

    # ---- prefill ----------------------------------------------------------------------------------------
    def _run_prefill(self, plan: SchedulerOutput, res: StepResult) -> None:
        items, owners = [], []
        for r, n in zip(plan.prefill_requests, plan.prefill_chunk_sizes):
            if r.is_finished or n <= 0:
                continue
            try:
                toks = r.prefill_tokens
                if not self._cache.has_sequence(r.seq_id):
                    h = self._cache.allocate_sequence(r.seq_id, toks, salt=self._cache_salt(r))
                    self._cache.mark_active(r.seq_id)
                    if h.num_cached_tokens and r.prefill_offset == 0:
                        r.prefill_offset = h.num_cached_tokens        # prefix already in the cache
                        n = min(n, r.remaining_prefill)
                start = r.prefill_offset
                items.append((r.seq_id, toks[start:start + n], start))
                owners.append((r, n))
            except Exception as exc:
                self._fail(r, exc, res)
        if not items:
            return
        # split into passes that respect the runner's limits
        passes, cur, cur_tok = [], [], 0
        for it, ow in zip(items, owners):
            if cur and (cur_tok + len(it[1]) > self._runner.max_tokens or len(cur) >= self._runner.max_batch_seqs):
                passes.append(cur)
                cur, cur_tok = [], 0
            cur.append((it, ow))
            cur_tok += len(it[1])
        passes.append(cur)
        for group in passes:
            its = [g[0] for g in group]
            ows = [g[1] for g in group]
            try:
                toks = self._runner.prefill(its, sampling=[_sampling_row(o[0]) for o in ows],
                                            adapters=[self._adapter_slot(o[0]) for o in ows]
                                            if self._lora is not None else None)
            except Exception as exc:
                for r, _ in ows:
                    self._fail(r, exc, res)
                continue
            for (r, n), tok in zip(ows, toks):
                res.num_prefill_tokens += n
                resumed = r.num_generated > 0            # re-prefill after preemption: next input is known
                self._sched.on_prefill_complete(r, n)
                if r.state == RequestState.DECODING and not resumed:
                    self._sched.on_token_generated(r, int(tok))
                    res.new_tokens[r.request_id] = int(tok)
                    res.tokens_generated += 1

    # ---- decode -----------------------------------------------------------------------------------------
    def _run_decode(self, reqs: List[InferenceRequest], res: StepResult) -> None:
        """One decode step for ``reqs``.

        Ordinary order: extend the cache, stage and launch the step, do host work for the next step while the device
        runs, read the tokens.  Pipelined (``pipeline_decode``): before the tokens of this step are read, the NEXT
        step is launched as well - its input tokens are gathered on the device from this step's choices - so the
        device never waits for the host between steps; the step after this call then only has to be read.  A launch
        made ahead is used by the requests that are still decoding when its turn comes (rows of requests that ended on
        a stop token in the meantime are ignored; the slot they wrote belongs to a sequence that no longer exists).
        """
        fly, self._inflight = self._inflight, None
        rows: Optional[List[int]] = None
        if fly is not None:
            where = {id(r): i for i, r in enumerate(fly.requests)}
            usable = all(id(r) in where and fly.generated[where[id(r)]] + 1 == r.num_generated
                         and r.params.repetition_penalty == 1.0 for r in reqs)
            if usable:
                rows = [where[id(r)] for r in reqs]
                ready, pending = list(reqs), fly.pending
            else:
                self._inflight = fly
                self._drop_inflight()
        if rows is None:
            # a request that was extended ahead of time (while the previous step ran on the device) is ready as it is
            todo = [r for r in reqs if not r.pre_extended]
            errs = dict(zip((id(r) for r in todo), self._cache.extend_batch([r.seq_id for r in todo])))
            ready = []
            for r in reqs:
                exc = None if r.pre_extended else errs[id(r)]
                r.pre_extended = False
                if exc is None:
                    ready.append(r)
                else:
                    self._fail(r, exc, res)
            if not ready:
                return
            pen = None
            if any(r.params.repetition_penalty != 1.0 for r in ready):
                pen = [(r.params.repetition_penalty, r.past_tokens) for r in ready]
            try:
                pending = self._runner.decode([r.seq_id for r in ready], [r.output_tokens[-1] for r in ready],
                                              sampling=[_sampling_row(r) for r in ready],
                                              adapters=[self._adapter_slot(r) for r in ready]
                                              if self._lora is not None else None, penalties=pen, defer=True)
            except Exception as exc:
                for r in ready:
                    self._fail(r, exc, res)
                return
            rows = list(range(len(ready)))
        try:
            # host work that overlaps the device step: the cache slot of the token after this one, for every
            # request that cannot end on this token by length (a stop token frees the sequence, slot included)
            ahead = [r for r in ready if r.num_generated + 1 < r.params.max_tokens
                     and r.params.timeout_ms is None]
            for r, exc in zip(ahead, self._cache.extend_batch([r.seq_id for r in ahead])):
                r.pre_extended = exc is None
            if self._pipeline:
                self._launch_ahead(ready, rows)
            toks_all = pending()
            toks = [toks_all[i] for i in rows]
        except Exception as exc:
            self._inflight = None
            for r in ready:
                self._fail(r, exc, res)
            return
        for r, tok in zip(ready, toks):
            self._sched.on_token_generated(r, int(tok))
            res.new_tokens[r.request_id] = int(tok)
        res.num_decode_tokens += len(ready)
        res.tokens_generated += len(ready)

    def _launch_ahead(self, ready: List[InferenceRequest], rows: List[int]) -> None:
        """Launches the decode step AFTER the one in progress for the requests that are sure to need it, unless
        something may rearrange the batch before its turn (work waiting for prefill, penalties that need the token
        history on the host, speculative decoding, a request without a slot for it)."""
        if self._spec is not None and self._spec.k > 0:
            return
        if (self._sched.num_waiting > 0 or self._sched.num_prefilling > 0
                or any(r.state != RequestState.DECODING for r in ready)):
            return
        nxt = [(r, row) for r, row in zip(ready, rows) if r.pre_extended]
        if not nxt or any(r.params.repetition_penalty != 1.0 for r, _ in nxt):
            return
        reqs = [r for r, _ in nxt]
        for r in reqs:
            r.pre_extended = False                     # the slot is used by the launch below
        try:
            pending = self._runner.decode([r.seq_id for r in reqs], None,
                                          sampling=[_sampling_row(r, ahead=1) for r in reqs],
                                          adapters=[self._adapter_slot(r) for r in reqs]
                                          if self._lora is not None else None, defer=True,
                                          ids_rows=[row for _, row in nxt])
        except Exception:
            for r in reqs:
                r.pre_extended = True
            raise
        self._inflight = _InFlight(reqs, [r.num_generated for r in reqs], pending)
        self.ahead_launches += 1

    def _drop_inflight(self) -> None:
        """Waits for a step that was launched ahead and discards what it chose; the requests keep the cache slot it
        used (the step that replaces it writes the same values there)."""
        fly, self._inflight = self._inflight, None
        if fly is None:
            return
        self.ahead_dropped += 1
        try:
            fly.pending()
        except Exception:
            pass
        for r, g in zip(fly.requests, fly.generated):
            if not r.is_finished and r.state == RequestState.DECODING and r.seq_id is not None \
                    and self._cache.has_sequence(r.seq_id):
                r.pre_extended = True

    def _run_speculative(self, reqs: List[InferenceRequest], res: StepResult) -> None:
        greedy = [r for r in reqs if r.params.greedy and r.params.repetition_penalty == 1.0]
        other = [r for r in reqs if r not in greedy]
        if other:
            self._run_decode(other, res)
        if greedy:
            try:
                produced = self._spec.step(greedy, self._sched,
                                           adapters=[self._adapter_slot(r) for r in greedy]
                                           if self._lora is not None else None)
                res.num_decode_tokens += len(greedy)
                res.tokens_generated += produced
                for r in greedy:
                    if r.output_tokens:
                        res.new_tokens[r.request_id] = int(r.output_tokens[-1])
            except Exception as exc:
                for r in greedy:
                    self._fail(r, exc, res)

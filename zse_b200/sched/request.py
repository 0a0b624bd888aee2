"""Request objects of the continuous-batching engine (zse-engine/zse_engine/zstreamer/request.py:18-228).

States WAITING -> PREFILLING -> DECODING -> (PREEMPTED) -> FINISHED / CANCELLED; finish reasons ``length``,
``stop``, ``cancelled``, ``error``, ``preempted``; urgency = TTFT deadline minus elapsed time; TTFT / TPOT /
tokens-per-second are computed when the request finishes.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from enum import Enum, auto
from typing import Callable, Dict, List, Optional


# Clock of every time-based DECISION (time-out, TTFT-deadline urgency, arrival order).  One process: the monotonic clock.
# Tensor-parallel workers install a clock that returns the value rank 0 broadcast for the current loop iteration, so
# all ranks finish a timed-out request in the same step and order their queues alike (each rank deciding on its own
# clock would split the group: different batch shapes, mismatched collectives).  Reported metrics keep the real clock.
_decision_clock: Optional[Callable[[], float]] = None


def set_decision_clock(fn: Optional[Callable[[], float]]) -> None:
    global _decision_clock
    _decision_clock = fn


def decision_now() -> float:
    return _decision_clock() if _decision_clock is not None else time.monotonic()


class RequestState(Enum):
    WAITING = auto()
    PREFILLING = auto()
    DECODING = auto()
    PREEMPTED = auto()
    FINISHED = auto()
    CANCELLED = auto()


class FinishReason(Enum):
    LENGTH = "length"
    STOP = "stop"
    CANCELLED = "cancelled"
    ERROR = "error"
    PREEMPTED = "preempted"


@dataclass
class GenerationParams:
    max_tokens: int = 128
    temperature: float = 1.0
    top_p: float = 0.9
    top_k: int = 50
    repetition_penalty: float = 1.0
    stop_tokens: Optional[List[int]] = None
    seed: Optional[int] = None
    timeout_ms: Optional[float] = None
    lora_id: Optional[str] = None

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1


@dataclass
class InferenceRequest:
    request_id: str
    prompt_tokens: List[int]
    params: GenerationParams = field(default_factory=GenerationParams)
    priority: int = 0
    deadline_ms: Optional[float] = None
    state: RequestState = RequestState.WAITING
    output_tokens: List[int] = field(default_factory=list)
    finish_reason: Optional[FinishReason] = None
    prefill_offset: int = 0          # prompt (or re-prefill) tokens whose KV is in the cache
    chunk_size: int = 0
    arrival_time: float = field(default_factory=decision_now)
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None
    seq_id: Optional[int] = None
    on_token: Optional[Callable[[int], None]] = None
    callback_error: Optional[str] = None
    on_finish: Optional[Callable[["RequestOutput"], None]] = None
    past_tokens: Dict[int, int] = field(default_factory=dict)
    error: Optional[str] = None
    num_preemptions: int = 0
    pre_extended: bool = False           # the cache slot of the next decode token is already allocated
    # speculative decoding statistics
    spec_drafted: int = 0
    spec_accepted: int = 0

    @property
    def lora_id(self) -> Optional[str]:
        return self.params.lora_id

    @property
    def prompt_len(self) -> int:
        return len(self.prompt_tokens)

    @property
    def num_generated(self) -> int:
        return len(self.output_tokens)

    @property
    def total_tokens(self) -> int:
        return self.prompt_len + self.num_generated

    @property
    def prefill_tokens(self) -> List[int]:
        """What must be in the cache before the next decode step: the prompt plus, after a preemption that dropped
        the KV, every token generated so far except the last (which is the next decode input)."""
        if self.output_tokens:
            return self.prompt_tokens + self.output_tokens[:-1]
        return self.prompt_tokens

    @property
    def remaining_prefill(self) -> int:
        return len(self.prefill_tokens) - self.prefill_offset

    @property
    def is_active(self) -> bool:
        return self.state in (RequestState.PREFILLING, RequestState.DECODING)

    @property
    def is_finished(self) -> bool:
        return self.state in (RequestState.FINISHED, RequestState.CANCELLED)

    @property
    def urgency(self) -> float:
        if self.deadline_ms is None:
            return float("inf")
        return self.deadline_ms - (decision_now() - self.arrival_time) * 1000.0

    @property
    def wait_time_ms(self) -> float:
        return (decision_now() - self.arrival_time) * 1000.0

    def mark_prefilling(self) -> None:
        self.state = RequestState.PREFILLING

    def mark_decoding(self) -> None:
        self.state = RequestState.DECODING

    def mark_preempted(self) -> None:
        self.state = RequestState.PREEMPTED
        self.pre_extended = False
        self.num_preemptions += 1

    def mark_finished(self, reason: FinishReason) -> None:
        self.state = RequestState.FINISHED
        self.finish_reason = reason
        self.finish_time = time.monotonic()

    def mark_cancelled(self) -> None:
        self.state = RequestState.CANCELLED
        self.finish_reason = FinishReason.CANCELLED
        self.finish_time = time.monotonic()

    def add_token(self, token_id: int) -> None:
        self.output_tokens.append(token_id)
        self.past_tokens[token_id] = self.past_tokens.get(token_id, 0) + 1
        if self.first_token_time is None:
            self.first_token_time = time.monotonic()
        if self.on_token is not None:
            try:
                self.on_token(token_id)
            except Exception as exc:     # a client's streaming callback must not take the serving loop down
                self.callback_error = f"on_token raised {exc!r}"
                self.on_token = None     # do not call it again

    def should_stop(self) -> Optional[FinishReason]:
        # a stop token that arrives as the last allowed token is still a natural end ("stop", not "length"; the
        # reference tests the length first, zse-engine/zse_engine/zstreamer/request.py:172-181)
        if self.output_tokens and self.params.stop_tokens and self.output_tokens[-1] in self.params.stop_tokens:
            return FinishReason.STOP
        if self.num_generated >= self.params.max_tokens:
            return FinishReason.LENGTH
        if self.params.timeout_ms is not None and self.wait_time_ms > self.params.timeout_ms:
            return FinishReason.LENGTH
        return None


@dataclass
class RequestOutput:
    request_id: str
    prompt_tokens: List[int]
    output_tokens: List[int]
    finish_reason: FinishReason
    ttft_ms: float
    total_time_ms: float
    tpot_ms: float
    tokens_per_sec: float
    error: Optional[str] = None

    @staticmethod
    def from_request(req: InferenceRequest) -> "RequestOutput":
        now = req.finish_time or time.monotonic()
        total_ms = (now - req.arrival_time) * 1000.0
        ttft_ms = (req.first_token_time - req.arrival_time) * 1000.0 if req.first_token_time else total_ms
        n = max(len(req.output_tokens), 1)
        decode_ms = (now - req.first_token_time) * 1000.0 if req.first_token_time else total_ms
        # time per output token after the first one
        tpot = decode_ms / (n - 1) if n > 1 else 0.0
        return RequestOutput(req.request_id, req.prompt_tokens, list(req.output_tokens),
                             req.finish_reason or FinishReason.ERROR, ttft_ms, total_ms, tpot,
                             n / (total_ms / 1000.0) if total_ms > 0 else 0.0, req.error)

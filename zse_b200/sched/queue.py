"""Priority queues for waiting and preempted requests (zse-engine/zse_engine/zstreamer/queue.py:19-176).

Two heaps keyed ``(urgency, -priority, arrival, counter)``; preempted requests resume before new ones; cancelling
marks the entry and it is dropped lazily when popped.
"""
from __future__ import annotations

import heapq
import itertools
import threading
from typing import Dict, List, Optional

from .request import InferenceRequest, RequestState


class RequestQueue:
    def __init__(self, max_queue_size: int = 256):
        self._max = max_queue_size
        self._waiting: List[tuple] = []
        self._preempted: List[tuple] = []
        self._live: Dict[str, InferenceRequest] = {}
        self._counter = itertools.count()
        self._lock = threading.Lock()
        self._total_added = self._total_rejected = self._total_cancelled = 0

    def _key(self, r: InferenceRequest) -> tuple:
        return (r.urgency, -r.priority, r.arrival_time, next(self._counter))

    def add(self, request: InferenceRequest, force: bool = False) -> bool:
        with self._lock:
            if not force and self._max > 0 and len(self._live) >= self._max:
                self._total_rejected += 1
                return False
            request.state = RequestState.WAITING
            heapq.heappush(self._waiting, (*self._key(request), request))
            self._live[request.request_id] = request
            self._total_added += 1
            return True

    def add_preempted(self, request: InferenceRequest) -> None:
        with self._lock:
            heapq.heappush(self._preempted, (*self._key(request), request))
            self._live[request.request_id] = request

    def cancel(self, request_id: str) -> Optional[InferenceRequest]:
        with self._lock:
            r = self._live.pop(request_id, None)
            if r is not None:
                r.mark_cancelled()
                self._total_cancelled += 1
            return r

    def _pop_live(self, heap: List[tuple]) -> Optional[InferenceRequest]:
        while heap:
            r = heapq.heappop(heap)[-1]
            if self._live.get(r.request_id) is r and not r.is_finished:
                del self._live[r.request_id]
                return r
        return None

    def _peek_live(self, heap: List[tuple]) -> Optional[InferenceRequest]:
        while heap:
            r = heap[0][-1]
            if self._live.get(r.request_id) is r and not r.is_finished:
                return r
            heapq.heappop(heap)
        return None

    def pop_next(self) -> Optional[InferenceRequest]:
        """Preempted requests come back before new ones, except when a new request outranks them: the request
        that a preemption made room for must not lose that room to the request it displaced."""
        with self._lock:
            p, w = self._peek_live(self._preempted), self._peek_live(self._waiting)
            if p is not None and w is not None and w.priority > p.priority:
                return self._pop_live(self._waiting)
            return self._pop_live(self._preempted) or self._pop_live(self._waiting)

    def pop_prefill_batch(self, max_requests: int, max_tokens: int) -> List[InferenceRequest]:
        out, tokens = [], 0
        while len(out) < max_requests:
            r = self.pop_next()
            if r is None:
                break
            need = r.remaining_prefill
            if out and tokens + need > max_tokens:
                self.push_back(r)
                break
            out.append(r)
            tokens += need
        return out

    def push_back(self, r: InferenceRequest) -> None:
        """Return a popped request to the queue it came from (keeps its original arrival order)."""
        with self._lock:
            heap = self._preempted if r.state == RequestState.PREEMPTED else self._waiting
            heapq.heappush(heap, (r.urgency, -r.priority, r.arrival_time, next(self._counter), r))
            self._live[r.request_id] = r

    def peek_waiting(self) -> List[InferenceRequest]:
        with self._lock:
            return [r for r in self._live.values()]

    def remove_finished(self, request_id: str) -> None:
        with self._lock:
            self._live.pop(request_id, None)

    def get(self, request_id: str) -> Optional[InferenceRequest]:
        """A queued (waiting or preempted) request by id."""
        with self._lock:
            return self._live.get(request_id)

    @property
    def num_preempted(self) -> int:
        with self._lock:
            return sum(1 for e in self._preempted if self._live.get(e[-1].request_id) is e[-1])

    @property
    def num_total(self) -> int:
        return len(self._live)

    @property
    def is_empty(self) -> bool:
        return not self._live

    @property
    def num_waiting(self) -> int:
        return len(self._live)

    def stats(self) -> dict:
        with self._lock:
            return {"waiting": len(self._live), "max_queue_size": self._max, "total_added": self._total_added,
                    "total_rejected": self._total_rejected, "total_cancelled": self._total_cancelled,
                    "preempted_waiting": sum(1 for r in self._live.values() if r.state == RequestState.PREEMPTED)}

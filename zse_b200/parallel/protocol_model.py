"""Host model of the flag protocol of ``tp_reduce_add_rmsnorm`` (csrc/comm.cu), one thread per rank over shared numpy
arrays.

It states the protocol in a form that runs without a GPU, so that its two claims can be tested on the CPU with ranks
that run at very different speeds: (1) two buffer slots are enough - a rank cannot start call c+2 before every rank
has finished its part of call c+1, so nothing a slow rank still reads for call c is overwritten; (2) a rank that does
not take part makes the others give up after a bounded wait with a status record instead of hanging, and the buffers
stay usable for the next call.

Per rank r (what the kernel keeps in symmetric memory):
    data[r]  [2 slots][rows][H]    fp16 row buffer that the peers read
    flags[r] [2 slots][tp][rows]   flags[r][s][q][row] != 0: rank q has published `row` for the call that uses slot s
One call for one row on rank r, slot s = call & 1:
    A. data[r][s][row] = fp16(sum of the local planes); for every rank q (r included): flags[q][s][r][row] = 1
    B. for every rank q: wait (bounded) until flags[r][s][q][row] != 0, then set it to 0
       result = sum over q in rank order of data[q][s][row]
The reference has no counterpart (its reduction is a library all-reduce,
zse-engine/zse_engine/orchestrator/model_runner.py:2622-2635).
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass
from typing import Callable, List, Optional

import numpy as np


@dataclass
class PeerTimeout:
    rank: int          # who gave up
    peer: int          # whose flag never came
    row: int
    call: int


class OneShotExchange:
    def __init__(self, tp: int, rows: int, hidden: int, slots: int = 2, wait_limit_s: float = 1.0):
        self.tp, self.rows, self.hidden, self.slots = tp, rows, hidden, slots
        self.wait_limit_s = wait_limit_s
        self.data = np.zeros((tp, slots, rows, hidden), dtype=np.float16)
        self.flags = np.zeros((tp, slots, tp, rows), dtype=np.uint32)
        self.status: List[PeerTimeout] = []
        self._status_lock = threading.Lock()

    def reduce_row(self, rank: int, call: int, row: int, partial: np.ndarray,
                   pause: Optional[Callable[[str], None]] = None) -> Optional[np.ndarray]:
        """Rank ``rank``'s part of call ``call`` for one row; returns the fp32 sum over ranks, or None after a
        bounded wait ran out (recorded in ``status``).  ``pause(where)`` lets a test slow a rank down between the
        phases."""
        s = call % self.slots
        self.data[rank, s, row] = partial.astype(np.float16)                   # phase A
        for q in range(self.tp):
            self.flags[q, s, rank, row] = 1                                    # st.release.sys
        if pause:
            pause("published")
        for q in range(self.tp):                                               # phase B
            t0 = time.monotonic()
            while self.flags[rank, s, q, row] == 0:                            # ld.acquire.sys, bounded
                if time.monotonic() - t0 > self.wait_limit_s:
                    with self._status_lock:
                        self.status.append(PeerTimeout(rank, q, row, call))
                    return None
                time.sleep(0)
            self.flags[rank, s, q, row] = 0
        if pause:
            pause("flags down")
        acc = np.zeros(self.hidden, dtype=np.float32)
        for q in range(self.tp):                                               # fixed order: reproducible sum
            acc += self.data[q, s, row].astype(np.float32)
        return acc

    def reset_flags(self) -> None:
        """What the host does after a reported timeout before the group is used again."""
        self.flags[:] = 0

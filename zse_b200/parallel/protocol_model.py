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


class ScatterGatherExchange:
    """Host model of the exchange for passes of many rows (csrc/gemm_w4.cu ``kEpiScatterF16`` / ``gather_wait_tile``,
    csrc/comm.cu ``tp_sp_sum_norm_gather_kernel``), one thread per rank over shared numpy arrays.

    Token rows are owned in blocks of ``block`` rows: block b belongs to rank b % tp.  Per rank r:
        inbox[r]  [slots][tp sources][own rows][H]   partial rows, written by every source's GEMM epilogue
        arrive[r] [slots][tp sources][blocks]        units a source has delivered for a block of rank r
        xg[r]     [rows][H]                          the gathered, normalised rows (every rank ends with all of them)
        gflag[r]  [blocks]                           epoch of the last call whose rows of that block have arrived
        epoch[r], ticket[r][blocks]                  local words: calls finished so far; rows of a block finished
    One call (slot = call % slots) on rank r:
        scatter  for every block b and every unit (a tile of the GEMM): store the unit's part of the partial rows into
                 inbox[owner(b)][slot][r], then arrive[owner(b)][slot][r][b] += 1
        reduce   for every row of every block that r owns: wait (bounded) until arrive[r][slot][q][b] == units for
                 all q; row = sum over q in rank order; store it into xg[k] for every rank k; the row that finishes
                 its block last takes the block's counters down and writes epoch + 1 into gflag[k][b] on every rank
        gather   (the next GEMM's prologue) wait (bounded) until gflag[r][b] == epoch + 1 for the blocks it reads
    What the tests check with ranks of very different speed: the counters can be taken down by the owner because a
    source only delivers again after its gather wait, i.e. after every owner has finished every block of the call
    before (without that wait a fast source overruns counters and rows the owner still uses; the second slot is margin,
    not what makes it safe); every rank ends with identical gathered rows; and a source that never delivers makes the
    owners give up after a bounded wait instead of hanging."""

    def __init__(self, tp: int, rows: int, hidden: int, block: int = 4, units: int = 3, slots: int = 2,
                 wait_limit_s: float = 1.0):
        self.tp, self.rows, self.hidden, self.block, self.units, self.slots = tp, rows, hidden, block, units, slots
        self.wait_limit_s = wait_limit_s
        self.n_blocks = (rows + block - 1) // block
        own = (self.n_blocks + tp - 1) // tp * block
        self.inbox = np.zeros((tp, slots, tp, own, hidden), dtype=np.float16)
        self.arrive = np.zeros((tp, slots, tp, self.n_blocks), dtype=np.int64)
        self.xg = np.zeros((tp, rows, hidden), dtype=np.float32)
        self.gflag = np.zeros((tp, self.n_blocks), dtype=np.int64)
        self.epoch = np.zeros(tp, dtype=np.int64)
        self.ticket = np.zeros((tp, self.n_blocks), dtype=np.int64)
        self.status: List[PeerTimeout] = []
        self.overruns: List[tuple] = []            # (owner, slot, source, block, count): a counter ran past `units`
        self._lock = threading.Lock()

    def _local(self, row: int) -> int:
        b = row // self.block
        return (b // self.tp) * self.block + row % self.block

    def scatter(self, rank: int, call: int, partial: np.ndarray, pause: Optional[Callable[[str], None]] = None) -> None:
        """The GEMM epilogue of ``rank``: ``partial`` [rows, H] goes, unit by unit, to the owners of its blocks."""
        s = call % self.slots
        cols = np.array_split(np.arange(self.hidden), self.units)
        for b in range(self.n_blocks):
            owner = b % self.tp
            r0, r1 = b * self.block, min(self.rows, (b + 1) * self.block)
            for u in range(self.units):
                for row in range(r0, r1):
                    self.inbox[owner, s, rank, self._local(row), cols[u]] = partial[row, cols[u]].astype(np.float16)
                with self._lock:                                              # red.add after the unit's stores
                    self.arrive[owner, s, rank, b] += 1
                    if self.arrive[owner, s, rank, b] > self.units:
                        self.overruns.append((owner, s, rank, b, int(self.arrive[owner, s, rank, b])))
            if pause:
                pause("scattered block")

    def reduce_gather(self, rank: int, call: int, pause: Optional[Callable[[str], None]] = None) -> bool:
        """The owner's part of the call: returns False when a bounded wait ran out."""
        s = call % self.slots
        epoch = int(self.epoch[rank]) + 1
        ok = True
        for b in range(rank, self.n_blocks, self.tp):
            r0, r1 = b * self.block, min(self.rows, (b + 1) * self.block)
            for row in range(r0, r1):
                for q in range(self.tp):
                    t0 = time.monotonic()
                    while self.arrive[rank, s, q, b] < self.units:
                        if time.monotonic() - t0 > self.wait_limit_s:
                            with self._lock:
                                self.status.append(PeerTimeout(rank, q, row, call))
                            ok = False
                            break
                        time.sleep(0)
                total = np.zeros(self.hidden, dtype=np.float32)
                for q in range(self.tp):                                       # rank order
                    total += self.inbox[rank, s, q, self._local(row)].astype(np.float32)
                for k in range(self.tp):
                    self.xg[k, row] = total
                self.ticket[rank, b] += 1
                if self.ticket[rank, b] == r1 - r0:                            # the block's last row
                    self.ticket[rank, b] = 0
                    self.arrive[rank, s, :, b] = 0
                    for k in range(self.tp):
                        self.gflag[k, b] = epoch
            if pause:
                pause("reduced block")
        self.epoch[rank] = epoch
        return ok

    def gather_wait(self, rank: int) -> bool:
        """The prologue of the GEMM that reads the gathered rows on ``rank`` (after its own reduce of the call)."""
        want = int(self.epoch[rank])
        for b in range(self.n_blocks):
            t0 = time.monotonic()
            while self.gflag[rank, b] != want:
                if time.monotonic() - t0 > self.wait_limit_s:
                    with self._lock:
                        self.status.append(PeerTimeout(rank, b % self.tp, b * self.block, want))
                    return False
                time.sleep(0)
        return True

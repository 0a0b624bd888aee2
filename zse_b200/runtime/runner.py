"""ModelRunner: turns scheduler decisions into passes of the decoder.

Capabilities of zse-engine/zse_engine/orchestrator/model_runner.py:51-2473 (``prefill``, ``decode_step``,
``batched_decode``, ``verify_tokens``, ``embed_pooled``, graph variants) on the new stack:

* ``prefill`` handles any chunk of any sequence at its true cache position (chunk >= 2 and speculative verification
  attend to the whole past; the reference restarts at position 0, model_runner.py:305,761-841);
* several sequences can be prefilled in one packed pass;
* ``decode`` is always batched; per batch-size bucket the whole step (all layers, lm_head, sampling) is captured in
  one CUDA graph and replayed with the inputs staged through pinned host memory;
* token selection happens on the device (``argmax`` / ``sample``), only token ids come back.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.cache_manager import KVCacheManager
from ..models.decoder import DecoderModel, StepBuffers


@dataclass
class SamplingRow:
    temperature: float = 0.0      # 0 = greedy
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1


GREEDY = SamplingRow()


def _bucket(n: int, buckets: Sequence[int]) -> int:
    for b in buckets:
        if n <= b:
            return b
    return buckets[-1]


class ModelRunner:
    DECODE_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)

    def __init__(self, model: DecoderModel, cache: KVCacheManager, max_batch_seqs: int = 64,
                 max_tokens_per_pass: int = 2048, max_seq_len: Optional[int] = None, use_graphs: Optional[bool] = None,
                 attn_splits: Optional[int] = None):
        self.model, self.cache = model, cache
        self.device = model.device
        c = model.config
        self.max_seq_len = min(max_seq_len or c.max_seq_len, c.max_seq_len)
        self.max_batch_seqs = max_batch_seqs
        self.max_tokens = max(max_tokens_per_pass, max_batch_seqs)
        self.max_blocks = (self.max_seq_len + cache.block_size - 1) // cache.block_size
        on_gpu = self.device.type == "cuda"
        self.use_graphs = on_gpu if use_graphs is None else (use_graphs and on_gpu)
        sm = torch.cuda.get_device_properties(self.device).multi_processor_count if on_gpu else 1
        self._sm = sm
        self.max_attn_splits = attn_splits or (16 if on_gpu else 1)
        logits_rows = max(max_batch_seqs, 64)
        self.buf = model.make_buffers(self.max_tokens, max_batch_seqs, self.max_blocks, logits_rows,
                                      max_planes=8, attn_splits=self.max_attn_splits)
        self._graphs: Dict[Tuple[int, int, bool], torch.cuda.CUDAGraph] = {}
        self._graph_launches: Dict[Tuple[int, int, bool], int] = {}
        self.kernel_launches = 0          # own kernels launched by decode steps (graph replays included)
        self.step_events = None           # list collecting (start, end) CUDA events of decode steps when set
        self._step = 0
        pin = on_gpu
        mk = lambda shape, dt: torch.zeros(shape, dtype=dt, pin_memory=pin)
        self.h_ids = mk(self.max_tokens, torch.int32)
        self.h_pos = mk(self.max_tokens, torch.int32)
        self.h_slots = mk(self.max_tokens, torch.int64)
        self.h_bt = mk((max_batch_seqs, self.max_blocks), torch.int32)
        self.h_lens = mk(max_batch_seqs, torch.int32)
        self.h_cu = mk(max_batch_seqs + 1, torch.int32)
        self.h_pos0 = mk(max_batch_seqs, torch.int32)
        self.h_rows = mk(logits_rows, torch.int64)
        self.h_temp = mk(logits_rows, torch.float32)
        self.h_topk = mk(logits_rows, torch.int32)
        self.h_topp = mk(logits_rows, torch.float32)
        self.h_seed = mk(logits_rows, torch.int64)
        self.h_adapter = mk(self.max_tokens, torch.int32)
        self.h_out = mk(logits_rows, torch.int32)
        # pipelined decode: tokens (and the device status word) of a step are copied out behind the step itself and
        # read after an event, into alternating buffers, while the next step already runs
        self.h_out2 = [mk(logits_rows, torch.int32), mk(logits_rows, torch.int32)]
        self.h_status2 = [mk(4, torch.int32), mk(4, torch.int32)]
        self._flip = 0
        self.h_src = mk(logits_rows, torch.int64)
        self._src_rows = torch.zeros(logits_rows, dtype=torch.int64, device=self.device)
        # numpy views of the pinned staging buffers: per-step host work is numpy slicing, not tensor indexing
        self._np = {"ids": self.h_ids.numpy(), "pos": self.h_pos.numpy(), "slots": self.h_slots.numpy(),
                    "bt": self.h_bt.numpy(), "lens": self.h_lens.numpy(), "rows": self.h_rows.numpy(),
                    "out": self.h_out.numpy()}
        self._arange = np.arange(max(logits_rows, self.max_tokens), dtype=np.int64)
        self.timings = {"prefill_passes": 0, "decode_steps": 0, "graph_replays": 0, "graph_captures": 0}

    # ---- staging ----------------------------------------------------------------------------------------
    def _staging_begin(self) -> None:
        """The pinned staging buffers may be rewritten only after the copies that read them have run.  With pipelined
        decode the host can be a whole step ahead of the device, so this is checked, not assumed (the event has
        normally completed long before)."""
        ev = self.__dict__.get("_staged")
        if ev is not None:
            ev.synchronize()

    def _staging_end(self) -> None:
        if self.device.type == "cuda":
            ev = self.__dict__.get("_staged")
            if ev is None:
                ev = self._staged = torch.cuda.Event()
            ev.record()

    def _upload(self, dst: torch.Tensor, src: torch.Tensor, n) -> None:
        dst[:n].copy_(src[:n], non_blocking=True)

    def _stage_sampling(self, rows: Sequence[SamplingRow], n_pad: int) -> bool:
        all_greedy = all(r.greedy for r in rows)
        if not all_greedy:
            n = len(rows)
            self.h_temp[:n] = torch.tensor([r.temperature for r in rows])
            self.h_topk[:n] = torch.tensor([r.top_k for r in rows], dtype=torch.int32)
            self.h_topp[:n] = torch.tensor([r.top_p for r in rows])
            self.h_seed[:n] = torch.tensor([r.seed & 0x7FFFFFFFFFFFFFFF for r in rows], dtype=torch.int64)
            if n_pad > n:
                self.h_temp[n:n_pad] = 0
            b = self.buf
            self._upload(b.temperature, self.h_temp, n_pad)
            self._upload(b.top_k, self.h_topk, n_pad)
            self._upload(b.top_p, self.h_topp, n_pad)
            self._upload(b.seeds, self.h_seed, n_pad)
        return all_greedy

    def _stage_adapters(self, per_token: Optional[Sequence[int]], M: int, M_pad: int) -> None:
        if self.model.lora is None:
            return
        if per_token is None:
            self.h_adapter[:M_pad] = -1
        else:
            self.h_adapter[:M] = torch.as_tensor(list(per_token), dtype=torch.int32)
            self.h_adapter[M:M_pad] = -1
        self._upload(self.buf.adapter_ids, self.h_adapter, M_pad)

    def _select(self, n_rows: int, greedy: bool) -> None:
        b, ops = self.buf, self.model.ops
        if self.model.comm is not None:
            self.model.comm.select_tokens(self, n_rows, greedy, 0)
        elif greedy:
            ops.argmax(b.logits, b.out_tokens, n_rows)
        else:
            ops.sample(b.logits, b.out_tokens, n_rows, b.temperature, b.top_k, b.top_p, b.seeds, 0)

    def _fetch_tokens(self, n: int) -> List[int]:
        self.h_out[:n].copy_(self.buf.out_tokens[:n], non_blocking=True)
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
        self.model.ops.check()
        return self.h_out[:n].tolist()

    def _fetch_async(self, n: int):
        """Enqueues the copy of the first ``n`` chosen tokens (and of the status word) to the host behind the work
        launched so far and returns a callable that waits for that copy only - later launches keep running - and gives
        the tokens."""
        h, hs = self.h_out2[self._flip], self.h_status2[self._flip]
        self._flip ^= 1
        h[:n].copy_(self.buf.out_tokens[:n], non_blocking=True)
        status = getattr(self.model.ops, "status", None)
        ev = None
        if self.device.type == "cuda":
            if status is not None:
                hs.copy_(status.buf, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()

        def wait() -> List[int]:
            if ev is not None:
                ev.synchronize()
                if status is not None and int(hs[0]) != 0:
                    status.check()                   # reads, clears and raises
            return h[:n].tolist()
        return wait

    # ---- prefill / chunk / verify -------------------------------------------------------------------------
    def prefill(self, items: Sequence[Tuple[int, Sequence[int], int]], sampling: Optional[Sequence[SamplingRow]] = None,
                all_logits: bool = False, adapters: Optional[Sequence[int]] = None, select: bool = True):
        """``items``: ``(seq_id, chunk_tokens, start_position)``; the cache must already hold blocks for positions
        ``start .. start+len-1`` of each sequence.  Returns the token chosen after each chunk's last token, or (with
        ``all_logits``) the fp16 logits of every row (device tensor view, valid until the next pass)."""
        b, cache = self.buf, self.cache
        S = len(items)
        total = sum(len(t) for _, t, _ in items)
        if S > self.max_batch_seqs or total > self.max_tokens:
            raise ValueError(f"prefill pass of {total} tokens / {S} sequences exceeds the pass limits "
                             f"({self.max_tokens} / {self.max_batch_seqs})")
        at, max_q, rows = 0, 0, []
        self._staging_begin()
        self.h_bt[:S].fill_(-1)
        per_tok_adapter = [] if adapters is not None else None
        for s, (sid, toks, start) in enumerate(items):
            n = len(toks)
            self.h_ids[at:at + n] = torch.as_tensor(list(toks), dtype=torch.int32)
            self.h_pos[at:at + n] = torch.arange(start, start + n, dtype=torch.int32)
            self.h_slots[at:at + n] = torch.from_numpy(cache.slots_for_range(sid, start, n))
            ids = cache.get_block_ids(sid)
            self.h_bt[s, :len(ids)] = torch.as_tensor(ids, dtype=torch.int32)
            self.h_cu[s] = at
            self.h_pos0[s] = start
            if per_tok_adapter is not None:
                per_tok_adapter += [adapters[s]] * n
            rows += list(range(at, at + n)) if all_logits else [at + n - 1]
            at += n
            max_q = max(max_q, n)
        self.h_cu[S] = at
        n_rows = len(rows)
        if n_rows > b.logits.shape[0]:
            raise ValueError(f"{n_rows} logits rows requested, buffer holds {b.logits.shape[0]}")
        self.h_rows[:n_rows] = torch.as_tensor(rows, dtype=torch.int64)
        for dst, src, n in ((b.ids, self.h_ids, total), (b.positions, self.h_pos, total), (b.slots, self.h_slots, total),
                            (b.block_tables, self.h_bt, S), (b.cu_q, self.h_cu, S + 1), (b.q_pos0, self.h_pos0, S),
                            (b.logit_rows, self.h_rows, n_rows)):
            self._upload(dst, src, n)
        self._stage_adapters(per_tok_adapter, total, total)
        greedy = self._stage_sampling(sampling or [GREEDY] * n_rows, n_rows) if select else True
        self._staging_end()
        ev = None
        if self.step_events is not None:         # a caller times the passes (speculative verification runs through here)
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        with self._nvtx(f"prefill[{total} tokens, {S} seqs]"):
            self.model.forward(b, cache.slab, total, "prefill", S, max_q, n_rows)
        if ev is not None:
            ev[1].record()
            self.step_events.append(ev)
        self.timings["prefill_passes"] += 1
        self._step += 1
        for sid, toks, start in items:
            cache.commit_tokens(sid, start + len(toks))
        if all_logits and not select:
            return b.logits[:n_rows]
        self._select(n_rows, greedy)
        toks = self._fetch_tokens(n_rows)
        return (toks, b.logits[:n_rows]) if all_logits else toks

    # ---- batched decode -----------------------------------------------------------------------------------
    def _pick_splits(self, S: int, max_len: int) -> int:
        if self.device.type != "cuda":
            return 1
        ctas = S * self.model.plan.num_kv_heads
        want = (2 * self._sm + ctas - 1) // ctas
        by_len = max(1, max_len // 128)              # at least 128 cached tokens per split
        n = int(max(1, min(want, by_len, self.max_attn_splits)))
        return 1 << (n.bit_length() - 1)              # powers of two: few distinct CUDA graphs as sequences grow

    def _apply_penalties(self, penalties, n_rows: int) -> None:
        """``penalties[i] = (penalty, {token: count})`` for logits row i (zse-engine/zse_engine/orchestrator/
        sampler.py:64-80), applied in place on the device through a sparse (row, token, count) list."""
        rows, toks, cnts, pens = [], [], [], []
        for i, (pen, counts) in enumerate(penalties[:n_rows]):
            pens.append(float(pen))
            if pen != 1.0:
                for t, c in counts.items():
                    rows.append(i)
                    toks.append(t)
                    cnts.append(c)
        if not rows:
            return
        dev = self.device
        mk = lambda v, dt: torch.tensor(v, dtype=dt, device=dev)
        self.model.ops.apply_repetition_penalty(self.buf.logits, mk(rows, torch.int32), mk(toks, torch.int32),
                                                mk(cnts, torch.int32), len(rows), mk(pens, torch.float32))

    def decode(self, seq_ids: Sequence[int], last_tokens: Sequence[int],
               sampling: Optional[Sequence[SamplingRow]] = None, adapters: Optional[Sequence[int]] = None,
               penalties=None, defer: bool = False, ids_rows: Optional[Sequence[int]] = None):
        """One new token for each sequence: ``last_tokens[i]`` is appended at the sequence's current length (the
        cache must already have been extended by one), attention covers the whole sequence.  With ``defer`` the step
        is only launched and a callable is returned that waits for it and gives the tokens, so that the caller can
        do host work while the device runs.  With ``ids_rows`` the input tokens are not known to the host yet: row i
        takes the token that the PREVIOUS decode step chose in its row ``ids_rows[i]`` (still on the device), which
        lets the caller launch a step before it has read the one before."""
        b, cache = self.buf, self.cache
        S = len(seq_ids)
        if S == 0:
            return (lambda: []) if defer else []
        if S > self.max_batch_seqs:
            raise ValueError(f"decode batch {S} exceeds max_batch_seqs {self.max_batch_seqs}")
        Sp = min(_bucket(S, self.DECODE_BUCKETS), self.max_batch_seqs) if self.use_graphs else S
        bs = cache.block_size
        n_ = self._np
        self._staging_begin()
        max_len = max(1, cache.stage_decode(seq_ids, n_["bt"], n_["lens"], n_["pos"], n_["slots"]))
        if ids_rows is None:
            n_["ids"][:S] = last_tokens
        else:
            src = self.h_src.numpy()
            src[:S] = ids_rows
            src[S:Sp] = 0
        if Sp > S:                                  # padding rows: empty sequences that write nothing
            n_["bt"][S:Sp].fill(-1)
            n_["ids"][S:Sp] = 0
            n_["pos"][S:Sp] = 0
            n_["slots"][S:Sp] = -1
            n_["lens"][S:Sp] = 0
        n_["rows"][:Sp] = self._arange[:Sp]
        for dst, src, n in ((b.positions, self.h_pos, Sp), (b.slots, self.h_slots, Sp),
                            (b.block_tables, self.h_bt, Sp), (b.seq_lens, self.h_lens, Sp),
                            (b.logit_rows, self.h_rows, Sp)):
            self._upload(dst, src, n)
        if ids_rows is None:
            self._upload(b.ids, self.h_ids, Sp)
        else:                                       # gather on the device, ordered behind the previous step's choice
            self._upload(self._src_rows, self.h_src, Sp)
            torch.index_select(b.out_tokens, 0, self._src_rows[:Sp], out=b.ids[:Sp])
        self._stage_adapters(adapters, S, Sp)
        greedy = self._stage_sampling(sampling or [GREEDY] * S, Sp)
        self._staging_end()
        splits = self._pick_splits(Sp, max_len)
        self._step += 1
        counter = self._launch_counter()
        before = counter[0]
        graphed = penalties is None and self.use_graphs and (self.model.comm is None or self.model.comm.graph_safe)
        g = None
        if graphed:
            key = (Sp, splits, greedy)
            g = self._graphs.get(key)
            if g is None:
                g = self._capture(Sp, splits, greedy)
                before = counter[0]
        ev = None
        if self.step_events is not None:
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        if g is not None:
            with self._nvtx(f"decode graph[{Sp} seqs]"):
                g.replay()
            self.timings["graph_replays"] += 1
            self.kernel_launches += self._graph_launches[key]
        else:
            self.model.forward(b, cache.slab, Sp, "decode", Sp, 1, Sp, splits)
            if penalties is not None:
                self._apply_penalties(penalties, S)
            self._select(Sp, greedy)
            self.kernel_launches += counter[0] - before
        if ev is not None:
            ev[1].record()
            self.step_events.append(ev)
        self.timings["decode_steps"] += 1
        wait = self._fetch_async(Sp)
        if defer:
            return lambda: wait()[:S]
        return wait()[:S]

    def _capture(self, Sp: int, splits: int, greedy: bool) -> "torch.cuda.CUDAGraph":
        b, cache = self.buf, self.cache
        t_begin = time.perf_counter()
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):            # warm-up outside capture (lazy attribute set-up, tensor maps)
            self.model.forward(b, cache.slab, Sp, "decode", Sp, 1, Sp, splits)
            self._select(Sp, greedy)
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        counter = self._launch_counter()
        n0 = counter[0]
        with torch.cuda.graph(g, stream=stream):
            self.model.forward(b, cache.slab, Sp, "decode", Sp, 1, Sp, splits)
            self._select(Sp, greedy)
        self._graphs[(Sp, splits, greedy)] = g
        self._graph_launches[(Sp, splits, greedy)] = counter[0] - n0
        self.timings["graph_captures"] += 1
        self.timings["graph_capture_s"] = self.timings.get("graph_capture_s", 0.0) + time.perf_counter() - t_begin
        return g

    def release_graphs(self) -> None:
        """Drops every captured decode graph.  Graphs that captured NCCL kernels keep their communicator busy, so
        this has to happen before the process group is destroyed."""
        self._graphs.clear()
        self._graph_launches.clear()

    @staticmethod
    def _nvtx(name: str):
        """NVTX range around a phase when ZSE_NVTX=1 (timeline tools), else a no-op context."""
        import contextlib
        from ..utils import env as _env
        if _env.flag("ZSE_NVTX") and torch.cuda.is_available():
            return torch.cuda.nvtx.range(name)
        return contextlib.nullcontext()

    def _launch_counter(self):
        if self.device.type == "cuda":
            from ..ops import native
            return native.LAUNCHES
        return [0]

    # ---- convenience ----------------------------------------------------------------------------------------
    def verify_tokens(self, seq_id: int, tokens: Sequence[int], start_position: int) -> torch.Tensor:
        """Logits (fp32, host) after each of ``tokens`` placed at ``start_position...``; the caller has extended the
        cache to cover them and truncates afterwards."""
        logits = self.prefill([(seq_id, tokens, start_position)], all_logits=True, select=False)
        return logits.float().cpu()

    def last_logits(self, tokens: Sequence[int], seq_id: int = 1_000_000_001) -> torch.Tensor:
        """fp32 host logits after the last of ``tokens`` (one prefill pass on a scratch sequence): what a Yes/No
        reranker reads."""
        self.cache.allocate_sequence(seq_id, num_tokens=len(tokens))
        try:
            self.prefill([(seq_id, tokens, 0)])
            return self.buf.logits[0].float().cpu()
        finally:
            self.cache.free_sequence(seq_id)

    def embed_pooled(self, tokens: Sequence[int], seq_id: int = 1_000_000_000) -> torch.Tensor:
        """Mean-pooled, L2-normalised final hidden state (dense retrieval embeddings), pooled on the device."""
        self.cache.allocate_sequence(seq_id, num_tokens=len(tokens))
        try:
            self.prefill([(seq_id, tokens, 0)], select=False, all_logits=False)
            h = self.model.hidden_rows(self.buf, len(tokens)).float().mean(dim=0)
            return torch.nn.functional.normalize(h, dim=0).cpu()
        finally:
            self.cache.free_sequence(seq_id)

    # ---- the reference's call forms (zse-engine/zse_engine/orchestrator/model_runner.py:675-2010) ---------------
    # There a caller passes the token, the sequence and its position, the runner extends the cache by one token
    # itself, and the fp16 logits come back as bytes (or, in the graph variants, the greedy token).  These wrappers
    # keep that contract on top of ``decode``; the serving loop uses ``decode`` / ``prefill`` directly.
    @property
    def hidden_size(self) -> int:
        return self.model.config.hidden_size

    @property
    def vocab_size(self) -> int:
        return self.model.config.vocab_size

    def _logit_rows_bytes(self, n: int) -> List[bytes]:
        rows = self.buf.logits[:n, : self.vocab_size].to(torch.float16).cpu().numpy()
        return [rows[i].tobytes() for i in range(n)]

    def batched_decode(self, token_ids: Sequence[int], seq_ids: Sequence[int], positions: Optional[Sequence[int]] = None,
                       lora_adapter=None, skip_logits_download: bool = False) -> Optional[List[bytes]]:
        """One token per sequence in one pass; ``positions`` must equal the sequences' current lengths (it is what the
        cache already knows, and is checked when given).  ``lora_adapter``: an adapter slot for every row, or None."""
        if len(token_ids) == 0:
            return []
        if positions is not None:
            for sid, pos in zip(seq_ids, positions):
                have = self.cache.num_tokens(sid)
                if have != pos:
                    raise ValueError(f"sequence {sid} holds {have} tokens, not {pos}")
        for sid in seq_ids:
            self.cache.extend_sequence(sid, 1)
        adapters = None if lora_adapter is None else [int(lora_adapter)] * len(seq_ids)
        self._last_tokens = self.decode(list(seq_ids), list(token_ids), adapters=adapters)
        return None if skip_logits_download else self._logit_rows_bytes(len(seq_ids))

    def decode_step(self, token_id: int, seq_id: int, position: Optional[int] = None, lora_adapter=None,
                    skip_logits_download: bool = False) -> Optional[bytes]:
        out = self.batched_decode([token_id], [seq_id], None if position is None else [position], lora_adapter,
                                  skip_logits_download)
        return None if out is None else out[0]

    def gpu_argmax(self, row_idx: int = 0) -> int:
        """Greedy token of row ``row_idx`` of the last decode pass: it was chosen on the device during the pass, so
        this reads four bytes' worth of host memory and launches nothing."""
        toks = getattr(self, "_last_tokens", None)
        if toks is None or not 0 <= row_idx < len(toks):
            raise IndexError(f"no decode row {row_idx} to read")
        return int(toks[row_idx])

    def batched_decode_graph(self, token_ids: Sequence[int], seq_ids: Sequence[int],
                             positions: Optional[Sequence[int]] = None) -> List[int]:
        """Greedy tokens of one batched step.  On a GPU the step replays the CUDA graph of its batch bucket (captured
        on first use); there is no separate un-graphed greedy path to fall back from."""
        self.batched_decode(token_ids, seq_ids, positions, skip_logits_download=True)
        return [int(t) for t in self._last_tokens]

    def decode_step_graph(self, token_id: int, seq_id: int, position: Optional[int] = None) -> int:
        return self.batched_decode_graph([token_id], [seq_id], None if position is None else [position])[0]

    def init_graph(self, max_seq_len: int = 2048) -> None:
        """Kept for callers of the reference: graphs need no set-up here beyond ``use_graphs`` (buffers are fixed from
        construction, buckets are captured on first use or by ``precapture_batched_graphs``)."""
        if max_seq_len > self.max_seq_len:
            raise ValueError(f"runner was built for sequences of {self.max_seq_len} tokens, not {max_seq_len}")

    def destroy_graph(self) -> None:
        self.release_graphs()

    def precapture_batched_graphs(self, batch_sizes=(1, 2, 4, 8), warmup_seq_ids=None) -> int:
        """Captures the decode graph of each batch size's bucket now rather than at its first use in serving.  Runs one
        throw-away step per bucket on scratch sequences (``warmup_seq_ids`` are accepted and ignored: no caller state
        is touched).  Returns how many graphs exist afterwards."""
        if not self.use_graphs:
            return 0
        base = 1_000_100_000
        for m in sorted({min(_bucket(int(x), self.DECODE_BUCKETS), self.max_batch_seqs) for x in batch_sizes}):
            sids = list(range(base, base + m))
            made = []
            try:
                for sid in sids:
                    self.cache.allocate_sequence(sid, num_tokens=1)
                    made.append(sid)
                self.decode(sids, [0] * m)
            finally:
                for sid in made:
                    self.cache.free_sequence(sid)
        return len(self._graphs)


class TPModelRunner(ModelRunner):
    """A runner over this rank's shard of the model (zse-engine/zse_engine/orchestrator/model_runner.py:2476-2885).
    The reference overrides the layer methods to add two all-reduces; here the model object carries the communication
    layer (``DecoderModel(..., comm=...)``: fused reduce + residual + norm kernels over peer memory, or NCCL), so the
    runner only checks that a sharded model has one and exposes the group's shape."""

    def __init__(self, model: DecoderModel, cache: KVCacheManager, *args, tp_group=None, **kwargs):
        if model.plan.tp_size > 1 and model.comm is None:
            raise ValueError("a sharded model needs a communication layer (pass comm= when the model is built)")
        if tp_group is not None and (tp_group.tp_size != model.plan.tp_size or tp_group.rank != model.plan.rank):
            raise ValueError(f"model shard {model.plan.rank}/{model.plan.tp_size} does not belong to "
                             f"rank {tp_group.rank}/{tp_group.tp_size}")
        super().__init__(model, cache, *args, **kwargs)
        self.tp_group = tp_group

    @property
    def tp_size(self) -> int:
        return self.model.plan.tp_size

    @property
    def tp_rank(self) -> int:
        return self.model.plan.rank

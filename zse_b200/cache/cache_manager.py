"""Thread-safe façade over the paged KV cache (zse-engine/zse_engine/cache/cache_manager.py:67-569).

Keeps the reference's semantics: adaptive block size, ``max_seq_len`` enforcement, eviction before allocation
(idle sequences first, lossy holes), sliding-window trimming, fork with copy-on-write, ``truncate_sequence`` for
speculative roll-back, ``mark_active/idle``, stats.  Differences:

* block sizes are multiples of 16 (the attention kernels stream 16-token MMA tiles): {16, 32, 64} instead of
  {8, 16, 32}; the choice still depends on context length and GQA ratio;
* prompt blocks are shared only along a common prefix and only after they were computed, and
  ``allocate_sequence`` reports how many leading prompt tokens are already cached so prefill can skip them.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Set

import numpy as np

from ..format.config import ModelConfig
from .attention_metadata import AttentionMetadata
from .block_pool import BlockPool
from .dedup import BlockDedup
from .evictor import Evictor
from .page_table import PageTable


@dataclass
class KVCacheHandle:
    seq_id: int
    num_tokens: int
    num_blocks: int
    num_cached_tokens: int = 0       # leading prompt tokens whose KV was found in shared blocks


@dataclass
class CacheStats:
    total_blocks: int
    allocated_blocks: int
    free_blocks: int
    total_bytes: int
    used_bytes: int
    utilization: float
    num_sequences: int
    total_cached_tokens: int
    eviction_count: int
    tokens_evicted: int
    eviction_policy: str
    dedup_hits: int
    dedup_hit_rate: float
    block_size_tokens: int
    block_bytes: int


class KVCacheManager:
    def __init__(self, config: ModelConfig, device=None, budget_bytes: int = 0, block_size: int = 0,
                 eviction_policy: str = "smart", enable_dedup: bool = True, num_kv_heads: Optional[int] = None,
                 num_blocks: int = 0):
        self._config = config
        self._lock = threading.RLock()
        self._block_size = block_size if block_size > 0 else self._auto_block_size(config)
        if self._block_size % 16:
            raise ValueError("block_size must be a multiple of 16")
        # local kv heads under tensor parallelism; rows of the widest layer when layers differ (Gemma-4)
        nkv, pool_hd = config.kv_pool_dims(num_kv_heads)
        if num_blocks > 0:
            self._pool = BlockPool(num_blocks, self._block_size, config.num_layers, nkv, pool_hd, device)
        else:
            if budget_bytes <= 0:
                raise ValueError("either budget_bytes or num_blocks is required")
            self._pool = BlockPool.from_budget(budget_bytes, self._block_size, config.num_layers, nkv,
                                               pool_hd, device)
        # a uniform window (Mistral) lets old blocks go; models that mix local and global layers keep everything and
        # apply the window inside attention
        self._windowed = bool(config.sliding_window and config.sliding_window > 0 and not config.layer_types)
        self._page_table = PageTable(self._pool)
        self._evictor = Evictor(eviction_policy)
        self._dedup = BlockDedup(self._pool) if enable_dedup else None
        self._prompt_lengths: Dict[int, int] = {}
        self._prompt_tokens: Dict[int, Sequence[int]] = {}
        self._registered_upto: Dict[int, int] = {}
        self._salts: Dict[int, int] = {}               # seq_id -> prefix-chain salt (sequences that run with an adapter)
        self._active: Set[int] = set()

    @staticmethod
    def _auto_block_size(config: ModelConfig) -> int:
        """<= 4096 context: 16; <= 32768: 32; longer: 64; halved (not below 16) for heavy GQA (kv/heads <= 1/4)."""
        base = 16 if config.max_seq_len <= 4096 else 32 if config.max_seq_len <= 32768 else 64
        if config.num_kv_heads / config.num_heads <= 0.25 and base > 16:
            base //= 2
        return base

    # ---- sequence life cycle --------------------------------------------------------------------------
    def allocate_sequence(self, seq_id: int, prompt_tokens: Optional[Sequence[int]] = None,
                          num_tokens: Optional[int] = None, salt: int = 0) -> KVCacheHandle:
        """Creates the sequence and reserves blocks for ``prompt_tokens`` (or ``num_tokens`` anonymous tokens).
        ``salt`` names the weights the sequence runs with (0: the base model; otherwise a value derived from the LoRA
        adapter): cached prefix blocks are only shared between sequences of equal salt."""
        with self._lock:
            n = len(prompt_tokens) if prompt_tokens is not None else int(num_tokens or 0)
            if n > self._config.max_seq_len:
                raise ValueError(f"prompt length {n} exceeds max_seq_len {self._config.max_seq_len}")
            if self._page_table.has_sequence(seq_id):
                raise ValueError(f"sequence {seq_id} already exists")
            bs = self._block_size
            shared: List[int] = []
            hashes: List[int] = []
            if self._dedup is not None and prompt_tokens is not None and n > bs:
                hashes = self._dedup.chain_hashes(prompt_tokens, salt)
                prev = salt
                for i, h in enumerate(hashes):
                    if (i + 1) * bs >= n:          # keep at least one token to compute
                        break
                    bid = self._dedup.lookup(h, prompt_tokens[i * bs:(i + 1) * bs], prev)
                    if bid is None:
                        break
                    shared.append(bid)
                    prev = h
            fresh_tokens = n - len(shared) * bs
            need = (fresh_tokens + bs - 1) // bs
            if need > self._pool.num_free and not self._evict_locked(need):
                raise RuntimeError(f"cannot allocate {need} KV blocks for sequence {seq_id}: "
                                   f"{self._pool.num_free} free and eviction did not help")
            e = self._page_table.create_sequence(seq_id)
            for i, bid in enumerate(shared):
                b = self._pool.get_block(bid)
                self._pool.increment_ref(b)
                e.blocks.append(b)
            e.touch()
            e.num_tokens = len(shared) * bs
            if fresh_tokens:
                self._page_table.append_tokens(seq_id, fresh_tokens)
            self._prompt_lengths[seq_id] = n
            self._track_blocks(e, 0)
            if prompt_tokens is not None:
                self._prompt_tokens[seq_id] = prompt_tokens
            self._registered_upto[seq_id] = len(shared)
            if salt:
                self._salts[seq_id] = salt
            return KVCacheHandle(seq_id, e.num_tokens, len(e.blocks), len(shared) * bs)

    def commit_tokens(self, seq_id: int, num_computed: int) -> None:
        """Tells the cache that the KV of the first ``num_computed`` tokens is now written, which makes the full
        prompt blocks among them shareable."""
        if self._dedup is None:
            return
        with self._lock:
            toks = self._prompt_tokens.get(seq_id)
            e = self._page_table.get_entry_or_none(seq_id)
            if toks is None or e is None:
                return
            bs = self._block_size
            upto = min(num_computed, len(toks)) // bs
            start = self._registered_upto.get(seq_id, 0)
            if upto <= start:
                return
            salt = self._salts.get(seq_id, 0)
            hashes = self._dedup.chain_hashes(toks[: upto * bs], salt)
            for i in range(start, upto):
                if i not in e.evicted_indices:
                    self._dedup.register(e.blocks[i].block_id, hashes[i], toks[i * bs:(i + 1) * bs],
                                         hashes[i - 1] if i else salt)
            self._registered_upto[seq_id] = upto

    def extend_sequence(self, seq_id: int, num_new_tokens: int = 1) -> None:
        if num_new_tokens <= 0:
            return
        with self._lock:
            cur = self._page_table.num_tokens(seq_id)
            if cur + num_new_tokens > self._config.max_seq_len:
                raise ValueError(f"extending sequence {seq_id} to {cur + num_new_tokens} tokens exceeds max_seq_len "
                                 f"{self._config.max_seq_len}")
            need = self._page_table.blocks_needed(seq_id, num_new_tokens)
            if need > self._pool.num_free and not self._evict_locked(need):
                raise RuntimeError(f"cannot extend sequence {seq_id}: need {need} KV blocks, "
                                   f"{self._pool.num_free} free")
            new_ids = self._page_table.append_tokens(seq_id, num_new_tokens)
            if new_ids:
                e = self._page_table.get_entry(seq_id)
                self._track_blocks(e, max(0, len(e.blocks) - len(new_ids) - 1))
            if self._windowed:
                self._trim_sliding_window(seq_id)

    def _track_blocks(self, e, first_idx: int) -> None:
        """Tells the evictor about blocks ``first_idx..`` of a sequence (new, shared or copied ones)."""
        bs = self._block_size
        prompt = self._prompt_lengths.get(e.seq_id, 0)
        for idx in range(first_idx, len(e.blocks)):
            if idx not in e.evicted_indices:
                b = e.blocks[idx]
                self._evictor.record_access(e.seq_id, idx, b.block_id, b.num_tokens or bs, idx * bs,
                                            idx * bs < prompt)

    def extend_batch(self, seq_ids) -> list:
        """One more token for each sequence (a decode step).  Returns one entry per sequence: None, or the exception
        that extending it raised.  A sequence whose private tail block still has room takes a short path that touches
        neither the pool nor the evictor."""
        errs = [None] * len(seq_ids)
        bs, limit = self._block_size, self._config.max_seq_len
        windowed = self._windowed
        with self._lock:
            for i, sid in enumerate(seq_ids):
                e = self._page_table.get_entry_or_none(sid)
                if e is not None and not windowed:
                    n = e.num_tokens
                    fill = n % bs
                    if fill and n < limit and e.blocks:
                        tail = e.blocks[-1]
                        if tail.ref_count == 1 and (len(e.blocks) - 1) not in e.evicted_indices:
                            tail.num_tokens = fill + 1
                            e.num_tokens = n + 1
                            continue
                try:
                    self.extend_sequence(sid, 1)
                except Exception as exc:          # reported per sequence: the rest of the batch still runs
                    errs[i] = exc
        return errs

    def free_sequence(self, seq_id: int) -> None:
        with self._lock:
            e = self._page_table.get_entry_or_none(seq_id)
            if e is None:
                return
            for i, b in enumerate(e.blocks):
                if i not in e.evicted_indices and b.ref_count == 1 and self._dedup is not None:
                    self._dedup.deregister_block(b.block_id)
            self._evictor.remove_sequence(seq_id)
            self._page_table.remove_sequence(seq_id)
            for d in (self._prompt_lengths, self._prompt_tokens, self._registered_upto, self._salts):
                d.pop(seq_id, None)
            self._active.discard(seq_id)

    def fork_sequence(self, src_id: int, dst_id: int) -> KVCacheHandle:
        with self._lock:
            e = self._page_table.fork_sequence(src_id, dst_id)
            self._prompt_lengths[dst_id] = self._prompt_lengths.get(src_id, 0)
            self._active.add(dst_id)
            return KVCacheHandle(dst_id, e.num_tokens, len(e.blocks))

    def truncate_sequence(self, seq_id: int, keep_tokens: int) -> None:
        """Rolls the sequence back to ``keep_tokens`` (speculative decoding rejects); frees whole blocks past it."""
        with self._lock:
            e = self._page_table.get_entry_or_none(seq_id)
            if e is None or keep_tokens >= e.num_tokens:
                return
            bs = self._block_size
            keep_blocks = (keep_tokens + bs - 1) // bs
            e.touch()
            while len(e.blocks) > keep_blocks:
                b = e.blocks.pop()
                idx = len(e.blocks)
                if idx in e.evicted_indices:
                    e.evicted_indices.discard(idx)
                    continue
                if self._dedup is not None and b.ref_count == 1:
                    self._dedup.deregister_block(b.block_id)
                self._evictor.remove_block(b.block_id, seq_id)
                self._pool.free(b)
            if e.blocks and keep_tokens > 0 and (keep_blocks - 1) not in e.evicted_indices:
                tail = e.blocks[-1]
                if not tail.is_shared:
                    tail.num_tokens = keep_tokens - (keep_blocks - 1) * bs
                    if self._dedup is not None and tail.num_tokens < bs:
                        self._dedup.deregister_block(tail.block_id)
            e.num_tokens = keep_tokens
            self._registered_upto[seq_id] = min(self._registered_upto.get(seq_id, 0), keep_tokens // bs)

    def mark_active(self, seq_id: int) -> None:
        with self._lock:
            self._active.add(seq_id)

    def mark_idle(self, seq_id: int) -> None:
        with self._lock:
            self._active.discard(seq_id)

    # ---- eviction -------------------------------------------------------------------------------------
    def evict_if_needed(self, blocks_needed: int) -> bool:
        with self._lock:
            return self._evict_locked(blocks_needed)

    def _evict_locked(self, blocks_needed: int) -> bool:
        if self._pool.num_free >= blocks_needed:
            return True
        shortage = blocks_needed - self._pool.num_free
        for exclude in (self._active, None):
            victims = self._evictor.select_victims(shortage * 2, exclude_seq_ids=exclude)
            for v in victims:
                if self._pool.num_free >= blocks_needed:
                    return True
                e = self._page_table.get_entry_or_none(v.seq_id)
                if e is None:
                    self._evictor.remove_block(v.block_id, v.seq_id)
                    continue
                for idx, b in enumerate(e.blocks):
                    if idx not in e.evicted_indices and b.block_id == v.block_id:
                        if self._dedup is not None and b.ref_count == 1:
                            self._dedup.deregister_block(b.block_id)
                        self._page_table.evict_block(v.seq_id, idx)
                        self._evictor.note_evicted(v.num_tokens)
                        break
                self._evictor.remove_block(v.block_id, v.seq_id)
            if self._pool.num_free >= blocks_needed:
                return True
        return self._pool.num_free >= blocks_needed

    def _trim_sliding_window(self, seq_id: int) -> None:
        e = self._page_table.get_entry_or_none(seq_id)
        window = self._config.sliding_window
        if e is None or e.num_tokens <= window:
            return
        for idx in range((e.num_tokens - window) // self._block_size):
            if idx not in e.evicted_indices:
                self._evictor.remove_block(e.blocks[idx].block_id, seq_id)
                self._page_table.evict_block(seq_id, idx)

    # ---- what the kernels need --------------------------------------------------------------------------
    def get_block_ids(self, seq_id: int) -> List[int]:
        with self._lock:
            return self._page_table.get_block_ids(seq_id)

    def block_ids_np(self, seq_id: int):
        with self._lock:
            return self._page_table.block_ids_np(seq_id)

    def stage_decode(self, seq_ids, block_tables, seq_lens, positions, slots) -> int:
        """Fills the decode-step arrays (numpy views of the runner's pinned staging buffers) for ``seq_ids`` in one
        pass: block table rows (-1 padded), lengths, the position of each sequence's newest token and the cache slot
        that token is written to (-1 when its block was evicted).  Returns the longest sequence length."""
        S = len(seq_ids)
        bs = self._block_size
        with self._lock:
            entries = [self._page_table.get_entry(sid) for sid in seq_ids]
            now = self._evictor.now()
            for sid in seq_ids:
                self._evictor.touch_sequence(sid, now)
            block_tables[:S].fill(-1)
            for s, e in enumerate(entries):
                ids = e.block_ids_np()
                block_tables[s, :ids.shape[0]] = ids
            seq_lens[:S] = [e.num_tokens for e in entries]
        n = seq_lens[:S]
        last = n - 1
        positions[:S] = last
        blk = block_tables[np.arange(S), np.maximum(last, 0) // bs].astype(np.int64)
        slots[:S] = np.where(blk < 0, -1, blk * bs + last % bs)
        return int(n.max()) if S else 0

    def num_tokens(self, seq_id: int) -> int:
        return self._page_table.num_tokens(seq_id)

    def has_sequence(self, seq_id: int) -> bool:
        return self._page_table.has_sequence(seq_id)

    def slot_for(self, seq_id: int, position: int) -> int:
        ids = self._page_table.get_block_ids(seq_id)
        b = ids[position // self._block_size]
        return -1 if b < 0 else b * self._block_size + position % self._block_size

    def slots_for_range(self, seq_id: int, start: int, count: int) -> np.ndarray:
        ids = np.asarray(self._page_table.get_block_ids(seq_id), dtype=np.int64)
        pos = np.arange(start, start + count, dtype=np.int64)
        blk = ids[pos // self._block_size]
        return np.where(blk < 0, -1, blk * self._block_size + pos % self._block_size)

    def get_attention_metadata(self, seq_ids: Sequence[int], is_prefill: Optional[List[bool]] = None,
                               record_access: bool = True, gpu_upload: bool = False) -> AttentionMetadata:
        """Block tables and lengths of a batch.  ``gpu_upload`` also copies them to the pool's device and fills the
        ``*_gpu_ptr`` fields (a list of booleans in second position is taken as ``is_prefill``, a bare ``True`` as the
        reference's ``gpu_upload`` flag)."""
        if isinstance(is_prefill, bool):
            gpu_upload, is_prefill = is_prefill, None
        with self._lock:
            tables, lens = [], []
            for sid in seq_ids:
                ids = self._page_table.get_block_ids(sid)
                tables.append(ids)
                lens.append(self._page_table.num_tokens(sid))
                if record_access:
                    self._evictor.record_batch_access(sid, ids, self._block_size, self._prompt_lengths.get(sid, 0))
            width = max((len(t) for t in tables), default=0)
            meta = AttentionMetadata(tables, lens, len(tables), max(lens, default=0), width, self._block_size,
                                     is_prefill)
        if gpu_upload and self._pool.slab is not None:
            meta.upload(self._pool.slab.device)
        return meta

    # ---- facts ----------------------------------------------------------------------------------------
    @property
    def pool(self) -> BlockPool:
        return self._pool

    @property
    def slab(self):
        return self._pool.slab

    @property
    def block_size(self) -> int:
        return self._block_size

    @property
    def num_free_blocks(self) -> int:
        return self._pool.num_free

    @property
    def num_total_blocks(self) -> int:
        return self._pool.num_blocks

    @property
    def num_sequences(self) -> int:
        return self._page_table.num_sequences

    @property
    def max_tokens_capacity(self) -> int:
        return self._pool.num_blocks * self._block_size

    def stats(self) -> CacheStats:
        with self._lock:
            pt = self._page_table.stats()
            return CacheStats(self._pool.num_blocks, self._pool.num_allocated, self._pool.num_free,
                              self._pool.total_bytes, self._pool.used_bytes, self._pool.utilization,
                              pt["num_sequences"], pt["total_tokens"], self._evictor.eviction_count,
                              self._evictor.total_tokens_evicted, self._evictor.policy,
                              self._dedup.dedup_hits if self._dedup else 0,
                              self._dedup.hit_rate if self._dedup else 0.0, self._block_size, self._pool.block_bytes)

    def summary(self) -> str:
        s = self.stats()
        return (f"KV cache: {s.allocated_blocks}/{s.total_blocks} blocks of {s.block_size_tokens} tokens "
                f"({s.used_bytes / 2**20:.1f}/{s.total_bytes / 2**20:.1f} MiB), {s.num_sequences} sequences, "
                f"{s.total_cached_tokens} tokens, {s.eviction_count} evictions ({s.eviction_policy}), "
                f"prefix hits {s.dedup_hits}")

    def destroy(self) -> None:
        with self._lock:
            self._pool.destroy()

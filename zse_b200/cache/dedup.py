"""Sharing of identical prompt blocks between sequences (prefix cache).

The reference hashes the token ids of each *full* block with FNV-1a-64 and shares blocks whose tokens match
(zse-engine/zse_engine/cache/dedup.py:15-140) without looking at what came before the block, although the keys and
values of a block depend on every earlier token.  Here the hash of block i chains the hash of block i-1, so only a
common *prefix* is ever shared, and a block becomes visible to other sequences only once its KV has been written
(``register`` is called after the pass that filled it).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

from .block_pool import BlockPool

_FNV_OFFSET = 0xCBF29CE484222325
_FNV_PRIME = 0x100000001B3
_MASK = 0xFFFFFFFFFFFFFFFF


def fnv1a_chain(prev_hash: int, token_ids: Sequence[int]) -> int:
    h = (_FNV_OFFSET ^ prev_hash) & _MASK
    for t in token_ids:
        for shift in (0, 8, 16, 24):
            h ^= (t >> shift) & 0xFF
            h = (h * _FNV_PRIME) & _MASK
    return h


def _fnv1a_hash(token_ids: Sequence[int]) -> int:
    return fnv1a_chain(0, token_ids)


class BlockDedup:
    def __init__(self, pool: BlockPool):
        self._pool = pool
        self._by_hash: Dict[int, Tuple[int, Tuple[int, ...], int]] = {}    # hash -> (block_id, tokens, prev_hash)
        self._hash_of_block: Dict[int, int] = {}
        self._hits = self._misses = self._collisions = 0

    def chain_hashes(self, tokens: Sequence[int], salt: int = 0) -> List[int]:
        """Chain hash of every full block.  ``salt`` starts the chain: sequences whose keys and values are computed
        with different weights (another LoRA adapter, or none) pass different salts and never share a block."""
        bs = self._pool.block_size_tokens
        out, h = [], salt & _MASK
        for i in range(len(tokens) // bs):
            h = fnv1a_chain(h, tokens[i * bs:(i + 1) * bs])
            out.append(h)
        return out

    def lookup(self, chain_hash: int, block_tokens: Sequence[int], prev_hash: int = 0) -> Optional[int]:
        hit = self._by_hash.get(chain_hash)
        if hit is None:
            self._misses += 1
            return None
        bid, toks, prev = hit
        if toks != tuple(block_tokens) or prev != prev_hash:
            self._collisions += 1
            return None
        self._hits += 1
        return bid

    def register(self, block_id: int, chain_hash: int, block_tokens: Sequence[int], prev_hash: int = 0) -> None:
        if chain_hash in self._by_hash or block_id in self._hash_of_block:
            return
        self._by_hash[chain_hash] = (block_id, tuple(block_tokens), prev_hash)
        self._hash_of_block[block_id] = chain_hash
        self._pool.get_block(block_id).content_hash = chain_hash

    def register_block(self, block_id: int, token_ids: Sequence[int], prev_hash: int = 0) -> Optional[int]:
        """The reference's one-call form (zse-engine/zse_engine/cache/dedup.py:50-95): returns the id of an existing
        block with the same content (and the same prefix chain, ``prev_hash``) after taking a reference on it, or
        registers ``block_id`` and returns None."""
        h = fnv1a_chain(prev_hash, token_ids)
        hit = self.lookup(h, token_ids, prev_hash)
        if hit is not None and hit != block_id:
            self._pool.increment_ref(self._pool.get_block(hit))
            return hit
        self.register(block_id, h, token_ids, prev_hash)
        return None

    def deregister_block(self, block_id: int) -> None:
        h = self._hash_of_block.pop(block_id, None)
        if h is not None:
            self._by_hash.pop(h, None)

    @property
    def dedup_hits(self) -> int:
        return self._hits

    @property
    def dedup_misses(self) -> int:
        return self._misses

    @property
    def collision_count(self) -> int:
        return self._collisions

    @property
    def hit_rate(self) -> float:
        n = self._hits + self._misses
        return self._hits / n if n else 0.0

    def stats(self) -> dict:
        return {"registered": len(self._by_hash), "hits": self._hits, "misses": self._misses,
                "collisions": self._collisions, "hit_rate": self.hit_rate}

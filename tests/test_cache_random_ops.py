"""Randomised operation sequences on the KV cache manager (allocate with shared prefixes, commit, extend one by one and
in batches, fork, truncate, free, eviction under pressure) with the book-keeping invariants checked after every
operation: a block is either free or referenced, reference counts equal the number of tables that hold the block,
nothing is lost when everything is freed."""
import random

import numpy as np
import pytest
import torch

from zse_b200.cache.cache_manager import KVCacheManager
from zse_b200.format import synth


def _check(m: KVCacheManager, live):
    pool = m.pool
    refs = {}
    for sid in live:
        assert m.has_sequence(sid)
        ids = m.get_block_ids(sid)
        n = m.num_tokens(sid)
        bs = m.block_size
        assert len(ids) >= (n + bs - 1) // bs or any(i < 0 for i in ids)
        for b in ids:
            if b >= 0:
                refs[b] = refs.get(b, 0) + 1
    for b, cnt in refs.items():
        blk = pool.get_block(b)
        assert blk.ref_count >= cnt, (b, blk.ref_count, cnt)      # the prefix index may hold one more reference
    assert pool.num_free + pool.num_allocated == pool.num_blocks
    assert pool.num_allocated >= len(refs)
    assert m.num_sequences == len(live)


@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_random_operation_sequences_keep_the_books_straight(seed):
    rng = random.Random(seed)
    cfg = synth.shape_config("tiny")
    m = KVCacheManager(cfg, torch.device("cpu"), block_size=16, num_blocks=48, enable_dedup=True)
    shared_prefix = [rng.randrange(1000) for _ in range(40)]
    live, next_id = [], 1
    for step in range(400):
        op = rng.random()
        try:
            if op < 0.25 and len(live) < 10:
                n = rng.randint(1, 60)
                toks = (shared_prefix[: rng.randint(0, 40)] if rng.random() < 0.5 else []) + \
                       [rng.randrange(1000) for _ in range(n)]
                h = m.allocate_sequence(next_id, toks)
                m.commit_tokens(next_id, len(toks))
                live.append(next_id)
                next_id += 1
            elif op < 0.55 and live:
                sid = rng.choice(live)
                m.extend_sequence(sid, rng.randint(1, 5))
            elif op < 0.65 and live:
                picks = rng.sample(live, min(len(live), rng.randint(1, 4)))
                errs = m.extend_batch(picks)
                assert len(errs) == len(picks)
            elif op < 0.72 and live and len(live) < 10:
                src = rng.choice(live)
                m.fork_sequence(src, next_id)
                live.append(next_id)
                next_id += 1
            elif op < 0.82 and live:
                sid = rng.choice(live)
                n = m.num_tokens(sid)
                if n > 1:
                    m.truncate_sequence(sid, rng.randint(1, n))
            elif op < 0.95 and live:
                sid = live.pop(rng.randrange(len(live)))
                m.free_sequence(sid)
            elif live:
                sid = rng.choice(live)
                (m.mark_active if rng.random() < 0.5 else m.mark_idle)(sid)
        except (RuntimeError, ValueError):
            pass                               # out of blocks / over the length limit: allowed outcomes, no corruption
        # a sequence whose every block was evicted may have been dropped by the manager
        live = [s for s in live if m.has_sequence(s)]
        _check(m, live)
        if live:                               # staging never reads outside the tables
            S = len(live)
            bt = np.full((S, 32), -1, dtype=np.int32)
            lens, pos = np.zeros(S, np.int32), np.zeros(S, np.int32)
            slots = np.zeros(S, np.int64)
            usable = [s for s in live if m.num_tokens(s) > 0]
            if usable:
                m.stage_decode(usable, bt, lens, pos, slots)
                assert (slots[: len(usable)] < m.num_total_blocks * m.block_size).all()
    for sid in live:
        m.free_sequence(sid)
    assert m.num_sequences == 0
    assert m.num_free_blocks == m.num_total_blocks, (m.num_free_blocks, m.num_total_blocks)

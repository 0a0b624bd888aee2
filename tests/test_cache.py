"""Paged KV cache on the host: pool, page table, copy-on-write, prefix sharing, eviction holes, truncation, and the
vectorised decode staging.  Mirrors the cases of zse-engine/tests/test_cache.py (pool/page-table/evictor/manager
classes) without a GPU: the slab lives on the CPU."""
import numpy as np
import pytest
import torch

from zse_b200.cache.block_pool import BlockPool
from zse_b200.cache.cache_manager import KVCacheManager
from zse_b200.cache.dedup import BlockDedup
from zse_b200.cache.evictor import Evictor
from zse_b200.cache.page_table import PageTable
from zse_b200.format import synth


def _cfg(**kw):
    c = synth.shape_config("tiny")
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def _mgr(num_blocks=32, block_size=16, **kw):
    return KVCacheManager(_cfg(), device=torch.device("cpu"), num_blocks=num_blocks, block_size=block_size, **kw)


# ---- pool ------------------------------------------------------------------------------------------------------
def test_pool_alloc_free_refcount():
    cfg = _cfg()
    pool = BlockPool(4, 16, cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, torch.device("cpu"))
    assert pool.num_free == 4 and pool.num_allocated == 0
    a, b = pool.alloc(1), pool.alloc(1)
    assert {a.block_id, b.block_id} <= set(range(4)) and a.block_id != b.block_id
    pool.increment_ref(a)
    assert a.is_shared
    assert pool.free(a) is False          # still referenced
    assert pool.free(a) is True
    assert pool.num_free == 3
    pool.alloc(); pool.alloc(); pool.alloc()
    with pytest.raises(Exception):
        pool.alloc()
    assert pool.block_bytes == 2 * cfg.num_layers * cfg.num_kv_heads * 16 * cfg.head_dim * 2 // cfg.num_layers * 1 \
        or pool.block_bytes > 0
    assert pool.total_bytes == pool.block_bytes * 4


def test_pool_from_budget_counts_blocks():
    cfg = _cfg()
    per_block = 2 * cfg.num_layers * cfg.num_kv_heads * 16 * cfg.head_dim * 2
    pool = BlockPool.from_budget(per_block * 7 + 5, 16, cfg.num_layers, cfg.num_kv_heads, cfg.head_dim,
                                 torch.device("cpu"))
    assert pool.num_blocks == 7


# ---- page table ------------------------------------------------------------------------------------------------
def test_page_table_growth_and_ids():
    cfg = _cfg()
    pool = BlockPool(8, 16, cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, torch.device("cpu"))
    pt = PageTable(pool)
    pt.create_sequence(5)
    assert pt.blocks_needed(5, 17) == 2
    new = pt.append_tokens(5, 17)
    assert len(new) == 2 and pt.num_tokens(5) == 17 and pt.num_blocks(5) == 2
    assert pt.blocks_needed(5, 15) == 0 and pt.blocks_needed(5, 16) == 1
    assert pt.get_block_ids(5) == new
    assert pt.block_ids_np(5).tolist() == new
    pt.append_tokens(5, 16)
    assert pt.block_ids_np(5).tolist() == pt.get_block_ids(5) and pt.num_blocks(5) == 3
    with pytest.raises(ValueError):
        pt.create_sequence(5)


def test_page_table_fork_is_copy_on_write():
    cfg = _cfg()
    pool = BlockPool(8, 16, cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, torch.device("cpu"))
    pt = PageTable(pool)
    pt.create_sequence(1)
    pt.append_tokens(1, 20)
    pool.slab[:, pt.get_block_ids(1)[1]] = 3.0
    pt.fork_sequence(1, 2)
    assert pt.get_block_ids(2) == pt.get_block_ids(1) and pool.num_allocated == 2
    assert pt.blocks_needed(2, 1) == 1                    # shared partly filled tail must be copied first
    pt.append_tokens(2, 1)
    a, b = pt.get_block_ids(1), pt.get_block_ids(2)
    assert a[0] == b[0] and a[1] != b[1] and pool.num_allocated == 3
    assert torch.equal(pool.slab[:, b[1]], pool.slab[:, a[1]])      # contents travelled with the copy
    assert pt.block_ids_np(2).tolist() == b
    pt.remove_sequence(1)
    assert pool.num_allocated == 2
    pt.remove_sequence(2)
    assert pool.num_allocated == 0


def test_page_table_eviction_leaves_hole():
    cfg = _cfg()
    pool = BlockPool(8, 16, cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, torch.device("cpu"))
    pt = PageTable(pool)
    pt.create_sequence(1)
    pt.append_tokens(1, 48)
    before = pt.get_block_ids(1)
    assert pt.evict_block(1, 1) is not None
    assert pt.evict_block(1, 1) is None
    ids = pt.get_block_ids(1)
    assert ids[1] == -1 and ids[0] == before[0] and ids[2] == before[2]
    assert pt.block_ids_np(1).tolist() == ids
    assert pt.num_tokens(1) == 48 and pool.num_allocated == 2
    assert pt.get_entry(1).tokens_evicted == 16


# ---- evictor / dedup -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("policy", ["lru", "lfu", "smart"])
def test_evictor_prefers_cold_blocks(policy):
    t = [0.0]
    ev = Evictor(policy, clock=lambda: t[0])
    for i in range(4):
        t[0] += 1.0
        ev.record_access(1, i, 100 + i, 16, token_start=16 * i, is_prompt=(i == 0))
    for _ in range(5):
        t[0] += 1.0
        ev.record_access(1, 3, 103, 16, token_start=48)
        ev.record_access(1, 0, 100, 16, is_prompt=True)
    victims = ev.select_victims(2)
    assert len(victims) == 2
    ids = [v.block_id for v in victims]
    assert 103 not in ids                              # the hot, most recent block stays
    assert 100 not in ids                              # the prompt block is hot too (and protected under "smart")
    with pytest.raises(ValueError):
        Evictor("random")
    assert ev.select_victims(2, exclude_seq_ids={1}) == []
    ev.remove_sequence(1)
    assert ev.select_victims(1) == []


def test_dedup_chain_hash_depends_on_prefix():
    cfg = _cfg()
    pool = BlockPool(4, 16, cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, torch.device("cpu"))
    d = BlockDedup(pool)
    a = list(range(32))
    b = list(range(16, 32)) + list(range(16, 32))
    ha, hb = d.chain_hashes(a), d.chain_hashes(b)
    assert len(ha) == 2 and ha[1] != hb[1]             # same second block, different prefix
    blk = pool.alloc()
    d.register(blk.block_id, ha[0], a[:16], 0)
    assert d.lookup(ha[0], a[:16], 0) == blk.block_id
    assert d.lookup(ha[0], [9] * 16, 0) is None        # same hash, other tokens: not a hit
    d.deregister_block(blk.block_id)
    assert d.lookup(ha[0], a[:16], 0) is None


# ---- manager ---------------------------------------------------------------------------------------------------
def test_manager_prefix_sharing_and_cached_tokens():
    m = _mgr()
    sys_prompt = list(range(100, 140))                  # 40 tokens: two full blocks + 8
    h1 = m.allocate_sequence(1, sys_prompt + [1, 2, 3])
    assert h1.num_cached_tokens == 0
    m.commit_tokens(1, len(sys_prompt) + 3)
    used = m.num_total_blocks - m.num_free_blocks
    h2 = m.allocate_sequence(2, sys_prompt + [7, 8, 9, 10])
    assert h2.num_cached_tokens == 32                   # the two full blocks are shared
    assert m.get_block_ids(2)[:2] == m.get_block_ids(1)[:2]
    assert m.num_total_blocks - m.num_free_blocks == used + 1
    st = m.stats()
    assert st.dedup_hits >= 2
    m.free_sequence(1)
    assert m.get_block_ids(2)[0] >= 0                   # still referenced by sequence 2
    m.free_sequence(2)
    assert m.num_free_blocks == m.num_total_blocks


def test_manager_identical_prompt_keeps_one_token_to_compute():
    m = _mgr()
    p = list(range(32))
    m.allocate_sequence(1, p)
    m.commit_tokens(1, 32)
    h = m.allocate_sequence(2, p)
    assert h.num_cached_tokens == 16                    # the last block is recomputed so that logits exist


def test_manager_extend_truncate_and_slots():
    m = _mgr()
    m.allocate_sequence(1, num_tokens=30)
    m.extend_sequence(1, 5)
    assert m.num_tokens(1) == 35 and len(m.get_block_ids(1)) == 3
    ids = m.get_block_ids(1)
    assert m.slot_for(1, 33) == ids[2] * 16 + 1
    assert m.slots_for_range(1, 14, 4).tolist() == [ids[0] * 16 + 14, ids[0] * 16 + 15, ids[1] * 16, ids[1] * 16 + 1]
    m.truncate_sequence(1, 17)
    assert m.num_tokens(1) == 17 and len(m.get_block_ids(1)) == 2
    assert m.block_ids_np(1).tolist() == m.get_block_ids(1)
    m.truncate_sequence(1, 16)
    assert len(m.get_block_ids(1)) == 1
    with pytest.raises(ValueError):
        m.extend_sequence(1, 10 ** 6)


def test_manager_evicts_idle_sequences_under_pressure():
    m = _mgr(num_blocks=6, enable_dedup=False)
    m.allocate_sequence(1, num_tokens=48)
    m.allocate_sequence(2, num_tokens=32)
    m.mark_active(2)
    assert m.num_free_blocks == 1
    m.allocate_sequence(3, num_tokens=48)               # needs 3: two come from idle sequence 1
    assert -1 in m.get_block_ids(1) and -1 not in m.get_block_ids(2)
    assert m.stats().eviction_count >= 2
    with pytest.raises(RuntimeError):
        m.allocate_sequence(4, num_tokens=16 * 7)           # more than the whole pool


def test_extend_batch_matches_extend_sequence():
    a, b = _mgr(), _mgr()
    lens = [1, 15, 16, 17, 31]
    for s, n in enumerate(lens):
        a.allocate_sequence(s, num_tokens=n)
        b.allocate_sequence(s, num_tokens=n)
    for _ in range(40):
        assert a.extend_batch(list(range(len(lens)))) == [None] * len(lens)
        for s in range(len(lens)):
            b.extend_sequence(s, 1)
    for s in range(len(lens)):
        assert a.num_tokens(s) == b.num_tokens(s) and len(a.get_block_ids(s)) == len(b.get_block_ids(s))
    errs = a.extend_batch([0, 99])
    assert errs[0] is None and errs[1] is not None       # unknown sequence is reported, the other one still grows


def test_stage_decode_against_per_sequence_queries():
    m = _mgr(num_blocks=64)
    lens = [5, 16, 17, 40, 1]
    for s, n in enumerate(lens):
        m.allocate_sequence(10 + s, num_tokens=n)
    m._page_table.evict_block(13, 1)                     # a hole in the middle of a sequence
    m._page_table.evict_block(11, 0)                     # the newest token's own block is gone
    S = len(lens)
    bt = np.zeros((8, 6), np.int32); sl = np.zeros(8, np.int32); pos = np.zeros(8, np.int32)
    slots = np.zeros(8, np.int64)
    mx = m.stage_decode([10 + s for s in range(S)], bt, sl, pos, slots)
    assert mx == 40
    for s, n in enumerate(lens):
        ids = m.get_block_ids(10 + s)
        assert bt[s, :len(ids)].tolist() == ids and (bt[s, len(ids):] == -1).all()
        assert sl[s] == n and pos[s] == n - 1
        blk = ids[(n - 1) // 16]
        assert slots[s] == (-1 if blk < 0 else blk * 16 + (n - 1) % 16)
    assert slots[1] == -1


def test_sliding_window_trims_old_blocks():
    m = KVCacheManager(_cfg(sliding_window=32), device=torch.device("cpu"), num_blocks=16, block_size=16)
    m.allocate_sequence(1, num_tokens=30)
    for _ in range(40):
        m.extend_sequence(1, 1)
    ids = m.get_block_ids(1)
    assert ids[0] == -1 and ids[1] == -1 and ids[-1] >= 0
    assert m.num_tokens(1) == 70

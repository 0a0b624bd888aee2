"""Unit tests of the KV cache's parts one by one - block pool arithmetic and addresses, eviction scores, chained block
hashes, packed attention metadata (the shape of the reference's tests/test_kv_cache.py, bookkeeping only: no device
slab).  The cache manager as a whole is in tests/test_cache.py and tests/test_cache_random_ops.py."""
import struct

import numpy as np
import pytest

from zse_b200.cache.attention_metadata import AttentionMetadata, build_attention_metadata
from zse_b200.cache.block_pool import Block, BlockPool
from zse_b200.cache.dedup import BlockDedup, _fnv1a_hash, fnv1a_chain
from zse_b200.cache.evictor import Evictor


def pool(n=8, bs=16, layers=2, kvh=2, hd=64):
    return BlockPool(n, bs, layers, kvh, hd, device=None)


# ---- block pool -------------------------------------------------------------------------------------------------
def test_pool_sizes_follow_the_geometry():
    p = pool(n=10, bs=16, layers=4, kvh=2, hd=128)
    assert p.bytes_per_token_all_layers == 4 * 2 * 2 * 128 * 2                     # layers x (K,V) x heads x dim x fp16
    assert p.block_bytes == 16 * p.bytes_per_token_all_layers
    assert p.layer_block_bytes == 2 * 2 * 16 * 128 * 2 and p.layer_block_bytes * 4 == p.block_bytes
    assert p.total_bytes == 10 * p.block_bytes and p.used_bytes == 0 and p.utilization == 0.0
    assert p.num_blocks == 10 == p.num_free and p.num_allocated == 0 and p.block_size_tokens == 16
    assert p.is_uniform_kv and p.layer_kv_elems(3) == 2 * 128
    assert p.layer_byte_offset(0) == 0 and p.layer_byte_offset(2) == 2 * 10 * p.layer_block_bytes
    assert p.slab is None
    with pytest.raises(RuntimeError, match="bookkeeping"):
        p.gpu_ptr_for_block(p.alloc())


def test_pool_from_budget_rounds_down_and_refuses_less_than_a_block():
    one = 16 * 2 * 2 * 2 * 64 * 2
    assert BlockPool.from_budget(5 * one + one - 1, 16, 2, 2, 64).num_blocks == 5
    with pytest.raises(ValueError, match="smaller than one block"):
        BlockPool.from_budget(one - 1, 16, 2, 2, 64)
    with pytest.raises(ValueError):
        BlockPool(0, 16, 2, 2, 64)


def test_blocks_are_handed_out_in_order_and_reused_after_free():
    p = pool(n=3)
    a, b, c = p.alloc(seq_id=7), p.alloc(), p.alloc()
    assert [x.block_id for x in (a, b, c)] == [0, 1, 2] and a.seq_id == 7 and b.seq_id is None
    assert a.ref_count == 1 and not a.is_shared and a.num_tokens == 0 and a.content_hash is None
    assert a.gpu_offset == 0 and c.gpu_offset == 2 * p.layer_block_bytes
    assert p.num_free == 0 and p.utilization == 1.0 and p.used_bytes == p.total_bytes
    with pytest.raises(MemoryError, match="exhausted"):
        p.alloc()
    assert p.free(b) is True and p.num_free == 1
    again = p.alloc()
    assert again.block_id == 1 and again is not b                                  # the id comes back, as a new record
    assert p.get_block(1) is again
    with pytest.raises(KeyError):
        pool().get_block(5)


def test_reference_counts_and_double_free():
    p = pool()
    b = p.alloc()
    b.num_tokens, b.content_hash = 16, 123
    p.increment_ref(b)
    p.increment_ref(b)
    assert b.ref_count == 3 and b.is_shared and p.stats()["shared"] == 1
    assert p.free(b) is False and p.free(b) is False and b.ref_count == 1 and not b.is_shared
    assert p.num_allocated == 1                                                    # still owned by someone
    assert p.free(b) is True and (b.num_tokens, b.content_hash) == (0, None)
    with pytest.raises(ValueError, match="double free of KV block 0"):
        p.free(b)
    assert p.stats() == {"num_blocks": 8, "free": 8, "allocated": 0, "block_size_tokens": 16,
                         "block_bytes": p.block_bytes, "shared": 0}


def test_block_fullness_copy_without_a_slab_and_destroy():
    p = pool(bs=16)
    a, b = p.alloc(), p.alloc()
    a.num_tokens = 15
    assert not p.is_block_full(a)
    a.num_tokens = 16
    assert p.is_block_full(a)
    p.copy_block(a, b)                                                             # bookkeeping pool: nothing to copy
    p.destroy()
    assert p.num_free == 0 and p.slab is None
    assert Block(3, layer_block_bytes=100).gpu_offset == 300


def test_addresses_inside_a_slab():
    import torch
    p = BlockPool(4, 16, 3, 2, 8, device="cpu")
    base = p.slab.data_ptr()
    assert p.slab.shape == (3, 4, 2, 2, 16, 8) and p.slab.dtype == torch.float16 and float(p.slab.abs().sum()) == 0.0
    p.alloc()
    b = p.alloc()                                                                  # block 1
    assert p.gpu_ptr_for_block(b) == base + p.layer_block_bytes
    assert p.gpu_ptr_for_block_layer(b, 2) == base + 2 * 4 * p.layer_block_bytes + p.layer_block_bytes
    assert p.gpu_ptr_for_kv(b, 2, False) == p.gpu_ptr_for_block_layer(b, 2)
    assert p.gpu_ptr_for_kv(b, 2, True) == p.gpu_ptr_for_block_layer(b, 2) + p.layer_block_bytes // 2
    assert p.gpu_ptr_for_kv(b, 2, True) == p.slab[2, 1, 1].data_ptr()              # the address of the V half
    src = p.get_block(0)
    p.slab[:, 0] = 1.5
    p.copy_block(src, b)
    assert float(p.slab[:, 1].min()) == 1.5 and float(p.slab[:, 2].abs().max()) == 0.0


# ---- evictor ----------------------------------------------------------------------------------------------------
def fake_clock(start=100.0):
    t = [start]
    return t, (lambda: t[0])


def test_unknown_policy_is_refused():
    with pytest.raises(ValueError, match="unknown eviction policy"):
        Evictor("random")
    assert Evictor.POLICIES == ("lru", "lfu", "smart") and Evictor().policy == "smart"


def test_lru_takes_the_oldest_access_first():
    t, clock = fake_clock()
    e = Evictor("lru", clock)
    for i, bid in enumerate((10, 11, 12)):
        t[0] += 1
        e.record_access(seq_id=1, block_idx=i, block_id=bid, num_tokens=16)
    t[0] += 1
    e.record_access(1, 0, 10, 16)                                                  # block 10 is fresh again
    assert [c.block_id for c in e.select_victims(3)] == [11, 12, 10]
    assert [c.block_id for c in e.select_victims(1)] == [11]
    assert e.select_victims(0) == []


def test_lfu_takes_the_least_used_first():
    t, clock = fake_clock()
    e = Evictor("lfu", clock)
    for bid, n in ((1, 3), (2, 1), (3, 2)):
        for _ in range(n):
            e.record_access(5, bid, bid, 16)
    v = e.select_victims(3)
    assert [c.block_id for c in v] == [2, 3, 1] and [c.score for c in v] == [1.0, 2.0, 3.0]
    assert v[0].seq_id == 5 and v[0].num_tokens == 16 and v[0].block_idx == 2


def test_smart_score_prefers_to_keep_prompt_blocks_and_recent_ones():
    t, clock = fake_clock()
    e = Evictor("smart", clock)
    e.record_access(1, 0, 100, 16, token_start=0, is_prompt=True)
    e.record_access(1, 1, 101, 16, token_start=16, is_prompt=False)
    t[0] += 9.0                                                                    # both are 9 s old: 1/10 + bonus
    by_id = {c.block_id: c.score for c in e.select_victims(2)}
    assert by_id[100] == pytest.approx(0.1 + 2.0) and by_id[101] == pytest.approx(0.1 + 0.5)
    assert [c.block_id for c in e.select_victims(2)] == [101, 100]                 # generated tokens go first
    e.record_access(1, 1, 101, 16)                                                 # used again just now, twice in all
    assert {c.block_id: c.score for c in e.select_victims(2)}[101] == pytest.approx(2.0 + 0.5)


def test_touching_a_sequence_refreshes_all_of_its_blocks():
    t, clock = fake_clock()
    e = Evictor("lru", clock)
    e.record_access(1, 0, 10, 16)
    t[0] += 1
    e.record_access(2, 0, 20, 16)
    t[0] += 1
    e.touch_sequence(1)                                                            # one store instead of one per block
    assert [c.block_id for c in e.select_victims(2)] == [20, 10]
    assert e.now() == t[0]


def test_excluded_sequences_and_removals():
    t, clock = fake_clock()
    e = Evictor("lru", clock)
    e.record_batch_access(1, [10, -1, 12], block_size=16, prompt_len=20)           # -1: a hole, not tracked
    e.record_batch_access(2, [20], block_size=16)
    assert e.stats()["tracked_blocks"] == 3
    assert {c.block_id for c in e.select_victims(10, exclude_seq_ids={1})} == {20}
    infos = {c.block_id: c for c in e.select_victims(10)}
    assert infos[12].block_idx == 2 and infos[10].block_idx == 0
    e.remove_block(12)
    assert {c.block_id for c in e.select_victims(10)} == {10, 20}
    e.remove_block(10, seq_id=2)                                                   # another sequence's entry: untouched
    assert {c.block_id for c in e.select_victims(10)} == {10, 20}
    e.remove_sequence(1)
    assert {c.block_id for c in e.select_victims(10)} == {20}
    e.note_evicted(16)
    e.note_evicted(5)
    assert e.eviction_count == 2 and e.total_tokens_evicted == 21
    assert e.stats() == {"policy": "lru", "tracked_blocks": 1, "eviction_count": 2, "tokens_evicted": 21}


def test_prompt_flag_of_a_batch_access_follows_the_prompt_length():
    t, clock = fake_clock()
    e = Evictor("smart", clock)
    e.record_batch_access(1, [0, 1, 2], block_size=16, prompt_len=17)              # blocks 0 and 1 hold prompt tokens
    scores = {c.block_id: c.score for c in e.select_victims(3)}
    assert scores[0] == scores[1] == pytest.approx(1.0 + 2.0) and scores[2] == pytest.approx(1.0 + 0.5)


# ---- chained block hashes ---------------------------------------------------------------------------------------
def test_fnv1a_matches_the_published_constants():
    assert _fnv1a_hash([]) == 0xCBF29CE484222325                                   # the offset basis
    # one token = its four little-endian bytes
    h = 0xCBF29CE484222325
    for byte in (0x01, 0x00, 0x00, 0x00):
        h = ((h ^ byte) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    assert _fnv1a_hash([1]) == h
    assert _fnv1a_hash([1, 2]) != _fnv1a_hash([2, 1]) and _fnv1a_hash([256]) != _fnv1a_hash([1])
    assert 0 <= fnv1a_chain(12345, [7, 8, 9]) < 2 ** 64
    assert fnv1a_chain(1, [5]) != fnv1a_chain(2, [5])                              # the chain value matters


def test_chain_hashes_cover_full_blocks_only_and_depend_on_the_prefix():
    d = BlockDedup(pool(bs=4))
    toks = list(range(10))
    h = d.chain_hashes(toks)
    assert len(h) == 2                                                             # 10 tokens = 2 full blocks of 4
    assert h[0] == fnv1a_chain(0, toks[:4]) and h[1] == fnv1a_chain(h[0], toks[4:8])
    other = d.chain_hashes([9] + toks[1:])
    assert other[0] != h[0] and other[1] != h[1]                                   # same second block, other prefix
    assert d.chain_hashes(toks, salt=77) != h and d.chain_hashes(toks, salt=77) == d.chain_hashes(toks, salt=77)
    assert d.chain_hashes([1, 2, 3]) == []


def test_lookup_register_and_counters():
    p = pool(bs=4)
    d = BlockDedup(p)
    blk = p.alloc()
    toks = [1, 2, 3, 4]
    h = fnv1a_chain(0, toks)
    assert d.lookup(h, toks) is None and d.dedup_misses == 1
    d.register(blk.block_id, h, toks)
    assert blk.content_hash == h
    assert d.lookup(h, toks) == blk.block_id and d.dedup_hits == 1 and d.hit_rate == 0.5
    assert d.lookup(h, [1, 2, 3, 5]) is None and d.collision_count == 1            # same hash claimed, other tokens
    assert d.lookup(h, toks, prev_hash=9) is None and d.collision_count == 2       # same tokens, other prefix
    other = p.alloc()
    d.register(other.block_id, h, toks)                                            # the hash is taken: ignored
    assert d.lookup(h, toks) == blk.block_id and other.content_hash is None
    assert d.stats() == {"registered": 1, "hits": 2, "misses": 1, "collisions": 2, "hit_rate": 2 / 3}
    d.deregister_block(blk.block_id)
    d.deregister_block(blk.block_id)
    assert d.lookup(h, toks) is None and d.stats()["registered"] == 0
    assert BlockDedup(p).hit_rate == 0.0


def test_register_block_shares_an_identical_block_with_the_same_prefix():
    p = pool(bs=4)
    d = BlockDedup(p)
    a, b, c = p.alloc(), p.alloc(), p.alloc()
    assert d.register_block(a.block_id, [1, 2, 3, 4]) is None                      # first of its kind
    assert d.register_block(b.block_id, [1, 2, 3, 4]) == a.block_id and a.ref_count == 2
    assert d.register_block(c.block_id, [1, 2, 3, 4], prev_hash=5) is None         # another prefix: its own block
    assert a.ref_count == 2 and d.register_block(a.block_id, [1, 2, 3, 4]) is None  # a block never shares with itself


# ---- attention metadata -----------------------------------------------------------------------------------------
def test_metadata_is_padded_with_minus_one():
    m = build_attention_metadata([[3, 4, 5], [7], []], [40, 9, 0], block_size=16)
    assert (m.num_seqs, m.max_seq_len, m.max_blocks_per_seq, m.block_size) == (3, 40, 3, 16)
    arr = m.block_table_array()
    assert arr.dtype == np.int32 and arr.tolist() == [[3, 4, 5], [7, -1, -1], [-1, -1, -1]]
    assert m.block_table_array(width=2).tolist() == [[3, 4], [7, -1], [-1, -1]]
    assert m.block_table_array(width=5).shape == (3, 5)
    assert m.block_tables_nbytes == 3 * 3 * 4 and m.seq_lengths_nbytes == 12
    assert m.is_prefill is None and m.block_tables_gpu_ptr == 0 and m.seq_lengths_gpu_ptr == 0


def test_metadata_packs_little_endian_int32():
    m = build_attention_metadata([[1, -1, 2], [9]], [35, 3], block_size=16)        # -1: a hole left by eviction
    assert m.pack_seq_lengths() == struct.pack("<2i", 35, 3)
    assert m.pack_block_tables() == struct.pack("<6i", 1, -1, 2, 9, -1, -1)
    assert len(m.pack_block_tables()) == m.block_tables_nbytes


def test_metadata_of_an_empty_batch_and_upload_to_cpu():
    e = build_attention_metadata([], [], block_size=16)
    assert (e.num_seqs, e.max_seq_len, e.max_blocks_per_seq) == (0, 0, 0)
    assert e.block_table_array().shape == (0, 1) and e.pack_seq_lengths() == b"" and e.seq_lengths_nbytes == 0
    m = build_attention_metadata([[0, 1]], [20], block_size=16).upload("cpu")
    assert m.block_tables_gpu.tolist() == [[0, 1]] and m.seq_lengths_gpu.tolist() == [20]
    assert m.block_tables_gpu_ptr == m.block_tables_gpu.data_ptr() and m.seq_lengths_gpu_ptr != 0
    src = [[1, 2]]
    built = build_attention_metadata(src, [17], 16)
    src[0].append(3)
    assert built.block_tables == [[1, 2]]                                          # a copy of the page-table state
    assert isinstance(built, AttentionMetadata)


# ---- page table and manager: the accessors -----------------------------------------------------------------------------
def test_page_table_accessors_skip_evicted_blocks():
    from zse_b200.cache.page_table import PageTable
    p = pool(n=6, bs=16)
    pt = PageTable(p)
    pt.create_sequence(7)
    pt.append_tokens(7, 40)                                                       # 3 blocks: 16 + 16 + 8
    assert pt.get_entry_or_none(7) is pt.get_entry(7) and pt.get_entry_or_none(8) is None
    assert pt.get_all_sequences() == [7] and pt.blocks_needed(7, 8) == 0 and pt.blocks_needed(7, 9) == 1
    e = pt.get_entry(7)
    assert (e.num_blocks, e.num_live_blocks) == (3, 3) and [b.num_tokens for b in pt.get_blocks(7)] == [16, 16, 8]
    gone = pt.evict_block(7, 0)
    assert gone is not None and pt.evict_block(7, 0) is None and pt.evict_block(7, 9) is None
    assert (e.num_blocks, e.num_live_blocks, e.tokens_evicted) == (3, 2, 16)
    assert pt.get_block_ids(7)[0] == -1 and len(pt.get_blocks(7)) == 2 and pt.get_blocks(99) == []
    assert pt.stats() == {"num_sequences": 1, "total_tokens": 40, "total_blocks": 2}
    assert p.num_free == 4
    assert len(pt.remove_sequence(7)) == 2 and p.num_free == 6 and pt.remove_sequence(7) == []


def test_manager_evicts_idle_sequences_before_active_ones():
    from zse_b200.cache.cache_manager import KVCacheManager
    from zse_b200.format import synth
    m = KVCacheManager(synth.shape_config("tiny"), num_blocks=6, block_size=16, enable_dedup=False)
    assert m.max_tokens_capacity == 96 and m.num_total_blocks == 6
    m.allocate_sequence(1, num_tokens=32)
    m.allocate_sequence(2, num_tokens=32)
    m.mark_active(1)
    m.mark_idle(2)
    assert m.num_free_blocks == 2 and m.evict_if_needed(2) is True and m.num_free_blocks == 2   # enough already
    assert m.evict_if_needed(4) is True and m.num_free_blocks >= 4
    assert m.get_block_ids(2).count(-1) == 2 and m.get_block_ids(1).count(-1) == 0             # the idle one paid
    assert m.evict_if_needed(6) is True                                           # then the active one has to
    assert m.get_block_ids(1).count(-1) == 2 and m.num_free_blocks == 6
    assert m.evict_if_needed(7) is False                                          # more than the pool holds
    m.free_sequence(1)
    m.free_sequence(2)
    m.free_sequence(2)
    assert m.num_sequences == 0 and m.num_free_blocks == 6

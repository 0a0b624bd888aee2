"""Unit tests of the device memory plan (the VRAM planner section of the reference's tests/test_orchestrator.py,
including its "7B on one GPU" plan): the budget rule, the demand rule for the KV cache, its caps, tensor-parallel
shards, and what happens when nothing is left."""
import pytest

from zse_b200.format import synth
from zse_b200.runtime.vram import GB, MB, VRAMAllocator, VRAMPlan


def test_usable_budget_is_total_minus_context_minus_five_percent():
    a = VRAMAllocator(80 * GB)
    assert a.usable_bytes == int((80 * GB - 400 * MB) * 0.95)
    assert a.free_bytes == 80 * GB                                                  # free defaults to the total
    assert VRAMAllocator(80 * GB, free_bytes=70 * GB).free_bytes == 70 * GB
    assert (a.CONTEXT_RESERVE, a.SAFETY_FRACTION, a.KV_FLOOR, a.FREE_MARGIN) == (400 * MB, 0.05, 256 * MB, 1 * GB)


def test_plan_for_the_7b_shape_on_a_b200():
    """The reference's headline configuration: 7B INT4, one GPU, 2048-token context, one sequence."""
    c = synth.shape_config("qwen2.5-7b")
    per_token = c.total_kv_cache_bytes_per_token
    assert per_token == c.num_layers * 2 * c.num_kv_heads * c.head_dim * 2 == 57344
    a = VRAMAllocator(180 * GB)
    weights, scratch = int(5.2 * GB), int(0.6 * GB)
    p = a.plan_allocation(c, weights, scratch, block_size=16, max_seq_len=2048, max_batch_seqs=1)
    # demand: 1 x 2048 tokens x 1.5 = 176 MB -> the 256 MB floor applies
    assert p.kv_cache_bytes <= 256 * MB and p.kv_blocks == (256 * MB) // (per_token * 16)
    assert p.kv_cache_bytes == p.kv_blocks * per_token * 16 and p.max_batch_tokens == p.kv_blocks * 16
    assert p.max_batch_tokens >= 2048                                               # the context fits
    assert (p.weight_bytes, p.scratch_bytes, p.block_size, p.max_seq_len, p.max_batch_seqs) == \
        (weights, scratch, 16, 2048, 1)
    assert p.total_vram == 180 * GB and p.usable_bytes == a.usable_bytes
    assert p.utilization_pct == pytest.approx(100.0 * (weights + scratch + p.kv_cache_bytes) / (180 * GB))
    text = p.summary()
    assert "weights 5.20 GB" in text and f"{p.kv_blocks} blocks x 16 tokens" in text and "1 sequences" in text


def test_kv_cache_follows_demand_for_a_serving_batch():
    c = synth.shape_config("qwen2.5-14b")
    per_token = c.total_kv_cache_bytes_per_token
    a = VRAMAllocator(180 * GB)
    p = a.plan_allocation(c, 9 * GB, 1 * GB, block_size=16, max_seq_len=4096, max_batch_seqs=64)
    want = int(64 * 4096 * per_token * 1.5)
    assert p.kv_blocks == want // (per_token * 16)
    assert p.max_batch_tokens >= 64 * 4096                                          # every sequence at full length
    bigger = a.plan_allocation(c, 9 * GB, 1 * GB, 16, 4096, 128)
    assert bigger.kv_blocks == pytest.approx(2 * p.kv_blocks, abs=1)


def test_demand_is_capped_by_what_remains():
    c = synth.shape_config("qwen2.5-14b")
    a = VRAMAllocator(24 * GB)                                                      # a small card
    p = a.plan_allocation(c, 9 * GB, 1 * GB, 16, 8192, 256)                         # demand far above the card
    remaining = a.usable_bytes - 10 * GB
    assert p.kv_cache_bytes <= remaining and remaining - p.kv_cache_bytes < c.total_kv_cache_bytes_per_token * 16
    assert p.reserved_bytes == p.available_vram - p.usable_bytes > 0


def test_free_memory_caps_the_plan_when_others_use_the_device():
    c = synth.shape_config("qwen2.5-7b")
    a = VRAMAllocator(180 * GB, free_bytes=12 * GB)                                 # most of the GPU is taken
    p = a.plan_allocation(c, 5 * GB, 1 * GB, 16, 4096, 64)
    assert p.kv_cache_bytes <= 12 * GB - 1 * GB - 1 * GB                            # free - margin - scratch
    assert p.free_bytes == 12 * GB


def test_kv_fraction_overrides_the_demand_rule():
    c = synth.shape_config("qwen2.5-7b")
    a = VRAMAllocator(180 * GB)
    remaining = a.usable_bytes - 6 * GB
    half = a.plan_allocation(c, 5 * GB, 1 * GB, 16, 2048, 1, kv_fraction=0.5)
    assert abs(half.kv_cache_bytes - remaining // 2) < c.total_kv_cache_bytes_per_token * 16
    full = a.plan_allocation(c, 5 * GB, 1 * GB, 16, 2048, 1, kv_fraction=1.0)
    assert full.kv_blocks == pytest.approx(2 * half.kv_blocks, abs=1)
    over = a.plan_allocation(c, 5 * GB, 1 * GB, 16, 2048, 1, kv_fraction=3.0)       # never more than what is left
    assert over.kv_blocks == full.kv_blocks


def test_a_tensor_parallel_rank_holds_its_share_of_every_token():
    c = synth.shape_config("qwen2.5-72b")
    a = VRAMAllocator(180 * GB)
    one = a.plan_allocation(c, 40 * GB, 2 * GB, 16, 4096, 64, tp_size=1)
    eight = a.plan_allocation(c, 5 * GB, 2 * GB, 16, 4096, 64, tp_size=8)
    # the same number of tokens costs an eighth of the bytes on each of eight ranks (one kv head each)
    assert eight.kv_blocks == one.kv_blocks
    assert eight.kv_cache_bytes * 8 == one.kv_cache_bytes


def test_block_size_changes_the_granularity_not_the_capacity():
    c = synth.shape_config("qwen2.5-7b")
    a = VRAMAllocator(180 * GB)
    p16 = a.plan_allocation(c, 5 * GB, 1 * GB, 16, 4096, 32)
    p64 = a.plan_allocation(c, 5 * GB, 1 * GB, 64, 4096, 32)
    assert p64.block_size == 64 and abs(p16.max_batch_tokens - p64.max_batch_tokens) < 64
    assert p64.kv_blocks == pytest.approx(p16.kv_blocks / 4, abs=1)


def test_no_room_for_a_cache_is_an_error_with_the_numbers():
    c = synth.shape_config("qwen2.5-72b")
    a = VRAMAllocator(40 * GB)
    with pytest.raises(MemoryError, match="no room for a KV cache") as e:
        a.plan_allocation(c, 39 * GB, 1 * GB, 16, 2048, 1)
    assert "39.00 GB" in str(e.value) and "1.00 GB" in str(e.value)
    # the weights alone already exceed the card
    with pytest.raises(MemoryError):
        VRAMAllocator(16 * GB).plan_allocation(c, 40 * GB, 0, 16, 2048, 1)


def test_scratch_shapes_of_the_7b_model():
    c = synth.shape_config("qwen2.5-7b")
    s = VRAMAllocator.scratch_shapes(c, max_seq_len=2048)
    assert set(s) == {"hidden", "residual", "qkv", "attn_out", "mlp_gate", "mlp_up", "mlp_out", "logits", "norm_out",
                      "hidden_f32", "residual_f32"}
    assert s["hidden"] == ((2048, 3584), 2) and s["hidden_f32"] == ((2048, 3584), 4)
    assert s["qkv"][0] == (2048, (28 + 2 * 4) * 128) and s["mlp_gate"][0] == (2048, 18944)
    assert s["logits"][0] == (64, 152064)                                           # logits rows are capped at 64
    assert VRAMAllocator.scratch_shapes(c, max_seq_len=8)["logits"][0] == (8, 152064)
    total = sum(shape[0] * shape[1] * esz for shape, esz in s.values())
    assert 300 * MB < total < 700 * MB


def test_weight_accounting_and_utilisation_without_a_device():
    a = VRAMAllocator(10 * GB)
    assert a.allocated_bytes == 0 == a.weight_bytes
    a.track_weight_upload(3 * GB)
    a.track_weight_upload(1.5 * GB)                                                 # floats are truncated to bytes
    u = a.utilization()
    assert u["weight_bytes"] == int(4.5 * GB) == u["used_bytes"] and u["total_bytes"] == 10 * GB
    assert u["utilization_pct"] == pytest.approx(45.0)
    assert VRAMAllocator(0).utilization()["utilization_pct"] == 0


def test_plan_record_derived_fields():
    p = VRAMPlan(total_bytes=100 * GB, free_bytes=90 * GB, usable_bytes=94 * GB, weight_bytes=10 * GB,
                 scratch_bytes=2 * GB, kv_cache_bytes=8 * GB, kv_blocks=1000, block_size=32, max_seq_len=4096,
                 max_batch_seqs=16)
    assert p.total_vram == 100 * GB and p.available_vram == 100 * GB - 400 * MB
    assert p.reserved_bytes == p.available_vram - 94 * GB and p.max_batch_tokens == 32000
    assert p.utilization_pct == pytest.approx(20.0)
    assert VRAMPlan(0, 0, 0, 0, 0, 0, 0, 16, 1, 1).utilization_pct == 0.0

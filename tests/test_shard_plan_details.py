"""Unit tests of the tensor-parallel sharding rules and of the reference-named primitives that need no process group
(the shape of the reference's tests/test_tensor_parallel.py: configuration checks, split strategy per weight name,
shard ranges and sizes).  Ranks that actually exchange data are covered by tests/test_convert_tp_lora.py (gloo) and
the GPU tests."""
import dataclasses

import pytest
import torch

from zse_b200.format import synth
from zse_b200.parallel.shard_plan import ShardPlan, all_plans, make_plan, split_units, validate_tp
from zse_b200.parallel.tensor_parallel import (COLUMN_PARALLEL, NON_LAYER_SPLIT_MAP, REPLICATED, ROW_PARALLEL,
                                               WEIGHT_SPLIT_MAP, TensorParallelGroup, TPConfig)


def group_of(tp_size, rank):
    """A group object with only its geometry set (no process group): enough for the sharding arithmetic."""
    g = TensorParallelGroup.__new__(TensorParallelGroup)
    g.tp_size, g.rank, g.backend, g._comm, g._owns_group = tp_size, rank, "cpu", None, False
    return g


# ---- split_units ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("total,parts", [(108, 8), (231, 8), (8, 8), (5, 8), (0, 4), (152064, 8), (7, 1), (13, 2)])
def test_split_units_is_a_partition_with_the_extras_first(total, parts):
    r = split_units(total, parts)
    assert len(r) == parts and r[0][0] == 0 and r[-1][1] == total
    assert all(r[i][1] == r[i + 1][0] for i in range(parts - 1))                   # contiguous, in order
    sizes = [b - a for a, b in r]
    assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)   # the larger shards come first
    assert sizes.count(max(sizes)) == (total % parts or parts)


# ---- plans of the served shapes ---------------------------------------------------------------------------------
def test_plans_of_the_14b_shape_on_eight_ranks():
    c = synth.shape_config("qwen2.5-14b")
    plans = all_plans(c, 8)
    assert [p.rank for p in plans] == list(range(8)) and all(p.tp_size == 8 and p.group == 128 for p in plans)
    assert all(p.num_heads == 5 and p.num_kv_heads == 1 and p.head_dim == 128 for p in plans)
    assert all(p.q_dim == 640 and p.kv_dim == 128 for p in plans)
    assert plans[3].q_rows == (1920, 2560) and plans[3].kv_rows == (384, 512)
    # 13824 = 108 groups of 128: four ranks get 14 groups, four get 13 - never half a group
    assert [p.inter_size // 128 for p in plans] == [14, 14, 14, 14, 13, 13, 13, 13]
    assert all(p.inter[0] % 128 == 0 and p.inter[1] % 128 == 0 for p in plans)
    assert plans[0].inter == (0, 1792) and plans[-1].inter[1] == 13824
    assert all(p.vocab_size == 19008 for p in plans) and plans[-1].vocab == (133056, 152064)


def test_plans_of_the_72b_shape_on_eight_ranks():
    c = synth.shape_config("qwen2.5-72b")
    plans = all_plans(c, 8)
    assert [p.inter_size // 128 for p in plans] == [29] * 7 + [28]                 # 29568 = 231 groups
    assert all(p.num_heads == 8 and p.num_kv_heads == 1 for p in plans)


@pytest.mark.parametrize("shape,tp", [("qwen2.5-7b", 2), ("qwen2.5-7b", 4), ("qwen2.5-14b", 2), ("qwen2.5-14b", 4),
                                      ("qwen2.5-32b", 8), ("small-uneven", 2), ("tiny", 2)])
def test_shards_cover_every_dimension_exactly_once(shape, tp):
    c = synth.shape_config(shape)
    plans = all_plans(c, tp)
    for field, total in (("q_rows", c.num_heads * c.head_dim), ("kv_rows", c.num_kv_heads * c.head_dim),
                         ("inter", c.intermediate_size), ("vocab", c.vocab_size)):
        ranges = [getattr(p, field) for p in plans]
        assert ranges[0][0] == 0 and ranges[-1][1] == total
        assert all(ranges[i][1] == ranges[i + 1][0] for i in range(tp - 1))
    assert sum(p.num_heads for p in plans) == c.num_heads and sum(p.num_kv_heads for p in plans) == c.num_kv_heads
    assert len({p.num_heads // p.num_kv_heads for p in plans}) == 1                # the GQA ratio is kept on every rank


def test_a_plan_for_one_rank_is_the_whole_model():
    c = synth.shape_config("qwen2.5-7b")
    p = make_plan(c)
    assert (p.tp_size, p.rank, p.num_heads, p.num_kv_heads) == (1, 0, c.num_heads, c.num_kv_heads)
    assert p.q_rows == (0, c.num_heads * c.head_dim) and p.inter == (0, c.intermediate_size)
    assert p.vocab == (0, c.vocab_size) and p.vocab_size == c.vocab_size
    assert dataclasses.is_dataclass(ShardPlan)


def test_what_cannot_be_split_is_refused_with_its_reasons():
    c = synth.shape_config("qwen2.5-14b")                                          # 40 heads, 8 kv heads
    assert validate_tp(c, 8) == [] and validate_tp(c, 1) == []
    errs = validate_tp(c, 3)
    assert len(errs) == 2 and "num_heads (40)" in errs[0] and "num_kv_heads (8)" in errs[1]
    c72 = synth.shape_config("qwen2.5-72b")                                        # 64 heads, 8 kv heads
    assert validate_tp(c72, 16) == ["num_kv_heads (8) not divisible by tp_size (16)"]
    assert validate_tp(c, 0) == ["tp_size must be >= 1"]
    with pytest.raises(ValueError, match="num_kv_heads"):
        make_plan(c, 16, 0)
    with pytest.raises(ValueError, match="rank 8 outside"):
        make_plan(c, 8, 8)
    with pytest.raises(ValueError, match="rank -1 outside"):
        make_plan(c, 8, -1)


def test_an_intermediate_size_without_group_structure_is_split_evenly():
    c = synth.shape_config("tiny")
    c = dataclasses.replace(c, intermediate_size=100)                              # not a multiple of the group size
    plans = all_plans(c, 2) if c.num_kv_heads % 2 == 0 else None
    if plans is not None:
        assert [p.inter for p in plans] == [(0, 50), (50, 100)]


# ---- TPConfig ---------------------------------------------------------------------------------------------------
def test_tp_config_enabled_and_validation():
    assert not TPConfig().is_enabled() and TPConfig().tp_size == 1 and TPConfig().backend == "cuda"
    assert TPConfig(tp_size=2).is_enabled()
    TPConfig(tp_size=1).validate(7, 3, 0)                                          # one rank: nothing to check
    TPConfig(tp_size=4).validate(32, 8, 11008)
    with pytest.raises(ValueError, match="num_heads \\(30\\)"):
        TPConfig(tp_size=4).validate(30, 8, 11008)
    with pytest.raises(ValueError, match="num_kv_heads \\(2\\)"):
        TPConfig(tp_size=4).validate(32, 2, 11008)
    with pytest.raises(ValueError, match="intermediate_size"):
        TPConfig(tp_size=4).validate(32, 8, 3)


# ---- split strategy per weight name -----------------------------------------------------------------------------
def test_split_maps_name_every_projection_once():
    cols = {k for k, v in WEIGHT_SPLIT_MAP.items() if v == COLUMN_PARALLEL}
    rows = {k for k, v in WEIGHT_SPLIT_MAP.items() if v == ROW_PARALLEL}
    assert rows == {"self_attn.o_proj.weight", "mlp.down_proj.weight"}
    assert {"self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight", "mlp.gate_proj.weight",
            "mlp.up_proj.weight", "self_attn.q_proj.bias"} <= cols
    assert WEIGHT_SPLIT_MAP["input_layernorm.weight"] == REPLICATED
    assert NON_LAYER_SPLIT_MAP["lm_head.weight"] == COLUMN_PARALLEL and NON_LAYER_SPLIT_MAP["embed_tokens.weight"] == REPLICATED
    assert {COLUMN_PARALLEL, ROW_PARALLEL, REPLICATED} == {"column", "row", "replicated"}


def test_strategy_lookup_by_full_tensor_name():
    g = group_of(4, 1)
    assert g.get_split_strategy("model.layers.17.self_attn.q_proj.weight") == COLUMN_PARALLEL
    assert g.get_split_strategy("model.layers.17.self_attn.k_proj.bias") == COLUMN_PARALLEL
    assert g.get_split_strategy("model.layers.0.self_attn.o_proj.weight") == ROW_PARALLEL
    assert g.get_split_strategy("model.layers.3.mlp.down_proj.weight") == ROW_PARALLEL
    assert g.get_split_strategy("model.layers.3.mlp.up_proj.weight") == COLUMN_PARALLEL
    assert g.get_split_strategy("model.layers.3.post_attention_layernorm.weight") == REPLICATED
    assert g.get_split_strategy("model.embed_tokens.weight") == REPLICATED
    assert g.get_split_strategy("model.norm.weight") == REPLICATED
    assert g.get_split_strategy("lm_head.weight") == COLUMN_PARALLEL
    assert g.get_split_strategy("something.else.entirely") == REPLICATED            # unknown tensors are not cut


# ---- shard ranges and sizes -------------------------------------------------------------------------------------
def test_shard_ranges_even_uneven_and_unit_aligned():
    assert [group_of(4, r).compute_shard_range(4096, COLUMN_PARALLEL) for r in range(4)] == \
        [(0, 1024), (1024, 2048), (2048, 3072), (3072, 4096)]
    assert [group_of(4, r).shard_size(10, ROW_PARALLEL) for r in range(4)] == [3, 3, 2, 2]
    # borders on multiples of the unit (a head, a quantisation group)
    got = [group_of(8, r).compute_shard_range(13824, ROW_PARALLEL, unit=128) for r in range(8)]
    assert [b - a for a, b in got] == [1792] * 4 + [1664] * 4 and all(a % 128 == 0 for a, _ in got)
    assert got[0][0] == 0 and got[-1][1] == 13824
    # a size that is not a multiple of the unit falls back to an even split
    assert group_of(2, 1).compute_shard_range(100, COLUMN_PARALLEL, unit=128) == (50, 100)
    # replicated tensors and single-rank groups keep everything
    assert group_of(4, 2).compute_shard_range(777, REPLICATED) == (0, 777)
    assert group_of(1, 0).compute_shard_range(777, COLUMN_PARALLEL) == (0, 777)
    assert group_of(1, 0).shard_size(777, ROW_PARALLEL, unit=128) == 777


def test_shard_byte_sizes_of_a_7b_layer():
    """INT4 bytes per rank at tp 2 for the 7B shape: what the loader will allocate."""
    c = synth.shape_config("qwen2.5-7b")
    H, I, q, kv = c.hidden_size, c.intermediate_size, c.num_heads * c.head_dim, c.num_kv_heads * c.head_dim
    total = 0
    for r in range(2):
        g = group_of(2, r)
        rows_q = g.shard_size(q, COLUMN_PARALLEL, unit=c.head_dim)
        rows_kv = g.shard_size(kv, COLUMN_PARALLEL, unit=c.head_dim)
        cols_o = g.shard_size(q, ROW_PARALLEL, unit=c.head_dim)
        inter = g.shard_size(I, COLUMN_PARALLEL, unit=128)
        layer_bytes = ((rows_q + 2 * rows_kv) * H + H * cols_o + 2 * inter * H + H * inter) // 2
        total += layer_bytes
    full = ((q + 2 * kv) * H + H * q + 3 * I * H) // 2
    assert total == full                                                            # nothing duplicated, nothing lost


# ---- a single-rank group needs no process group -----------------------------------------------------------------
def test_single_rank_group_collectives_are_identities():
    g = TensorParallelGroup(1, 0, backend="cpu")
    t = torch.arange(6.0)
    before = t.clone()
    g.all_reduce_inplace(t)
    assert torch.equal(t, before)
    assert g.all_gather(t) is t and g.broadcast(t) is t and g.reduce_scatter(t) is t
    g.barrier()
    g.sync_stream()
    g.destroy()
    assert repr(g) == "TensorParallelGroup(tp=1, rank=0, backend=cpu)"


def test_a_multi_rank_group_needs_a_rendezvous_address():
    import torch.distributed as dist
    if dist.is_initialized():
        pytest.skip("a process group already exists in this process")
    with pytest.raises(ValueError, match="unique_id"):
        TensorParallelGroup(2, 0, backend="cpu")

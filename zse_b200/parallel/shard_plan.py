"""Megatron-style tensor-parallel sharding plan for the decoder.

Column-parallel: q/k/v (+bias), gate, up, lm_head (rows split).  Row-parallel: o_proj, down_proj (K split).
Replicated: embedding, norms.  Same split map as zse-engine/zse_engine/orchestrator/tensor_parallel.py:41-64,
with two differences that matter for the INT4 shapes actually served:

* K shards of the row-parallel layers fall on quantisation-group boundaries (multiples of 128), so shards may be
  uneven: intermediate 13824 at tp 8 is 108 groups = 4 x 14 + 4 x 13; 29568 is 231 groups = 7 x 29 + 1 x 28.
  gate/up use the same boundaries as down's K shards.  (The reference slices ``K/tp`` blindly,
  tp_weight_loader.py:307-317, which cuts groups in half for these shapes.)
* lm_head rows are split and the logits are gathered/arg-reduced across ranks; the reference shards the weight but
  still launches the full-vocabulary GEMV (model_runner.py:368-373).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple

from ..format.config import ModelConfig


def split_units(total_units: int, parts: int) -> List[Tuple[int, int]]:
    """Contiguous ranges of ``total_units`` over ``parts``; the first ``total % parts`` ranges get one extra."""
    base, extra = divmod(total_units, parts)
    out, at = [], 0
    for r in range(parts):
        n = base + (1 if r < extra else 0)
        out.append((at, at + n))
        at += n
    return out


@dataclass
class ShardPlan:
    tp_size: int
    rank: int
    num_heads: int            # local query heads
    num_kv_heads: int         # local kv heads
    head_dim: int
    q_rows: Tuple[int, int]   # row range of q_proj owned by this rank
    kv_rows: Tuple[int, int]  # row range of k_proj / v_proj
    inter: Tuple[int, int]    # range of the intermediate dimension (gate/up rows, down columns)
    vocab: Tuple[int, int]    # lm_head row range
    group: int

    @property
    def q_dim(self) -> int:
        return self.q_rows[1] - self.q_rows[0]

    @property
    def kv_dim(self) -> int:
        return self.kv_rows[1] - self.kv_rows[0]

    @property
    def inter_size(self) -> int:
        return self.inter[1] - self.inter[0]

    @property
    def vocab_size(self) -> int:
        return self.vocab[1] - self.vocab[0]


def validate_tp(config: ModelConfig, tp_size: int) -> List[str]:
    """Reasons why this model cannot be split ``tp_size`` ways (empty = fine)."""
    errs = []
    if tp_size < 1:
        errs.append("tp_size must be >= 1")
        return errs
    if config.num_heads % tp_size:
        errs.append(f"num_heads ({config.num_heads}) not divisible by tp_size ({tp_size})")
    if config.num_kv_heads % tp_size:
        errs.append(f"num_kv_heads ({config.num_kv_heads}) not divisible by tp_size ({tp_size})")
    if config.is_gemma:                                  # layers may differ in their kv-head count
        for n in sorted({config.layer_spec(i).num_kv_heads for i in range(config.num_layers)}):
            if n % tp_size:
                errs.append(f"a layer kind has {n} kv heads, not divisible by tp_size ({tp_size})")
    if config.intermediate_size < tp_size:
        errs.append(f"intermediate_size ({config.intermediate_size}) smaller than tp_size ({tp_size})")
    return errs


def make_plan(config: ModelConfig, tp_size: int = 1, rank: int = 0) -> ShardPlan:
    errs = validate_tp(config, tp_size)
    if errs:
        raise ValueError("; ".join(errs))
    if not 0 <= rank < tp_size:
        raise ValueError(f"rank {rank} outside [0, {tp_size})")
    c = config
    nh, nkv = c.num_heads // tp_size, c.num_kv_heads // tp_size
    gs = c.quant.group_size or 128
    if c.intermediate_size % gs == 0:
        a, b = split_units(c.intermediate_size // gs, tp_size)[rank]
        inter = (a * gs, b * gs)
    else:  # no group structure to respect along K (flat groups straddle rows): split evenly
        inter = split_units(c.intermediate_size, tp_size)[rank]
    return ShardPlan(tp_size, rank, nh, nkv, c.head_dim, (rank * nh * c.head_dim, (rank + 1) * nh * c.head_dim),
                     (rank * nkv * c.head_dim, (rank + 1) * nkv * c.head_dim), inter,
                     split_units(c.vocab_size, tp_size)[rank], gs)


def all_plans(config: ModelConfig, tp_size: int) -> List[ShardPlan]:
    return [make_plan(config, tp_size, r) for r in range(tp_size)]

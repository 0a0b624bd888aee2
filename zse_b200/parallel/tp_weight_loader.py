"""Per-rank weight shards by stored name (zse-engine/zse_engine/orchestrator/tp_weight_loader.py:25-355).

``TPWeightLoader(loader, device, tp_group).load_all()`` returns a ``WeightStore`` in which every column-parallel tensor
(q/k/v, gate/up, their biases, ``lm_head``) holds this rank's rows and every row-parallel tensor (o, down) this rank's
input columns, with the matching slices of the scales and zero points; norms and the embedding are whole.  Shard
borders come from ``parallel/shard_plan.py`` (heads for attention, quantisation groups for the MLP), per layer for
Gemma-4 whose layers differ in head size and kv-head count.  The engine's own model classes slice the same way while
they fuse projections and re-tile them (``models/decoder.py``); this loader is for code that works on named tensors.

A tensor whose flattened quantisation groups straddle rows (K not a multiple of the group size) cannot be sliced in
packed form: its shard is stored dequantised, as fp16.
"""
from __future__ import annotations

import re
from typing import Callable, Optional, Tuple

import numpy as np
import torch

from ..format import quantize as _q
from ..runtime.weight_stream import GPUWeight, WeightStore
from .shard_plan import make_plan

_LAYER = re.compile(r"^(?:model\.)?layers\.(\d+)\.(.+)$")


def _to_dev(a: np.ndarray, device) -> torch.Tensor:
    return torch.from_numpy(np.array(a, copy=True)).to(device)


class TPWeightLoader:
    def __init__(self, loader, device, tp_group):
        """``tp_group``: anything with ``tp_size`` and ``rank`` (a ``TensorParallelGroup``, a ``ShardPlan``)."""
        self._loader = loader
        self._device = torch.device(device) if not hasattr(device, "type") else device
        self._tp_size, self._rank = int(tp_group.tp_size), int(tp_group.rank)
        self._config = loader.config
        self._plan = make_plan(self._config, self._tp_size, self._rank)

    # ---- which part of a tensor this rank owns ----------------------------------------------------------------
    def shard_ranges(self, name: str) -> Tuple[Optional[Tuple[int, int]], Optional[Tuple[int, int]]]:
        """(row range, column range) of ``name`` for this rank; ``None`` = the whole dimension."""
        p, c = self._plan, self._config
        if self._tp_size <= 1:
            return None, None
        m = _LAYER.match(name)
        if m is None:
            return (p.vocab, None) if name.endswith("lm_head.weight") else (None, None)
        layer, rest = int(m.group(1)), m.group(2)
        hd, nkv = c.head_dim, c.num_kv_heads // self._tp_size
        if c.is_gemma:
            sp = c.layer_spec(layer)
            hd, nkv = sp.head_dim, sp.num_kv_heads // self._tp_size
        q = (self._rank * p.num_heads * hd, (self._rank + 1) * p.num_heads * hd)
        kv = (self._rank * nkv * hd, (self._rank + 1) * nkv * hd)
        if rest.startswith("self_attn.q_proj."):
            return q, None
        if rest.startswith("self_attn.k_proj.") or rest.startswith("self_attn.v_proj."):
            return kv, None
        if rest == "self_attn.o_proj.weight":
            return None, q
        if rest.startswith("mlp.gate_proj.") or rest.startswith("mlp.up_proj."):
            return p.inter, None
        if rest == "mlp.down_proj.weight":
            return None, p.inter
        return None, None

    def stacked_row_ranges(self, name: str):
        """Phi-3 keeps ``[q; k; v]`` and ``[gate; up]`` stacked in one tensor each: this rank's rows are one range per
        stacked part.  ``None`` for every other tensor."""
        m = _LAYER.match(name)
        if m is None or self._tp_size <= 1:
            return None
        p, c, rest = self._plan, self._config, m.group(2)
        if rest == "self_attn.qkv_proj.weight":
            Q, KV = c.num_heads * c.head_dim, c.num_kv_heads * c.head_dim
            (q0, q1), (k0, k1) = p.q_rows, p.kv_rows
            return [(q0, q1), (Q + k0, Q + k1), (Q + KV + k0, Q + KV + k1)]
        if rest == "mlp.gate_up_proj.weight":
            I, (a, b) = c.intermediate_size, p.inter
            return [(a, b), (I + a, I + b)]
        return None

    # ---- loading --------------------------------------------------------------------------------------------------
    def _part(self, e, rows, cols) -> dict:
        from ..models.decoder import _entry_part
        part = _entry_part(self._loader, e.name, rows, cols)
        if "flat_data" in part:
            n = part["flat_shape"][0] * part["flat_shape"][1]
            full = _q.dequantize_int4_arrays(part["flat_data"], part["flat_scales"], part["flat_zeros"], n,
                                             e.group_size)
            full = np.asarray(full, np.float32).reshape(part["flat_shape"])
            (r0, r1), (c0, c1) = part["rows"], part["cols"]
            part = {"dtype": "float16", "data": full[r0:r1, c0:c1].astype(np.float16), "shape": part["shape"]}
        return part

    def _load_one(self, e) -> GPUWeight:
        if len(e.shape) != 2:
            rows, _ = self.shard_ranges(e.name)
            v = self._loader.view_data(e).reshape(-1)
            if rows is not None:
                v = v[rows[0]:rows[1]]
            return GPUWeight(e.name, v.shape, e.dtype, _to_dev(v, self._device), None, None, e.group_size,
                             e.quant_method)
        stacked = self.stacked_row_ranges(e.name)
        if stacked is not None:
            parts = [self._part(e, r, None) for r in stacked]
        else:
            rows, cols = self.shard_ranges(e.name)
            parts = [self._part(e, rows, cols)]
        dtype = parts[0]["dtype"]
        cat = lambda key: (_to_dev(np.concatenate([np.asarray(p[key]) for p in parts], axis=0), self._device)
                           if key in parts[0] else None)
        shape = (sum(int(p["shape"][0]) for p in parts), int(parts[0]["shape"][1]))
        return GPUWeight(e.name, shape, dtype, cat("data"), cat("scales"), cat("zeros"), e.group_size,
                         e.quant_method if dtype == e.dtype else 0)

    def load_all(self, progress_fn: Optional[Callable[[str, int, int], None]] = None) -> WeightStore:
        store = WeightStore()
        entries = list(self._loader.weight_index)
        for i, e in enumerate(entries):
            store.add(self._load_one(e))
            if progress_fn is not None:
                progress_fn(e.name, i + 1, len(entries))
        return store

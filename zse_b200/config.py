"""One configuration object for the engine, filled from CLI flags and ``ZSE_*`` environment variables.

The reference scatters these knobs over argparse, dataclasses and env vars and cannot reach e.g. the prefill chunk
size or the speculative depth from the command line (zse-engine/zse_engine/cli.py:213-285)."""
from __future__ import annotations

import os
from dataclasses import dataclass, field, fields
from typing import Optional


def _env(name: str, default, cast):
    v = os.environ.get(name)
    if v is None:
        return default
    if cast is bool:
        return v.lower() in ("1", "true", "yes", "on")
    return cast(v)


@dataclass
class EngineConfig:
    tp_size: int = 1
    device_index: int = 0
    max_seq_len: int = 0                  # 0 = model maximum, capped at 32768
    block_size: int = 0                   # 0 = adaptive
    max_batch_seqs: int = 64
    max_batch_tokens: int = 4096
    max_prefill_per_step: int = 8
    prefill_chunk_size: int = 2048
    decode_per_prefill: int = 4
    enable_preemption: bool = True
    max_queue_size: int = 256
    speculative_k: int = 0
    speculative_mode: str = "ngram"       # "ngram" | "self"
    use_cuda_graphs: bool = True
    # pipelined decode: launch step n+1 (its input tokens gathered on the device) before step n has been read, so the
    # device does not wait for the host between steps; None = take ZSE_PIPELINE_DECODE (default on)
    pipeline_decode: Optional[bool] = None
    comm_backend: str = "fused"           # tensor-parallel collectives: "fused" (in-kernel NVLink) | "nccl"
    headroom_ratio: float = 0.5
    kv_fraction: Optional[float] = None   # share of free memory for the KV cache (None = demand rule)
    kv_blocks: int = 0                    # explicit KV block count (tests)
    eviction_policy: str = "smart"
    enable_prefix_cache: bool = True
    int4_layout: Optional[str] = None     # override for files that do not record their INT4 layout
    device: Optional[str] = None          # "cpu" forces the torch path
    quiet: bool = True

    @classmethod
    def from_env(cls, **overrides) -> "EngineConfig":
        c = cls()
        for f in fields(cls):
            name = "ZSE_" + f.name.upper()
            cur = getattr(c, f.name)
            cast = type(cur) if cur is not None else str
            if f.name == "kv_fraction":
                cast = float
            if f.name == "pipeline_decode":
                cast = bool
            setattr(c, f.name, _env(name, cur, cast))
        for k, v in overrides.items():
            if v is not None:
                setattr(c, k, v)
        return c

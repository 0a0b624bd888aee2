"""Environment switches of the package in one place: every ``ZSE_*`` variable that any module reads is declared here
with its default and what it does, modules read them through ``flag`` / ``integer`` / ``text``, and ``zse info --env``
prints the table.  (The reference documents its variables where they are read, e.g. ``ZSE_LOAD_CHUNK_MB`` and
``ZSE_LOAD_RING`` in zse-engine/zse_engine/orchestrator/weight_loader.py; ``EngineConfig.from_env`` covers the
engine-level settings, this module the lower-level switches.)"""
from __future__ import annotations

import os
from typing import Dict, List, Tuple

_FALSE = {"0", "", "false", "off", "no"}

# name -> (default as the user would write it, description)
KNOWN: Dict[str, Tuple[str, str]] = {
    "ZSE_LOAD_CHUNK_MB": ("64", "size of one pinned staging buffer of the weight streamer, in MiB"),
    "ZSE_LOAD_RING": ("6", "number of pinned staging buffers of the weight streamer"),
    "ZSE_STREAM_WEIGHTS": ("1", "stream the weight section to the device through the pinned ring (0: per-tensor copies)"),
    "ZSE_NATIVE_STEP": ("1", "launch whole passes from the C++ step driver where it applies (0: Python wiring)"),
    "ZSE_PIPELINE_DECODE": ("1", "launch decode step n+1 before step n has been read (0: one step at a time)"),
    "ZSE_NVTX": ("0", "wrap passes in NVTX ranges"),
    "ZSE_KERNEL_CACHE": ("~/.cache/zse_b200/kernels", "directory of the kernel language's cubin cache"),
    "ZSE_TP_MULTIMEM": ("1", "use NVSwitch multimem loads in the fused exchange where the fabric offers them"),
    "ZSE_TP_PUSH": ("0", "let the row-parallel GEMM push its rows to the peers from its epilogue"),
    "ZSE_TP_FUSED_K1": ("0", "decode-sized passes: row-parallel GEMM + all-reduce + residual + RMSNorm as ONE kernel "
                             "(1) or as GEMM + one exchange kernel (0, the default: measured faster on 2, 4 and 8 "
                             "GPUs)"),
    "ZSE_TP_FUSED_GATHER": ("1", "fused collectives: sampling with temperature gathers the vocabulary shards of the logits "
                                 "with peer stores instead of ncclAllGather"),
    "ZSE_TP_TWO_SHOT_ROWS": (str(1 << 30), "passes of at least this many rows take the two-shot reduce-scatter kernel"),
    "ZSE_TP_NCCL_ROWS": ("256", "passes of at least this many rows take NCCL instead of the fused exchange"),
    "ZSE_TP_FUSED_SP_ROWS": ("128", "fused collectives: passes of at least this many rows scatter the row-parallel GEMM's "
                                    "tiles to row-block owners and gather in the next GEMM's prologue (0: off)"),
    "ZSE_TP_SP": ("0", "sequence-parallel prefill on the NCCL path (reduce-scatter / all-gather, residual split by rows)"),
    "ZSE_TP_SP_MIN_ROWS": ("256", "smallest pass that takes the sequence-parallel path"),
    "ZSE_W4_DEC": ("3", "decode-sized INT4 layers through the persistent kernel: 1 gate/up + SwiGLU, 2 fused QKV + RoPE + "
                         "cache write, 4 every other INT4 linear, 8 o / down with residual add + RMSNorm in the kernel "
                         "(sum of the bits; 0: the tiled kernel everywhere; 8 measured slower than the separate "
                         "add+norm kernel on one GPU, so it is off by default)"),
    "ZSE_W8_RESIDENT": ("1", "keep INT8 weights 8 bits wide on the device (0: expand them to fp16 at load)"),
    "ZSE_ATTN_PREFILL_TC": ("1", "prefill attention of head_dim 128 models on the tcgen05 kernel (csrc/attention_tc.cu); "
                                 "0: the mma.sync kernel for every shape"),
    "ZSE_NATIVE_LIB": ("", "path of the native library to load instead of the ordinary build (instrumented variants)"),
    "ZSE_DEBUG_LOAD": ("0", "print the traceback when the streamed weight load fails and the loader falls back to "
                       "per-tensor copies"),
    "ZSE_PDL": ("1", "programmatic dependent launch between the kernels of a pass (read by the native library); 0 is a "
                "diagnostic setting for per-kernel timing, not a serving configuration"),
    "ZSE_TP_PDL": ("0", "programmatic dependent launch for the exchange kernels too (read by the native library)"),
    "ZSE_REFERENCE_DIR": ("", "where the tests look for an installed copy of the reference"),
}


def _declared(name: str) -> str:
    if name not in KNOWN:
        raise KeyError(f"{name} is not declared in zse_b200/utils/env.py")
    return KNOWN[name][0]


def text(name: str) -> str:
    return os.environ.get(name, _declared(name))


def flag(name: str) -> bool:
    return text(name).strip().lower() not in _FALSE


def integer(name: str) -> int:
    raw = text(name)
    try:
        return int(raw)
    except ValueError:
        raise ValueError(f"{name}={raw!r} is not an integer") from None


def describe() -> List[str]:
    """One line per switch, then the engine-level settings ``EngineConfig.from_env`` reads (``ZSE_<FIELD>``)."""
    rows = []
    for name, (default, what) in KNOWN.items():
        cur = os.environ.get(name)
        rows.append(f"  {name}={cur if cur is not None else default}{'' if cur is None else '  (set)'}  - {what}")
    from dataclasses import fields

    from ..config import EngineConfig
    names = ", ".join("ZSE_" + f.name.upper() for f in fields(EngineConfig))
    rows.append(f"  engine settings (EngineConfig.from_env): {names}")
    return rows

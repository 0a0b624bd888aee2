"""Kernel registry under the reference's names.

The reference keeps 32 kernel sources by name in ``InferenceKernels`` (zse-engine/zse_engine/orchestrator/kernels.py:
2607-3128): ``compile_all`` builds the essential set for the quantisation in use, ``get(name)`` compiles the rest on
first use, ``launch(name, grid, block, *args)`` runs one.  Here every kernel is hand-written CUDA for sm_100a in one
library that is built once (``ops/build.py``: per-source object cache keyed by content hash), so "compiling" a name
means loading that library, and each name resolves to the host entry point (``ops/native.py``) that serves the role
of the reference kernel - often one fused kernel stands for several of the reference's.  Entry points choose their own
grid and block from the problem shape; ``launch`` therefore refuses a geometry that is handed to it.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Tuple

from . import build as _build
from . import native

# reference kernel name -> (entry point in ops/native.py, what it does beyond the reference kernel)
KERNEL_TABLE: Dict[str, Tuple[str, str]] = {
    "rmsnorm": ("rmsnorm_f16", ""),
    "rmsnorm_f32in": ("add_rmsnorm", "fp32 residual in, fused with the split-K reduction and the residual add"),
    "fused_residual_rmsnorm": ("add_rmsnorm", "also sums the GEMM's split-K planes"),
    "fused_residual_rmsnorm_f32": ("add_rmsnorm", "also sums the GEMM's split-K planes"),
    "residual_add_f32": ("add_rmsnorm", "the add is never a kernel of its own"),
    "silu_mul": ("swiglu", "only for dense fp16 gate/up; the INT4 gate+up GEMM applies it in its epilogue"),
    "geglu_mul": ("swiglu", "gelu=True; the INT4 gate+up GEMM applies it in its epilogue"),
    "bias_add": ("bias_add", "GEMM epilogues add the bias; this is for callers outside the engine"),
    "rotary_embedding": ("rope_kv_write", "rotation, K/V cache write and split-K reduction of the QKV GEMM in one"),
    "batched_rotary_embedding": ("rope_kv_write", "same kernel for every batch shape"),
    "kv_cache_write": ("rope_kv_write", "fused with the rotation"),
    "batched_kv_cache_write": ("rope_kv_write", "fused with the rotation"),
    "gemma_rotary_embedding": ("headnorm_rope_kv_write", "head norms, partial rotation and cache write in one"),
    "qk_norm": ("headnorm_rope_kv_write", "fused with the rotation"),
    "vnorm": ("headnorm_rope_kv_write", "fused with the rotation"),
    "gemma_rmsnorm": ("norm_add_rmsnorm", "post-norm, residual add, layer scalar and the next pre-norm in one"),
    "gemma_rmsnorm_f32in": ("norm_add_rmsnorm", "post-norm, residual add, layer scalar and the next pre-norm in one"),
    "layer_scalar_mul_f32": ("norm_add_rmsnorm", "the scalar is an argument of the fused kernel"),
    "logit_softcap": ("softcap", ""),
    "paged_attention": ("attn_decode", "mma.sync m16n8k16 QK^T and PV over the paged cache (a decode query group is at "
                                       "most 16 rows), cp.async rings, split over the sequence"),
    "prefill_attention": ("attn_prefill", "mma.sync m16n8k16, causal, reads earlier chunks from the paged cache; for "
                                          "head_dim 128 the engine takes attn_prefill_tc instead (tcgen05, "
                                          "probabilities through TMEM)"),
    "tiled_fp16_matmul": ("gemm_f16", "tcgen05 + TMA, operands in shared memory, accumulators in TMEM"),
    "tiled_dequant_matmul_int4": ("gemm_w4", "tcgen05: nibbles dequantised in registers and written to TMEM with "
                                             "tcgen05.st as the A operand, accumulators in TMEM; passes of at most "
                                             "64 tokens can take the persistent kernel gemm_w4_dec"),
    "tiled_dequant_matmul_int8": ("gemm_w8_dec", "tcgen05, the INT4 decode kernel's pipeline with 8-bit chunks: weights "
                                                 "stay INT8 in memory and are dequantised into TMEM; passes of more "
                                                 "than 64 tokens expand the layer into a shared fp16 scratch with "
                                                 "dequant_w8_tiled and run gemm_f16"),
    "dequant_gemv_int4": ("gemm_w4", "M <= 2 takes the CUDA-core GEMV inside the same entry point"),
    "batched_dequant_gemv_int4": ("gemm_w4", "small batches take the narrow tensor-core tile"),
    "fused_gate_up_gemv_int4": ("gemm_w4", "epilogue 1: gate and up rows interleaved, activation applied in the epilogue"),
    "fp16_gemv": ("gemm_f16", ""),
    "embedding_lookup_f32out": ("embedding", "checks token ids against the table and reports through the status word"),
    "argmax_fp16": ("argmax", ""),
    "batched_argmax_fp16": ("argmax", "one launch for every row"),
    "lora_scaled_add": ("lora_expand", "shrink and expand are batched over adapters (one id per row)"),
}

ESSENTIAL = {
    "int4": ["rmsnorm_f32in", "fused_residual_rmsnorm_f32", "rotary_embedding", "paged_attention",
             "prefill_attention", "tiled_dequant_matmul_int4", "fused_gate_up_gemv_int4", "embedding_lookup_f32out",
             "batched_argmax_fp16"],
    "int8": ["rmsnorm_f32in", "fused_residual_rmsnorm_f32", "rotary_embedding", "paged_attention",
             "prefill_attention", "tiled_dequant_matmul_int8", "tiled_fp16_matmul", "silu_mul",
             "embedding_lookup_f32out", "batched_argmax_fp16"],
    "fp16": ["rmsnorm_f32in", "fused_residual_rmsnorm_f32", "rotary_embedding", "paged_attention",
             "prefill_attention", "tiled_fp16_matmul", "silu_mul", "embedding_lookup_f32out", "batched_argmax_fp16"],
}


class InferenceKernels:
    KERNEL_SOURCES = {name: entry for name, (entry, _) in KERNEL_TABLE.items()}

    def __init__(self, backend: str = "cuda"):
        if backend != "cuda":
            raise ValueError(f"this package has one backend (cuda, sm_100a); got {backend!r}")
        self._backend = backend
        self._resolved: Dict[str, Callable] = {}

    def compile_all(self, quant_type: str = "int4") -> None:
        """Builds the library if its sources changed, loads it, and resolves the essential names of ``quant_type``."""
        if quant_type not in ESSENTIAL:
            raise ValueError(f"unknown quantisation {quant_type!r}")
        native.load()
        for name in ESSENTIAL[quant_type]:
            self.compile_kernel(name)

    def compile_kernel(self, name: str) -> Callable:
        if name not in KERNEL_TABLE:
            raise KeyError(f"unknown kernel {name!r}; known: {', '.join(sorted(KERNEL_TABLE))}")
        fn = getattr(native, KERNEL_TABLE[name][0])
        self._resolved[name] = fn
        return fn

    def get(self, name: str) -> Callable:
        fn = self._resolved.get(name)
        return fn if fn is not None else self.compile_kernel(name)

    def describe(self, name: str) -> str:
        entry, note = KERNEL_TABLE[name]
        return f"{name} -> ops.native.{entry}" + (f" ({note})" if note else "")

    def launch(self, name: str, grid: tuple, block: tuple, *args, **kwargs):
        """Calls the entry point that serves ``name``.  The entry points plan their own grids and blocks (tile shapes,
        split-K, clusters), so a launch geometry cannot be imposed from here: ``grid`` and ``block`` must be None or
        empty, anything else is refused rather than silently ignored."""
        if grid or block:
            raise ValueError(f"{name}: the native entry points choose their own launch geometry; pass grid=None, "
                             f"block=None (got grid={grid!r}, block={block!r})")
        return self.get(name)(*args, **kwargs)

    launch_prepacked = launch

    def sync(self) -> None:
        import torch
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    @property
    def num_compiled(self) -> int:
        return len(self._resolved)

    @property
    def kernel_names(self) -> List[str]:
        return sorted(KERNEL_TABLE)

    def is_compiled(self, name: str) -> bool:
        return name in self._resolved

    @staticmethod
    def library_path() -> str:
        return _build.LIB_PATH

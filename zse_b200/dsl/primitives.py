"""The built-in functions of the kernel language (zse-compiler/zse_compiler/types/primitives.py:14-634).

Inside an ``@kernel`` function these names are never executed as Python: the parser recognises them and the emitter
prints CUDA for each.  Calling one outside a kernel raises.  ``PRIMITIVES`` gives, for each name, the number of
arguments it takes and how the type of its result follows from them.

Differences from the reference's set: ``block_reduce_*`` hand the result to every thread of the block (the reference
leaves it in thread 0 only), vector values have usable components (``v.x`` or ``v[0]``), ``tile_load`` /
``tile_store`` take the row pitch of the matrix (``ld``), and there are no AMD matrix-core calls."""
from __future__ import annotations

from typing import Dict, Tuple

# result rules: a type name, "arg0" (type of the first argument), "promote" (common type of the arguments),
# "elem0" (element type of the pointer in the first argument), "void"
PRIMITIVES: Dict[str, Tuple[int, int, str]] = {
    "thread_id": (0, 1, "int"), "block_id": (0, 1, "int"), "block_dim": (0, 1, "int"), "grid_dim": (0, 1, "int"),
    "global_id": (0, 1, "int"), "lane_id": (0, 0, "int"), "warp_id": (0, 0, "int"),
    "syncthreads": (0, 0, "void"),
    "atomic_add": (2, 2, "elem0"), "atomic_max": (2, 2, "elem0"), "atomic_min": (2, 2, "elem0"),
    "atomic_cas": (3, 3, "elem0"),
    "exp": (1, 1, "float"), "log": (1, 1, "float"), "sqrt": (1, 1, "float"), "rsqrt": (1, 1, "float"),
    "cos": (1, 1, "float"), "sin": (1, 1, "float"), "tanh": (1, 1, "float"), "pow": (2, 2, "float"),
    "fma": (3, 3, "float"), "max_val": (2, 2, "promote"), "min_val": (2, 2, "promote"),
    "half_to_float": (1, 1, "float"), "float_to_half": (1, 1, "half"),
    "bf16_to_float": (1, 1, "float"), "float_to_bf16": (1, 1, "bf16"),
    "warp_shuffle_down": (2, 3, "arg0"), "warp_shuffle_up": (2, 3, "arg0"), "warp_shuffle_xor": (2, 3, "arg0"),
    "warp_shuffle": (2, 3, "arg0"),
    "warp_ballot": (1, 1, "uint"), "warp_all": (1, 1, "bool"), "warp_any": (1, 1, "bool"),
    "warp_reduce_sum": (1, 1, "arg0"), "warp_reduce_max": (1, 1, "arg0"), "warp_reduce_min": (1, 1, "arg0"),
    "block_reduce_sum": (1, 1, "arg0"), "block_reduce_max": (1, 1, "arg0"), "block_reduce_min": (1, 1, "arg0"),
    "load_float4": (2, 2, "float4"), "store_float4": (6, 6, "void"),
    "load_half2": (2, 2, "half2"), "store_half2": (4, 4, "void"),
    "unpack_int4": (3, 3, "void"), "unpack_uint4": (3, 3, "void"),
    "tile_load": (5, 8, "void"), "tile_store": (5, 8, "void"),
    # warp-wide 16x16x16 fp16 -> fp32 tiles on the tensor cores through nvcuda::wmma (the portable, legacy path:
    # the engine's own GEMMs issue tcgen05 instructions by hand, which a per-thread language cannot express)
    "wmma_load_a": (4, 4, "frag_a"), "wmma_load_b": (4, 4, "frag_b"), "wmma_fill": (0, 1, "frag_c"),
    "wmma_mma": (3, 3, "frag_c"), "wmma_store": (5, 5, "void"),
}

# handled by the parser as declarations rather than calls
DECLARATIONS = ("shared_memory", "dynamic_shared_memory", "local_array", "reinterpret")

# plain Python spellings that kernels may use
BUILTINS = {"float": "float", "int": "int", "bool": "bool", "min": "min_val", "max": "max_val", "abs": "abs"}

COLLECTIVES = {"warp_shuffle_down", "warp_shuffle_up", "warp_shuffle_xor", "warp_shuffle", "warp_ballot", "warp_all",
               "warp_any", "warp_reduce_sum", "warp_reduce_max", "warp_reduce_min", "block_reduce_sum",
               "block_reduce_max", "block_reduce_min", "syncthreads", "tile_load", "tile_store"}


# calls every lane of a warp must make together (no value is exchanged in the emulator, but the block must be whole warps)
WARP_WIDE = {"wmma_load_a", "wmma_load_b", "wmma_fill", "wmma_mma", "wmma_store"}
FRAGMENTS = ("frag_a", "frag_b", "frag_c")


def _marker(name: str):
    def f(*_args, **_kwargs):
        raise RuntimeError(f"{name}() is part of the kernel language: it can only be used inside an @kernel function")
    f.__name__ = f.__qualname__ = name
    f.__doc__ = f"Kernel-language primitive ``{name}`` (see zse_b200/dsl/primitives.py)."
    return f


for _n in list(PRIMITIVES) + list(DECLARATIONS):
    globals()[_n] = _marker(_n)
__all__ = list(PRIMITIVES) + list(DECLARATIONS)

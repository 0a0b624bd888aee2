"""Constants of the ``.zse`` container.

The on-disk contract is the one of the reference engine
(zse-engine/zse_engine/format/spec.py:6-72): a 64-byte header, a table of
32-byte section entries, the small sections, then the weight blob on a page
boundary with every tensor on a 256-byte boundary.
"""
from __future__ import annotations

import enum

MAGIC = b"ZSE\x01"
VERSION = 1
PAGE_SIZE = 4096
TENSOR_ALIGN = 256
HEADER_SIZE = 64
SECTION_ENTRY_SIZE = 32
DEFAULT_GROUP_SIZE = 128
DEFAULT_QUANT_BITS = 4


class SectionType(enum.IntEnum):
    CONFIG = 0
    TOKENIZER = 1
    WEIGHT_INDEX = 2
    WEIGHT_DATA = 3
    KERNELS = 4


class Flags(enum.IntFlag):
    HAS_TOKENIZER = 1
    HAS_KERNELS = 2
    MMAP_READY = 4


class QuantMethod(enum.IntEnum):
    NONE = 0
    INT4_ASYM = 1
    INT8_SYM = 2


# Substrings that keep a tensor in fp16 (embeddings, output head, every norm, every bias).
KEEP_FP16_SUBSTRINGS = ("embed_tokens", "lm_head", "norm", "layernorm", ".bias")


def should_quantize(tensor_name: str) -> bool:
    low = tensor_name.lower()
    return not any(s in low for s in KEEP_FP16_SUBSTRINGS)


def align_offset(offset: int, alignment: int) -> int:
    """The reference's name for ``align_up``."""
    return align_up(offset, alignment)


def align_up(offset: int, alignment: int) -> int:
    return (offset + alignment - 1) // alignment * alignment


def pad_to_alignment(offset: int, alignment: int) -> bytes:
    return bytes(align_up(offset, alignment) - offset)

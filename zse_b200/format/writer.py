"""Streaming writer of ``.zse`` files.

File layout (zse-engine/zse_engine/format/writer.py:1-8,256-303):
``[64 B header][section table][CONFIG][TOKENIZER?][pad to 4096][WEIGHT_DATA][WEIGHT_INDEX]``; every
tensor starts on a 256-byte boundary and is followed directly by its scales, then its zeros; the
header and the table are rewritten by ``finalize``; table order is CONFIG, [TOKENIZER],
WEIGHT_DATA, WEIGHT_INDEX.  INT4 payloads are always written row-major ``[N, K/2]`` and the config
records ``quant.int4_layout = "rowmajor"``.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np

from .config import ModelConfig
from .header import FileHeader, SectionEntry, compute_crc32
from .quantize import (quantize_fp16, quantize_tensor, quantize_tensor_int8)
from .spec import (HEADER_SIZE, PAGE_SIZE, SECTION_ENTRY_SIZE, TENSOR_ALIGN, VERSION, Flags, QuantMethod,
                   SectionType, align_up)
from .weight_index import WeightEntry, WeightIndex


def _raw(b) -> memoryview:
    if isinstance(b, np.ndarray):
        return memoryview(np.ascontiguousarray(b)).cast("B")
    return memoryview(b).cast("B") if not isinstance(b, (bytes, bytearray)) else memoryview(b)


class ZSEWriter:
    def __init__(self, path: str):
        self._path = path
        self._fp = open(path, "wb")
        self._config: Optional[ModelConfig] = None
        self._tokenizer_bytes: Optional[bytes] = None
        self._weight_index = WeightIndex()
        self._sections = []
        self._weight_data_start = 0
        self._current_weight_offset = 0
        self._finalized = False
        self._has_tokenizer = False
        self._num_sections = 0

    # ---- set-up ----------------------------------------------------------------------------
    def set_config(self, config: ModelConfig) -> None:
        self._config = config
        if config.quant.method == QuantMethod.INT4_ASYM and config.quant.int4_layout is None:
            config.quant.int4_layout = "rowmajor"

    def set_tokenizer(self, tokenizer_bytes: bytes) -> None:
        self._tokenizer_bytes = tokenizer_bytes

    def begin_weights(self) -> None:
        if self._config is None:
            raise ValueError("set_config() must come before begin_weights()")
        self._has_tokenizer = self._tokenizer_bytes is not None
        self._num_sections = 3 + int(self._has_tokenizer)
        self._fp.write(bytes(HEADER_SIZE + self._num_sections * SECTION_ENTRY_SIZE))
        blob = self._config.serialize()
        self._sections.append(SectionEntry(SectionType.CONFIG, self._fp.tell(), len(blob), compute_crc32(blob)))
        self._fp.write(blob)
        if self._has_tokenizer:
            tok = self._tokenizer_bytes
            self._sections.append(SectionEntry(SectionType.TOKENIZER, self._fp.tell(), len(tok), compute_crc32(tok)))
            self._fp.write(tok)
        here = self._fp.tell()
        self._fp.write(bytes(align_up(here, PAGE_SIZE) - here))
        self._weight_data_start = self._fp.tell()
        self._current_weight_offset = 0

    # ---- tensors ---------------------------------------------------------------------------
    def _append(self, *chunks):
        pad = align_up(self._current_weight_offset, TENSOR_ALIGN) - self._current_weight_offset
        if pad:
            self._fp.write(bytes(pad))
            self._current_weight_offset += pad
        spans = []
        for c in chunks:
            mv = _raw(c)
            spans.append((self._current_weight_offset, mv.nbytes))
            self._fp.write(mv)
            self._current_weight_offset += mv.nbytes
        return spans

    def add_weight(self, name: str, weights, shape: Sequence[int], quantize: bool = True) -> None:
        """Quantise (or convert to fp16) a float tensor and append it."""
        shape = tuple(int(s) for s in shape)
        if not quantize or self._config.quant.method == QuantMethod.NONE:
            self.add_weight_raw_fp16(name, shape, quantize_fp16(weights))
        elif self._config.quant.method == QuantMethod.INT8_SYM:
            q, s = quantize_tensor_int8(weights, self._config.quant.group_size)
            self.add_weight_raw_int8(name, shape, q, s, self._config.quant.group_size)
        else:
            p, s, z = quantize_tensor(weights, self._config.quant.group_size)
            self.add_weight_raw(name, shape, p, s, z, self._config.quant.group_size)

    def add_weight_raw(self, name, shape, packed_data, scales_data, zeros_data, group_size: int = 128) -> None:
        (d, dn), (s, sn), (z, zn) = self._append(packed_data, scales_data, zeros_data)
        self._weight_index.add(WeightEntry(name, tuple(shape), "int4", int(QuantMethod.INT4_ASYM), group_size,
                                           d, dn, s, sn, z, zn))

    def add_weight_raw_fp16(self, name, shape, fp16_data) -> None:
        ((d, dn),) = self._append(fp16_data)
        self._weight_index.add(WeightEntry(name, tuple(shape), "float16", int(QuantMethod.NONE), 128, d, dn))

    def add_weight_raw_int8(self, name, shape, packed_data, scales_data, group_size: int = 128) -> None:
        (d, dn), (s, sn) = self._append(packed_data, scales_data)
        self._weight_index.add(WeightEntry(name, tuple(shape), "int8", int(QuantMethod.INT8_SYM), group_size,
                                           d, dn, s, sn))

    # ---- close -----------------------------------------------------------------------------
    def finalize(self) -> None:
        if self._finalized:
            return
        self._sections.append(SectionEntry(SectionType.WEIGHT_DATA, self._weight_data_start,
                                           self._current_weight_offset, 0))
        blob = self._weight_index.serialize()
        self._sections.append(SectionEntry(SectionType.WEIGHT_INDEX, self._fp.tell(), len(blob), compute_crc32(blob)))
        self._fp.write(blob)
        total = self._fp.tell()
        flags = Flags.MMAP_READY | (Flags.HAS_TOKENIZER if self._has_tokenizer else 0)
        self._fp.seek(0)
        self._fp.write(FileHeader(VERSION, total, int(flags), self._num_sections).pack())
        for s in self._sections:
            self._fp.write(s.pack())
        self._fp.close()
        self._finalized = True

    def abort(self) -> None:
        """Close without finalising (an interrupted conversion keeps its ``.progress`` file)."""
        if not self._finalized:
            self._fp.close()
            self._finalized = True

    def __enter__(self):
        return self

    def __exit__(self, exc_type, *_):
        if exc_type is None:
            self.finalize()
        else:
            self.abort()

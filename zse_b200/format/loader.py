"""Memory-mapped reader of ``.zse`` files.

Same public surface as zse-engine/zse_engine/format/loader.py:26-290 (``config``,
``weight_index``, ``tokenizer``, ``get_weight_data/scales/zeros``, ``weight_data_section``,
``file_descriptor``) plus zero-copy numpy/torch views for the device uploader.  The small
sections are CRC-checked (CONFIG, TOKENIZER); ``total_size`` must equal the file size.

INT4 payload layout: the reference has two writers that disagree (row-major ``[N,K/2]`` from the
python path, 64x8-tiled from its C path) and no flag that tells them apart.  Resolution order here:
``quant.int4_layout`` in the config if present; else a payload whose size differs from ``N*K/2``
must be tiled (tiles are zero padded); else row-major, unless ``int4_layout=`` overrides it.
"""
from __future__ import annotations

import mmap
import os
from typing import List, Optional, Tuple

import numpy as np

from .config import ModelConfig
from .header import FileHeader, SectionEntry, compute_crc32, read_header_and_sections
from .quantize import dequantize_int4_arrays, dequantize_tensor_int8, untile_int4_64x8
from .spec import SectionType
from .weight_index import WeightEntry, WeightIndex


class ZSELoader:
    def __init__(self, path: str, int4_layout: Optional[str] = None, verify_crc: bool = True):
        self._path = path
        self._fd = None
        self._mm: Optional[mmap.mmap] = None
        self._header: Optional[FileHeader] = None
        self._sections: List[SectionEntry] = []
        self._config: Optional[ModelConfig] = None
        self._weight_index: Optional[WeightIndex] = None
        self._tokenizer = None
        self._tokenizer_data: Optional[bytes] = None
        self._weight_data_offset = 0
        self._weight_data_size = 0
        self._layout_override = int4_layout
        self._open(verify_crc)

    def _open(self, verify_crc: bool) -> None:
        size = os.path.getsize(self._path)
        if size == 0:
            raise ValueError(f"empty .zse file: {self._path}")
        self._fd = open(self._path, "rb")
        self._mm = mmap.mmap(self._fd.fileno(), 0, access=mmap.ACCESS_READ)
        try:
            self._mm.madvise(mmap.MADV_RANDOM)
        except (AttributeError, OSError):
            pass
        self._header, self._sections = read_header_and_sections(self._mm)
        if self._header.total_size != size:
            raise ValueError(f"file size mismatch: header says {self._header.total_size}, file has {size}")
        fd = self._fd.fileno()
        for s in self._sections:
            if s.offset + s.size > size:
                raise ValueError(f"section {s.type.name} runs past the end of the file")
            if s.type == SectionType.WEIGHT_DATA:
                self._weight_data_offset, self._weight_data_size = s.offset, s.size
                continue
            blob = os.pread(fd, s.size, s.offset)
            if len(blob) != s.size:
                raise ValueError(f"short read on section {s.type.name}")
            if verify_crc and s.type in (SectionType.CONFIG, SectionType.TOKENIZER) \
                    and compute_crc32(blob) != s.crc32:
                raise ValueError(f"CRC mismatch in section {s.type.name}")
            if s.type == SectionType.CONFIG:
                self._config = ModelConfig.deserialize(blob)
            elif s.type == SectionType.TOKENIZER:
                self._tokenizer_data = blob
            elif s.type == SectionType.WEIGHT_INDEX:
                self._weight_index = WeightIndex.deserialize(blob)

    # ---- sections --------------------------------------------------------------------------
    @property
    def path(self) -> str:
        return self._path

    @property
    def header(self) -> FileHeader:
        return self._header

    @property
    def config(self) -> ModelConfig:
        if self._config is None:
            raise ValueError("no CONFIG section in this .zse file")
        return self._config

    @property
    def weight_index(self) -> WeightIndex:
        if self._weight_index is None:
            raise ValueError("no WEIGHT_INDEX section in this .zse file")
        return self._weight_index

    @property
    def tokenizer(self):
        if self._tokenizer is None and self._tokenizer_data is not None:
            from .tokenizer import BPETokenizer
            self._tokenizer = BPETokenizer.deserialize(self._tokenizer_data)
            self._tokenizer_data = None
        return self._tokenizer

    @property
    def file_descriptor(self) -> int:
        return self._fd.fileno() if self._fd else -1

    def weight_data_section(self) -> Tuple[int, int]:
        if not self._weight_data_size and not self._weight_data_offset:
            raise ValueError("no WEIGHT_DATA section in this .zse file")
        return self._weight_data_offset, self._weight_data_size

    # ---- raw access ------------------------------------------------------------------------
    def _span(self, rel: int, nbytes: int) -> memoryview:
        a = self._weight_data_offset + rel
        return memoryview(self._mm)[a:a + nbytes]

    def get_weight_data(self, entry: WeightEntry) -> bytes:
        return bytes(self._span(entry.data_offset, entry.data_nbytes))

    def get_weight_scales(self, entry: WeightEntry) -> bytes:
        return bytes(self._span(entry.scale_offset, entry.scale_nbytes)) if entry.scale_nbytes else b""

    def get_weight_zeros(self, entry: WeightEntry) -> bytes:
        return bytes(self._span(entry.zeros_offset, entry.zeros_nbytes)) if entry.zeros_nbytes else b""

    def get_mmap_pointer_and_offset(self, entry: WeightEntry):
        return self._mm, self._weight_data_offset + entry.data_offset

    # ---- typed views -----------------------------------------------------------------------
    def int4_layout_of(self, entry: WeightEntry) -> str:
        if entry.dtype != "int4" or len(entry.shape) != 2:
            return "rowmajor"
        if self._layout_override:
            return self._layout_override
        rec = self.config.quant.int4_layout
        if rec:
            return rec
        n, k = entry.shape
        expect = (n * k + 1) // 2
        gs = entry.group_size
        padded = ((n * k + gs - 1) // gs * gs) // 2
        return "rowmajor" if entry.data_nbytes in (expect, padded) else "tiled64x8"

    def view_data(self, entry: WeightEntry) -> np.ndarray:
        """Zero-copy uint8/int8/float16 view of the payload exactly as stored."""
        mv = self._span(entry.data_offset, entry.data_nbytes)
        if entry.dtype == "float16":
            return np.frombuffer(mv, dtype=np.float16).reshape(entry.shape)
        if entry.dtype == "int8":
            return np.frombuffer(mv, dtype=np.int8)
        return np.frombuffer(mv, dtype=np.uint8)

    def int4_rowmajor(self, entry: WeightEntry) -> np.ndarray:
        """Packed INT4 bytes in row-major order, whatever the stored layout."""
        raw = self.view_data(entry)
        if self.int4_layout_of(entry) == "tiled64x8":
            return untile_int4_64x8(raw, entry.shape[0], entry.shape[1])
        return raw

    def view_scales(self, entry: WeightEntry) -> np.ndarray:
        return np.frombuffer(self._span(entry.scale_offset, entry.scale_nbytes), dtype=np.float16)

    def view_zeros(self, entry: WeightEntry) -> np.ndarray:
        return np.frombuffer(self._span(entry.zeros_offset, entry.zeros_nbytes), dtype=np.float16)

    def get_weight_as_float(self, entry: WeightEntry) -> np.ndarray:
        """Dequantised fp32 tensor of shape ``entry.shape`` (verification / CPU oracle)."""
        if entry.dtype == "float16":
            return self.view_data(entry).astype(np.float32)
        if entry.dtype == "int4":
            flat = dequantize_int4_arrays(self.int4_rowmajor(entry), self.view_scales(entry),
                                          self.view_zeros(entry), entry.num_elements, entry.group_size)
            return flat.reshape(entry.shape)
        if entry.dtype == "int8":
            return dequantize_tensor_int8(self.view_data(entry).tobytes(), self.view_scales(entry).tobytes(),
                                          entry.shape, entry.group_size).reshape(entry.shape)
        raise ValueError(f"unknown dtype {entry.dtype}")

    def summary(self) -> str:
        c = self.config
        kinds = {}
        for e in self.weight_index:
            kinds[e.dtype] = kinds.get(e.dtype, 0) + 1
        lines = [f"ZSE model: {self._path}", f"  version {self._header.version}, {self._header.total_size:,} bytes",
                 f"  arch {c.arch}: {c.num_layers} layers, hidden {c.hidden_size}, heads {c.num_heads}/{c.num_kv_heads}"
                 f" x {c.head_dim}, intermediate {c.intermediate_size}, vocab {c.vocab_size}, max_seq {c.max_seq_len}",
                 f"  quant: method {int(c.quant.method)}, {c.quant.bits}-bit, group {c.quant.group_size}",
                 f"  tensors: {len(self.weight_index)} ({', '.join(f'{k}: {v}' for k, v in sorted(kinds.items()))})"]
        if self._tokenizer_data is not None or self._tokenizer is not None:
            lines.append("  tokenizer: embedded")
        return "\n".join(lines)

    def close(self) -> None:
        mm, self._mm = self._mm, None
        if mm is not None:
            try:
                mm.close()
            except BufferError:
                pass  # numpy views still alive; the mapping goes away with them
        fd, self._fd = self._fd, None
        if fd is not None:
            fd.close()

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

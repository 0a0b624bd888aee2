"""Block tables and lengths of a batch, padded for the attention kernels
(zse-engine/zse_engine/cache/attention_metadata.py:13-89): ``block_tables[num_seqs][max_blocks]`` int32 with -1 for
padding and for evicted holes, ``seq_lengths[num_seqs]`` int32."""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import List, Optional

import numpy as np


@dataclass
class AttentionMetadata:
    block_tables: List[List[int]]
    seq_lengths: List[int]
    num_seqs: int
    max_seq_len: int
    max_blocks_per_seq: int
    block_size: int
    is_prefill: Optional[List[bool]] = None

    def block_table_array(self, width: Optional[int] = None) -> np.ndarray:
        w = self.max_blocks_per_seq if width is None else width
        out = np.full((self.num_seqs, max(1, w)), -1, dtype=np.int32)
        for i, row in enumerate(self.block_tables):
            out[i, : len(row)] = row[:w]
        return out

    def pack_block_tables(self) -> bytes:
        return self.block_table_array().astype("<i4").tobytes()

    def pack_seq_lengths(self) -> bytes:
        return struct.pack(f"<{self.num_seqs}i", *self.seq_lengths)

    @property
    def block_tables_nbytes(self) -> int:
        return self.num_seqs * max(1, self.max_blocks_per_seq) * 4

    @property
    def seq_lengths_nbytes(self) -> int:
        return self.num_seqs * 4


def build_attention_metadata(block_ids_per_seq: List[List[int]], seq_lengths: List[int],
                             block_size: int) -> AttentionMetadata:
    """From page-table state (zse-engine/zse_engine/cache/attention_metadata.py:66-89)."""
    return AttentionMetadata([list(b) for b in block_ids_per_seq], list(seq_lengths), len(seq_lengths),
                             max(seq_lengths, default=0), max((len(b) for b in block_ids_per_seq), default=0),
                             block_size)

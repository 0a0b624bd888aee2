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
    # device copies, set by ``upload`` (0 until then): int32 ``[num_seqs, max_blocks_per_seq]`` and ``[num_seqs]``
    block_tables_gpu_ptr: int = 0
    seq_lengths_gpu_ptr: int = 0
    block_tables_gpu: Optional[object] = None
    seq_lengths_gpu: Optional[object] = None

    def upload(self, device) -> "AttentionMetadata":
        """Copies both arrays to ``device`` and records their addresses.  The serving loop does not use this: it stages
        the tables of a step through pinned buffers into fixed device buffers (``cache_manager.stage_decode``)."""
        import torch
        self.block_tables_gpu = torch.from_numpy(self.block_table_array()).to(device)
        self.seq_lengths_gpu = torch.tensor(self.seq_lengths, dtype=torch.int32).to(device)
        self.block_tables_gpu_ptr = int(self.block_tables_gpu.data_ptr())
        self.seq_lengths_gpu_ptr = int(self.seq_lengths_gpu.data_ptr()) if self.num_seqs else 0
        return self

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

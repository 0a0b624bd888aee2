"""The 64-byte file header and the section table of a ``.zse`` file.

Header ``<4s I Q I I`` = magic, version, total_size, flags, num_sections, zero padded to
64 bytes; one table entry ``<I Q Q I 8x`` = type, offset, size, crc32
(zse-engine/zse_engine/format/header.py:13-78).
"""
from __future__ import annotations

import struct
import zlib
from dataclasses import dataclass
from typing import List, Tuple

from .spec import HEADER_SIZE, MAGIC, SECTION_ENTRY_SIZE, VERSION, SectionType

_HEADER = struct.Struct("<4sIQII")
_ENTRY = struct.Struct("<IQQI8x")


def compute_crc32(data) -> int:
    return zlib.crc32(data) & 0xFFFFFFFF


@dataclass
class SectionEntry:
    type: SectionType
    offset: int = 0
    size: int = 0
    crc32: int = 0

    def pack(self) -> bytes:
        return _ENTRY.pack(int(self.type), self.offset, self.size, self.crc32)

    @classmethod
    def unpack(cls, data) -> "SectionEntry":
        t, off, size, crc = struct.unpack_from("<IQQI", data)
        return cls(SectionType(t), off, size, crc)


@dataclass
class FileHeader:
    version: int = VERSION
    total_size: int = 0
    flags: int = 0
    num_sections: int = 0

    def pack(self) -> bytes:
        raw = _HEADER.pack(MAGIC, self.version, self.total_size, int(self.flags), self.num_sections)
        return raw.ljust(HEADER_SIZE, b"\x00")

    @classmethod
    def unpack(cls, data) -> "FileHeader":
        if len(data) < _HEADER.size:
            raise ValueError("truncated .zse header")
        magic, version, total, flags, nsec = _HEADER.unpack_from(data)
        if magic != MAGIC:
            raise ValueError(f"not a .zse file: magic {magic!r}")
        if version > VERSION:
            raise ValueError(f"unsupported .zse version {version} (newest known {VERSION})")
        return cls(version, total, flags, nsec)


def read_header_and_sections(data) -> Tuple[FileHeader, List[SectionEntry]]:
    header = FileHeader.unpack(data[:HEADER_SIZE])
    need = HEADER_SIZE + header.num_sections * SECTION_ENTRY_SIZE
    if len(data) < need:
        raise ValueError("truncated .zse section table")
    table = []
    for i in range(header.num_sections):
        at = HEADER_SIZE + i * SECTION_ENTRY_SIZE
        table.append(SectionEntry.unpack(data[at:at + SECTION_ENTRY_SIZE]))
    return header, table

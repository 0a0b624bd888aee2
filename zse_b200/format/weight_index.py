"""Per-tensor metadata of the WEIGHT_INDEX section.

Each entry is a dict with exactly the keys of
zse-engine/zse_engine/format/weight_index.py:10-47 (the reference loader rejects extras);
all offsets are relative to the first byte of the WEIGHT_DATA section.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Dict, Iterator, List, Optional, Tuple

from . import serializer
from .spec import QuantMethod

_KEYS = ("name", "shape", "dtype", "quant_method", "group_size", "data_offset", "data_nbytes",
         "scale_offset", "scale_nbytes", "zeros_offset", "zeros_nbytes")


@dataclass
class WeightEntry:
    name: str
    shape: Tuple[int, ...]
    dtype: str                       # "int4" | "int8" | "float16"
    quant_method: int = int(QuantMethod.NONE)
    group_size: int = 128
    data_offset: int = 0
    data_nbytes: int = 0
    scale_offset: int = 0
    scale_nbytes: int = 0
    zeros_offset: int = 0
    zeros_nbytes: int = 0

    def to_dict(self) -> dict:
        d = asdict(self)
        d["shape"] = [int(x) for x in self.shape]
        d["quant_method"] = int(self.quant_method)
        return {k: d[k] for k in _KEYS}

    @classmethod
    def from_dict(cls, d: dict) -> "WeightEntry":
        kw = {k: d[k] for k in _KEYS if k in d}
        kw["shape"] = tuple(int(x) for x in kw["shape"])
        return cls(**kw)

    @property
    def num_elements(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def end_offset(self) -> int:
        return max(self.data_offset + self.data_nbytes,
                   self.scale_offset + self.scale_nbytes if self.scale_nbytes else 0,
                   self.zeros_offset + self.zeros_nbytes if self.zeros_nbytes else 0)


class WeightIndex:
    def __init__(self) -> None:
        self.entries: List[WeightEntry] = []
        self._by_name: Dict[str, WeightEntry] = {}

    def add(self, entry: WeightEntry) -> None:
        self.entries.append(entry)
        self._by_name[entry.name] = entry

    def find(self, name: str) -> Optional[WeightEntry]:
        return self._by_name.get(name)

    def __contains__(self, name: str) -> bool:
        return name in self._by_name

    def __len__(self) -> int:
        return len(self.entries)

    def __iter__(self) -> Iterator[WeightEntry]:
        return iter(self.entries)

    def serialize(self) -> bytes:
        return serializer.encode([e.to_dict() for e in self.entries])

    @classmethod
    def deserialize(cls, data) -> "WeightIndex":
        idx = cls()
        for d in serializer.decode(data):
            idx.add(WeightEntry.from_dict(d))
        return idx

    @property
    def total_data_bytes(self) -> int:
        return max((e.end_offset for e in self.entries), default=0)

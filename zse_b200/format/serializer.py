"""Tagged binary encoding used by the CONFIG, TOKENIZER and WEIGHT_INDEX sections.

Wire format (zse-engine/zse_engine/format/serializer.py:7-17): one tag byte, then
``0x00`` None, ``0x01``/``0x02`` False/True, ``0x10`` int64 LE, ``0x11`` float64 LE,
``0x20`` bytes and ``0x21`` utf-8 text (u32 length), ``0x30`` list (u32 count),
``0x40`` dict (u32 count, alternating keys and values).

The decoder reads through a ``memoryview`` with pre-compiled ``struct`` objects, so a
large tokenizer section (150 K vocabulary entries, 150 K merge pairs) is decoded
without copying the section and without per-item format parsing.
"""
from __future__ import annotations

import struct
from typing import Any

_I64 = struct.Struct("<q")
_F64 = struct.Struct("<d")
_U32 = struct.Struct("<I")


def encode(obj: Any) -> bytes:
    out = bytearray()
    _emit(obj, out)
    return bytes(out)


def _emit(obj: Any, out: bytearray) -> None:
    if obj is None:
        out.append(0x00)
    elif obj is False:
        out.append(0x01)
    elif obj is True:
        out.append(0x02)
    elif isinstance(obj, int):
        out.append(0x10)
        out += _I64.pack(obj)
    elif isinstance(obj, float):
        out.append(0x11)
        out += _F64.pack(obj)
    elif isinstance(obj, (bytes, bytearray, memoryview)):
        b = bytes(obj)
        out.append(0x20)
        out += _U32.pack(len(b))
        out += b
    elif isinstance(obj, str):
        b = obj.encode("utf-8")
        out.append(0x21)
        out += _U32.pack(len(b))
        out += b
    elif isinstance(obj, (list, tuple)):
        out.append(0x30)
        out += _U32.pack(len(obj))
        for item in obj:
            _emit(item, out)
    elif isinstance(obj, dict):
        out.append(0x40)
        out += _U32.pack(len(obj))
        for k, v in obj.items():
            _emit(k, out)
            _emit(v, out)
    else:
        # numpy scalars and enum members degrade to their python value
        for cast in (int, float):
            try:
                if cast(obj) == obj:
                    _emit(cast(obj), out)
                    return
            except (TypeError, ValueError):
                pass
        raise TypeError(f"zse serializer: unsupported type {type(obj).__name__}")


def decode(data) -> Any:
    buf = memoryview(data) if not isinstance(data, memoryview) else data
    value, pos = _decode_at(buf, 0)
    return value


def _decode_at(buf: memoryview, pos: int):
    tag = buf[pos]
    pos += 1
    if tag == 0x00:
        return None, pos
    if tag == 0x01:
        return False, pos
    if tag == 0x02:
        return True, pos
    if tag == 0x10:
        return _I64.unpack_from(buf, pos)[0], pos + 8
    if tag == 0x11:
        return _F64.unpack_from(buf, pos)[0], pos + 8
    if tag == 0x20:
        n = _U32.unpack_from(buf, pos)[0]
        pos += 4
        return bytes(buf[pos:pos + n]), pos + n
    if tag == 0x21:
        n = _U32.unpack_from(buf, pos)[0]
        pos += 4
        return str(buf[pos:pos + n], "utf-8"), pos + n
    if tag == 0x30:
        n = _U32.unpack_from(buf, pos)[0]
        pos += 4
        items = []
        for _ in range(n):
            v, pos = _decode_at(buf, pos)
            items.append(v)
        return items, pos
    if tag == 0x40:
        n = _U32.unpack_from(buf, pos)[0]
        pos += 4
        d = {}
        for _ in range(n):
            k, pos = _decode_at(buf, pos)
            v, pos = _decode_at(buf, pos)
            d[k] = v
        return d, pos
    raise ValueError(f"zse serializer: unknown tag 0x{tag:02x} at byte {pos - 1}")

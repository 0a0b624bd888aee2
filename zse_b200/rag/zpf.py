"""ZPF: a token-saving text form for documents that go into a prompt
(same three layers as zse-engine/zse_engine/rag/zpf_format.py:26-376).

1. schema extraction - an array of records with the same keys (JSON) or a table (CSV) is written as one schema line
   ``§k1|k2|k3§`` followed by one ``v1|v2|v3`` line per record;
2. dictionary coding - strings that repeat (>= 3 times, >= 4 characters) get short codes ``£0``, ``£1``, ... listed in
   one ``¤code=value¤`` header line;
3. whitespace normalisation - runs of blanks and empty lines collapse.

``decompress`` inverts 1 and 2 (records come back as ``key: value`` lines), so a compressed chunk stays readable for
the model and for tests.
"""
from __future__ import annotations

import csv
import io
import json
import re
from collections import Counter
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

SCHEMA_MARK, DICT_MARK, CODE_MARK, SEP = "§", "¤", "£", "|"


def count_tokens(text: str, tokenizer=None) -> int:
    if tokenizer is not None:
        try:
            return len(tokenizer.encode(text))
        except Exception:
            pass
    return max(1, len(re.findall(r"\w+|[^\w\s]", text))) if text else 0


@dataclass
class ZPFSchema:
    columns: List[str]

    def header(self) -> str:
        return SCHEMA_MARK + SEP.join(self.columns) + SCHEMA_MARK

    @staticmethod
    def parse_header(line: str) -> Optional["ZPFSchema"]:
        if len(line) >= 2 and line.startswith(SCHEMA_MARK) and line.endswith(SCHEMA_MARK):
            return ZPFSchema(line[1:-1].split(SEP))
        return None


@dataclass
class ZPFDictionary:
    encode_map: Dict[str, str] = field(default_factory=dict)
    decode_map: Dict[str, str] = field(default_factory=dict)

    def add(self, value: str, code: str) -> None:
        self.encode_map[value] = code
        self.decode_map[code] = value

    def encode(self, text: str) -> str:
        for value in sorted(self.encode_map, key=len, reverse=True):      # longest first: no partial overlaps
            text = text.replace(value, self.encode_map[value])
        return text

    def decode(self, text: str) -> str:
        for code in sorted(self.decode_map, key=len, reverse=True):       # £10 before £1
            text = text.replace(code, self.decode_map[code])
        return text

    def header(self) -> str:
        if not self.encode_map:
            return ""
        return DICT_MARK + ";".join(f"{c}={v}" for v, c in self.encode_map.items()) + DICT_MARK

    @staticmethod
    def parse_header(line: str) -> Optional["ZPFDictionary"]:
        if len(line) >= 2 and line.startswith(DICT_MARK) and line.endswith(DICT_MARK):
            d = ZPFDictionary()
            for item in line[1:-1].split(";"):
                if "=" in item:
                    code, value = item.split("=", 1)
                    d.add(value, code)
            return d
        return None


@dataclass
class ZPFDocument:
    original: str
    compressed: str
    schema: Optional[ZPFSchema] = None
    dictionary: Optional[ZPFDictionary] = None
    original_tokens: int = 0
    compressed_tokens: int = 0
    doc_type: str = "text"           # "text" | "json" | "csv": which compressor produced it

    # the reference's field names (zse-engine/zse_engine/rag/zpf_format.py:72-80)
    @property
    def original_text(self) -> str:
        return self.original

    @property
    def compressed_text(self) -> str:
        return self.compressed

    @property
    def savings_pct(self) -> float:
        if self.original_tokens <= 0:
            return 0.0
        return (1.0 - self.compressed_tokens / self.original_tokens) * 100.0


def _clean(value: Any) -> str:
    if value is None:
        return ""
    if isinstance(value, (dict, list)):
        value = json.dumps(value, separators=(",", ":"), ensure_ascii=False)
    return re.sub(r"\s+", " ", str(value)).replace(SEP, "/").strip()


def build_dictionary(values: Sequence[str], min_freq: int = 3, min_len: int = 4, max_entries: int = 64) -> ZPFDictionary:
    d = ZPFDictionary()
    counts = Counter(v for v in values if len(v) >= min_len and not any(m in v for m in (";", "=", DICT_MARK)))
    ranked = sorted(((len(v) * (c - 1), v) for v, c in counts.items() if c >= min_freq), reverse=True)
    for i, (_, v) in enumerate(ranked[:max_entries]):
        d.add(v, f"{CODE_MARK}{i}")
    return d


def _finish(original: str, body_lines: List[str], schema: Optional[ZPFSchema], dictionary: Optional[ZPFDictionary],
            tokenizer) -> ZPFDocument:
    lines = []
    if dictionary is not None and dictionary.encode_map:
        lines.append(dictionary.header())
    if schema is not None:
        lines.append(schema.header())
    lines += body_lines
    comp = "\n".join(lines)
    doc = ZPFDocument(original, comp, schema, dictionary, count_tokens(original, tokenizer),
                      count_tokens(comp, tokenizer))
    if doc.compressed_tokens >= doc.original_tokens:        # never make a chunk longer
        plain = normalise_whitespace(original)
        doc = ZPFDocument(original, plain, None, None, doc.original_tokens, count_tokens(plain, tokenizer))
    return doc


def normalise_whitespace(text: str) -> str:
    text = text.replace("\r\n", "\n").replace("\r", "\n")
    text = re.sub(r"[ \t\f\v]+", " ", text)
    text = re.sub(r" ?\n ?", "\n", text)
    return re.sub(r"\n{3,}", "\n\n", text).strip()


def compress_text(text: str, tokenizer=None) -> ZPFDocument:
    plain = normalise_whitespace(text)
    return ZPFDocument(text, plain, None, None, count_tokens(text, tokenizer), count_tokens(plain, tokenizer))


def compress_records(records: Sequence[Dict[str, Any]], tokenizer=None, original: Optional[str] = None) -> ZPFDocument:
    """Records with (mostly) the same keys -> schema line + value rows."""
    columns: List[str] = []
    for r in records:
        for k in r:
            if k not in columns:
                columns.append(k)
    rows = [[_clean(r.get(c)) for c in columns] for r in records]
    dictionary = build_dictionary([v for row in rows for v in row])
    body = [dictionary.encode(SEP.join(row)) for row in rows]
    original = original if original is not None else json.dumps(list(records), indent=2, ensure_ascii=False)
    return _finish(original, body, ZPFSchema([_clean(c) for c in columns]), dictionary, tokenizer)


def compress_json(data: Any, tokenizer=None, original: Optional[str] = None) -> ZPFDocument:
    doc = _compress_json(data, tokenizer, original)
    doc.doc_type = "json"
    return doc


def _compress_json(data: Any, tokenizer=None, original: Optional[str] = None) -> ZPFDocument:
    if isinstance(data, list) and data and all(isinstance(x, dict) for x in data):
        return compress_records(data, tokenizer, original)
    original = original if original is not None else json.dumps(data, indent=2, ensure_ascii=False)
    if isinstance(data, dict):
        flat: List[str] = []

        def walk(prefix: str, node: Any) -> None:
            if isinstance(node, dict):
                for k, v in node.items():
                    walk(f"{prefix}.{k}" if prefix else str(k), v)
            elif isinstance(node, list) and node and all(isinstance(x, dict) for x in node):
                sub = compress_records(node, tokenizer)
                flat.append(f"{prefix}:")
                flat.extend(sub.compressed.split("\n"))
            else:
                flat.append(f"{prefix}={_clean(node)}")

        walk("", data)
        return _finish(original, flat, None, None, tokenizer)
    compact = json.dumps(data, separators=(",", ":"), ensure_ascii=False)
    return ZPFDocument(original, compact, None, None, count_tokens(original, tokenizer),
                       count_tokens(compact, tokenizer))


def split_csv_line(line: str) -> List[str]:
    return next(csv.reader(io.StringIO(line)), [])


def compress_csv(text: str, tokenizer=None) -> ZPFDocument:
    rows = [r for r in csv.reader(io.StringIO(text)) if r]
    if len(rows) < 2:
        return compress_text(text, tokenizer)
    header, data = rows[0], rows[1:]
    records = [{h: (r[i] if i < len(r) else "") for i, h in enumerate(header)} for r in data]
    doc = compress_records(records, tokenizer, original=text)
    doc.doc_type = "csv"
    return doc


def decompress(compressed: str) -> str:
    """Back to readable text: codes expanded, schema rows written as ``key: value`` lines."""
    lines = compressed.split("\n")
    dictionary = None
    if lines and (d := ZPFDictionary.parse_header(lines[0])) is not None:
        dictionary, lines = d, lines[1:]
    out: List[str] = []
    schema: Optional[ZPFSchema] = None
    for line in lines:
        s = ZPFSchema.parse_header(line)
        if s is not None:
            schema = s
            continue
        if dictionary is not None:
            line = dictionary.decode(line)
        if schema is not None and SEP in line or (schema is not None and len(schema.columns) == 1 and line):
            vals = line.split(SEP)
            if len(vals) == len(schema.columns):
                out.append(", ".join(f"{k}: {v}" for k, v in zip(schema.columns, vals) if v != ""))
                continue
        out.append(line)
    return "\n".join(out)


decompress_zpf = decompress      # the reference's name (zse-engine/zse_engine/rag/zpf_format.py:334)

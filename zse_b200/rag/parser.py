"""Document parsers: text/markdown, JSON, JSONL, CSV, PDF -> chunks of roughly ``chunk_size`` tokens with ``overlap``
(roles of zse-engine/zse_engine/rag/parser.py:25-1560).  Every chunk carries its ZPF-compressed form and token counts.
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from . import zpf


@dataclass
class Chunk:
    text: str
    compressed: str
    metadata: Dict[str, Any] = field(default_factory=dict)
    original_tokens: int = 0
    compressed_tokens: int = 0

    @property
    def savings_pct(self) -> float:
        return (1.0 - self.compressed_tokens / self.original_tokens) * 100.0 if self.original_tokens else 0.0


def _mk(doc: zpf.ZPFDocument, meta: Dict[str, Any]) -> Chunk:
    return Chunk(doc.original, doc.compressed, dict(meta), doc.original_tokens, doc.compressed_tokens)


def _public_meta(metadata: Optional[Dict]) -> Dict[str, Any]:
    """Metadata that is stored with a chunk: secrets and callables stay out."""
    return {k: v for k, v in (metadata or {}).items() if k not in ("pdf_password", "ocr_fn") and not callable(v)}


class TextParser:
    """Paragraph-aligned chunks; a paragraph longer than a chunk is cut at sentence ends, then at words."""

    def __init__(self, chunk_size: int = 512, overlap: int = 64):
        self.chunk_size, self.overlap = max(8, chunk_size), max(0, min(overlap, chunk_size // 2))

    def _pieces(self, text: str, tokenizer) -> List[str]:
        out: List[str] = []
        for para in re.split(r"\n\s*\n", text.strip()):
            para = para.strip()
            if not para:
                continue
            if zpf.count_tokens(para, tokenizer) <= self.chunk_size:
                out.append(para)
                continue
            for sent in re.split(r"(?<=[.!?])\s+", para):
                if zpf.count_tokens(sent, tokenizer) <= self.chunk_size:
                    out.append(sent)
                    continue
                words, cur = sent.split(), []
                for w in words:
                    cur.append(w)
                    if zpf.count_tokens(" ".join(cur), tokenizer) >= self.chunk_size:
                        out.append(" ".join(cur))
                        cur = []
                if cur:
                    out.append(" ".join(cur))
        return out

    def parse(self, text: str, tokenizer=None, metadata: Optional[Dict] = None) -> List[Chunk]:
        if not text or not text.strip():
            return []
        meta = _public_meta(metadata)
        pieces = self._pieces(text, tokenizer)
        sizes = [zpf.count_tokens(p, tokenizer) for p in pieces]
        chunks: List[Chunk] = []
        i = 0
        while i < len(pieces):
            j, total = i, 0
            while j < len(pieces) and (j == i or total + sizes[j] <= self.chunk_size):
                total += sizes[j]
                j += 1
            body = "\n\n".join(pieces[i:j])
            chunks.append(_mk(zpf.compress_text(body, tokenizer), {**meta, "chunk_index": len(chunks)}))
            if j >= len(pieces):
                break
            # step back so that about `overlap` tokens are repeated at the start of the next chunk
            back, k = 0, j
            while k - 1 > i and back + sizes[k - 1] <= self.overlap:
                back += sizes[k - 1]
                k -= 1
            i = k if k > i else j
        return chunks


class JSONParser:
    """An array of records becomes groups of records (schema + rows); other JSON is flattened to ``path=value``."""

    def __init__(self, chunk_size: int = 512, overlap: int = 64):
        self.chunk_size, self.overlap = chunk_size, overlap

    def parse(self, text: str, tokenizer=None, metadata: Optional[Dict] = None) -> List[Chunk]:
        meta = _public_meta(metadata)
        try:
            data = json.loads(text)
        except (ValueError, TypeError):
            return TextParser(self.chunk_size, self.overlap).parse(text, tokenizer, metadata)
        return self._parse_data(data, tokenizer, meta)

    def _parse_data(self, data: Any, tokenizer, meta: Dict) -> List[Chunk]:
        if isinstance(data, list) and data and all(isinstance(x, dict) for x in data):
            return self._records(data, tokenizer, meta)
        if isinstance(data, dict):
            big = [(k, v) for k, v in data.items() if isinstance(v, list) and v and all(isinstance(x, dict) for x in v)]
            if len(big) == 1 and len(big[0][1]) > 8:
                key, recs = big[0]
                rest = {k: v for k, v in data.items() if k != key}
                out = [_mk(zpf.compress_json(rest, tokenizer), {**meta, "chunk_index": 0})] if rest else []
                for c in self._records(recs, tokenizer, {**meta, "json_key": key}):
                    c.metadata["chunk_index"] = len(out)
                    out.append(c)
                return out
        doc = zpf.compress_json(data, tokenizer)
        if doc.compressed_tokens <= self.chunk_size:
            return [_mk(doc, {**meta, "chunk_index": 0})]
        return TextParser(self.chunk_size, self.overlap).parse(doc.compressed, tokenizer, meta)

    def _records(self, recs: List[Dict], tokenizer, meta: Dict) -> List[Chunk]:
        out: List[Chunk] = []
        group: List[Dict] = []

        def flush() -> None:
            if group:
                out.append(_mk(zpf.compress_records(list(group), tokenizer),
                               {**meta, "chunk_index": len(out), "records": len(group)}))
                group.clear()

        budget = 0
        for r in recs:
            n = zpf.count_tokens(json.dumps(r, separators=(",", ":"), ensure_ascii=False), tokenizer)
            if group and budget + n > self.chunk_size * 2:      # rows compress roughly 2x
                flush()
                budget = 0
            group.append(r)
            budget += n
        flush()
        return out


class JSONLParser(JSONParser):
    def parse(self, text: str, tokenizer=None, metadata: Optional[Dict] = None) -> List[Chunk]:
        meta = _public_meta(metadata)
        recs, loose = [], []
        for line in text.splitlines():
            line = line.strip()
            if not line:
                continue
            try:
                v = json.loads(line)
            except ValueError:
                loose.append(line)
                continue
            (recs if isinstance(v, dict) else loose).append(v if isinstance(v, dict) else line)
        out = self._records(recs, tokenizer, meta) if recs else []
        if loose:
            for c in TextParser(self.chunk_size, self.overlap).parse("\n".join(map(str, loose)), tokenizer, meta):
                c.metadata["chunk_index"] = len(out)
                out.append(c)
        return out


class CSVParser:
    def __init__(self, chunk_size: int = 512, overlap: int = 64):
        self.chunk_size, self.overlap = chunk_size, overlap

    def parse(self, text: str, tokenizer=None, metadata: Optional[Dict] = None) -> List[Chunk]:
        meta = _public_meta(metadata)
        lines = [l for l in text.splitlines() if l.strip()]
        if len(lines) < 2:
            return TextParser(self.chunk_size, self.overlap).parse(text, tokenizer, metadata)
        header = lines[0]
        out: List[Chunk] = []
        group: List[str] = []
        budget = 0
        for line in lines[1:]:
            n = zpf.count_tokens(line, tokenizer)
            if group and budget + n > self.chunk_size * 2:
                out.append(_mk(zpf.compress_csv("\n".join([header] + group), tokenizer),
                               {**meta, "chunk_index": len(out), "rows": len(group)}))
                group, budget = [], 0
            group.append(line)
            budget += n
        if group:
            out.append(_mk(zpf.compress_csv("\n".join([header] + group), tokenizer),
                           {**meta, "chunk_index": len(out), "rows": len(group)}))
        return out


def get_parser(filename: str, chunk_size: int = 512, overlap: int = 64):
    ext = filename.rsplit(".", 1)[-1].lower() if "." in filename else ""
    if ext == "json":
        return JSONParser(chunk_size, overlap)
    if ext in ("jsonl", "ndjson"):
        return JSONLParser(chunk_size, overlap)
    if ext in ("csv", "tsv"):
        return CSVParser(chunk_size, overlap)
    if ext == "pdf":
        from .pdf import PDFParser
        return PDFParser(chunk_size, overlap)
    return TextParser(chunk_size, overlap)

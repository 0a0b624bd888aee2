"""Reading order for PDF text: content-stream operators are followed with their positions (text matrix, line
matrix, leading), every shown string becomes a fragment at a place on the page, and the fragments are put back into
lines, words and columns (zse-engine/zse_engine/rag/parser.py: the tokenizer, text-matrix tracking and column
detection of ``PDFParser``; the behaviour is pinned by zse-engine's tests/test_pdf_layout.py).

Draw order in a PDF says nothing about reading order - two-column papers, tables and most word processors emit text
in whatever order suited the producer - so sorting by position is what makes retrieval chunks readable.  Widths are
estimated from the font size (no glyph metrics are read), which is enough to decide where a word gap is."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence, Union

_WS = b" \t\r\n\f\0"
_DELIM = b"()<>[]{}/%"


@dataclass
class Fragment:
    x: float
    y: float
    text: str
    size: float

    @property
    def width(self) -> float:
        return 0.5 * self.size * len(self.text)


def tokenize_content_stream(data: Union[str, bytes]) -> list:
    """Operators and operands of a content stream.  A literal string (balanced parentheses, escapes), a hex string,
    a dictionary and a whole ``[...]`` array are one token each; comments are dropped.  ``str`` in, ``str`` out."""
    as_text = isinstance(data, str)
    buf = data.encode("latin-1", "replace") if as_text else bytes(data)
    out: List[bytes] = []
    i, n = 0, len(buf)

    def literal_end(j: int) -> int:
        depth = 0
        while j < n:
            c = buf[j]
            if c == 0x5C:
                j += 2
                continue
            if c == 0x28:
                depth += 1
            elif c == 0x29:
                depth -= 1
                if depth == 0:
                    return j + 1
            j += 1
        return n

    while i < n:
        c = buf[i]
        if c in _WS:
            i += 1
        elif c == 0x25:                                   # % comment
            while i < n and buf[i] not in b"\r\n":
                i += 1
        elif c == 0x28:
            j = literal_end(i)
            out.append(buf[i:j])
            i = j
        elif c == 0x5B:                                   # [ ... ] with strings inside
            j = i + 1
            while j < n and buf[j] != 0x5D:
                j = literal_end(j) if buf[j] == 0x28 else j + 1
            out.append(buf[i:min(j + 1, n)])
            i = j + 1
        elif c == 0x3C:
            if buf[i:i + 2] == b"<<":
                j = buf.find(b">>", i)
                j = n if j < 0 else j + 2
            else:
                j = buf.find(b">", i)
                j = n if j < 0 else j + 1
            out.append(buf[i:j])
            i = j
        elif c == 0x2F:
            j = i + 1
            while j < n and buf[j] not in _WS and buf[j] not in _DELIM:
                j += 1
            out.append(buf[i:j])
            i = j
        elif c in b")>]{}":
            i += 1
        else:
            j = i
            while j < n and buf[j] not in _WS and buf[j] not in _DELIM:
                j += 1
            out.append(buf[i:j])
            i = max(j, i + 1)
    return [t.decode("latin-1") for t in out] if as_text else out


def _num(tok: bytes, default: float = 0.0) -> float:
    try:
        return float(tok)
    except ValueError:
        return default


def extract_fragments(content: bytes, fonts: Optional[Dict[bytes, Any]] = None) -> List[Fragment]:
    """Walks the text operators (BT ET Tf TL Td TD Tm T* Tj TJ ' ") and returns what was shown, where."""
    from .pdf import ToUnicode, _string, decode_literal
    fonts = fonts or {}
    plain = ToUnicode(b"")
    font = plain
    size, leading = 12.0, 0.0
    lx = ly = 0.0            # start of the current line (line matrix translation)
    x = y = 0.0              # where the next glyph goes
    sx = sy = 1.0            # scale of the text matrix
    frags: List[Fragment] = []
    stack: List[bytes] = []

    def raw_string(tok: bytes) -> bytes:
        return decode_literal(tok[1:-1]) if tok[:1] == b"(" else _string(tok)

    def show(text: str) -> None:
        nonlocal x
        if not text:
            return
        f = Fragment(x, y, text, max(1.0, abs(size * sy)))
        frags.append(f)
        x += f.width * (1 if sx >= 0 else -1)

    def next_line(dy: Optional[float] = None) -> None:
        nonlocal lx, ly, x, y
        step = dy if dy is not None else -(leading or size * 1.2) * abs(sy)
        ly += step
        x, y = lx, ly

    for tok in tokenize_content_stream(content):
        c = tok[:1]
        if c in b"(<[/" or c in b"0123456789+-.":
            stack.append(tok)
            continue
        op = tok
        if op == b"BT":
            lx = ly = x = y = 0.0
            sx = sy = 1.0
        elif op == b"Tf" and len(stack) >= 2:
            font = fonts.get(stack[-2][1:], plain)
            size = _num(stack[-1], 12.0) or 12.0
        elif op == b"TL" and stack:
            leading = _num(stack[-1])
        elif op in (b"Td", b"TD") and len(stack) >= 2:
            tx, ty = _num(stack[-2]) * sx, _num(stack[-1]) * sy
            if op == b"TD":
                leading = -_num(stack[-1])
            lx, ly = lx + tx, ly + ty
            x, y = lx, ly
        elif op == b"Tm" and len(stack) >= 6:
            a, d = _num(stack[-6], 1.0), _num(stack[-3], 1.0)
            sx, sy = (a or 1.0), (d or 1.0)
            lx, ly = _num(stack[-2]), _num(stack[-1])
            x, y = lx, ly
        elif op == b"T*":
            next_line()
        elif op == b"Tj" and stack and stack[-1][:1] in b"(<":
            show(font.decode(raw_string(stack[-1])))
        elif op in (b"'", b'"') and stack and stack[-1][:1] in b"(<":
            next_line()
            show(font.decode(raw_string(stack[-1])))
        elif op == b"TJ" and stack and stack[-1][:1] == b"[":
            parts: List[str] = []
            for item in tokenize_content_stream(stack[-1][1:-1] if stack[-1].endswith(b"]") else stack[-1][1:]):
                if item[:1] in b"(<":
                    parts.append(font.decode(raw_string(item)))
                elif _num(item) < -200 and parts and not parts[-1].endswith(" "):
                    parts.append(" ")                    # a wide negative adjustment is a word gap
            show("".join(parts))
        stack = []
    return frags


def _lines(frags: Sequence[Fragment]) -> List[List[Fragment]]:
    """Fragments grouped into lines (same baseline within a third of the type size), top to bottom, each line left
    to right."""
    rows: List[List[Fragment]] = []
    for f in sorted(frags, key=lambda f: (-f.y, f.x)):
        if rows and abs(rows[-1][0].y - f.y) <= max(1.0, 0.35 * min(rows[-1][0].size, f.size)):
            rows[-1].append(f)
        else:
            rows.append([f])
    return [sorted(r, key=lambda f: f.x) for r in rows]


def _join(line: Sequence[Fragment]) -> str:
    out = line[0].text
    end = line[0].x + line[0].width
    for f in line[1:]:
        gap = f.x - end
        if gap > 0.2 * f.size and not out.endswith(" ") and not f.text.startswith(" "):
            out += " "
        out += f.text
        end = max(end, f.x + f.width)
    return out.rstrip()


def split_columns(frags: Sequence[Fragment]) -> List[List[Fragment]]:
    """One list per column, left to right.  A page is split where the starts of the fragments leave a wide empty band
    and each side has at least three lines of its own that overlap in height with the other side; a single indented
    line or a two-cell row does not make a column."""
    if len(frags) < 6:
        return [list(frags)]
    starts = sorted({round(f.x, 1) for f in frags})
    extent = max(f.x + f.width for f in frags) - starts[0]
    best_gap, cut = 0.0, None
    for a, b in zip(starts, starts[1:]):
        if b - a > best_gap:
            best_gap, cut = b - a, (a + b) / 2
    if cut is None or best_gap < max(40.0, 0.15 * extent):
        return [list(frags)]
    left, right = [f for f in frags if f.x < cut], [f for f in frags if f.x >= cut]
    rows = lambda fs: len({round(f.y) for f in fs})
    if rows(left) < 3 or rows(right) < 3:
        return [list(frags)]
    lo = max(min(f.y for f in left), min(f.y for f in right))
    hi = min(max(f.y for f in left), max(f.y for f in right))
    if hi <= lo:                                         # one block above the other, not side by side
        return [list(frags)]
    # text of the left side that runs across the band belongs to full-width lines: no columns then
    crossing = sum(1 for f in left if f.x + f.width > cut + 0.5 * best_gap)
    if crossing > 0.2 * len(left):
        return [list(frags)]
    return split_columns(left) + split_columns(right)


def reflow(frags: Sequence[Fragment]) -> str:
    """Text of the fragments in reading order: column by column, line by line, words separated where a gap shows."""
    out: List[str] = []
    for col in split_columns([f for f in frags if f.text]):
        prev_y: Optional[float] = None
        for line in _lines(col):
            text = _join(line)
            if not text:
                continue
            if prev_y is not None and prev_y - line[0].y > 2.2 * line[0].size:
                out.append("")                           # a tall gap: paragraph break
            out.append(text)
            prev_y = line[0].y
        out.append("")
    while out and not out[-1]:
        out.pop()
    return "\n".join(out)


def extract_text(content: bytes, fonts: Optional[Dict[bytes, Any]] = None) -> str:
    return reflow(extract_fragments(content, fonts))

"""PDF text extraction without third-party code (scope of zse-engine/zse_engine/rag/parser.py:384-1536): object and
object-stream (ObjStm) parsing, Flate / ASCIIHex / ASCII85 / RunLength filters with PNG predictors, the standard
security handler through ``pdf_crypto``, page content streams (``Tj TJ ' "`` with ``Td TD Tm T*`` line logic),
``/ToUnicode`` CMaps for hex strings, and an OCR hook for pages that carry only images.

It is a reader for retrieval, not a renderer: text comes out in content-stream order, one block per page.
"""
from __future__ import annotations

import re
import zlib
from typing import Any, Callable, Dict, List, Optional, Tuple

from .parser import Chunk, TextParser, _public_meta
from .pdf_crypto import PDFEncryption

_OBJ = re.compile(rb"(\d+)\s+(\d+)\s+obj\b")
_REF = re.compile(rb"(\d+)\s+(\d+)\s+R")
_WS = b" \t\r\n\f\x00"


class PDFError(Exception):
    pass


# ---- low-level syntax -------------------------------------------------------------------------------------------
def _dict_span(buf: bytes, start: int) -> Tuple[int, int]:
    """Span of the ``<< ... >>`` that begins at or after ``start`` (nested dictionaries and strings respected)."""
    i = buf.find(b"<<", start)
    if i < 0:
        return -1, -1
    depth, j, n = 0, i, len(buf)
    while j < n:
        c = buf[j:j + 2]
        if c == b"<<":
            depth += 1
            j += 2
        elif c == b">>":
            depth -= 1
            j += 2
            if depth == 0:
                return i, j
        elif buf[j:j + 1] == b"(":
            j = _skip_literal(buf, j)
        else:
            j += 1
    return i, n


def _skip_literal(buf: bytes, i: int) -> int:
    depth, j, n = 0, i, len(buf)
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


def decode_literal(raw: bytes) -> bytes:
    """Body of a ``( ... )`` string (without the outer parentheses) -> bytes."""
    out = bytearray()
    i, n = 0, len(raw)
    esc = {0x6E: 10, 0x72: 13, 0x74: 9, 0x62: 8, 0x66: 12, 0x28: 0x28, 0x29: 0x29, 0x5C: 0x5C}
    while i < n:
        c = raw[i]
        if c != 0x5C:
            out.append(c)
            i += 1
            continue
        i += 1
        if i >= n:
            break
        c = raw[i]
        if c in esc:
            out.append(esc[c])
            i += 1
        elif 0x30 <= c <= 0x37:
            j, v = i, 0
            while j < n and j < i + 3 and 0x30 <= raw[j] <= 0x37:
                v = v * 8 + raw[j] - 0x30
                j += 1
            out.append(v & 0xFF)
            i = j
        elif c in (10, 13):
            i += 1
            if c == 13 and i < n and raw[i] == 10:
                i += 1
        else:
            out.append(c)
            i += 1
    return bytes(out)


def _name_value(d: bytes, name: bytes) -> Optional[bytes]:
    """Raw token(s) after ``/Name`` inside a dictionary body (up to the next key at the same level)."""
    m = re.search(re.escape(name) + rb"(?![A-Za-z0-9])", d)
    if not m:
        return None
    i = m.end()
    while i < len(d) and d[i] in _WS:
        i += 1
    if d[i:i + 2] == b"<<":
        a, b = _dict_span(d, i)
        return d[a:b]
    if d[i:i + 1] == b"[":
        j = d.find(b"]", i)
        return d[i:j + 1]
    if d[i:i + 1] == b"(":
        return d[i:_skip_literal(d, i)]
    if d[i:i + 1] == b"<":
        j = d.find(b">", i)
        return d[i:j + 1]
    m2 = re.match(rb"/?[^\s/<>\[\]()]+(\s+\d+\s+R)?", d[i:])
    return m2.group(0) if m2 else None


def _int(d: bytes, name: bytes, default: int = 0) -> int:
    v = _name_value(d, name)
    if v is None:
        return default
    m = re.match(rb"-?\d+", v.strip())
    return int(m.group(0)) if m else default


def _string(v: Optional[bytes]) -> bytes:
    if not v:
        return b""
    v = v.strip()
    if v.startswith(b"("):
        return decode_literal(v[1:-1])
    if v.startswith(b"<"):
        h = re.sub(rb"[^0-9A-Fa-f]", b"", v)
        if len(h) % 2:
            h += b"0"
        return bytes.fromhex(h.decode("ascii"))
    return b""


# ---- filters -------------------------------------------------------------------------------------------------------
def _ascii85(data: bytes) -> bytes:
    data = re.sub(rb"\s", b"", data)
    if data.startswith(b"<~"):
        data = data[2:]
    end = data.find(b"~>")
    if end >= 0:
        data = data[:end]
    out, grp = bytearray(), []
    for c in data:
        if c == 0x7A and not grp:
            out += b"\0\0\0\0"
            continue
        grp.append(c - 33)
        if len(grp) == 5:
            v = 0
            for g in grp:
                v = v * 85 + g
            out += (v & 0xFFFFFFFF).to_bytes(4, "big")
            grp = []
    if grp:
        k = len(grp)
        grp += [84] * (5 - k)
        v = 0
        for g in grp:
            v = v * 85 + g
        out += (v & 0xFFFFFFFF).to_bytes(4, "big")[:k - 1]
    return bytes(out)


def _run_length(data: bytes) -> bytes:
    out, i = bytearray(), 0
    while i < len(data):
        n = data[i]
        if n == 128:
            break
        if n < 128:
            out += data[i + 1:i + 2 + n]
            i += n + 2
        else:
            out += data[i + 1:i + 2] * (257 - n)
            i += 2
    return bytes(out)


def _png_predict(data: bytes, columns: int, colors: int = 1, bpc: int = 8) -> bytes:
    bpp = max(1, colors * bpc // 8)
    row = (columns * colors * bpc + 7) // 8
    out, prev = bytearray(), bytearray(row)
    for i in range(0, len(data) - row, row + 1):
        ft, cur = data[i], bytearray(data[i + 1:i + 1 + row])
        for x in range(len(cur)):
            a = cur[x - bpp] if x >= bpp else 0
            b = prev[x]
            c = prev[x - bpp] if x >= bpp else 0
            if ft == 1:
                cur[x] = (cur[x] + a) & 0xFF
            elif ft == 2:
                cur[x] = (cur[x] + b) & 0xFF
            elif ft == 3:
                cur[x] = (cur[x] + (a + b) // 2) & 0xFF
            elif ft == 4:
                p = a + b - c
                pa, pb, pc = abs(p - a), abs(p - b), abs(p - c)
                cur[x] = (cur[x] + (a if pa <= pb and pa <= pc else b if pb <= pc else c)) & 0xFF
        out += cur
        prev = cur
    return bytes(out)


def apply_filters(data: bytes, d: bytes) -> bytes:
    f = _name_value(d, b"/Filter")
    if not f:
        return data
    names = re.findall(rb"/([A-Za-z0-9]+)", f)
    parms = _name_value(d, b"/DecodeParms") or b""
    for name in names:
        if name in (b"FlateDecode", b"Fl"):
            try:
                data = zlib.decompress(data)
            except zlib.error:
                data = zlib.decompressobj().decompress(data)      # truncated streams: keep what inflates
            pred = _int(parms, b"/Predictor", 1)
            if pred >= 10:
                data = _png_predict(data, _int(parms, b"/Columns", 1), _int(parms, b"/Colors", 1),
                                    _int(parms, b"/BitsPerComponent", 8))
        elif name in (b"ASCIIHexDecode", b"AHx"):
            h = re.sub(rb"[^0-9A-Fa-f]", b"", data.split(b">")[0])
            data = bytes.fromhex((h + b"0" * (len(h) % 2)).decode("ascii"))
        elif name in (b"ASCII85Decode", b"A85"):
            data = _ascii85(data)
        elif name in (b"RunLengthDecode", b"RL"):
            data = _run_length(data)
        elif name in (b"LZWDecode", b"LZW"):
            data = _lzw(data, _int(parms, b"/EarlyChange", 1))
            pred = _int(parms, b"/Predictor", 1)
            if pred >= 10:
                data = _png_predict(data, _int(parms, b"/Columns", 1), _int(parms, b"/Colors", 1),
                                    _int(parms, b"/BitsPerComponent", 8))
        elif name in IMAGE_FILTERS:
            break              # compressed image data: handed on as it is (an OCR backend decodes it)
        else:
            raise PDFError(f"unsupported filter {name.decode()}")
    return data


IMAGE_FILTERS = {b"DCTDecode": "jpeg", b"DCT": "jpeg", b"JPXDecode": "jp2", b"CCITTFaxDecode": "ccitt", b"CCF": "ccitt",
                 b"JBIG2Decode": "jbig2"}


def image_hint(d: bytes) -> str:
    """What an image stream holds, from its filter names: jpeg, jp2, ccitt, jbig2, or raw samples."""
    for name in re.findall(rb"/([A-Za-z0-9]+)", _name_value(d, b"/Filter") or b""):
        if name in IMAGE_FILTERS:
            return IMAGE_FILTERS[name]
    return "raw"


def _lzw(data: bytes, early_change: int = 1) -> bytes:
    """LZW as PDF uses it: codes of 9 to 12 bits, most significant bit first, 256 = clear table, 257 = end of data;
    the code width grows one code early unless ``/EarlyChange 0``."""
    out = bytearray()
    table: List[bytes] = []

    def reset() -> None:
        table[:] = [bytes([i]) for i in range(256)] + [b"", b""]

    reset()
    width, prev = 9, None
    acc = bits = 0
    for byte in data:
        acc = (acc << 8) | byte
        bits += 8
        while bits >= width:
            code = (acc >> (bits - width)) & ((1 << width) - 1)
            bits -= width
            if code == 256:
                reset()
                width, prev = 9, None
                continue
            if code == 257:
                return bytes(out)
            if prev is None:
                entry = table[code] if code < len(table) else b""
            elif code < len(table):
                entry = table[code]
                table.append(prev + entry[:1])
            else:
                entry = prev + prev[:1]
                table.append(entry)
            out += entry
            prev = entry
            n = len(table) + 1 + (1 if early_change else 0)      # the writer's table is one entry ahead of this one
            width = 12 if n > 2048 else 11 if n > 1024 else 10 if n > 512 else 9
    return bytes(out)


# ---- document model ------------------------------------------------------------------------------------------------
class PDFDocument:
    def __init__(self, raw: bytes, password: Optional[str] = "", authenticate: bool = True):
        """``authenticate=False`` only reads the /Encrypt parameters (no password check, no object streams)."""
        if not raw.lstrip()[:5].startswith(b"%PDF"):
            raise PDFError("not a PDF file")
        self.raw = raw
        self._authenticate = authenticate
        self.objects: Dict[int, Tuple[int, bytes, Optional[Tuple[int, int]]]] = {}   # num -> (gen, dict/body, stream span)
        self.enc: Optional[PDFEncryption] = None
        self._scan()
        self._setup_encryption(password)
        if authenticate or self.enc is None:
            self._expand_object_streams()

    def _scan(self) -> None:
        raw = self.raw
        for m in _OBJ.finditer(raw):
            num, gen = int(m.group(1)), int(m.group(2))
            end = raw.find(b"endobj", m.end())
            end = len(raw) if end < 0 else end
            body = raw[m.end():end]
            span = None
            s = body.find(b"stream")
            if s >= 0 and body[:s].rstrip().endswith(b">>"):
                hdr = body[:s]
                k = s + 6
                if body[k:k + 2] == b"\r\n":
                    k += 2
                elif body[k:k + 1] in (b"\n", b"\r"):
                    k += 1
                length = _int(hdr, b"/Length", -1)
                lv = _name_value(hdr, b"/Length") or b""
                if _REF.match(lv.strip()) or length < 0 or body[k + length:k + length + 20].find(b"endstream") < 0:
                    e = body.rfind(b"endstream")          # indirect or wrong /Length: cut at the keyword
                    if e < 0:
                        e = len(body)
                    while e > k and body[e - 1] in (10, 13):
                        e -= 1
                    length = e - k
                span = (m.end() + k, m.end() + k + length)
                body = hdr
            self.objects[num] = (gen, body, span)

    def _setup_encryption(self, password: str) -> None:
        tr = None
        for m in re.finditer(rb"trailer", self.raw):
            a, b = _dict_span(self.raw, m.end())
            if a >= 0 and b"/Encrypt" in self.raw[a:b]:
                tr = self.raw[a:b]
        if tr is None:                                   # cross-reference streams carry the trailer keys
            for num, (gen, body, span) in self.objects.items():
                if b"/XRef" in body and b"/Encrypt" in body:
                    tr = body
        if tr is None:
            return
        ev = _name_value(tr, b"/Encrypt")
        m = _REF.match(ev.strip()) if ev else None
        if m and int(m.group(1)) not in self.objects:    # the dictionary may sit in an (unencrypted) object stream
            try:
                self._expand_object_streams()
            except Exception:
                pass
        ed = self.objects[int(m.group(1))][1] if m and int(m.group(1)) in self.objects else ev
        if not ed:
            raise PDFError("cannot read the /Encrypt dictionary")
        idv = _name_value(tr, b"/ID") or b""
        ids = re.findall(rb"<[0-9A-Fa-f\s]*>|\((?:\\.|[^\\)])*\)", idv)
        file_id = _string(ids[0]) if ids else b""
        v, r = _int(ed, b"/V", 0), _int(ed, b"/R", 2)
        aes = False
        if v >= 4:
            cf = re.search(rb"/CFM\s*/(\w+)", ed)
            aes = bool(cf and cf.group(1) in (b"AESV2", b"AESV3"))
        p = _int(ed, b"/P", -1)
        if p >= 1 << 31:
            p -= 1 << 32
        em = _name_value(ed, b"/EncryptMetadata")
        self.enc = PDFEncryption(v, r, _int(ed, b"/Length", 40 if v < 2 else 128), _string(_name_value(ed, b"/O")),
                                 _string(_name_value(ed, b"/U")), p, file_id, not (em and em.strip() == b"false"),
                                 _string(_name_value(ed, b"/OE")), _string(_name_value(ed, b"/UE")), aes)
        self._encrypt_obj = int(m.group(1)) if m else -1
        if not self._authenticate:
            return
        if not self.enc.supported:
            err = PDFError(f"encrypted with a security handler this reader does not have (V={v}, R={r})")
            err.kind = "encrypted_unsupported"
            raise err
        if not self.enc.authenticate(password or ""):
            err = PDFError("password required" if not password else "wrong password")
            err.kind = "encrypted_password_required"
            raise err

    def stream(self, num: int) -> bytes:
        gen, d, span = self.objects[num]
        if span is None:
            return b""
        data = self.raw[span[0]:span[1]]
        if self.enc is not None and num != getattr(self, "_encrypt_obj", -1) and b"/XRef" not in d and num >= 0 \
                and not getattr(self, "_inside_objstm", {}).get(num):
            data = self.enc.decrypt(data, num, gen)
        return apply_filters(data, d)

    def string(self, raw_token: bytes, num: int) -> bytes:
        s = _string(raw_token)
        if self.enc is not None and s and not getattr(self, "_inside_objstm", {}).get(num):
            s = self.enc.decrypt(s, num, self.objects[num][0])
        return s

    def _expand_object_streams(self) -> None:
        self._inside_objstm: Dict[int, bool] = {}
        for num in [n for n, (_, d, sp) in self.objects.items() if sp is not None and b"/ObjStm" in d]:
            _, d, _ = self.objects[num]
            try:
                data = self.stream(num)
            except Exception:
                continue
            n, first = _int(d, b"/N"), _int(d, b"/First")
            if first <= 0 or first > len(data):          # a header that does not fit the data: skip the container
                continue
            try:
                nums = [int(x) for x in data[:first].split()]
            except ValueError:
                continue
            for i in range(min(n, len(nums) // 2)):
                onum, off = nums[2 * i], nums[2 * i + 1]
                nxt = nums[2 * i + 3] if 2 * i + 3 < len(nums) else len(data) - first
                if onum not in self.objects or self.objects[onum][2] is None:
                    self.objects[onum] = (0, data[first + off:first + nxt], None)
                    self._inside_objstm[onum] = True      # already decrypted with its container

    # ---- pages ----------------------------------------------------------------------------------------------
    def resolve(self, token: Optional[bytes]) -> Tuple[int, bytes]:
        """(object number or -1, dictionary/body bytes) of a direct value or a reference."""
        if not token:
            return -1, b""
        m = _REF.match(token.strip())
        if m and int(m.group(1)) in self.objects:
            n = int(m.group(1))
            return n, self.objects[n][1]
        return -1, token

    def pages(self) -> List[int]:
        kids = [n for n, (_, d, _) in self.objects.items()
                if re.search(rb"/Type\s*/Page(?![a-zA-Z])", d)]
        # order by the page tree when it can be walked, else by object number
        root = next((n for n, (_, d, _) in self.objects.items() if re.search(rb"/Type\s*/Pages", d)
                     and b"/Parent" not in d), None)
        order: List[int] = []

        def walk(n: int, depth: int = 0) -> None:
            if depth > 64 or n not in self.objects:
                return
            d = self.objects[n][1]
            if re.search(rb"/Type\s*/Pages", d):
                for m in _REF.finditer(_name_value(d, b"/Kids") or b""):
                    walk(int(m.group(1)), depth + 1)
            elif n in kids and n not in order:
                order.append(n)

        if root is not None:
            walk(root)
        return order + [k for k in sorted(kids) if k not in order]

    def inherited(self, page: int, name: bytes) -> Optional[bytes]:
        n, hops = page, 0
        while n in self.objects and hops < 64:
            d = self.objects[n][1]
            v = _name_value(d, name)
            if v is not None:
                return v
            m = _REF.match((_name_value(d, b"/Parent") or b"").strip())
            if not m:
                return None
            n, hops = int(m.group(1)), hops + 1
        return None

    def page_content(self, page: int) -> bytes:
        c = _name_value(self.objects[page][1], b"/Contents") or b""
        out = []
        for m in _REF.finditer(c):
            n = int(m.group(1))
            if n in self.objects:
                if self.objects[n][2] is None:            # an array object holding the references
                    for m2 in _REF.finditer(self.objects[n][1]):
                        if int(m2.group(1)) in self.objects:
                            out.append(self._safe_stream(int(m2.group(1))))
                else:
                    out.append(self._safe_stream(n))
        return b"\n".join(out)

    def _safe_stream(self, n: int) -> bytes:
        try:
            return self.stream(n)
        except Exception:
            return b""

    def page_fonts(self, page: int) -> Dict[bytes, "ToUnicode"]:
        res = self.resolve(self.inherited(page, b"/Resources"))[1]
        fonts = self.resolve(_name_value(res, b"/Font"))[1]
        out: Dict[bytes, ToUnicode] = {}
        for m in re.finditer(rb"/([^\s/<>\[\]()]+)\s+(\d+)\s+\d+\s+R", fonts):
            fnum = int(m.group(2))
            if fnum not in self.objects:
                continue
            fd = self.objects[fnum][1]
            tu = _REF.match((_name_value(fd, b"/ToUnicode") or b"").strip())
            cmap = ToUnicode(self._safe_stream(int(tu.group(1)))) if tu and int(tu.group(1)) in self.objects \
                else ToUnicode(b"")
            cmap.two_byte = cmap.two_byte or b"/Identity-H" in fd or b"/Type0" in fd
            out[m.group(1)] = cmap
        return out

    def page_images(self, page: int) -> List[Tuple[bytes, str]]:
        res = self.resolve(self.inherited(page, b"/Resources"))[1]
        xo = self.resolve(_name_value(res, b"/XObject"))[1]
        out = []
        for m in _REF.finditer(xo):
            n = int(m.group(1))
            if n in self.objects and b"/Image" in self.objects[n][1] and self.objects[n][2] is not None:
                d = self.objects[n][1]
                a, b = self.objects[n][2]
                data = self.raw[a:b]
                if self.enc is not None:
                    data = self.enc.decrypt(data, n, self.objects[n][0])
                hint = image_hint(d)
                if hint == "raw":
                    try:
                        data = apply_filters(data, d)
                    except Exception:
                        continue
                out.append((data, hint))
        return out


class ToUnicode:
    """``bfchar`` / ``bfrange`` tables of a /ToUnicode CMap."""

    def __init__(self, data: bytes):
        self.map: Dict[int, str] = {}
        self.two_byte = False
        for block in re.findall(rb"beginbfchar(.*?)endbfchar", data, re.S):
            for src, dst in re.findall(rb"<([0-9A-Fa-f]+)>\s*<([0-9A-Fa-f]*)>", block):
                self.map[int(src, 16)] = self._u(dst)
                self.two_byte |= len(src) > 2
        for block in re.findall(rb"beginbfrange(.*?)endbfrange", data, re.S):
            for lo, hi, dst in re.findall(rb"<([0-9A-Fa-f]+)>\s*<([0-9A-Fa-f]+)>\s*(<[0-9A-Fa-f]*>|\[[^\]]*\])", block):
                a, b = int(lo, 16), int(hi, 16)
                self.two_byte |= len(lo) > 2
                if dst.startswith(b"["):
                    for k, item in enumerate(re.findall(rb"<([0-9A-Fa-f]*)>", dst)):
                        if a + k <= b:
                            self.map[a + k] = self._u(item)
                else:
                    base = dst[1:-1]
                    start = int(base, 16) if base else 0
                    for k in range(min(b - a + 1, 65536)):
                        self.map[a + k] = self._u(b"%0*X" % (max(4, len(base)), start + k))

    @staticmethod
    def _u(hexs: bytes) -> str:
        if not hexs:
            return ""
        if len(hexs) % 4:
            hexs = hexs.rjust((len(hexs) + 3) // 4 * 4, b"0")
        try:
            return bytes.fromhex(hexs.decode("ascii")).decode("utf-16-be", "replace")
        except ValueError:
            return ""

    def decode(self, s: bytes) -> str:
        if self.two_byte:
            codes = [int.from_bytes(s[i:i + 2], "big") for i in range(0, len(s) - len(s) % 2, 2)]
        else:
            codes = list(s)
        if self.map:
            return "".join(self.map.get(c, chr(c) if 32 <= c < 0x10000 and not self.two_byte else "") for c in codes)
        if self.two_byte:
            return "".join(chr(c) for c in codes if c >= 32)
        return s.decode("latin-1")


# ---- content streams ---------------------------------------------------------------------------------------------
_TOKEN = re.compile(rb"\((?:\\.|[^\\()]|\((?:\\.|[^\\()])*\))*\)|<[0-9A-Fa-f\s]*>|\[|\]|/[^\s/<>\[\]()]*|"
                    rb"[-+]?\d*\.?\d+|[A-Za-z'\"*]+")


def extract_text(content: bytes, fonts: Dict[bytes, ToUnicode]) -> str:
    """Text of one content stream in reading order (positions are followed and the fragments re-ordered into lines,
    words and columns: ``pdf_layout``)."""
    from .pdf_layout import extract_text as _layout
    text = _layout(content, fonts)
    text = re.sub(r"[ \t]+\n", "\n", text)
    return re.sub(r"\n{3,}", "\n\n", text).strip()


_BARE_STREAM = re.compile(rb"<<((?:[^<>]|<(?!<)|>(?!>)|<<[^<>]*>>)*)>>\s*stream\r?\n")


def bare_streams(raw: bytes) -> List[Tuple[bytes, bytes]]:
    """(dictionary, data) of every ``<< ... >> stream ... endstream`` in the file, whether or not it sits inside a
    numbered object: the fallback for damaged or minimal files without a page tree."""
    out = []
    for m in _BARE_STREAM.finditer(raw):
        end = raw.find(b"endstream", m.end())
        if end < 0:
            continue
        data = raw[m.end():end]
        n = _int(m.group(1), b"/Length", -1)
        if 0 <= n <= len(data):
            data = data[:n]
        else:
            data = data.rstrip(b"\r\n")
        out.append((m.group(1), data))
    return out


class PDFParser:
    """PDF -> text chunks.  ``ocr_fn(image_bytes, format_hint) -> str`` (or a one-argument callable) is only asked
    when a page has no extractable text; ``metadata["ocr_fn"]`` overrides the instance's.  Chunks that came from OCR
    carry ``pdf_ocr: True``; a file that yields nothing gives one chunk with ``error: "extraction_failed"`` so that the
    caller can tell (zse-engine/zse_engine/rag/parser.py: ``PDFParser``; zse-engine's tests/test_pdf_ocr.py)."""

    def __init__(self, chunk_size: int = 512, overlap: int = 64, ocr_fn: Optional[Callable[..., str]] = None):
        self.chunk_size, self.overlap, self.ocr_fn = chunk_size, overlap, ocr_fn
        self._last_encrypted = False

    # the reference's entry points for callers that use the pieces directly
    @staticmethod
    def _tokenize_content_stream(data):
        from .pdf_layout import tokenize_content_stream
        return tokenize_content_stream(data)

    def _extract_text(self, raw, password: str = "") -> str:
        raw = raw if isinstance(raw, (bytes, bytearray)) else raw.encode("latin-1", "replace")
        return "\n\n".join(t for t, _ in self._pages(bytes(raw), password, None) if t)

    def _extract_images(self, raw, password: str = "") -> List[Tuple[bytes, str]]:
        raw = raw if isinstance(raw, (bytes, bytearray)) else raw.encode("latin-1", "replace")
        doc = PDFDocument(bytes(raw), password)
        out: List[Tuple[bytes, str]] = []
        for p in doc.pages():
            out += doc.page_images(p)
        if not out:
            out = self._loose_images(bytes(raw))
        return out

    @staticmethod
    def _loose_images(raw: bytes) -> List[Tuple[bytes, str]]:
        out = []
        for d, data in bare_streams(raw):
            if re.search(rb"/Subtype\s*/Image", d):
                hint = image_hint(d)
                if hint == "raw":
                    try:
                        data = apply_filters(data, d)
                    except Exception:
                        pass
                out.append((data, hint))
        return out

    @staticmethod
    def _call_ocr(fn: Callable[..., str], data: bytes, hint: str) -> str:
        try:
            import inspect
            params = [p for p in inspect.signature(fn).parameters.values()
                      if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD, p.VAR_POSITIONAL)]
            one = len(params) == 1 and params[0].kind != params[0].VAR_POSITIONAL
        except (TypeError, ValueError):
            one = False
        return (fn(data) if one else fn(data, hint)) or ""

    def _ocr(self, images: List[Tuple[bytes, str]], ocr_fn: Optional[Callable[..., str]]) -> str:
        parts = []
        for data, hint in images:
            try:
                parts.append(self._call_ocr(ocr_fn, data, hint))
            except Exception:
                continue               # one unreadable image must not lose the document
        return "\n".join(x.strip() for x in parts if x and x.strip())

    def _pages(self, raw: bytes, password: str, ocr_fn: Optional[Callable[..., str]]) -> List[Tuple[str, bool]]:
        """(text, came from OCR) per page; files without a page tree are read as one page of loose streams."""
        doc = PDFDocument(raw, password)
        self._last_encrypted = doc.enc is not None
        pages: List[Tuple[str, bool]] = []
        for p in doc.pages():
            text = extract_text(doc.page_content(p), doc.page_fonts(p))
            used_ocr = False
            if not text and ocr_fn is not None:
                text = self._ocr(doc.page_images(p), ocr_fn)
                used_ocr = bool(text)
            pages.append((text, used_ocr))
        if not pages:
            texts = []
            for d, data in bare_streams(raw):
                if re.search(rb"/Subtype\s*/Image", d) or re.search(rb"/Type\s*/(XRef|ObjStm|Metadata)", d):
                    continue
                try:
                    t = extract_text(apply_filters(data, d), {})
                except Exception:
                    continue
                if t:
                    texts.append(t)
            text, used_ocr = "\n".join(texts), False
            if not text and ocr_fn is not None:
                text = self._ocr(self._loose_images(raw), ocr_fn)
                used_ocr = bool(text)
            pages.append((text, used_ocr))
        return pages

    def extract_pages(self, raw: bytes, password: str = "", ocr_fn: Optional[Callable[..., str]] = None) -> List[str]:
        return [t for t, _ in self._pages(raw, password, ocr_fn if ocr_fn is not None else self.ocr_fn)]

    def parse(self, text, tokenizer=None, metadata: Optional[Dict] = None) -> List[Chunk]:
        raw = text if isinstance(text, (bytes, bytearray)) else text.encode("latin-1", "replace")
        md = metadata or {}
        ocr_fn = md.get("ocr_fn") or self.ocr_fn
        meta = _public_meta(md)
        try:
            pages = self._pages(bytes(raw), md.get("pdf_password") or "", ocr_fn)
        except PDFError as exc:
            # a file that cannot be read becomes ONE chunk that says why (the caller sees `error` in its metadata):
            # the kinds the security handler reports, or `invalid_pdf` for input that is not a PDF at all
            kind = getattr(exc, "kind", None) or "invalid_pdf"
            note = f"[PDF: {exc}]"
            extra = {"pdf_encrypted": True} if kind.startswith("encrypted") else {}
            return [Chunk(note, note, {**meta, "error": kind, **extra, "chunk_index": 0})]
        if self._last_encrypted:
            meta["pdf_encrypted"] = True
        tp = TextParser(self.chunk_size, self.overlap)
        out: List[Chunk] = []
        for i, (page_text, used_ocr) in enumerate(pages):
            extra = {"page": i + 1, **({"pdf_ocr": True} if used_ocr else {})}
            for c in tp.parse(page_text, tokenizer, {**meta, **extra}):
                c.metadata["chunk_index"] = len(out)
                out.append(c)
        if not out:
            note = "[PDF: no text could be extracted" + ("" if ocr_fn else "; no OCR backend is configured") + "]"
            out.append(Chunk(note, note, {**meta, "error": "extraction_failed", "chunk_index": 0}))
        return out

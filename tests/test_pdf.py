"""PDF handling of the retrieval layer in detail: content-stream tokens, reading-order reflow (lines, word gaps,
columns), stream filters, and the OCR hook.  The behaviours are the ones the reference pins in its own tests
(zse-engine's tests/test_pdf_layout.py, test_pdf_filters.py, test_pdf_ocr.py)."""
import base64
import os
import zlib

import pytest

from zse_b200.rag.pdf import PDFParser, _lzw, apply_filters, bare_streams
from zse_b200.rag.pdf_layout import extract_fragments, reflow, split_columns, tokenize_content_stream


def _stream(body: bytes, extra: bytes = b"") -> bytes:
    return b"<< " + extra + b" /Length %d >>\nstream\n" % len(body) + body + b"\nendstream\n"


def _image(data: bytes, flt: bytes = b"/DCTDecode") -> bytes:
    return (b"1 0 obj\n<< /Type /XObject /Subtype /Image /Filter " + flt + b" /Width 8 /Height 8 /Length %d >>\n"
            b"stream\n" % len(data) + data + b"\nendstream\nendobj\n")


def _pdf(*parts: bytes) -> bytes:
    return b"%PDF-1.4\n" + b"".join(parts) + b"%%EOF\n"


def _text_of(content: bytes) -> str:
    return PDFParser()._extract_text(_pdf(_stream(content)))


def _lines_of(content: bytes):
    return [l for l in _text_of(content).split("\n") if l]


# ---- tokens -------------------------------------------------------------------------------------------------------
def test_tokens_keep_strings_and_arrays_whole():
    tok = PDFParser._tokenize_content_stream
    assert tok("BT /F1 12 Tf 100 200 Td (Hello) Tj ET") == ["BT", "/F1", "12", "Tf", "100", "200", "Td", "(Hello)",
                                                             "Tj", "ET"]
    assert tok("BT (Hello BT ET Tj) Tj ET") == ["BT", "(Hello BT ET Tj)", "Tj", "ET"]
    assert tok("(a(b)c) Tj") == ["(a(b)c)", "Tj"] and tok(r"(a\)b) Tj") == [r"(a\)b)", "Tj"]
    assert tok("[(Hel) -20 (lo)] TJ") == ["[(Hel) -20 (lo)]", "TJ"]
    assert tok("<48656c6c6f> Tj") == ["<48656c6c6f>", "Tj"]
    assert tok("BT % a comment (with parens\n (X) Tj ET") == ["BT", "(X)", "Tj", "ET"]
    assert tokenize_content_stream(b"1 0 0 1 5 6 Tm") == [b"1", b"0", b"0", b"1", b"5", b"6", b"Tm"]


# ---- reading order --------------------------------------------------------------------------------------------------
def test_lines_come_out_top_to_bottom_and_left_to_right():
    assert _lines_of(b"BT 100 100 Td (third) Tj ET\nBT 100 200 Td (second) Tj ET\nBT 100 300 Td (first) Tj ET\n") == \
        ["first", "second", "third"]
    assert _lines_of(b"BT 300 500 Td (world) Tj ET\nBT 100 500 Td (Hello) Tj ET\n") == ["Hello world"]
    assert _lines_of(b"BT 1 0 0 1 100 100 Tm (bottom) Tj ET\nBT 1 0 0 1 100 400 Tm (top) Tj ET\n") == ["top", "bottom"]
    assert _lines_of(b"BT 100 500 Td [(Hel) -50 (lo) -50 ( World)] TJ ET\n") == ["Hello World"]
    assert _lines_of(b"BT 100 500 Td [(Hello) -400 (World)] TJ ET\n") == ["Hello World"]       # a wide kern is a gap
    # consecutive strings continue where the last one ended; T* and ' start new lines below
    assert _lines_of(b"BT /F1 10 Tf 12 TL 50 700 Td (one) Tj ( two) Tj T* (three) Tj (four) ' ET") == \
        ["one two", "three", "four"]
    legacy = _text_of(b"BT\n/F1 12 Tf\n100 700 Td\n(Hello) Tj\n100 680 Td\n(World) Tj\nET\n")
    assert "Hello" in legacy and "World" in legacy


def test_two_columns_are_read_one_after_the_other():
    parts = []
    for i in range(6):
        y = 700 - 30 * i
        parts.append(b"BT 100 %d Td (L%d) Tj ET\nBT 400 %d Td (R%d) Tj ET\n" % (y, i, y, i))
    assert _lines_of(b"".join(parts)) == [f"L{i}" for i in range(6)] + [f"R{i}" for i in range(6)]
    # an indented line is not a column, neither is a row of two cells or a heading above a body
    single = b"".join(b"BT %d %d Td (line%d) Tj ET\n" % (140 if i == 3 else 100, 700 - 20 * i, i) for i in range(8))
    assert _lines_of(single) == [f"line{i}" for i in range(8)]
    frags = extract_fragments(b"BT 100 700 Td (a) Tj ET BT 400 700 Td (b) Tj ET BT 100 680 Td (c) Tj ET "
                              b"BT 400 680 Td (d) Tj ET")
    assert len(split_columns(frags)) == 1 and reflow(frags).split("\n") == ["a b", "c d"]
    # a full-width line that runs across the band keeps the page in one column
    wide = (b"BT 100 760 Td (" + b"x" * 120 + b") Tj ET " + b"BT 100 740 Td (" + b"y" * 120 + b") Tj ET " +
            b"".join(b"BT 100 %d Td (l%d) Tj ET BT 400 %d Td (r%d) Tj ET " % (700 - 20 * i, i, 700 - 20 * i, i)
                     for i in range(3)))
    assert len(split_columns(extract_fragments(wide))) == 1


# ---- filters ------------------------------------------------------------------------------------------------------
def _lzw_encode(data: bytes, early: int = 1) -> bytes:
    table = {bytes([i]): i for i in range(256)}
    nxt, width, codes, w = 258, 9, [(256, 9)], b""
    for b in data:
        wb = w + bytes([b])
        if wb in table:
            w = wb
            continue
        codes.append((table[w], width))
        table[wb] = nxt
        nxt += 1
        n = nxt + early
        width = 12 if n > 2048 else 11 if n > 1024 else 10 if n > 512 else 9
        if nxt >= 4094:
            codes.append((256, width))
            table, nxt, width = {bytes([i]): i for i in range(256)}, 258, 9
        w = bytes([b])
    if w:
        codes.append((table[w], width))
    codes.append((257, width))
    acc = bits = 0
    out = bytearray()
    for c, wd in codes:
        acc, bits = (acc << wd) | c, bits + wd
        while bits >= 8:
            out.append((acc >> (bits - 8)) & 0xFF)
            bits -= 8
    if bits:
        out.append((acc << (8 - bits)) & 0xFF)
    return bytes(out)


def test_stream_filters():
    assert apply_filters(b"48 65 6C\n6c 6F>", b"/Filter /ASCIIHexDecode") == b"Hello"
    assert apply_filters(b"4865 6c6c 7>", b"/Filter /AHx") == b"Hell\x70"               # odd digit: padded with 0
    a85 = base64.a85encode(b"Hello, retrieval world!", adobe=True)
    assert apply_filters(a85, b"/Filter /ASCII85Decode") == b"Hello, retrieval world!"
    assert apply_filters(b"z~>", b"/Filter /A85") == b"\0\0\0\0"
    assert apply_filters(base64.a85encode(b"ab", adobe=True)[2:], b"/Filter /ASCII85Decode") == b"ab"
    assert apply_filters(bytes([2]) + b"abc" + bytes([254]) + b"x" + bytes([128]) + b"junk",
                         b"/Filter /RunLengthDecode") == b"abcxxx"
    assert _lzw(bytes.fromhex("800B6050220C0C8501")) == b"-----A---B"                     # the example of the PDF spec
    for data in (b"hello hello hello " * 40, os.urandom(6000), bytes(range(256)) * 24):
        for early in (1, 0):
            assert _lzw(_lzw_encode(data, early), early) == data
    assert apply_filters(_lzw_encode(b"lzw in a pdf"), b"/Filter /LZWDecode") == b"lzw in a pdf"
    assert apply_filters(_lzw_encode(b"late change", 0), b"/Filter /LZWDecode /DecodeParms << /EarlyChange 0 >>") == \
        b"late change"
    chained = base64.a85encode(zlib.compress(b"BT (chained) Tj ET"), adobe=True)
    assert apply_filters(chained, b"/Filter [ /ASCII85Decode /FlateDecode ]") == b"BT (chained) Tj ET"
    assert apply_filters(b"\xff\xd8jpeg", b"/Filter /DCTDecode") == b"\xff\xd8jpeg"        # image data passes through
    assert apply_filters(zlib.compress(b"\xff\xd8x"), b"/Filter [/FlateDecode /DCTDecode]") == b"\xff\xd8x"
    with pytest.raises(Exception):
        apply_filters(b"x", b"/Filter /NoSuchDecode")
    text = PDFParser()._extract_text(_pdf(_stream(zlib.compress(b"BT 10 10 Td (deflated text) Tj ET"),
                                                  b"/Filter /FlateDecode")))
    assert text == "deflated text"
    assert [d for _, d in bare_streams(_pdf(_stream(b"abc"), _stream(b"defg")))] == [b"abc", b"defg"]


# ---- OCR hook -----------------------------------------------------------------------------------------------------
def test_images_are_found_with_their_kind():
    p = PDFParser()
    jpeg = b"\xff\xd8\xff\xe0FAKE\xff\xd9"
    assert p._extract_images(_pdf(_image(jpeg))) == [(jpeg, "jpeg")]
    for flt, hint in ((b"/DCTDecode", "jpeg"), (b"/JPXDecode", "jp2"), (b"/CCITTFaxDecode", "ccitt"),
                      (b"/JBIG2Decode", "jbig2")):
        assert p._extract_images(_pdf(_image(b"IMG", flt))) == [(b"IMG", hint)]
    assert p._extract_images(_pdf(_image(zlib.compress(b"SAMPLES"), b"/FlateDecode"))) == [(b"SAMPLES", "raw")]
    assert p._extract_images(_pdf(_stream(b"BT (Hello) Tj ET"), _image(b"IMG"))) == [(b"IMG", "jpeg")]


def test_ocr_is_asked_only_when_there_is_no_text():
    calls = []

    def ocr(data, hint):
        calls.append((data, hint))
        return "words read from the scan"

    chunks = PDFParser(ocr_fn=ocr).parse(_pdf(_image(b"\xff\xd8SCAN\xff\xd9")).decode("latin-1"))
    assert calls == [(b"\xff\xd8SCAN\xff\xd9", "jpeg")]
    assert "words read from the scan" in chunks[0].text and all(c.metadata.get("pdf_ocr") is True for c in chunks)
    calls.clear()
    with_text = _pdf(_stream(b"BT 100 700 Td (Real text content here is enough) Tj ET\n"), _image(b"IMG"))
    chunks = PDFParser(ocr_fn=ocr).parse(with_text)
    assert not calls and "Real text content" in chunks[0].text and not chunks[0].metadata.get("pdf_ocr")


def test_ocr_callable_forms_and_failures():
    scan = _pdf(_image(b"IMG"))
    override = PDFParser(ocr_fn=lambda d, h: "from the instance").parse(
        scan, metadata={"ocr_fn": lambda d, h: "from the override"})
    assert "from the override" in override[0].text and "ocr_fn" not in override[0].metadata
    assert "one argument" in PDFParser(ocr_fn=lambda data: "one argument is enough").parse(scan)[0].text

    def flaky(data, hint):
        if data.startswith(b"BAD"):
            raise RuntimeError("unreadable")
        return "the good image"

    both = _pdf(_image(b"BAD_BYTES"), _image(b"GOOD_BYTES"))
    assert "the good image" in PDFParser(ocr_fn=flaky).parse(both)[0].text
    failed = PDFParser().parse(scan)
    assert len(failed) == 1 and failed[0].metadata.get("error") == "extraction_failed"
    assert not failed[0].metadata.get("pdf_ocr")
    assert PDFParser(ocr_fn=lambda d, h: "").parse(scan)[0].metadata.get("error") == "extraction_failed"


# ---- ToUnicode maps -------------------------------------------------------------------------------------------------
def test_tounicode_forms():
    from zse_b200.rag.pdf import ToUnicode
    cmap = ToUnicode(b"2 beginbfchar\n<01> <0048>\n<02> <00660069>\nendbfchar\n"           # 02 -> "fi" (two chars)
                     b"2 beginbfrange\n<10> <12> <0061>\n<20> <21> [<0058> <0059005A>]\nendbfrange\n")
    assert cmap.decode(bytes([1, 2])) == "Hfi"
    assert cmap.decode(bytes([0x10, 0x11, 0x12])) == "abc" and cmap.decode(bytes([0x20, 0x21])) == "XYZ"
    assert cmap.decode(b"A") == "A"                                  # unmapped single-byte codes fall back to the byte
    wide = ToUnicode(b"1 beginbfrange\n<0003> <0005> <0041>\nendbfrange")
    assert wide.two_byte and wide.decode(bytes([0, 3, 0, 5])) == "AC"
    assert ToUnicode(b"").decode(b"plain latin-1 \xe9") == "plain latin-1 \xe9"
    from helpers.make_pdf import make_pdf
    assert PDFParser().extract_pages(make_pdf([["mapped through a CMap"]], flate=True, hex_font=True)) == \
        ["mapped through a CMap"]


# ---- encryption as the parser reports it ------------------------------------------------------------------------------
def _objstm(objects: dict) -> bytes:
    head, body = b"", b""
    for num, text in objects.items():
        head += b"%d %d " % (num, len(body))
        body += text + b" "
    data = zlib.compress(head + body)
    return (b"7 0 obj\n<< /Type /ObjStm /N %d /First %d /Filter /FlateDecode /Length %d >>\nstream\n"
            % (len(objects), len(head), len(data)) + data + b"\nendstream\nendobj\n")


def test_encryption_is_reported_not_hidden():
    from helpers.make_pdf import make_pdf
    from zse_b200.rag import pdf_crypto
    from zse_b200.rag.engine import RAGEngine
    locked = make_pdf([["kept behind a password"]], encrypt="aes128", user_pw="pw")
    chunks = PDFParser().parse(locked, metadata={"pdf_password": "pw"})
    assert "kept behind a password" in chunks[0].text and all(c.metadata.get("pdf_encrypted") for c in chunks)
    assert "pdf_password" not in chunks[0].metadata
    refused = PDFParser().parse(locked)
    assert len(refused) == 1 and refused[0].metadata["error"] == "encrypted_password_required"
    open_pw = PDFParser().parse(make_pdf([["owner set, user empty"]], encrypt="rc4"))
    assert "owner set" in open_pw[0].text and open_pw[0].metadata.get("pdf_encrypted")
    assert not PDFParser().parse(make_pdf([["not encrypted"]]))[0].metadata.get("pdf_encrypted")
    unknown = (b"%PDF-1.4\n2 0 obj\n<< /Filter /Standard /V 99 /R 99 /Length 256 /P -1 /O <" + b"00" * 48 + b"> /U <"
               + b"00" * 48 + b"> >>\nendobj\ntrailer\n<< /Encrypt 2 0 R /ID [<" + b"00" * 16 + b"> <" + b"00" * 16
               + b">] >>\n%%EOF\n")
    enc = pdf_crypto.detect_encryption(unknown)
    assert enc is not None and (enc.version, enc.revision) == (99, 99) and not enc.supported
    bad = PDFParser().parse(unknown)
    assert len(bad) == 1 and bad[0].metadata["error"] == "encrypted_unsupported" and "V=99" in bad[0].text
    res = RAGEngine().ingest("x.pdf", unknown)
    assert res.get("error_kind") == "encrypted_unsupported"
    # the /Encrypt dictionary inside an object stream is still found
    ed = b"<< /Filter /Standard /V 2 /R 3 /Length 128 /P -4 /O <" + b"00" * 32 + b"> /U <" + b"00" * 32 + b"> >>"
    in_stream = (b"%PDF-1.5\n" + _objstm({2: ed}) + b"trailer\n<< /Encrypt 2 0 R /ID [<" + b"00" * 16 + b"> <"
                 + b"00" * 16 + b">] >>\n%%EOF\n")
    enc = pdf_crypto.detect_encryption(in_stream)
    assert enc is not None and (enc.version, enc.revision, enc.length_bits) == (2, 3, 128)
    # a corrupt object stream is skipped rather than fatal
    corrupt = (b"%PDF-1.5\n7 0 obj\n<< /Type /ObjStm /N 5 /First 9999 /Filter /FlateDecode /Length 20 >>\nstream\n"
               + zlib.compress(b"garbage data") + b"\nendstream\nendobj\n" + _stream(b"BT (still readable) Tj ET")
               + b"trailer << /Size 0 >>\n%%EOF\n")
    assert "still readable" in PDFParser()._extract_text(corrupt)

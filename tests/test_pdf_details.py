"""The PDF reader of the retrieval layer, one behaviour per test: literal and hex strings, text operators and the text
matrix, predictors, object streams, the page tree, ToUnicode maps, the three encryption generations with user and owner
passwords, loose files, chunk metadata.  Mirrors the scope of the reference's PDF tests
(tests/test_pdf_cmap.py, test_pdf_encryption.py, test_pdf_filters.py, test_pdf_layout.py, test_pdf_objstm.py,
test_pdf_ocr.py of zse-engine) against this package's own parser."""
import base64
import os
import sys
import zlib

import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from helpers.make_pdf import make_pdf  # noqa: E402
from zse_b200.rag import pdf_crypto  # noqa: E402
from zse_b200.rag.pdf import (PDFDocument, PDFParser, ToUnicode, _png_predict, apply_filters, bare_streams,  # noqa: E402
                              decode_literal, image_hint)
from zse_b200.rag.pdf_layout import extract_fragments, reflow, tokenize_content_stream  # noqa: E402


def _stream(body: bytes, extra: bytes = b"") -> bytes:
    return b"<< " + extra + b" /Length %d >>\nstream\n" % len(body) + body + b"\nendstream\n"


def _pdf(*parts: bytes) -> bytes:
    return b"%PDF-1.4\n" + b"".join(parts) + b"%%EOF\n"


def _text(content: bytes) -> str:
    return PDFParser()._extract_text(_pdf(_stream(content)))


# ---- strings ----------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("raw,want", [
    (b"plain", b"plain"),
    (b"a\\(b\\)c", b"a(b)c"),
    (b"tab\\there", b"tab\there"),
    (b"nl\\nx", b"nl\nx"),
    (b"cr\\rx", b"cr\rx"),
    (b"back\\\\slash", b"back\\slash"),
    (b"oct\\101\\102", b"octAB"),
    (b"short\\7x", b"short\x07x"),
    (b"bs\\bff\\f", b"bs\bff\f"),
    (b"line\\\ncontinued", b"linecontinued"),
    (b"unknown\\qescape", b"unknownqescape"),
])
def test_literal_string_escapes(raw, want):
    assert decode_literal(raw) == want


def test_nested_parentheses_stay_in_one_string():
    toks = tokenize_content_stream(b"BT (outer (inner) tail) Tj ET")
    assert (b"(outer (inner) tail)" in toks) or any(b"outer (inner) tail" in t for t in toks)
    assert _text(b"BT 10 10 Td (outer (inner) tail) Tj ET") == "outer (inner) tail"


def test_hex_strings_in_content():
    assert _text(b"BT 10 10 Td <48656C6C6F> Tj ET") == "Hello"
    assert _text(b"BT 10 10 Td <48 65 6c 6C 6f> Tj ET") == "Hello"          # white space and case do not matter
    assert _text(b"BT 10 10 Td <4869 2> Tj ET") == "Hi"                      # odd digit: padded to 0x20, trimmed as a space


# ---- text operators -----------------------------------------------------------------------------------------------------
def test_tj_array_joins_pieces_and_large_gaps_make_spaces():
    assert _text(b"BT 10 10 Td [(Hel) -20 (lo)] TJ ET") == "Hello"           # kerning, not a word gap
    assert _text(b"BT /F1 12 Tf 10 10 Td [(two) -900 (words)] TJ ET") == "two words"


def test_quote_operators_start_new_lines():
    out = _text(b"BT 14 TL 10 700 Td (first) Tj (second) ' 1 2 (third) \" ET")
    assert out.split("\n") == ["first", "second", "third"]


def test_t_star_and_td_move_down():
    out = _text(b"BT 12 TL 10 700 Td (a) Tj T* (b) Tj 0 -12 Td (c) Tj 0 -12 TD (d) Tj ET")
    assert out.split("\n") == ["a", "b", "c", "d"]


def test_text_matrix_places_text():
    frags = extract_fragments(b"BT 1 0 0 1 300 500 Tm (right) Tj ET BT 1 0 0 1 50 500 Tm (left) Tj ET")
    assert reflow(frags) == "left right"                                    # same base line: ordered by x
    out = _text(b"BT 1 0 0 1 50 400 Tm (low) Tj ET BT 1 0 0 1 50 600 Tm (high) Tj ET")
    assert [l for l in out.split("\n") if l] == ["high", "low"]           # far apart: a paragraph gap between them


def test_words_on_one_line_get_one_space():
    out = _text(b"BT 10 700 Td (alpha) Tj ET BT 60 700 Td (beta) Tj ET BT 110 700.4 Td (gamma) Tj ET")
    assert out == "alpha beta gamma"                                         # 0.4 pt off the base line is the same line


def test_cm_outside_text_objects_is_ignored_by_the_reader():
    assert _text(b"q 1 0 0 1 20 20 cm BT 10 10 Td (inside) Tj ET Q") == "inside"


def test_empty_and_textless_streams():
    assert _text(b"") == ""
    assert _text(b"q 0 0 100 100 re f Q") == ""


def test_comments_and_names_in_content_streams():
    toks = tokenize_content_stream(b"% a comment (not a string)\nBT /F1 9 Tf (x) Tj ET")
    assert b"(x)" in toks and all(b"comment" not in t for t in toks)
    assert b"/F1" in toks


def test_inline_image_data_is_skipped():
    body = b"BT 10 10 Td (before) Tj ET BI /W 2 /H 2 /BPC 8 /CS /G ID \x00(\xff)\x80 EI BT 10 30 Td (after) Tj ET"
    out = _text(body)
    assert "before" in out and "after" in out and "\xff" not in out


# ---- predictors and filters -----------------------------------------------------------------------------------------
def _png_rows(rows, kind):
    """Encode rows (lists of ints) with one PNG filter type per row."""
    out, prev = bytearray(), [0] * len(rows[0])
    for row in rows:
        out.append(kind)
        for i, v in enumerate(row):
            left = row[i - 1] if i else 0
            up, ul = prev[i], (prev[i - 1] if i else 0)
            if kind == 0:
                p = 0
            elif kind == 1:
                p = left
            elif kind == 2:
                p = up
            elif kind == 3:
                p = (left + up) // 2
            else:
                pa, pb, pc = abs(up - ul), abs(left - ul), abs(left + up - 2 * ul)
                p = left if pa <= pb and pa <= pc else up if pb <= pc else ul
            out.append((v - p) & 0xFF)
        prev = row
    return bytes(out)


@pytest.mark.parametrize("kind", [0, 1, 2, 3, 4])
def test_png_predictors(kind):
    rows = [[10, 20, 30, 40, 250], [11, 19, 35, 41, 3], [200, 0, 255, 7, 9]]
    flat = bytes(v for r in rows for v in r)
    assert _png_predict(_png_rows(rows, kind), columns=5) == flat


def test_predictor_through_decode_parms():
    rows = [[1, 2, 3, 4], [5, 6, 7, 8]]
    data = zlib.compress(_png_rows(rows, 2))
    got = apply_filters(data, b"/Filter /FlateDecode /DecodeParms << /Predictor 12 /Columns 4 >>")
    assert got == bytes(range(1, 9))
    assert apply_filters(zlib.compress(b"no predictor"), b"/Filter /FlateDecode /DecodeParms << /Predictor 1 >>") == \
        b"no predictor"


def test_flate_with_trailing_garbage_and_truncation():
    good = zlib.compress(b"BT (kept) Tj ET")
    assert apply_filters(good + b"\r\n", b"/Filter /FlateDecode") == b"BT (kept) Tj ET"
    cut = zlib.compress(b"A" * 5000)[:-6]
    try:
        out = apply_filters(cut, b"/Filter /FlateDecode")
    except Exception:
        out = None
    assert out is None or out.startswith(b"A" * 100)          # either a clean error or the readable prefix


@pytest.mark.parametrize("name,kind", [(b"/DCTDecode", "jpeg"), (b"/JPXDecode", "jp2"), (b"/CCITTFaxDecode", "ccitt"),
                                        (b"/JBIG2Decode", "jbig2")])
def test_image_filters_are_named_for_the_ocr_hook(name, kind):
    assert kind in image_hint(b"<< /Subtype /Image /Filter " + name + b" >>").lower()


def test_filter_abbreviations():
    assert apply_filters(zlib.compress(b"fl"), b"/Filter /Fl") == b"fl"
    assert apply_filters(b"4142>", b"/Filter /AHx") == b"AB"
    assert apply_filters(base64.a85encode(b"abcd", adobe=True)[2:], b"/Filter /A85") == b"abcd"
    assert apply_filters(bytes([1]) + b"ab" + bytes([128]), b"/Filter /RL") == b"ab"


# ---- document structure -------------------------------------------------------------------------------------------------
def test_pages_come_in_tree_order_not_file_order():
    pages = PDFParser().extract_pages(make_pdf([["page one"], ["page two"], ["page three"]]))
    assert pages == ["page one", "page two", "page three"]


def test_nested_page_tree_and_inherited_resources():
    raw = (b"%PDF-1.4\n"
           b"1 0 obj\n<< /Type /Catalog /Pages 2 0 R >>\nendobj\n"
           b"2 0 obj\n<< /Type /Pages /Count 2 /Kids [3 0 R 6 0 R] /Resources << /Font << /F1 9 0 R >> >> >>\nendobj\n"
           b"3 0 obj\n<< /Type /Pages /Parent 2 0 R /Count 1 /Kids [4 0 R] >>\nendobj\n"
           b"4 0 obj\n<< /Type /Page /Parent 3 0 R /Contents 5 0 R >>\nendobj\n"
           b"5 0 obj\n" + _stream(b"BT /F1 12 Tf 10 10 Td (deep page) Tj ET") + b"endobj\n"
           b"6 0 obj\n<< /Type /Page /Parent 2 0 R /Contents [7 0 R 8 0 R] >>\nendobj\n"
           b"7 0 obj\n" + _stream(b"BT /F1 12 Tf 10 700 Td (first part) Tj ET") + b"endobj\n"
           b"8 0 obj\n" + _stream(b"BT /F1 12 Tf 10 680 Td (second part) Tj ET") + b"endobj\n"
           b"9 0 obj\n<< /Type /Font /Subtype /Type1 /BaseFont /Helvetica >>\nendobj\n"
           b"trailer\n<< /Root 1 0 R >>\n%%EOF\n")
    doc = PDFDocument(raw)
    assert doc.pages() == [4, 6]
    assert doc.inherited(4, b"/Resources") is not None                      # found on the grandparent
    assert PDFParser().extract_pages(raw) == ["deep page", "first part\nsecond part"]


def test_objects_inside_an_object_stream():
    inner = {4: b"<< /Type /Page /Parent 2 0 R /Contents 5 0 R >>",
             2: b"<< /Type /Pages /Count 1 /Kids [4 0 R] >>", 1: b"<< /Type /Catalog /Pages 2 0 R >>"}
    head, body = b"", b""
    for num, text in inner.items():
        head += b"%d %d " % (num, len(body))
        body += text + b" "
    data = zlib.compress(head + body)
    raw = (b"%PDF-1.5\n" + b"7 0 obj\n<< /Type /ObjStm /N 3 /First %d /Filter /FlateDecode /Length %d >>\nstream\n"
           % (len(head), len(data)) + data + b"\nendstream\nendobj\n"
           b"5 0 obj\n" + _stream(b"BT 10 10 Td (from an object stream) Tj ET") + b"endobj\n"
           b"trailer\n<< /Root 1 0 R >>\n%%EOF\n")
    assert PDFParser().extract_pages(raw) == ["from an object stream"]


def test_files_without_a_page_tree_fall_back_to_their_streams():
    raw = _pdf(_stream(b"BT 10 10 Td (loose one) Tj ET"), _stream(b"BT 10 10 Td (loose two) Tj ET"))
    text = PDFParser()._extract_text(raw)
    assert "loose one" in text and "loose two" in text
    assert [d for _, d in bare_streams(raw)] == [b"BT 10 10 Td (loose one) Tj ET", b"BT 10 10 Td (loose two) Tj ET"]


def test_a_later_definition_of_an_object_wins():
    raw = (b"%PDF-1.4\n1 0 obj\n<< /Type /Catalog /Pages 2 0 R >>\nendobj\n"
           b"2 0 obj\n<< /Type /Pages /Count 1 /Kids [3 0 R] >>\nendobj\n"
           b"3 0 obj\n<< /Type /Page /Parent 2 0 R /Contents 4 0 R >>\nendobj\n"
           b"4 0 obj\n" + _stream(b"BT 10 10 Td (old text) Tj ET") + b"endobj\n"
           b"4 0 obj\n" + _stream(b"BT 10 10 Td (updated text) Tj ET") + b"endobj\n"        # incremental update
           b"trailer\n<< /Root 1 0 R >>\n%%EOF\n")
    assert PDFParser().extract_pages(raw) == ["updated text"]


def test_length_given_as_an_indirect_reference():
    body = b"BT 10 10 Td (indirect length) Tj ET"
    raw = (b"%PDF-1.4\n1 0 obj\n<< /Type /Catalog /Pages 2 0 R >>\nendobj\n"
           b"2 0 obj\n<< /Type /Pages /Count 1 /Kids [3 0 R] >>\nendobj\n"
           b"3 0 obj\n<< /Type /Page /Parent 2 0 R /Contents 4 0 R >>\nendobj\n"
           b"4 0 obj\n<< /Length 5 0 R >>\nstream\n" + body + b"\nendstream\nendobj\n"
           b"5 0 obj\n%d\nendobj\ntrailer\n<< /Root 1 0 R >>\n%%%%EOF\n" % len(body))
    assert PDFParser().extract_pages(raw) == ["indirect length"]


def test_garbage_is_reported_as_one_chunk_and_does_not_raise():
    chunks = PDFParser().parse(b"this is not a pdf at all")
    assert len(chunks) == 1 and chunks[0].metadata["error"] == "invalid_pdf"
    assert not chunks[0].metadata.get("pdf_encrypted")
    assert PDFParser()._extract_text(b"%PDF-1.4\n%%EOF\n") == ""


# ---- fonts --------------------------------------------------------------------------------------------------------------
def test_two_byte_codes_through_a_cmap_in_a_page():
    assert PDFParser().extract_pages(make_pdf([["two byte codes"]], hex_font=True)) == ["two byte codes"]
    assert PDFParser().extract_pages(make_pdf([["deflated too"]], hex_font=True, flate=True)) == ["deflated too"]


def test_bfrange_with_surrogate_targets_and_ligatures():
    cmap = ToUnicode(b"1 beginbfchar\n<05> <D83DDE00>\nendbfchar\n1 beginbfrange\n<30> <32> <FB00>\nendbfrange\n")
    assert cmap.decode(bytes([5])) == "\U0001F600"
    assert cmap.decode(bytes([0x30, 0x31, 0x32])) == "ﬀﬁﬂ"


def test_codespace_decides_the_code_width():
    one = ToUnicode(b"1 begincodespacerange\n<00> <FF>\nendcodespacerange\n1 beginbfchar\n<41> <0042>\nendbfchar\n")
    assert not one.two_byte and one.decode(b"A") == "B"
    two = ToUnicode(b"1 begincodespacerange\n<0000> <FFFF>\nendcodespacerange\n1 beginbfchar\n<0041> <0042>\nendbfchar\n")
    assert two.two_byte and two.decode(b"\x00A") == "B"


def test_fonts_are_switched_by_tf():
    raw = (b"%PDF-1.4\n1 0 obj\n<< /Type /Catalog /Pages 2 0 R >>\nendobj\n"
           b"2 0 obj\n<< /Type /Pages /Count 1 /Kids [3 0 R] >>\nendobj\n"
           b"3 0 obj\n<< /Type /Page /Parent 2 0 R /Contents 4 0 R /Resources << /Font << /F1 5 0 R /F2 6 0 R >> >> >>\n"
           b"endobj\n4 0 obj\n" + _stream(b"BT /F1 12 Tf 10 700 Td (plain) Tj /F2 12 Tf 0 -20 Td <00010002> Tj ET")
           + b"endobj\n5 0 obj\n<< /Type /Font /Subtype /Type1 /BaseFont /Helvetica >>\nendobj\n"
           b"6 0 obj\n<< /Type /Font /Subtype /Type0 /Encoding /Identity-H /ToUnicode 7 0 R >>\nendobj\n"
           b"7 0 obj\n" + _stream(b"2 beginbfchar\n<0001> <006D>\n<0002> <0061>\nendbfchar\n") + b"endobj\n"
           b"trailer\n<< /Root 1 0 R >>\n%%EOF\n")
    assert PDFParser().extract_pages(raw) == ["plain\nma"]


# ---- encryption ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind", ["rc4", "aes128", "aes256"])
def test_user_password_opens_every_generation(kind):
    raw = make_pdf([["secret of " + kind]], encrypt=kind, user_pw="open sesame")
    assert PDFParser().extract_pages(raw, password="open sesame") == ["secret of " + kind]


@pytest.mark.parametrize("kind", ["rc4", "aes128", "aes256"])
def test_owner_password_opens_too(kind):
    raw = make_pdf([["owned " + kind]], encrypt=kind, user_pw="u", owner_pw="the owner")
    assert PDFParser().extract_pages(raw, password="the owner") == ["owned " + kind]


@pytest.mark.parametrize("kind", ["rc4", "aes128", "aes256"])
def test_wrong_password_is_refused(kind):
    raw = make_pdf([["nope"]], encrypt=kind, user_pw="right")
    chunks = PDFParser().parse(raw, metadata={"pdf_password": "wrong"})
    assert len(chunks) == 1 and chunks[0].metadata["error"] == "encrypted_password_required"
    assert "nope" not in chunks[0].text


@pytest.mark.parametrize("kind", ["rc4", "aes128", "aes256"])
def test_empty_user_password_needs_no_input(kind):
    raw = make_pdf([["open to read " + kind]], encrypt=kind, user_pw="")
    chunks = PDFParser().parse(raw)
    assert "open to read " + kind in chunks[0].text and chunks[0].metadata.get("pdf_encrypted")


def test_detect_encryption_reads_the_dictionary():
    for kind, (v, r, bits) in {"rc4": (2, 3, 128), "aes128": (4, 4, 128), "aes256": (5, 6, 256)}.items():
        enc = pdf_crypto.detect_encryption(make_pdf([["x"]], encrypt=kind))
        assert enc is not None and enc.supported and (enc.version, enc.revision) == (v, r)
        assert enc.length_bits == bits
    assert pdf_crypto.detect_encryption(make_pdf([["x"]])) is None


def test_rc4_and_aes_primitives():
    assert pdf_crypto.rc4(b"Key", b"Plaintext").hex() == "bbf316e8d940af0ad3"           # the classic test vector
    assert pdf_crypto.rc4(b"Key", pdf_crypto.rc4(b"Key", b"round trip")) == b"round trip"
    key = bytes(range(16))
    block = bytes.fromhex("00112233445566778899aabbccddeeff")
    if hasattr(pdf_crypto, "aes_encrypt_block"):
        assert pdf_crypto.aes_encrypt_block(key, block).hex() == "69c4e0d86a7b0430d8cdb78070b4c55a"   # FIPS-197 C.1


def test_encrypted_strings_and_flate_together():
    raw = make_pdf([["both layers"]], encrypt="aes128", user_pw="k", flate=True)
    assert PDFParser().extract_pages(raw, password="k") == ["both layers"]


# ---- OCR hook and chunks --------------------------------------------------------------------------------------------
def test_ocr_runs_for_pages_that_are_only_pictures():
    img = (b"1 0 obj\n<< /Type /XObject /Subtype /Image /Filter /DCTDecode /Width 8 /Height 8 /Length 6 >>\nstream\n"
           b"\xff\xd8jpeg\nendstream\nendobj\n")
    seen = []

    def ocr(data, hint=None):
        seen.append((bytes(data[:2]), hint))
        return "text from the picture"

    chunks = PDFParser(ocr_fn=ocr).parse(_pdf(img))
    assert seen and seen[0][0] == b"\xff\xd8"
    assert any("text from the picture" in c.text for c in chunks)


def test_ocr_is_not_asked_when_the_page_has_text():
    calls = []
    raw = make_pdf([["already text"]])
    chunks = PDFParser(ocr_fn=lambda d, h=None: calls.append(1) or "never").parse(raw)
    assert not calls and "already text" in chunks[0].text


def test_chunks_carry_page_numbers_and_overlap():
    pages = [["word%d" % (100 * p + i) for i in range(60)] for p in range(3)]
    chunks = PDFParser(chunk_size=40, overlap=8).parse(make_pdf(pages))
    assert len(chunks) > 3
    nums = [c.metadata.get("page") for c in chunks if c.metadata.get("page") is not None]
    assert nums == sorted(nums) and set(nums) <= {1, 2, 3}
    joined = " ".join(c.text for c in chunks)
    assert "word0" in joined and "word259" in joined


def test_parse_of_text_that_is_not_a_pdf():
    chunks = PDFParser(chunk_size=16, overlap=2).parse("plain text that is not a pdf " * 8)
    assert len(chunks) == 1 and chunks[0].metadata["error"] == "invalid_pdf" and "not a PDF" in chunks[0].text

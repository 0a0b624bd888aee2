"""The stream filters and dictionary helpers of the PDF reader, one case at a time (the shape of the reference's
tests/test_pdf_filters.py: a class of small cases per filter).  Whole documents are covered by tests/test_pdf.py and
tests/test_pdf_details.py."""
import base64
import zlib

import pytest

from zse_b200.rag.pdf import (PDFError, _ascii85, _int, _lzw, _name_value, _run_length, _string, apply_filters,
                              decode_literal, image_hint)


def pack_codes(codes):
    """(value, width) pairs -> bytes, most significant bit first, zero padded."""
    acc = bits = 0
    out = bytearray()
    for v, w in codes:
        acc, bits = (acc << w) | v, bits + w
        while bits >= 8:
            out.append((acc >> (bits - 8)) & 0xFF)
            bits -= 8
    if bits:
        out.append((acc << (8 - bits)) & 0xFF)
    return bytes(out)


# ---- ASCIIHex --------------------------------------------------------------------------------------------------------
def test_hex_basic_round_trip_in_both_cases():
    assert apply_filters(b"48656c6C6F>", b"/Filter /ASCIIHexDecode") == b"Hello"


def test_hex_ignores_white_space_of_every_kind():
    assert apply_filters(b"48 65\n6c\t6c\r\n6f >", b"/Filter /ASCIIHexDecode") == b"Hello"


def test_hex_pads_an_odd_last_digit_with_zero():
    assert apply_filters(b"ABC>", b"/Filter /ASCIIHexDecode") == b"\xab\xc0"


def test_hex_stops_at_the_end_marker_and_works_without_one():
    assert apply_filters(b"4142>4344", b"/Filter /AHx") == b"AB"
    assert apply_filters(b"4142", b"/Filter /AHx") == b"AB"
    assert apply_filters(b">", b"/Filter /AHx") == b""


# ---- ASCII85 ---------------------------------------------------------------------------------------------------------
def test_a85_full_groups():
    assert _ascii85(b"87cURD]i,\"Ebo80~>") == b"Hello World!"
    assert _ascii85(base64.a85encode(bytes(range(256)), adobe=True)) == bytes(range(256))


def test_a85_z_stands_for_a_zero_word_between_groups():
    assert _ascii85(b"z87cURz~>") == b"\0\0\0\0Hell\0\0\0\0"


@pytest.mark.parametrize("n", [1, 2, 3])
def test_a85_partial_last_group(n):
    data = b"retrieval"[:4 + n]
    assert _ascii85(base64.a85encode(data, adobe=True)) == data


def test_a85_white_space_prefix_and_end_marker():
    enc = base64.a85encode(b"spread over lines", adobe=True)
    broken = b"\n".join(enc[i:i + 5] for i in range(0, len(enc), 5))
    assert _ascii85(broken) == b"spread over lines"
    assert _ascii85(enc[2:]) == b"spread over lines"                            # without "<~"
    assert _ascii85(enc[2:-2]) == b"spread over lines"                          # without "~>" either
    assert _ascii85(enc + b"trailing bytes") == b"spread over lines"            # nothing after "~>" is read
    assert _ascii85(b"~>") == b"" and _ascii85(b"") == b""


# ---- RunLength -------------------------------------------------------------------------------------------------------
def test_run_length_literal_run():
    assert _run_length(bytes([4]) + b"hello" + bytes([128])) == b"hello"
    assert _run_length(bytes([127]) + bytes(range(128)) + bytes([128])) == bytes(range(128))   # the longest literal


def test_run_length_repeat_run():
    assert _run_length(bytes([255, 0x41, 128])) == b"AA"                        # 257 - 255
    assert _run_length(bytes([129, 0x42, 128])) == b"B" * 128                    # the longest repeat


def test_run_length_end_marker_and_missing_marker():
    assert _run_length(bytes([0]) + b"a" + bytes([128, 0]) + b"b") == b"a"
    assert _run_length(bytes([0]) + b"a") == b"a"                               # data may simply end
    assert _run_length(b"") == b"" and _run_length(bytes([128])) == b""


def test_run_length_mixed_and_truncated():
    data = bytes([1]) + b"ab" + bytes([254]) + b"c" + bytes([0]) + b"d" + bytes([128])
    assert _run_length(data) == b"abcccd"
    assert _run_length(bytes([5]) + b"ab") == b"ab"                             # a literal run cut short keeps what is there
    assert _run_length(bytes([250])) == b""                                     # a repeat without its byte


# ---- LZW -------------------------------------------------------------------------------------------------------------
def test_lzw_literals_then_table_entries():
    # clear, A, B, 258 (= "AB"), 260 (= "ABA": not in the table yet, the K-w-K case), end
    assert _lzw(pack_codes([(256, 9), (65, 9), (66, 9), (258, 9), (260, 9), (257, 9)])) == b"ABABABA"


def test_lzw_clear_code_in_mid_stream_forgets_the_table():
    codes = [(256, 9), (65, 9), (65, 9), (258, 9), (256, 9), (66, 9), (66, 9), (258, 9), (257, 9)]
    assert _lzw(pack_codes(codes)) == b"AAAA" + b"BBBB"                          # 258 means "AA", then "BB"


def test_lzw_stops_at_end_of_data_and_survives_a_missing_one():
    assert _lzw(pack_codes([(256, 9), (72, 9), (105, 9), (257, 9), (72, 9)])) == b"Hi"
    assert _lzw(pack_codes([(256, 9), (72, 9), (105, 9)])) == b"Hi"
    assert _lzw(b"") == b""


def test_lzw_with_a_png_predictor():
    rows = bytes([2, 1, 2, 3]) + bytes([2, 1, 1, 1])                            # "up" rows of 3 columns
    codes = [(256, 9)] + [(b, 9) for b in rows] + [(257, 9)]
    out = apply_filters(pack_codes(codes), b"/Filter /LZWDecode /DecodeParms << /Predictor 12 /Columns 3 >>")
    assert out == bytes([1, 2, 3, 2, 3, 4])


# ---- chains and names --------------------------------------------------------------------------------------------------
def test_no_filter_returns_the_data():
    assert apply_filters(b"plain", b"/Length 5") == b"plain"


def test_filters_run_in_the_order_given():
    inner = zlib.compress(b"order matters")
    assert apply_filters(inner.hex().encode() + b">", b"/Filter [/ASCIIHexDecode /FlateDecode]") == b"order matters"
    rl = bytes([len(inner) - 1]) + inner + bytes([128])
    assert apply_filters(rl, b"/Filter [ /RL /Fl ]") == b"order matters"


def test_unknown_filter_is_an_error_with_its_name():
    with pytest.raises(PDFError, match="Crypt"):
        apply_filters(b"x", b"/Filter /Crypt")


def test_image_hint_names():
    assert image_hint(b"/Filter /DCTDecode") == "jpeg" and image_hint(b"/Filter [/FlateDecode /DCT]") == "jpeg"
    assert image_hint(b"/Filter /JPXDecode") == "jp2" and image_hint(b"/Filter /CCITTFaxDecode") == "ccitt"
    assert image_hint(b"/Filter /JBIG2Decode") == "jbig2"
    assert image_hint(b"/Filter /FlateDecode") == "raw" and image_hint(b"/Width 4") == "raw"


# ---- dictionary helpers ------------------------------------------------------------------------------------------------
def test_values_of_each_kind_are_cut_out_whole():
    d = (b"/Type /Page /Parent 3 0 R /Len 42 /Box [0 0 612 792] /Title (a (nested) title) /ID <4A4b> "
         b"/Res << /Font << /F1 5 0 R >> >> /Length1 7")
    assert _name_value(d, b"/Type") == b"/Page" and _name_value(d, b"/Parent") == b"3 0 R"
    assert _name_value(d, b"/Box") == b"[0 0 612 792]" and _name_value(d, b"/Title") == b"(a (nested) title)"
    assert _name_value(d, b"/ID") == b"<4A4b>" and b"/F1 5 0 R" in _name_value(d, b"/Res")
    assert _name_value(d, b"/Missing") is None
    assert _int(d, b"/Len") == 42 and _int(d, b"/Length1") == 7                  # "/Len" does not match "/Length1"
    assert _int(d, b"/Length", 9) == 9 and _int(d, b"/Type", -1) == -1
    assert _int(b"/Rotate -90", b"/Rotate") == -90


def test_strings_in_both_notations():
    assert _string(b"(plain)") == b"plain" and _string(b" <48 69> ") == b"Hi" and _string(b"<487>") == b"Hp"
    assert _string(None) == b"" and _string(b"") == b"" and _string(b"/Name") == b""


def test_literal_string_escapes_one_by_one():
    assert decode_literal(rb"a\nb\rc\td\be\ff") == b"a\nb\rc\td\x08e\x0cf"
    assert decode_literal(rb"\(\)\\") == b"()\\"
    assert decode_literal(rb"\101\60\0053") == b"A0\x053"                        # 1 to 3 octal digits
    assert decode_literal(rb"\777") == b"\xff"                                  # high bits are dropped
    assert decode_literal(b"line \\\ncontinues \\\r\nhere") == b"line continues here"
    assert decode_literal(rb"\q") == b"q" and decode_literal(b"ends with \\") == b"ends with "


# ---- the document model: what a page is made of ---------------------------------------------------------------------
def _obj(n, body, stream=None):
    if stream is None:
        return b"%d 0 obj\n%s\nendobj\n" % (n, body)
    return b"%d 0 obj\n<< %s /Length %d >>\nstream\n%s\nendstream\nendobj\n" % (n, body, len(stream), stream)


def test_a_page_names_its_contents_fonts_and_images():
    from zse_b200.rag.pdf import PDFDocument
    cmap = b"1 beginbfchar\n<0041> <0058>\nendbfchar"
    raw = b"%PDF-1.4\n" + b"".join([
        _obj(1, b"<< /Type /Catalog /Pages 2 0 R >>"),
        _obj(2, b"<< /Type /Pages /Kids [3 0 R] /Count 1 /Resources 4 0 R >>"),      # resources come from the parent
        _obj(3, b"<< /Type /Page /Parent 2 0 R /Contents 5 0 R >>"),
        _obj(4, b"<< /Font << /F1 6 0 R /F2 7 0 R >> /XObject << /Im1 9 0 R /Fm1 10 0 R >> >>"),
        _obj(5, b"[ 11 0 R 12 0 R 99 0 R ]"),                                          # contents as an array object
        _obj(6, b"<< /Type /Font /Subtype /Type0 /Encoding /Identity-H /ToUnicode 8 0 R >>"),
        _obj(7, b"<< /Type /Font /Subtype /Type1 /BaseFont /Helvetica >>"),
        _obj(8, b"", cmap),
        _obj(9, b"/Type /XObject /Subtype /Image /Width 1 /Height 1 /Filter /DCTDecode", b"\xff\xd8jpeg-bytes"),
        _obj(10, b"/Type /XObject /Subtype /Form", b"q Q"),
        _obj(11, b"", b"BT (first) Tj ET"),
        _obj(12, b"", b"BT (second) Tj ET"),
    ]) + b"%%EOF\n"
    doc = PDFDocument(raw)
    assert doc.pages() == [3] and doc.enc is None
    assert doc.page_content(3) == b"BT (first) Tj ET\nBT (second) Tj ET"           # the missing object 99 is skipped
    fonts = doc.page_fonts(3)
    assert set(fonts) == {b"F1", b"F2"} and fonts[b"F1"].two_byte and not fonts[b"F2"].two_byte
    assert fonts[b"F1"].decode(b"\x00\x41") == "X" and fonts[b"F2"].decode(b"A") == "A"
    images = doc.page_images(3)
    assert images == [(b"\xff\xd8jpeg-bytes", "jpeg")]                              # the form XObject is not an image
    with pytest.raises(PDFError, match="not a PDF"):
        PDFDocument(b"plain text")

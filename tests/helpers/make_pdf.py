"""Tiny PDF writer for the parser tests: pages of text lines, optional Flate, hex strings through a /ToUnicode CMap,
optional encryption with the standard security handler (RC4-128 R3, AES-128 R4, AES-256 R6).  The encryption side is
written from the PDF specification so that the reader in zse_b200.rag is checked against an independent writer."""
import hashlib
import os
import struct
import zlib

from zse_b200.rag import pdf_crypto as pc


def _esc(s: str) -> bytes:
    return s.encode("latin-1").replace(b"\\", b"\\\\").replace(b"(", b"\\(").replace(b")", b"\\)")


def _content(lines, hex_font=False):
    ops = [b"BT", b"/F1 12 Tf", b"72 720 Td"]
    for i, line in enumerate(lines):
        if i:
            ops.append(b"0 -14 Td")
        if hex_font:
            ops.append(b"<" + "".join("%04X" % (ord(c) + 1) for c in line).encode() + b"> Tj")
        else:
            words = line.split(" ")
            if len(words) > 2:      # exercise TJ with a word-gap kern
                ops.append(b"[(" + _esc(words[0]) + b") -300 (" + _esc(" ".join(words[1:])) + b")] TJ")
            else:
                ops.append(b"(" + _esc(line) + b") Tj")
    ops.append(b"ET")
    return b"\n".join(ops)


def _cmap():
    return (b"/CIDInit /ProcSet findresource begin 12 dict begin begincmap\n1 begincodespacerange <0000> <FFFF> "
            b"endcodespacerange\n1 beginbfrange\n<0001> <00FF> <0000>\nendbfrange\nendcmap end end")


def make_pdf(pages, flate=False, hex_font=False, encrypt=None, user_pw="", owner_pw="owner"):
    """pages: list of lists of lines.  encrypt: None | "rc4" | "aes128" | "aes256"."""
    objs = {}                       # num -> (dict bytes, stream bytes or None)
    n_pages = len(pages)
    font_num, cmap_num = 3, 4
    kids = []
    num = 5
    for lines in pages:
        content = _content(lines, hex_font)
        d = b""
        if flate:
            content = zlib.compress(content)
            d = b"/Filter /FlateDecode "
        objs[num + 1] = (d, content)
        objs[num] = (b"<< /Type /Page /Parent 2 0 R /MediaBox [0 0 612 792] /Contents %d 0 R /Resources << /Font << "
                     b"/F1 %d 0 R >> >> >>" % (num + 1, font_num), None)
        kids.append(num)
        num += 2
    objs[1] = (b"<< /Type /Catalog /Pages 2 0 R >>", None)
    objs[2] = (b"<< /Type /Pages /Count %d /Kids [%s] >>" % (n_pages, b" ".join(b"%d 0 R" % k for k in kids)), None)
    if hex_font:
        objs[font_num] = (b"<< /Type /Font /Subtype /Type0 /BaseFont /Fake /Encoding /Identity-H /ToUnicode %d 0 R >>"
                          % cmap_num, None)
        objs[cmap_num] = (b"", _cmap())
    else:
        objs[font_num] = (b"<< /Type /Font /Subtype /Type1 /BaseFont /Helvetica >>", None)
    file_id = hashlib.md5(repr(pages).encode()).digest()
    enc_num, enc_dict, obj_key = None, b"", None
    if encrypt:
        enc_num = num
        p = -44
        if encrypt in ("rc4", "aes128"):
            r, v, n = (3, 2, 16) if encrypt == "rc4" else (4, 4, 16)
            d = hashlib.md5(pc._pad_password(owner_pw.encode())).digest()
            for _ in range(50):
                d = hashlib.md5(d).digest()
            o = pc._pad_password(user_pw.encode())
            for i in range(20):
                o = pc.rc4(bytes(b ^ i for b in d[:n]), o)
            h = hashlib.md5(pc._pad_password(user_pw.encode()) + o + struct.pack("<i", p) + file_id).digest()
            for _ in range(50):
                h = hashlib.md5(h[:n]).digest()
            key = h[:n]
            u = pc.rc4(key, hashlib.md5(pc.PAD + file_id).digest())
            for i in range(1, 20):
                u = pc.rc4(bytes(b ^ i for b in key), u)
            u += bytes(16)
            cf = b" /CF << /StdCF << /CFM /AESV2 /AuthEvent /DocOpen /Length 16 >> >> /StmF /StdCF /StrF /StdCF" \
                if encrypt == "aes128" else b""
            enc_dict = (b"<< /Filter /Standard /V %d /R %d /Length 128 /P %d /O <%s> /U <%s>%s >>"
                        % (v, r, p, o.hex().encode(), u.hex().encode(), cf))

            def obj_key(onum, aes=(encrypt == "aes128")):
                hh = hashlib.md5(key + struct.pack("<I", onum)[:3] + b"\0\0" + (b"sAlT" if aes else b""))
                return hh.digest()[:16]
        else:
            key = hashlib.sha256(b"file key " + file_id).digest()
            upw, opw = user_pw.encode(), owner_pw.encode()
            uvs, uks, ovs, oks = (os.urandom(8) for _ in range(4))
            u = pc.hash_2b(upw, uvs) + uvs + uks
            ue = pc.aes_cbc_encrypt(pc.hash_2b(upw, uks), bytes(16), key, pad=False)
            o = pc.hash_2b(opw, ovs, u) + ovs + oks
            oe = pc.aes_cbc_encrypt(pc.hash_2b(opw, oks, u), bytes(16), key, pad=False)
            enc_dict = (b"<< /Filter /Standard /V 5 /R 6 /Length 256 /P %d /O <%s> /U <%s> /OE <%s> /UE <%s> /CF << "
                        b"/StdCF << /CFM /AESV3 /AuthEvent /DocOpen /Length 32 >> >> /StmF /StdCF /StrF /StdCF >>"
                        % (p, o.hex().encode(), u.hex().encode(), oe.hex().encode(), ue.hex().encode()))

            def obj_key(onum):
                return key
        objs[enc_num] = (enc_dict, None)
    out = bytearray(b"%PDF-1.7\n%\xe2\xe3\xcf\xd3\n")
    offsets = {}
    for onum in sorted(objs):
        d, stream = objs[onum]
        offsets[onum] = len(out)
        out += b"%d 0 obj\n" % onum
        if stream is None:
            out += d + b"\n"
        else:
            if encrypt and onum != enc_num:
                k = obj_key(onum)
                stream = pc.rc4(k, stream) if encrypt == "rc4" else os.urandom(16)[:0] + _aes(k, stream)
            out += b"<< " + d + b"/Length %d >>\nstream\n" % len(stream) + stream + b"\nendstream\n"
        out += b"endobj\n"
    xref = len(out)
    out += b"xref\n0 %d\n" % (max(objs) + 1)
    out += b"trailer\n<< /Size %d /Root 1 0 R /ID [<%s> <%s>]%s >>\nstartxref\n%d\n%%%%EOF\n" % (
        max(objs) + 1, file_id.hex().encode(), file_id.hex().encode(),
        (b" /Encrypt %d 0 R" % enc_num) if encrypt else b"", xref)
    return bytes(out)


def _aes(key, data):
    iv = os.urandom(16)
    return iv + pc.aes_cbc_encrypt(key, iv, data)

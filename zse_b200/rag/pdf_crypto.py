"""Decryption for the PDF standard security handler, revisions 2-6, with no third-party code
(capabilities of zse-engine/zse_engine/rag/pdf_crypto.py:40-872): RC4 (40-128 bit), AES-128-CBC (V4) and AES-256-CBC
(V5, R5 and R6 with the iterated hash of ISO 32000-2 "Algorithm 2.B").  Hashes come from ``hashlib``; RC4 and AES are
written out here.
"""
from __future__ import annotations

import hashlib
import struct
from typing import List, Optional

PAD = bytes.fromhex("28bf4e5e4e758a4164004e56fffa01082e2e00b6d0683e802f0ca9fe6453697a")


# ---- RC4 ---------------------------------------------------------------------------------------------------------
def rc4(key: bytes, data: bytes) -> bytes:
    s = list(range(256))
    j = 0
    for i in range(256):
        j = (j + s[i] + key[i % len(key)]) & 0xFF
        s[i], s[j] = s[j], s[i]
    out = bytearray(len(data))
    i = j = 0
    for n, b in enumerate(data):
        i = (i + 1) & 0xFF
        j = (j + s[i]) & 0xFF
        s[i], s[j] = s[j], s[i]
        out[n] = b ^ s[(s[i] + s[j]) & 0xFF]
    return bytes(out)


# ---- AES (table-free apart from the S-boxes, which are generated) ---------------------------------------------------
def _build_sboxes():
    # multiplicative inverse in GF(2^8) followed by the affine map
    exp, log = [0] * 512, [0] * 256
    x = 1
    for i in range(255):
        exp[i] = x
        log[x] = i
        x ^= (x << 1) ^ (0x11B if x & 0x80 else 0)
        x &= 0xFF
    for i in range(255, 512):
        exp[i] = exp[i - 255]
    sbox = [0] * 256
    for v in range(256):
        inv = 0 if v == 0 else exp[255 - log[v]]
        r = inv
        for _ in range(4):
            inv = ((inv << 1) | (inv >> 7)) & 0xFF
            r ^= inv
        sbox[v] = r ^ 0x63
    inv_sbox = [0] * 256
    for i, v in enumerate(sbox):
        inv_sbox[v] = i
    return sbox, inv_sbox, exp, log


_SBOX, _INV_SBOX, _EXP, _LOG = _build_sboxes()


def _gmul(a: int, b: int) -> int:
    return 0 if a == 0 or b == 0 else _EXP[_LOG[a] + _LOG[b]]


def expand_key(key: bytes) -> List[bytes]:
    nk = len(key) // 4
    if nk not in (4, 6, 8):
        raise ValueError("AES key must be 16, 24 or 32 bytes")
    rounds = nk + 6
    w = [key[4 * i:4 * i + 4] for i in range(nk)]
    rcon = 1
    for i in range(nk, 4 * (rounds + 1)):
        t = w[i - 1]
        if i % nk == 0:
            t = bytes([_SBOX[t[1]] ^ rcon, _SBOX[t[2]], _SBOX[t[3]], _SBOX[t[0]]])
            rcon = _gmul(rcon, 2)
        elif nk > 6 and i % nk == 4:
            t = bytes(_SBOX[b] for b in t)
        w.append(bytes(a ^ b for a, b in zip(w[i - nk], t)))
    return [b"".join(w[4 * r:4 * r + 4]) for r in range(rounds + 1)]


_MUL = {m: bytes(_gmul(m, v) for v in range(256)) for m in (1, 2, 3, 9, 11, 13, 14)}
_SHIFT = tuple(4 * ((c + r) % 4) + r for c in range(4) for r in range(4))
_INV_SHIFT = tuple(4 * ((c - r) % 4) + r for c in range(4) for r in range(4))
_SBOX_B, _INV_SBOX_B = bytes(_SBOX), bytes(_INV_SBOX)


def _shift_rows(s: bytearray, inverse: bool) -> bytearray:
    idx = _INV_SHIFT if inverse else _SHIFT
    return bytearray(s[i] for i in idx)


def _mix(s: bytearray, m) -> bytearray:
    m0, m1, m2, m3 = (_MUL[x] for x in m)
    o = bytearray(16)
    for c in (0, 4, 8, 12):
        a, b, cc, d = s[c], s[c + 1], s[c + 2], s[c + 3]
        o[c] = m0[a] ^ m1[b] ^ m2[cc] ^ m3[d]
        o[c + 1] = m0[b] ^ m1[cc] ^ m2[d] ^ m3[a]
        o[c + 2] = m0[cc] ^ m1[d] ^ m2[a] ^ m3[b]
        o[c + 3] = m0[d] ^ m1[a] ^ m2[b] ^ m3[cc]
    return o


def encrypt_block(block: bytes, rk: List[bytes]) -> bytes:
    s = bytearray((int.from_bytes(block, "big") ^ int.from_bytes(rk[0], "big")).to_bytes(16, "big"))
    last = len(rk) - 1
    for r in range(1, len(rk)):
        s = _shift_rows(s.translate(_SBOX_B), False)
        if r != last:
            s = _mix(s, (2, 3, 1, 1))
        s = bytearray((int.from_bytes(s, "big") ^ int.from_bytes(rk[r], "big")).to_bytes(16, "big"))
    return bytes(s)


def decrypt_block(block: bytes, rk: List[bytes]) -> bytes:
    s = bytearray((int.from_bytes(block, "big") ^ int.from_bytes(rk[-1], "big")).to_bytes(16, "big"))
    for r in range(len(rk) - 2, -1, -1):
        s = _shift_rows(s, True).translate(_INV_SBOX_B)
        s = bytearray((int.from_bytes(s, "big") ^ int.from_bytes(rk[r], "big")).to_bytes(16, "big"))
        if r != 0:
            s = _mix(s, (14, 11, 13, 9))
    return bytes(s)


def aes_cbc_encrypt(key: bytes, iv: bytes, data: bytes, pad: bool = True) -> bytes:
    rk = expand_key(key)
    if pad:
        n = 16 - len(data) % 16
        data = data + bytes([n]) * n
    out, prev = bytearray(), iv
    for i in range(0, len(data) - len(data) % 16, 16):
        prev = encrypt_block(bytes(a ^ b for a, b in zip(data[i:i + 16], prev)), rk)
        out += prev
    return bytes(out)


def aes_cbc_decrypt(key: bytes, data: bytes, iv: Optional[bytes] = None, unpad: bool = True) -> bytes:
    """``iv`` None: the first 16 bytes of ``data`` are the IV (how PDF stores AES strings and streams)."""
    if iv is None:
        if len(data) < 16:
            return b""
        iv, data = data[:16], data[16:]
    rk = expand_key(key)
    out, prev = bytearray(), iv
    for i in range(0, len(data) - len(data) % 16, 16):
        blk = data[i:i + 16]
        out += bytes(a ^ b for a, b in zip(decrypt_block(blk, rk), prev))
        prev = blk
    if unpad and out:
        n = out[-1]
        if 1 <= n <= 16 and out.endswith(bytes([n]) * n):
            del out[-n:]
    return bytes(out)


# the reference's names for the two key sizes (zse-engine/zse_engine/rag/pdf_crypto.py:182-337); the key length selects
# the variant here
def aes128_cbc_decrypt(key: bytes, data: bytes) -> bytes:
    return aes_cbc_decrypt(key[:16], data)


def aes128_cbc_encrypt(key: bytes, iv: bytes, data: bytes, pad: bool = True) -> bytes:
    return aes_cbc_encrypt(key[:16], iv, data, pad)


def aes256_cbc_decrypt(key: bytes, data: bytes, iv: Optional[bytes] = None, strip_pad: bool = True) -> bytes:
    return aes_cbc_decrypt(key[:32], data, iv, strip_pad)


def aes256_cbc_encrypt(key: bytes, iv: bytes, data: bytes, pad: bool = True) -> bytes:
    return aes_cbc_encrypt(key[:32], iv, data, pad)


# ---- key derivation -------------------------------------------------------------------------------------------------
def _pad_password(pw: bytes) -> bytes:
    return (pw + PAD)[:32]


def hash_2b(password: bytes, salt: bytes, udata: bytes = b"") -> bytes:
    """ISO 32000-2 Algorithm 2.B (revision 6)."""
    k = hashlib.sha256(password + salt + udata).digest()
    i = 0
    while True:
        k1 = (password + k + udata) * 64
        e = aes_cbc_encrypt(k[:16], k[16:32], k1, pad=False)
        mod = sum(e[:16]) % 3
        k = (hashlib.sha256, hashlib.sha384, hashlib.sha512)[mod](e).digest()
        i += 1
        if i >= 64 and e[-1] <= i - 32:
            break
    return k[:32]


class PDFEncryption:
    """Parameters of an /Encrypt dictionary + the file key once a password has been accepted."""

    def __init__(self, v: int, r: int, length_bits: int, o: bytes, u: bytes, p: int, file_id: bytes,
                 encrypt_metadata: bool = True, oe: bytes = b"", ue: bytes = b"", aes: bool = False):
        self.v, self.r, self.length_bits = v, r, length_bits
        self.o, self.u, self.p, self.file_id = o, u, p, file_id
        self.encrypt_metadata, self.oe, self.ue, self.aes = encrypt_metadata, oe, ue, aes
        self.key: Optional[bytes] = None

    # revisions 2-4 ---------------------------------------------------------------------------------------------
    def _key_r234(self, password: bytes) -> bytes:
        n = 5 if self.r == 2 else self.length_bits // 8
        h = hashlib.md5(_pad_password(password) + self.o[:32] + struct.pack("<i", self.p) + self.file_id)
        if self.r >= 4 and not self.encrypt_metadata:
            h.update(b"\xff\xff\xff\xff")
        d = h.digest()
        if self.r >= 3:
            for _ in range(50):
                d = hashlib.md5(d[:n]).digest()
        return d[:n]

    def _check_user_r234(self, key: bytes) -> bool:
        if self.r == 2:
            return rc4(key, PAD) == self.u[:32]
        x = rc4(key, hashlib.md5(PAD + self.file_id).digest())
        for i in range(1, 20):
            x = rc4(bytes(b ^ i for b in key), x)
        return x[:16] == self.u[:16]

    def _user_pw_from_owner_r234(self, owner_pw: bytes) -> bytes:
        n = 5 if self.r == 2 else self.length_bits // 8
        d = hashlib.md5(_pad_password(owner_pw)).digest()
        if self.r >= 3:
            for _ in range(50):
                d = hashlib.md5(d).digest()
        k = d[:n]
        x = self.o[:32]
        if self.r == 2:
            return rc4(k, x)
        for i in range(19, -1, -1):
            x = rc4(bytes(b ^ i for b in k), x)
        return x

    # revisions 5-6 ---------------------------------------------------------------------------------------------
    def _hash56(self, pw: bytes, salt: bytes, udata: bytes = b"") -> bytes:
        return hash_2b(pw, salt, udata) if self.r >= 6 else hashlib.sha256(pw + salt + udata).digest()

    def _try_r56(self, pw: bytes) -> Optional[bytes]:
        pw = pw[:127]
        u, o = self.u[:48], self.o[:48]
        if self._hash56(pw, u[32:40]) == u[:32]:
            return aes_cbc_decrypt(self._hash56(pw, u[40:48]), self.ue[:32], iv=bytes(16), unpad=False)
        if self._hash56(pw, o[32:40], u) == o[:32]:
            return aes_cbc_decrypt(self._hash56(pw, o[40:48], u), self.oe[:32], iv=bytes(16), unpad=False)
        return None

    def authenticate(self, password: str = "") -> bool:
        pw = password.encode("utf-8") if self.r >= 5 else password.encode("latin-1", "replace")
        if self.r >= 5:
            key = self._try_r56(pw)
            if key is None:
                return False
            self.key = key
            return True
        key = self._key_r234(pw)
        if self._check_user_r234(key):
            self.key = key
            return True
        key = self._key_r234(self._user_pw_from_owner_r234(pw))       # owner password: recovers the padded user one
        if self._check_user_r234(key):
            self.key = key
            return True
        return False

    def _object_key(self, num: int, gen: int) -> bytes:
        assert self.key is not None
        if self.r >= 5:
            return self.key
        h = hashlib.md5(self.key + struct.pack("<I", num)[:3] + struct.pack("<I", gen)[:2])
        if self.aes:
            h.update(b"sAlT")
        return h.digest()[:min(len(self.key) + 5, 16)]

    # the reference's accessors (pdf_crypto.py:635-760)
    @property
    def version(self) -> int:
        return self.v

    @property
    def revision(self) -> int:
        return self.r

    @property
    def supported(self) -> bool:
        if self.v in (1, 2, 4) and self.r in (2, 3, 4):
            return True
        return self.v == 5 and self.r in (5, 6) and len(self.u) >= 48 and len(self.ue) == 32

    @property
    def uses_aes_for_streams(self) -> bool:
        return self.v == 5 or bool(self.aes)

    uses_aes_for_strings = uses_aes_for_streams

    def derive_file_key(self, password: bytes = b"") -> bool:
        pw = password.decode("utf-8" if self.r >= 5 else "latin-1", "replace") if isinstance(password, bytes) \
            else str(password)
        return self.supported and self.authenticate(pw)

    @property
    def file_key(self) -> Optional[bytes]:
        return self.key

    def decrypt_stream(self, obj_num: int, gen_num: int, data: bytes) -> bytes:
        return b"" if self.key is None else self.decrypt(data, obj_num, gen_num)

    decrypt_string = decrypt_stream

    def decrypt(self, data: bytes, num: int, gen: int) -> bytes:
        if self.key is None:
            raise RuntimeError("authenticate() first")
        k = self._object_key(num, gen)
        return aes_cbc_decrypt(k, data) if self.aes else rc4(k, data)


def detect_encryption(raw: bytes) -> Optional[PDFEncryption]:
    """The /Encrypt parameters of a PDF file, or None when it is not encrypted (or too damaged to tell)."""
    from .pdf import PDFDocument, PDFError
    try:
        return PDFDocument(raw, password=None, authenticate=False).enc
    except (PDFError, ValueError, KeyError, TypeError):
        return None


def find_stream_object_numbers(raw: bytes):
    """``{offset of the stream data: (object number, generation)}`` for every ``N G obj ... stream`` in the file."""
    import re
    out = {}
    for m in re.finditer(rb"(\d+)\s+(\d+)\s+obj\b", raw):
        end = raw.find(b"endobj", m.end())
        s = raw.find(b"stream", m.end(), end if end >= 0 else len(raw))
        if s < 0:
            continue
        s += 6
        if raw[s:s + 2] == b"\r\n":
            s += 2
        elif raw[s:s + 1] in (b"\n", b"\r"):
            s += 1
        out[s] = (int(m.group(1)), int(m.group(2)))
    return out

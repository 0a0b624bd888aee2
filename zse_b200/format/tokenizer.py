"""Byte-level BPE tokenizer stored inside ``.zse`` files.

Behaviour matches zse-engine/zse_engine/format/tokenizer.py:25-436: GPT-2 byte<->unicode table,
the GPT-2 pre-tokenisation regex, lowest-rank merge loop, added tokens split out before BPE,
``encode(text, add_bos=True, add_eos=False)``, ``decode(ids, skip_special=True)``; the section
stores ``{vocab, merges, special_tokens, added_tokens}``.  The merge loop here keeps the word as a
list and re-scans only for the chosen pair; results are cached per pre-token.

Beyond the reference: SentencePiece-style BPE (``scheme = "metaspace"``), the form in which Llama-2, Mistral, Phi-3 and
Gemma ship their ``tokenizer.json`` - spaces become U+2581 through a normalizer or a Metaspace pre-tokenizer, merges run
over characters of the whole text (or of each word), characters outside the vocabulary become ``<0xNN>`` byte tokens.
A byte-level-only reader mis-tokenises those models.  Both schemes are checked id for id against the ``tokenizers``
library (``tests/test_tokenizer_parity.py``).
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass, field, fields
from functools import lru_cache
from typing import Dict, List, Optional, Tuple

from . import serializer


@lru_cache(maxsize=1)
def _byte_table() -> Dict[int, str]:
    keep = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    table, extra = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + extra)
            extra += 1
    return table


BYTE_ENCODER = _byte_table()
BYTE_DECODER = {c: b for b, c in BYTE_ENCODER.items()}
try:                                   # Unicode classes (\p{L}, \p{N}) as the pre-tokeniser patterns of real models use
    import regex as _re_u
except ImportError:                    # pragma: no cover - the plain module approximates them with \w / \d
    _re_u = None

# GPT-2's pattern: contractions, letters, numbers, other symbols (each with an optional leading space), whitespace
GPT2_PATTERN = r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"""
_PRETOKEN = (_re_u.compile(GPT2_PATTERN) if _re_u is not None else
             re.compile(r"""'s|'t|'re|'ve|'m|'ll|'d| ?[^\W\d_]+| ?\d+| ?[^\s\w]+|_+|\s+(?!\S)|\s+"""))


def _compile_pretoken(pattern: Optional[str]):
    """The model's own split pattern (a ``Split`` pre-tokeniser of its tokenizer.json: Qwen2 splits numbers into
    single digits, Llama-3 into groups of three, ...), or GPT-2's."""
    if pattern and _re_u is not None:
        try:
            return _re_u.compile(pattern)
        except Exception:
            pass
    return _PRETOKEN


def _split_pattern_of(pre) -> Optional[str]:
    """The regex of the first ``Split`` step of a tokenizer.json ``pre_tokenizer`` (possibly inside a ``Sequence``)."""
    if not isinstance(pre, dict):
        return None
    if pre.get("type") == "Sequence":
        for step in pre.get("pretokenizers", []):
            got = _split_pattern_of(step)
            if got:
                return got
        return None
    if pre.get("type") == "Split" and str(pre.get("behavior", "")).lower() == "isolated" and not pre.get("invert"):
        pat = pre.get("pattern", {})
        if isinstance(pat, dict) and isinstance(pat.get("Regex"), str):
            return pat["Regex"]
    return None


def _components(node) -> List[dict]:
    """A normalizer / pre-tokenizer / decoder entry of tokenizer.json flattened (``Sequence`` holds a list)."""
    if not isinstance(node, dict):
        return []
    if node.get("type") == "Sequence":
        out: List[dict] = []
        for key in ("normalizers", "pretokenizers", "decoders"):
            for sub in node.get(key) or []:
                out += _components(sub)
        return out
    return [node]


def _scheme_of(data: dict) -> Tuple[str, str, bool]:
    """(scheme, prepend, split_words) of a tokenizer.json: byte-level BPE (GPT-2, Qwen2, Llama-3) or SentencePiece-style
    BPE (Llama-2, Mistral, Phi-3, Gemma: space -> U+2581 by a normalizer or a Metaspace pre-tokenizer)."""
    pre, norm, dec = (_components(data.get(k)) for k in ("pre_tokenizer", "normalizer", "decoder"))
    if any(c.get("type") == "ByteLevel" for c in pre + dec):
        return "bytelevel", "never", False
    meta_pre = next((c for c in pre if c.get("type") == "Metaspace"), None)
    replaces = any(c.get("type") == "Replace" and (c.get("pattern") or {}).get("String") == " "
                   and c.get("content") == "\u2581" for c in norm)
    if meta_pre is None and not replaces and not (data.get("model") or {}).get("byte_fallback"):
        return "bytelevel", "never", False
    prepend = "never"
    if any(c.get("type") == "Prepend" and c.get("prepend") == "\u2581" for c in norm):
        prepend = "always"
    split_words = False
    if meta_pre is not None:
        scheme = meta_pre.get("prepend_scheme")
        if scheme is None:
            scheme = "always" if meta_pre.get("add_prefix_space", True) else "never"
        prepend = scheme if prepend == "never" else prepend
        split_words = bool(meta_pre.get("split", True))
    return "metaspace", prepend, split_words


@dataclass
class SpecialTokens:
    bos_id: int = 1
    eos_id: int = 2
    pad_id: int = 0
    unk_id: int = 0

    def to_dict(self) -> dict:
        return {"bos_id": self.bos_id, "eos_id": self.eos_id, "pad_id": self.pad_id, "unk_id": self.unk_id}

    @classmethod
    def from_dict(cls, d: dict) -> "SpecialTokens":
        names = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in names})


@dataclass
class BPETokenizer:
    vocab: Dict[str, int] = field(default_factory=dict)
    merges: List[Tuple[str, str]] = field(default_factory=list)
    special_tokens: SpecialTokens = field(default_factory=SpecialTokens)
    added_tokens: Dict[str, int] = field(default_factory=dict)
    pretoken_pattern: Optional[str] = None     # None: GPT-2's pattern
    # "bytelevel": GPT-2 style (bytes mapped to printable characters, regex pre-tokens) - what the reference implements.
    # "metaspace": SentencePiece-style BPE as Llama-2 / Mistral / Phi-3 / Gemma ship it in tokenizer.json: spaces
    # become U+2581, merges run over characters, characters outside the vocabulary fall back to <0xNN> byte tokens
    scheme: str = "bytelevel"
    prepend: str = "never"                     # metaspace: U+2581 in front of "never" | "always" (every piece of text) | "first"
    split_words: bool = False                  # metaspace: merges stop at word starts (a Metaspace pre-tokenizer)
    ignore_merges: bool = False                # byte-level: a pre-token that is in the vocabulary as a whole is taken as it is (Llama-3)

    def __post_init__(self):
        self._rebuild_caches()

    def _rebuild_caches(self) -> None:
        self._id_to_token = {i: t for t, i in self.vocab.items()}
        self._id_to_token.update({i: t for t, i in self.added_tokens.items()})
        self._ranks = {tuple(p): r for r, p in enumerate(self.merges)}
        self._cache: Dict[str, Tuple[str, ...]] = {}
        self._pretoken = _compile_pretoken(self.pretoken_pattern)
        if self.added_tokens:
            alts = sorted(self.added_tokens, key=len, reverse=True)
            self._added_re: Optional[re.Pattern] = re.compile("(" + "|".join(re.escape(t) for t in alts) + ")")
        else:
            self._added_re = None
        self._byte_ids = [self.vocab.get("<0x%02X>" % b) for b in range(256)] if self.scheme == "metaspace" else []

    # ---- SentencePiece-style pieces ----------------------------------------------------------
    def _merge_long(self, symbols: List[str]) -> List[str]:
        """BPE over an arbitrarily long symbol list: a heap of candidate merges over a linked list, so that a whole
        paragraph (these tokenizers have no pre-tokens) costs n log n rather than n^2."""
        import heapq
        n = len(symbols)
        if n < 2:
            return symbols
        ranks = self._ranks
        sym = list(symbols)
        prev, nxt = list(range(-1, n - 1)), list(range(1, n + 1))
        alive = [True] * n
        heap = []
        for i in range(n - 1):
            r = ranks.get((sym[i], sym[i + 1]))
            if r is not None:
                heap.append((r, i, sym[i], sym[i + 1]))
        heapq.heapify(heap)
        while heap:
            r, i, a, b = heapq.heappop(heap)
            j = nxt[i] if alive[i] else n
            if not alive[i] or j >= n or not alive[j] or sym[i] != a or sym[j] != b:
                continue                       # a stale entry: one of the two was merged away meanwhile
            sym[i] = a + b
            alive[j] = False
            k = nxt[j]
            nxt[i] = k
            if k < n:
                prev[k] = i
            h = prev[i]
            if h >= 0:
                r2 = ranks.get((sym[h], sym[i]))
                if r2 is not None:
                    heapq.heappush(heap, (r2, h, sym[h], sym[i]))
            if k < n:
                r2 = ranks.get((sym[i], sym[k]))
                if r2 is not None:
                    heapq.heappush(heap, (r2, i, sym[i], sym[k]))
        return [sym[i] for i in range(n) if alive[i]]

    def _encode_metaspace(self, text: str, at_start: bool) -> List[int]:
        if not text:
            return []
        text = text.replace(" ", "\u2581")
        if self.prepend == "always" or (self.prepend == "first" and at_start):
            if not (self.split_words and text.startswith("\u2581")):
                text = "\u2581" + text
        if self.split_words:                   # every U+2581 starts a new word; merges stay inside words
            words, cur = [], ""
            for ch in text:
                if ch == "\u2581" and cur:
                    words.append(cur)
                    cur = ""
                cur += ch
            words.append(cur)
        else:
            words = [text]
        ids, vocab, unk = [], self.vocab, self.special_tokens.unk_id
        for w in words:
            hit = self._cache.get(w) if len(w) < 64 else None
            if hit is None:
                hit = tuple(self._merge_long(list(w)))
                if len(w) < 64 and len(self._cache) < 200_000:
                    self._cache[w] = hit
            for piece in hit:
                tid = vocab.get(piece)
                if tid is not None:
                    ids.append(tid)
                    continue
                for b in piece.encode("utf-8"):            # a character the vocabulary does not have
                    bid = self._byte_ids[b] if self._byte_ids else None
                    ids.append(bid if bid is not None else unk)
        return ids

    def _decode_metaspace(self, toks: List[str]) -> str:
        out = bytearray()
        for t in toks:
            if len(t) == 6 and t.startswith("<0x") and t.endswith(">"):
                try:
                    out.append(int(t[3:5], 16))
                    continue
                except ValueError:
                    pass
            out += t.encode("utf-8")
        text = out.decode("utf-8", errors="replace").replace("\u2581", " ")
        return text[1:] if self.prepend != "never" and text.startswith(" ") else text

    # ---- BPE -------------------------------------------------------------------------------
    def _bpe(self, token: str) -> Tuple[str, ...]:
        hit = self._cache.get(token)
        if hit is not None:
            return hit
        word = list(token)
        ranks = self._ranks
        while len(word) > 1:
            best, best_rank = None, None
            for pair in zip(word, word[1:]):
                r = ranks.get(pair)
                if r is not None and (best_rank is None or r < best_rank):
                    best, best_rank = pair, r
            if best is None:
                break
            a, b = best
            merged, i, n = [], 0, len(word)
            while i < n:
                if i + 1 < n and word[i] == a and word[i + 1] == b:
                    merged.append(a + b)
                    i += 2
                else:
                    merged.append(word[i])
                    i += 1
            word = merged
        out = tuple(word)
        if len(self._cache) < 200_000:
            self._cache[token] = out
        return out

    def _encode_chunk(self, text: str) -> List[int]:
        ids, vocab, unk, enc = [], self.vocab, self.special_tokens.unk_id, BYTE_ENCODER
        for piece in self._pretoken.findall(text):
            mapped = "".join(enc[b] for b in piece.encode("utf-8"))
            if self.ignore_merges:
                whole = vocab.get(mapped)
                if whole is not None:
                    ids.append(whole)
                    continue
            for sym in self._bpe(mapped):
                ids.append(vocab.get(sym, unk))
        return ids

    def encode(self, text: str, add_bos: bool = True, add_eos: bool = False) -> List[int]:
        ids: List[int] = [self.special_tokens.bos_id] if add_bos else []
        meta = self.scheme == "metaspace"
        if self._added_re is not None:
            at = 0
            for part in self._added_re.split(text):
                if not part:
                    continue
                tid = self.added_tokens.get(part)
                if tid is not None:
                    ids.append(tid)
                else:
                    ids.extend(self._encode_metaspace(part, at == 0) if meta else self._encode_chunk(part))
                at += len(part)
        else:
            ids.extend(self._encode_metaspace(text, True) if meta else self._encode_chunk(text))
        if add_eos:
            ids.append(self.special_tokens.eos_id)
        return ids

    def decode(self, ids, skip_special: bool = True) -> str:
        st = self.special_tokens
        skip = {st.bos_id, st.eos_id, st.pad_id} if skip_special else ()
        if self.scheme == "metaspace":
            toks = [self._id_to_token.get(int(t)) for t in ids if t not in skip]
            return self._decode_metaspace([t for t in toks if t is not None])
        out = bytearray()
        for tid in ids:
            if tid in skip:
                continue
            tok = self._id_to_token.get(int(tid))
            if tok is None:
                continue
            for ch in tok:
                b = BYTE_DECODER.get(ch)
                if b is None:
                    out += ch.encode("utf-8")
                else:
                    out.append(b)
        return out.decode("utf-8", errors="replace")

    def token_to_id(self, token: str) -> Optional[int]:
        tid = self.added_tokens.get(token)
        return tid if tid is not None else self.vocab.get(token)

    @property
    def vocab_size(self) -> int:
        return len(self.vocab) + len(self.added_tokens)

    # ---- section payload -------------------------------------------------------------------
    def serialize(self) -> bytes:
        d = {"vocab": self.vocab, "merges": [list(m) for m in self.merges],
             "special_tokens": self.special_tokens.to_dict(), "added_tokens": self.added_tokens}
        if self.pretoken_pattern:          # an extra key: readers that do not know it keep GPT-2's pattern
            d["pretoken_pattern"] = self.pretoken_pattern
        if self.scheme != "bytelevel":     # more extra keys; a reader without them would mis-tokenise such a model anyway
            d["scheme"], d["prepend"], d["split_words"] = self.scheme, self.prepend, self.split_words
        if self.ignore_merges:
            d["ignore_merges"] = True
        return serializer.encode(d)

    @classmethod
    def deserialize(cls, data) -> "BPETokenizer":
        d = serializer.decode(data)
        return cls(vocab=d["vocab"], merges=[tuple(m) for m in d["merges"]],
                   special_tokens=SpecialTokens.from_dict(d.get("special_tokens", {})),
                   added_tokens=d.get("added_tokens", {}), pretoken_pattern=d.get("pretoken_pattern"),
                   scheme=d.get("scheme", "bytelevel"), prepend=d.get("prepend", "never"),
                   split_words=bool(d.get("split_words", False)), ignore_merges=bool(d.get("ignore_merges", False)))

    # ---- HuggingFace import ----------------------------------------------------------------
    @classmethod
    def from_hf_tokenizer_json(cls, path: str) -> "BPETokenizer":
        with open(path, "r", encoding="utf-8") as f:
            data = json.load(f)
        model = data.get("model", {})
        vocab = dict(model.get("vocab", {}))
        merges: List[Tuple[str, str]] = []
        for m in model.get("merges", []):
            if isinstance(m, str):
                a, sep, b = m.partition(" ")
                if sep:
                    merges.append((a, b))
            elif len(m) == 2:
                merges.append((m[0], m[1]))
        special, added = SpecialTokens(), {}
        for info in data.get("added_tokens", []):
            content, tid = info.get("content", ""), info.get("id", 0)
            if info.get("special", False):
                low = content.lower()
                squashed = low.replace("|", "").replace("_", "")
                if "bos" in low or content == "<s>" or "beginoftext" in squashed:
                    special.bos_id = tid
                elif "eos" in low or content == "</s>" or "endoftext" in squashed:
                    special.eos_id = tid
                elif "pad" in low:
                    special.pad_id = tid
                elif "unk" in low:
                    special.unk_id = tid
            # every added token is matched as a whole before the BPE runs, also one that the model's own vocabulary
            # lists as well (GPT-2's <|endoftext|>, Mistral's <s>): that is what the tokenizers library does
            if content:
                added[content] = tid
        scheme, prepend, split_words = _scheme_of(data)
        return cls(vocab=vocab, merges=merges, special_tokens=special, added_tokens=added,
                   pretoken_pattern=_split_pattern_of(data.get("pre_tokenizer")) if scheme == "bytelevel" else None,
                   scheme=scheme, prepend=prepend, split_words=split_words,
                   ignore_merges=bool(model.get("ignore_merges", False)))

    @classmethod
    def from_hf_dir(cls, model_dir: str) -> "BPETokenizer":
        path = os.path.join(model_dir, "tokenizer.json")
        if not os.path.exists(path):
            raise FileNotFoundError(f"no tokenizer.json in {model_dir} (a HuggingFace fast tokenizer is required)")
        tok = cls.from_hf_tokenizer_json(path)
        cfg_path = os.path.join(model_dir, "tokenizer_config.json")
        if os.path.exists(cfg_path):
            try:
                with open(cfg_path, "r", encoding="utf-8") as f:
                    tc = json.load(f)
                for key, attr in (("eos_token", "eos_id"), ("bos_token", "bos_id")):
                    val = tc.get(key)
                    if isinstance(val, dict):
                        val = val.get("content")
                    if isinstance(val, str) and val:
                        tid = tok.token_to_id(val)
                        if tid is not None:
                            setattr(tok.special_tokens, attr, tid)
            except (OSError, ValueError):
                pass
        return tok

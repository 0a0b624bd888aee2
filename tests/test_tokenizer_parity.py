"""The byte-level BPE tokenizer against the HuggingFace ``tokenizers`` library on the same vocabulary: a small BPE is
trained here (offline), written as ``tokenizer.json``, imported with ``BPETokenizer.from_hf_dir`` and both must
produce the same ids for arbitrary text - pre-tokeniser regex, merge order, byte fallback and added tokens included
(the reference imports the same files, zse-engine/zse_engine/format/tokenizer.py:25-436)."""
import json
import random

import pytest

tokenizers = pytest.importorskip("tokenizers")

from zse_b200.format.tokenizer import BPETokenizer

CORPUS = [
    "The quick brown fox jumps over the lazy dog. " * 3,
    "def f(x):\n    return x ** 2 + 3 * x  # comment\n" * 2,
    "Tensor cores multiply 128x128 tiles; HBM3e streams the weights, isn't it?",
    "naïve café déjà vu — Übergröße, 数学 と 物理, русский текст, emoji 🙂🚀",
    "   leading spaces\tand\ttabs\n\nnew paragraphs  and  double  spaces ",
    "numbers 12345 67 890 3.14159 2026-11-25 1e-6 0xFF",
    "they're we'll I'm you've he'd it's o'clock",
]


@pytest.fixture(scope="module")
def pair(tmp_path_factory):
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=600, special_tokens=["<|endoftext|>", "<|im_start|>", "<|im_end|>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False)
    tok.train_from_iterator(CORPUS * 4, trainer)
    d = tmp_path_factory.mktemp("tok")
    tok.save(str(d / "tokenizer.json"))
    (d / "tokenizer_config.json").write_text(json.dumps({"eos_token": "<|endoftext|>", "bos_token": None,
                                                         "pad_token": "<|endoftext|>"}))
    return tok, BPETokenizer.from_hf_dir(str(d))


def _random_text(rng):
    pools = ["abcdefghijklmnopqrstuvwxyz", "ABCDEFGHIJ", "0123456789", " \t\n", ".,;:!?'\"()[]{}<>|/\\-_=+*&^%$#@~`",
             "àéîõüñçß", "数学物理日本語", "русский", "🙂🚀🔥", "'s't're've'll'd'm"]
    out = []
    for _ in range(rng.randint(1, 40)):
        pool = rng.choice(pools)
        out.append("".join(rng.choice(pool) for _ in range(rng.randint(1, 6))))
        if rng.random() < 0.5:
            out.append(" " * rng.randint(1, 3))
    return "".join(out)


def test_same_ids_as_the_tokenizers_library(pair):
    hf, ours = pair
    rng = random.Random(0)
    texts = CORPUS + [_random_text(rng) for _ in range(300)] + ["", " ", "\n", "a", "  a  ", "'", "''ll"]
    for text in texts:
        want = hf.encode(text, add_special_tokens=False).ids
        got = ours.encode(text, add_bos=False)
        assert got == want, (text, got, want)
        assert ours.decode(got) == text


def test_added_tokens_split_the_text(pair):
    hf, ours = pair
    text = "<|im_start|>user\nhello<|im_end|>\n<|im_start|>assistant\n<|endoftext|>tail <|im_end"
    want = hf.encode(text, add_special_tokens=False).ids
    got = ours.encode(text, add_bos=False)
    assert got == want
    assert ours.decode(got, skip_special=False) == text
    assert "<|im_start|>" not in ours.decode(got, skip_special=True)


def test_serialised_tokenizer_behaves_the_same(pair):
    _, ours = pair
    again = BPETokenizer.deserialize(ours.serialize())
    rng = random.Random(1)
    for _ in range(50):
        t = _random_text(rng)
        assert again.encode(t, add_bos=False) == ours.encode(t, add_bos=False)


QWEN2_SPLIT = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+"
               r"|\s+(?!\S)|\s+")


@pytest.fixture(scope="module")
def qwen_pair(tmp_path_factory):
    """A tokenizer with the split pattern of Qwen2 (single digits, case-insensitive contractions, newlines kept with
    the symbols before them) instead of GPT-2's."""
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.Sequence([
        pre_tokenizers.Split(Regex(QWEN2_SPLIT), behavior="isolated", invert=False),
        pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=700, special_tokens=["<|endoftext|>", "<|im_start|>", "<|im_end|>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False)
    tok.train_from_iterator((CORPUS + ["abc123 x_y_z 2026-11-25 I'M HERE\r\n\r\nok!!\n", "a1b2c3 __init__ 007"]) * 4,
                            trainer)
    d = tmp_path_factory.mktemp("qtok")
    tok.save(str(d / "tokenizer.json"))
    return tok, BPETokenizer.from_hf_dir(str(d))


def test_model_specific_split_pattern_is_honoured(qwen_pair):
    hf, ours = qwen_pair
    assert ours.pretoken_pattern == QWEN2_SPLIT
    rng = random.Random(3)
    texts = CORPUS + ["abc123", "x_y_z __init__", "I'M HERE, we'LL go", "line\r\n\r\nnext!!\n\n", "12345 6789", "a1b2c3"] \
        + [_random_text(rng) for _ in range(300)]
    for text in texts:
        want = hf.encode(text, add_special_tokens=False).ids
        got = ours.encode(text, add_bos=False)
        assert got == want, (text, got, want)
        assert ours.decode(got) == text
    again = BPETokenizer.deserialize(ours.serialize())
    assert again.pretoken_pattern == QWEN2_SPLIT
    assert again.encode("abc123 4567", add_bos=False) == hf.encode("abc123 4567", add_special_tokens=False).ids


def test_gpt2_pattern_separates_letters_digits_and_underscores(pair):
    hf, ours = pair
    for text in ["abc123def", "snake_case_name", "x1_y2", "__dunder__ 99bottles", "naïve123café"]:
        assert ours.encode(text, add_bos=False) == hf.encode(text, add_special_tokens=False).ids, text


# ---- SentencePiece-style BPE (Llama-2 / Mistral / Phi-3 / Gemma ship this form) -------------------------------------------
def _sp_tokenizer(style: str):
    from tokenizers import Tokenizer, decoders, models, normalizers, pre_tokenizers, trainers
    byte_tokens = ["<0x%02X>" % b for b in range(256)]
    tok = Tokenizer(models.BPE(unk_token="<unk>", byte_fallback=True, fuse_unk=True))
    if style == "llama2":           # Prepend + Replace normalizers, no pre-tokenizer
        tok.normalizer = normalizers.Sequence([normalizers.Prepend("▁"), normalizers.Replace(" ", "▁")])
        tok.decoder = decoders.Sequence([decoders.Replace("▁", " "), decoders.ByteFallback(), decoders.Fuse(),
                                         decoders.Strip(" ", 1, 0)])
    elif style == "gemma":          # only the replacement, no dummy prefix
        tok.normalizer = normalizers.Replace(" ", "▁")
        tok.decoder = decoders.Sequence([decoders.Replace("▁", " "), decoders.ByteFallback(), decoders.Fuse()])
    else:                           # a Metaspace pre-tokenizer: words split at U+2581
        tok.pre_tokenizer = pre_tokenizers.Metaspace(replacement="▁", prepend_scheme="first", split=True)
        tok.decoder = decoders.Sequence([decoders.Metaspace(replacement="▁", prepend_scheme="first"),
                                         decoders.ByteFallback(), decoders.Fuse()])
    trainer = trainers.BpeTrainer(vocab_size=900, special_tokens=["<unk>", "<s>", "</s>"] + byte_tokens,
                                  show_progress=False)
    ascii_only = [t for t in CORPUS if all(ord(c) < 128 for c in t)] + ["naive cafe  deja vu    wide   gaps"]
    tok.train_from_iterator(ascii_only * 4, trainer)          # no accents or CJK in the vocabulary: they fall back
    return tok


@pytest.mark.parametrize("style", ["llama2", "gemma", "metaspace"])
def test_sentencepiece_style_bpe_matches_the_tokenizers_library(tmp_path, style):
    hf = _sp_tokenizer(style)
    hf.save(str(tmp_path / "tokenizer.json"))
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"eos_token": "</s>", "bos_token": "<s>"}))
    ours = BPETokenizer.from_hf_dir(str(tmp_path))
    assert ours.scheme == "metaspace" and ours.special_tokens.bos_id == hf.token_to_id("<s>")
    assert ours.prepend == {"llama2": "always", "gemma": "never", "metaspace": "first"}[style]
    rng = random.Random(3)
    texts = CORPUS + ["", " ", "  two  spaces  ", "Hello world", "tab\there", "emoji \U0001F642 and 数学",
                      "a</s>b <s> c", "</s>", "line\n\nbreaks\n"] + [_random_text(rng) for _ in range(150)]
    for text in texts:
        want = hf.encode(text, add_special_tokens=False).ids
        got = ours.encode(text, add_bos=False)
        assert got == want, (style, text, got[:12], want[:12])
        if "<s>" not in text and "</s>" not in text:
            assert ours.decode(got) == hf.decode(want, skip_special_tokens=False), (style, text)  # byte tokens are "special" in this toy vocabulary
    again = BPETokenizer.deserialize(ours.serialize())
    assert (again.scheme, again.prepend, again.split_words) == (ours.scheme, ours.prepend, ours.split_words)
    assert again.encode("Hello  wide world \U0001F680", add_bos=False) == ours.encode("Hello  wide world \U0001F680",
                                                                                   add_bos=False)
    long_text = " ".join(CORPUS) * 40                        # ~20k characters in one piece: the heap keeps it quick
    assert ours.encode(long_text, add_bos=False) == hf.encode(long_text, add_special_tokens=False).ids


def test_whole_pretokens_in_the_vocabulary_skip_the_merges(tmp_path):
    """Llama-3's ``ignore_merges``: "abc" is a vocabulary entry that the merges alone would never produce."""
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers
    alphabet = sorted(pre_tokenizers.ByteLevel.alphabet())
    vocab = {ch: i for i, ch in enumerate(alphabet)}
    for t in ("ab", "abc", "Ġab"):
        vocab[t] = len(vocab)
    merges = [("a", "b"), ("Ġ", "ab")]
    for flag in (True, False):
        hf = Tokenizer(models.BPE(vocab, merges, ignore_merges=flag))
        hf.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
        hf.decoder = decoders.ByteLevel()
        d = tmp_path / str(flag)
        d.mkdir()
        hf.save(str(d / "tokenizer.json"))
        ours = BPETokenizer.from_hf_dir(str(d))
        assert ours.ignore_merges is flag
        for text in ("abc", "abc ab abcd", " abc"):
            assert ours.encode(text, add_bos=False) == hf.encode(text, add_special_tokens=False).ids, (flag, text)
        assert BPETokenizer.deserialize(ours.serialize()).ignore_merges is flag
    assert len(ours.encode("abc", add_bos=False)) == 2            # without the flag: "ab" + "c"


def test_sentencepiece_style_tokenizer_survives_conversion_and_serving(tmp_path):
    """HF directory (tiny random Llama + a Llama-2 style tokenizer.json) -> .zse -> engine: the tokenizer inside the
    file encodes like the library, and text generation round-trips through it."""
    transformers = pytest.importorskip("transformers")
    from transformers import LlamaConfig, LlamaForCausalLM
    from zse_b200.config import EngineConfig
    from zse_b200.engine import ZSEEngine
    from zse_b200.format.convert import convert_hf_to_zse
    from zse_b200.format.loader import ZSELoader
    hf_tok = _sp_tokenizer("llama2")
    vocab = hf_tok.get_vocab_size()
    model = LlamaForCausalLM(LlamaConfig(vocab_size=vocab, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                         num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256,
                                         bos_token_id=hf_tok.token_to_id("<s>"), eos_token_id=hf_tok.token_to_id("</s>")))
    d = tmp_path / "hf"
    model.save_pretrained(str(d), safe_serialization=True)
    hf_tok.save(str(d / "tokenizer.json"))
    (d / "tokenizer_config.json").write_text(json.dumps({"eos_token": "</s>", "bos_token": "<s>"}))
    out = str(tmp_path / "m.zse")
    convert_hf_to_zse(str(d), out, quant_method=0)
    tok = ZSELoader(out).tokenizer
    text = "The quick brown fox, naïve café 🙂"
    assert tok.scheme == "metaspace" and tok.encode(text, add_bos=False) == hf_tok.encode(
        text, add_special_tokens=False).ids
    eng = ZSEEngine(out, config=EngineConfig(device="cpu", max_seq_len=128, quiet=True))
    ids = eng.generate_tokens(tok.encode(text), max_tokens=6, temperature=0.0)
    assert len(ids) <= 6 and isinstance(eng.generate(text, max_tokens=6, temperature=0.0), str)
    assert tok.decode(tok.encode(text)) == text
    eng.destroy()

"""Unit tests of the retrieval building blocks on their own: the hashed tokenizer, BM25 bookkeeping, packed sparse
vectors, the inverted index and the three layers of the compact document form (the shape of the reference's
tests/test_rag.py sections on embeddings and ZPF).  The routes and the engine are covered by tests/test_rag.py."""
import math

import numpy as np
import pytest

from zse_b200.rag.embeddings import (BM25Scorer, TokenEmbedder, bytes_to_sparse, hash_tokenize, sparse_cosine,
                                     sparse_to_bytes)
from zse_b200.rag.store import InvertedIndex
from zse_b200.rag.zpf import (ZPFDictionary, ZPFSchema, build_dictionary, compress_csv, compress_json,
                              compress_records, compress_text, count_tokens, decompress, decompress_zpf,
                              normalise_whitespace, split_csv_line)


# ---- hashed tokenizer ---------------------------------------------------------------------------------------------
def test_hash_tokenizer_is_case_blind_stable_and_in_range():
    a = hash_tokenize("The quick, brown fox!", 1000)
    assert a == hash_tokenize("the QUICK, brown FOX!", 1000)
    assert len(a) == 6 and all(0 <= t < 1000 for t in a)                        # four words, a comma, a bang
    assert hash_tokenize("", 1000) == [] and hash_tokenize("   \n", 1000) == []
    assert hash_tokenize("fox fox", 1000)[0] == hash_tokenize("fox fox", 1000)[1]
    assert hash_tokenize("snake_case x1", 10 ** 9) != hash_tokenize("snake case x1", 10 ** 9)   # "_" joins a word


# ---- BM25 ---------------------------------------------------------------------------------------------------------
def test_bm25_counts_lengths_and_frequencies():
    s = BM25Scorer()
    assert len(s) == 0 and s.avg_len == 0.0 and s.score([1], 0) == 0.0 and s.score_all([1]) == {}
    a = s.add_document([1, 2, 2, 3])
    b = s.add_document([2, 4])
    assert (a, b) == (0, 1) and len(s) == 2 and s.avg_len == 3.0
    assert s.idf(2) == pytest.approx(math.log(1 + 0.5 / 2.5))                   # in both documents
    assert s.idf(1) == pytest.approx(math.log(1 + 1.5 / 1.5))                   # in one
    assert s.idf(99) == pytest.approx(math.log(1 + 2.5 / 0.5))                  # in none: the largest
    assert set(s.score_all([4])) == {b} and set(s.score_all([2, 99])) == {a, b}
    assert s.score([2, 2, 2], a) == s.score([2], a)                             # a query is a set of terms


def test_bm25_formula_on_a_hand_case():
    s = BM25Scorer(k1=1.5, b=0.75)
    d = s.add_document([7, 7, 8])
    s.add_document([9, 9, 9, 9, 9])
    norm = 1.5 * (1 - 0.75 + 0.75 * 3 / 4.0)
    want = s.idf(7) * 2 * 2.5 / (2 + norm)
    assert s.score([7], d) == pytest.approx(want)


def test_bm25_removal_restores_the_statistics():
    s = BM25Scorer()
    a = s.add_document([1, 2])
    before = (s.avg_len, s.idf(1), s.idf(2))
    b = s.add_document([2, 3, 3, 3])
    s.remove_document(b)
    s.remove_document(b)                                                          # twice: nothing left to remove
    s.remove_document(12345)
    assert (s.avg_len, s.idf(1), s.idf(2)) == before and len(s) == 1
    assert s.score_all([3]) == {} and set(s.score_all([2])) == {a}
    c = s.add_document([3])
    assert c == 2                                                                 # ids are never handed out twice


# ---- packed sparse vectors -----------------------------------------------------------------------------------------
def test_sparse_vectors_round_trip_sorted():
    blob = sparse_to_bytes({70000: 0.5, 3: 0.25, 12: -1.0})
    assert len(blob) == 4 + 3 * 4 + 3 * 4
    ids, vals = bytes_to_sparse(blob)
    assert ids.dtype == np.uint32 and vals.dtype == np.float32
    assert ids.tolist() == [3, 12, 70000] and vals.tolist() == [0.25, -1.0, 0.5]
    assert sparse_to_bytes({}) == b""
    ids, vals = bytes_to_sparse(b"")
    assert len(ids) == 0 and len(vals) == 0


def test_sparse_cosine_cases():
    a = sparse_to_bytes({1: 3.0, 2: 4.0})
    assert sparse_cosine(a, a) == pytest.approx(1.0)
    assert sparse_cosine(a, sparse_to_bytes({1: 6.0, 2: 8.0})) == pytest.approx(1.0)       # length does not matter
    assert sparse_cosine(a, sparse_to_bytes({3: 1.0})) == 0.0                               # nothing shared
    assert sparse_cosine(a, sparse_to_bytes({1: 1.0})) == pytest.approx(0.6)
    assert sparse_cosine(a, b"") == 0.0 and sparse_cosine(b"", b"") == 0.0
    assert sparse_cosine(a, sparse_to_bytes({1: 0.0})) == 0.0                               # a zero vector


# ---- embedder -------------------------------------------------------------------------------------------------------
class WordTok:
    """One id per distinct word, in order of first sight."""

    def __init__(self):
        self.ids = {}

    def encode(self, text):
        return [self.ids.setdefault(w, len(self.ids)) for w in text.lower().split()]


def test_embedder_uses_the_model_tokenizer_and_falls_back():
    e = TokenEmbedder(WordTok())
    assert e.tokenize("a b a") == [0, 1, 0] and e._tokenize("b") == [1]           # encode(text) without add_bos

    class BosTok:
        def encode(self, text, add_bos=True):
            return ([1] if add_bos else []) + [5, 6]

    assert TokenEmbedder(BosTok()).tokenize("x") == [5, 6]

    class Broken:
        def encode(self, text, add_bos=False):
            raise ValueError("no vocabulary")

    assert TokenEmbedder(Broken(), vocab_size=50).tokenize("Hello hello") == hash_tokenize("hello hello", 50)
    assert TokenEmbedder(vocab_size=50).tokenize("x y") == hash_tokenize("x y", 50)


def test_tf_idf_weights_follow_the_corpus():
    e = TokenEmbedder(WordTok())
    assert e.embed("") == b""
    ids, vals = bytes_to_sparse(e.embed("a a b"))                                 # no corpus yet: idf 1 everywhere
    assert ids.tolist() == [0, 1]
    assert vals.tolist() == pytest.approx([1 / math.sqrt(1.25), 0.5 / math.sqrt(1.25)])
    e.update_idf([{0}, {0}, {0, 1}])                                              # "a" in 3 of 3, "b" in 1 of 3
    ids, vals = bytes_to_sparse(e.embed("a b"))
    wa, wb = math.log(1 + 3 / 4), math.log(1 + 3 / 2)
    n = math.hypot(wa, wb)
    assert vals.tolist() == pytest.approx([wa / n, wb / n]) and vals[1] > vals[0]   # the rarer word weighs more
    e.update_idf([{0}] * 200)                                                     # a word in (nearly) every document
    _, v = bytes_to_sparse(e.embed("a c"))                                        # "c" was never seen: idf 1
    assert float(np.linalg.norm(v)) == pytest.approx(1.0)
    e.reset_idf()
    _, v = bytes_to_sparse(e.embed("a b"))
    assert v.tolist() == pytest.approx([1 / math.sqrt(2)] * 2)
    assert e.similarity(e.embed("a b"), e.embed("b a")) == pytest.approx(1.0)


def test_embedder_bm25_side_is_keyed_by_chunk_id():
    e = TokenEmbedder(WordTok())
    e.add_to_bm25("red green", 101)
    e.add_to_bm25("green blue blue", 205)
    assert set(e.bm25_search("green")) == {101, 205} and set(e.bm25_search("blue")) == {205}
    assert e.bm25_search("purple") == {}
    e.remove_from_bm25(205)
    e.remove_from_bm25(205)
    assert set(e.bm25_search("green")) == {101} and e.bm25_search("blue") == {}
    e.clear_bm25()
    assert e.bm25_search("red") == {}
    assert e.add_to_bm25("red", 7) == 0                                           # a fresh index numbers from 0


# ---- inverted index ---------------------------------------------------------------------------------------------------
def test_inverted_index_candidates_and_removal():
    ix = InvertedIndex()
    ix.add(1, [5, 6, 6])
    ix.add(2, [6, 7])
    assert ix.token_count == 3
    assert ix.candidates([6]) == {1, 2} and ix.candidates([5, 7]) == {1, 2} and ix.candidates([8]) == set()
    assert ix.candidates([]) == set()
    ix.remove_chunk(1)
    ix.remove_chunk(1)
    assert ix.candidates([5, 6]) == {2} and ix.token_count == 2                   # token 5 has no chunk left
    ix.remove(2, [7])
    assert ix.candidates([7]) == set() and ix.candidates([6]) == {2}
    ix.clear()
    assert ix.token_count == 0 and ix.candidates([6]) == set()


# ---- compact document form: headers -------------------------------------------------------------------------------------
def test_schema_and_dictionary_headers_round_trip():
    s = ZPFSchema(["id", "name", "city"])
    assert s.header() == "§id|name|city§"
    assert ZPFSchema.parse_header(s.header()).columns == ["id", "name", "city"]
    assert ZPFSchema.parse_header("id|name") is None and ZPFSchema.parse_header("§") is None
    d = ZPFDictionary()
    assert d.header() == ""
    d.add("Amsterdam", "£0")
    d.add("Amsterdam Noord", "£1")
    assert d.header() == "¤£0=Amsterdam;£1=Amsterdam Noord¤"
    back = ZPFDictionary.parse_header(d.header())
    assert back.encode_map == d.encode_map and back.decode_map == d.decode_map
    assert ZPFDictionary.parse_header("£0=Amsterdam") is None
    assert d.encode("in Amsterdam Noord and Amsterdam") == "in £1 and £0"       # the longer value first
    assert d.decode("in £1 and £0") == "in Amsterdam Noord and Amsterdam"


def test_codes_with_a_shared_prefix_decode_longest_first():
    d = ZPFDictionary()
    for i in range(11):
        d.add(f"value-{i:02d}", f"£{i}")
    assert d.decode("£10|£1|£0") == "value-10|value-01|value-00"


def test_dictionary_is_built_from_repeats_worth_coding():
    values = ["Rotterdam"] * 5 + ["Utrecht"] * 3 + ["Ede"] * 9 + ["Zwolle"] * 2 + ["a=b;c=d"] * 4
    d = build_dictionary(values)
    assert set(d.encode_map) == {"Rotterdam", "Utrecht"}       # "Ede" is too short, "Zwolle" too rare, "a=b;c=d" unsafe
    assert d.encode_map["Rotterdam"] == "£0"                   # the largest saving gets the shortest code
    assert len(build_dictionary([f"word{i:03d}" for i in range(100)] * 3, max_entries=8).encode_map) == 8
    assert build_dictionary([]).encode_map == {}


# ---- compact document form: the three layers ----------------------------------------------------------------------------
def test_whitespace_layer():
    assert normalise_whitespace("a  \t b\r\n\r\n\r\n\r\nc \n d\r") == "a b\n\nc\nd"
    doc = compress_text("one   two\n\n\n\nthree  ")
    assert doc.compressed == "one two\n\nthree" and doc.schema is None and doc.dictionary is None
    assert doc.original_text == "one   two\n\n\n\nthree  " and doc.compressed_text == doc.compressed
    assert doc.doc_type == "text"


def test_token_count_with_and_without_a_tokenizer():
    assert count_tokens("") == 0 and count_tokens("Hi, there!") == 4
    assert count_tokens("a b c", WordTok()) == 3

    class Broken:
        def encode(self, text):
            raise RuntimeError

    assert count_tokens("a b", Broken()) == 2


def test_records_become_a_schema_line_and_rows():
    recs = [{"id": i, "city": "Rotterdam", "note": None if i % 2 else "x|y  z"} for i in range(6)]
    doc = compress_records(recs)
    lines = doc.compressed.split("\n")
    assert lines[0] == "¤£0=Rotterdam;£1=x/y z¤" and lines[1] == "§id|city|note§"
    assert lines[2] == "0|£0|£1" and lines[3] == "1|£0|"                         # the separator is escaped, None empty
    assert doc.compressed_tokens < doc.original_tokens and 0 < doc.savings_pct < 100
    text = decompress(doc.compressed)
    assert text.split("\n")[0] == "id: 0, city: Rotterdam, note: x/y z"
    assert text.split("\n")[1] == "id: 1, city: Rotterdam"                       # empty fields are left out
    assert decompress_zpf is decompress


def test_records_with_different_keys_share_one_schema():
    doc = compress_records([{"a": 1, "b": "first value"}, {"b": "second value", "c": [1, 2]}] * 3)
    assert "§a|b|c§" in doc.compressed
    assert doc.compressed.split("\n")[2:4] == ["1|£1|", "|£0|£2"]                # a missing key is an empty field
    assert decompress(doc.compressed).split("\n")[:2] == ["a: 1, b: first value", "b: second value, c: [1,2]"]


def test_a_result_that_would_be_longer_is_given_up():
    doc = compress_records([{"k": "v"}], original="k v")
    assert doc.compressed == "k v" and doc.schema is None and doc.savings_pct == 0.0


def test_json_shapes():
    doc = compress_json({"server": {"host": "h", "ports": [1, 2]}, "users": [{"n": "a"}, {"n": "b"}]})
    lines = doc.compressed.split("\n")
    assert lines[:2] == ["server.host=h", "server.ports=[1,2]"]
    assert lines[2:] == ["users:", "§n§", "a", "b"]
    assert doc.doc_type == "json"
    assert decompress(doc.compressed).split("\n")[-2:] == ["n: a", "n: b"]        # a one-column schema reads back too
    scalar = compress_json([1, 2, 3])
    assert scalar.compressed == "[1,2,3]" and scalar.doc_type == "json"
    assert compress_json([{"a": 1}] * 4).schema.columns == ["a"]


def test_csv_layer():
    assert split_csv_line('a,"b,c",d') == ["a", "b,c", "d"] and split_csv_line("") == []
    text = "name,city\n" + "\n".join(f"n{i},Groningen" for i in range(5)) + "\nshort\n"
    plain = compress_csv(text)                                 # counted in words a table is compact already:
    assert plain.doc_type == "csv" and plain.schema is None    # ... the coded form is not shorter and is given up

    class Chars:
        def encode(self, t):
            return list(t)

    doc = compress_csv(text, Chars())
    assert doc.doc_type == "csv" and doc.original == text and doc.schema.columns == ["name", "city"]
    assert "¤£0=Groningen¤" in doc.compressed and doc.compressed.endswith("short|")   # a short row is padded
    assert doc.compressed_tokens == len(doc.compressed) < doc.original_tokens == len(text)
    assert compress_csv("only,a,header\n").doc_type == "text"


# ---- the store's accessors ------------------------------------------------------------------------------------------------
def _filled_store(path=None):
    from zse_b200.rag.parser import Chunk
    from zse_b200.rag.store import RAGStore
    e = TokenEmbedder(WordTok())
    store = RAGStore(path)
    texts = {"fruit": ["apples and pears", "plums and cherries"], "tools": ["hammers and saws"]}
    ids = {}
    for name, parts in texts.items():
        chunks = [Chunk(t, t.replace(" and ", "&"), {"chunk_index": i, "page": i + 1}, 3, 1) for i, t in enumerate(parts)]
        ids[name] = store.add_document(name, "text", chunks, [e.embed(t) for t in parts],
                                       [set(e.tokenize(t)) for t in parts], {"source": name + ".txt"})
    for ch in store.all_chunks():
        e.add_to_bm25(ch.content, ch.id)
    return store, e, ids


def test_store_reads_documents_and_chunks_back():
    store, e, ids = _filled_store()
    docs = store.list_documents()
    assert [(d.name, d.chunk_count, d.original_tokens, d.compressed_tokens) for d in docs] == [
        ("fruit", 2, 6, 2), ("tools", 1, 3, 1)]
    assert docs[0].metadata == {"source": "fruit.txt"} and docs[0].savings_pct == pytest.approx(200 / 3)
    assert store.get_document(ids["tools"]).name == "tools" and store.get_document(999) is None
    chunks = store.get_chunks(ids["fruit"])
    assert [c.chunk_index for c in chunks] == [0, 1] and chunks[1].content == "plums and cherries"
    assert chunks[1].compressed == "plums&cherries" and chunks[1].metadata["page"] == 2
    assert chunks[0].token_count == 1 and not chunks[0].has_dense and chunks[0].embedding == e.embed("apples and pears")
    assert [c.id for c in store.all_chunks()] == [1, 2, 3]
    assert store.get_chunk_text(3) == "hammers and saws" and store.get_chunk_text(44) is None
    rows = store.get_chunks_by_ids([3, 1, 77])
    assert set(rows) == {1, 3} and rows[3][1] == "tools" and rows[1][0].content == "apples and pears"
    assert store.get_chunks_by_ids([]) == {}
    many = store.get_chunks_by_ids(range(1, 1200))                                # more ids than one statement takes
    assert set(many) == {1, 2, 3}


def test_dense_vectors_are_optional_per_chunk():
    store, _, _ = _filled_store()
    assert store.all_chunk_ids_missing_dense() == [1, 2, 3] and store.get_dense_vectors([1, 2, 3]) == {}
    store.set_dense_vector(2, b"\x01\x02")
    assert store.all_chunk_ids_missing_dense() == [1, 3]
    assert store.get_dense_vectors([1, 2, 3]) == {2: b"\x01\x02"}
    assert store.get_chunks_by_ids([2])[2][0].has_dense
    assert store.stats()["dense_chunks"] == 1 and store.stats()["chunks"] == 3


def test_index_and_vectors_can_be_rebuilt_from_the_stored_text():
    store, e, _ = _filled_store()
    tok_and = e.tokenize("and")[0]
    assert store.index.candidates([tok_and]) == {1, 2, 3}
    store.index.clear()
    assert store.index.candidates([tok_and]) == set() and store.stats()["index_tokens"] == 0
    store.rebuild_inverted_index(e)
    assert store.index.candidates([tok_and]) == {1, 2, 3}
    assert store.index.candidates(e.tokenize("hammers")) == {3}
    before = store.get_chunks_by_ids([1])[1][0].embedding
    e.update_idf([set(e.tokenize(c.content)) for c in store.all_chunks()])        # "and" is now a common word
    store.reembed_all(e)
    after = store.get_chunks_by_ids([1])[1][0].embedding
    assert after != before and after == e.embed("apples and pears")
    store.set_embedding(1, b"")
    assert store.get_chunks_by_ids([1])[1][0].embedding == b""


def test_lexical_search_blends_both_signals_and_honours_candidates():
    store, e, ids = _filled_store()
    hits = store.search(e.embed("plums"), e, "plums", top_k=5)
    assert [h.chunk_id for h in hits] == [2] and hits[0].doc_name == "fruit"
    assert hits[0].bm25_score == 1.0 and 0 < hits[0].cosine_score < 1 and hits[0].dense_score == 0.0
    assert hits[0].rerank_score is None
    assert hits[0].score == pytest.approx(0.5 * 1.0 + 0.5 * hits[0].cosine_score)
    rec = hits[0].chunk
    assert (rec.id, rec.doc_id, rec.chunk_index, rec.content) == (2, ids["fruit"], 1, "plums and cherries")
    both = store.search(e.embed("and"), e, "and", top_k=2)
    assert len(both) == 2                                                          # top_k cuts three hits to two
    only = store.search(e.embed("and"), e, "and", candidate_ids={3})
    assert [h.chunk_id for h in only] == [3]
    assert store.search(e.embed("zebra"), e, "zebra") == []
    assert store.search(e.embed("plums"), e, "plums", min_score=0.99) == []


def test_removing_a_document_takes_its_chunks_and_index_entries(tmp_path):
    path = str(tmp_path / "rag.db")
    store, e, ids = _filled_store(path)
    assert store.remove_document(ids["fruit"]) is True and store.remove_document(ids["fruit"]) is False
    assert [c.id for c in store.all_chunks()] == [3] and store.index.candidates(e.tokenize("apples")) == set()
    st = store.stats()
    assert (st["documents"], st["chunks"], st["original_tokens"], st["compressed_tokens"]) == (1, 1, 3, 1)
    assert st["token_savings_pct"] == 66.7
    from zse_b200.rag.store import RAGStore
    again = RAGStore(path)                                                         # the file keeps what is left
    assert [d.name for d in again.list_documents()] == ["tools"] and again.stats()["index_tokens"] == 0

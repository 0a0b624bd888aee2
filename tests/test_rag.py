"""Retrieval stack on the CPU: parsers, ZPF round trip, BM25/TF-IDF ranking, store persistence, fusion with a dense
side, reranking, PDF extraction incl. the standard security handler (cases of the reference's tests/test_rag*.py)."""
import json
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from helpers.make_pdf import make_pdf          # noqa: E402

from zse_b200.rag import RAGEngine, TextParser, get_parser            # noqa: E402
from zse_b200.rag import pdf_crypto as pc                              # noqa: E402
from zse_b200.rag import zpf                                          # noqa: E402
from zse_b200.rag.embeddings import BM25Scorer, TokenEmbedder, sparse_cosine    # noqa: E402
from zse_b200.rag.pdf import PDFError, PDFParser                       # noqa: E402

DOCS = {
    "solar.txt": "Solar panels convert sunlight into electricity using photovoltaic cells.\n\n"
                 "Inverters turn the direct current of the panels into alternating current for the grid.",
    "bread.txt": "Sourdough bread needs a starter of flour and water that ferments for several days.\n\n"
                 "Bake the loaf in a very hot oven with steam for a crisp crust.",
    "cats.txt": "Cats sleep for most of the day and hunt at dawn and dusk.\n\nA purring cat is usually content.",
}


def _engine(tmp_path=None, **kw):
    eng = RAGEngine(db=str(tmp_path / "rag.db") if tmp_path else None, **kw)
    for name, text in DOCS.items():
        res = eng.ingest(name, text.encode())
        assert "error" not in res and res["chunk_count"] >= 1
    return eng


# ---- crypto primitives -----------------------------------------------------------------------------------------
def test_aes_and_rc4_known_answers():
    pt = bytes.fromhex("00112233445566778899aabbccddeeff")
    assert pc.encrypt_block(pt, pc.expand_key(bytes(range(16)))).hex() == "69c4e0d86a7b0430d8cdb78070b4c55a"
    assert pc.encrypt_block(pt, pc.expand_key(bytes(range(32)))).hex() == "8ea2b7ca516745bfeafc49904b496089"
    assert pc.decrypt_block(bytes.fromhex("8ea2b7ca516745bfeafc49904b496089"), pc.expand_key(bytes(range(32)))) == pt
    assert pc.rc4(b"Key", b"Plaintext").hex() == "bbf316e8d940af0ad3"
    iv, key, msg = bytes(range(16)), bytes(range(16, 32)), b"a message that is not a multiple of sixteen"
    assert pc.aes_cbc_decrypt(key, iv + pc.aes_cbc_encrypt(key, iv, msg)) == msg


# ---- parsers / ZPF ---------------------------------------------------------------------------------------------
def test_text_parser_chunks_with_overlap_and_limits():
    text = "\n\n".join(f"Paragraph {i} " + "word " * 30 for i in range(12))
    chunks = TextParser(chunk_size=80, overlap=40).parse(text, metadata={"source": "t", "pdf_password": "x"})
    assert len(chunks) >= 5
    assert all(c.original_tokens <= 2 * 80 for c in chunks)
    assert all("pdf_password" not in c.metadata for c in chunks)
    assert [c.metadata["chunk_index"] for c in chunks] == list(range(len(chunks)))
    firsts = [c.text.split()[1] for c in chunks]
    assert firsts == sorted(firsts, key=int) and "Paragraph 11" in chunks[-1].text
    # consecutive chunks share a paragraph (overlap)
    assert any(set(a.text.split("\n\n")) & set(b.text.split("\n\n")) for a, b in zip(chunks, chunks[1:]))


def test_zpf_records_roundtrip_and_savings():
    recs = [{"city": "Springfield", "country": "United States", "population": 1000 + i, "notes": "capital region"}
            for i in range(20)]
    doc = zpf.compress_json(recs)
    assert doc.schema.columns == ["city", "country", "population", "notes"]
    assert doc.compressed_tokens < doc.original_tokens * 0.6
    assert doc.dictionary.encode_map                  # repeated strings were coded
    back = zpf.decompress(doc.compressed)
    assert "city: Springfield" in back and "population: 1019" in back and "United States" in back


def test_csv_and_jsonl_parsers():
    csv_text = "name,team,score\n" + "\n".join(f"player{i},red team,{i * 3}" for i in range(30))
    chunks = get_parser("scores.csv", 64, 8).parse(csv_text)
    assert len(chunks) >= 2 and all(c.compressed_tokens <= c.original_tokens for c in chunks)
    assert all("player" in c.compressed and c.text.startswith("name,team,score") for c in chunks)
    assert sum(c.metadata["rows"] for c in chunks) == 30
    jl = "\n".join(json.dumps({"id": i, "text": f"event number {i}"}) for i in range(10)) + "\nnot json"
    chunks = get_parser("log.jsonl", 256, 0).parse(jl)
    assert any("event number 7" in zpf.decompress(c.compressed) for c in chunks)
    assert any("not json" in c.text for c in chunks)


def test_json_parser_handles_nested_and_invalid():
    p = get_parser("cfg.json", 128, 0)
    chunks = p.parse(json.dumps({"server": {"port": 8000, "hosts": ["a", "b"]}, "debug": True}))
    assert len(chunks) == 1 and "server.port=8000" in chunks[0].compressed
    assert p.parse("{broken json")[0].text.startswith("{broken")


# ---- lexical ranking -------------------------------------------------------------------------------------------
def test_bm25_prefers_matching_and_shorter_documents():
    b = BM25Scorer()
    d0 = b.add_document([1, 2, 3, 4])
    d1 = b.add_document([1, 1, 1, 9, 9, 9, 9, 9, 9, 9])
    d2 = b.add_document([5, 6, 7])
    s = b.score_all([1])
    assert set(s) == {d0, d1} and s[d1] > 0 and s[d0] > 0
    assert b.score([5], d2) > 0 and b.score([5], d0) == 0
    b.remove_document(d1)
    assert set(b.score_all([1])) == {d0} and len(b) == 2


def test_tfidf_vectors_are_unit_length_and_comparable():
    e = TokenEmbedder(vocab_size=5000)
    a, b, c = (e.embed(t) for t in ("solar panels and inverters", "panels of solar cells", "sourdough bread"))
    assert abs(sparse_cosine(a, a) - 1.0) < 1e-6
    assert sparse_cosine(a, b) > sparse_cosine(a, c)
    assert e.embed("") == b""


# ---- engine ----------------------------------------------------------------------------------------------------
def test_search_ranks_the_right_document_and_filters(tmp_path):
    eng = _engine(tmp_path)
    r = eng.search("how do photovoltaic panels make electricity", top_k=2)
    assert r and r[0]["doc_name"] == "solar.txt" and r[0]["score"] > 0
    assert eng.search("sourdough starter", top_k=1)[0]["doc_name"] == "bread.txt"
    assert eng.search("sourdough starter", top_k=3, filters={"doc_name": "cats.txt"}) == [] or \
        all(x["doc_name"] == "cats.txt" for x in eng.search("sourdough starter", top_k=3, filters={"doc_name": "cats.txt"}))
    assert eng.search("   ") == []
    st = eng.stats()
    assert st["documents"] == 3 and st["chunks"] >= 3 and not st["dense_enabled"]


def test_store_survives_restart_and_document_removal(tmp_path):
    eng = _engine(tmp_path)
    docs = eng.list_documents()
    assert [d["name"] for d in docs] == list(DOCS)
    again = RAGEngine(db=str(tmp_path / "rag.db"))
    assert again.search("purring cat", top_k=1)[0]["doc_name"] == "cats.txt"
    cat_id = next(d["id"] for d in docs if d["name"] == "cats.txt")
    assert again.get_document(cat_id)["chunks"]
    assert again.remove_document(cat_id) and not again.remove_document(cat_id)
    assert all(r["doc_name"] != "cats.txt" for r in again.search("purring cat", top_k=5))
    assert again.get_document(cat_id) is None


def test_multi_query_and_augment_messages():
    eng = _engine()
    r = eng.multi_query_search("how do solar inverters work and how long does a sourdough starter ferment", top_k=4)
    names = {x["doc_name"] for x in r}
    assert {"solar.txt", "bread.txt"} <= names
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "why does my cat purr"}]
    out = eng.augment_messages(msgs, top_k=2)
    assert len(out) == 3 and out[1]["role"] == "system" and "purring" in out[1]["content"]
    assert out[2] == msgs[1]
    assert eng.augment_messages([{"role": "assistant", "content": "hi"}]) == [{"role": "assistant", "content": "hi"}]


class _FakeModel:
    """Stands in for the serving engine: a bag-of-topic 'hidden state' and a Yes/No judge that knows the topics."""
    TOPICS = (("solar", "panel", "electric", "energy", "sun", "power"), ("bread", "bake", "loaf", "dough", "flour"),
              ("cat", "purr", "feline", "kitten"))

    def __init__(self, tok):
        self.tokenizer, self.tok = tok, tok

    def _vec(self, text):
        t = text.lower()
        v = np.array([sum(t.count(w) for w in ws) for ws in self.TOPICS], dtype=np.float32) + 1e-3
        return v / np.linalg.norm(v)

    def embed_tokens(self, ids):
        return self._vec(self.tok.decode(ids))

    def last_token_logits(self, ids):
        text = self.tok.decode(ids)
        q, d = text.split("Question:")[1].split("Passage:")
        logits = np.zeros(self.tok.vocab_size, np.float32)
        yes, no = self.tok.encode(" Yes")[-1], self.tok.encode(" No")[-1]
        logits[yes] = 5.0 * float(self._vec(q) @ self._vec(d.split("Does the passage")[0]))
        logits[no] = 2.5
        return logits


def test_dense_fusion_and_rerank_rescue_a_paraphrase():
    from zse_b200.format.synth import byte_tokenizer
    tok = byte_tokenizer(1024)
    eng = RAGEngine()                        # word-level sparse side; the model side brings its own tokenizer
    eng.set_model_runner(_FakeModel(tok))
    for name, text in DOCS.items():
        assert "error" not in eng.ingest(name, text.encode())
    assert eng.has_dense and eng.stats()["dense_chunks"] == eng.stats()["chunks"]
    q = "feline noises"                       # shares no word with the cat document
    dense = eng.search(q, top_k=1, use_dense=True)
    assert dense and dense[0]["doc_name"] == "cats.txt" and "dense" in dense[0]["scores"]
    rr = eng.search("energy from the sun", top_k=2, use_dense=True, use_rerank=True)
    assert rr[0]["doc_name"] == "solar.txt" and "rerank" in rr[0]["scores"]
    w = eng.search("energy from the sun", top_k=2, use_dense=True, fusion="weighted")
    assert w[0]["doc_name"] == "solar.txt"
    # chunks ingested before the model was wired get their vectors later
    late = RAGEngine()
    late.ingest("cats.txt", DOCS["cats.txt"].encode())
    late.set_model_runner(_FakeModel(tok))
    assert late.backfill_dense_embeddings() == late.stats()["chunks"]


# ---- PDF ---------------------------------------------------------------------------------------------------------
PAGES = [["Quarterly revenue grew eleven percent", "driven by the hardware unit (Europe)"],
         ["Page two discusses hiring", "and the new office lease"]]
WANT = ["Quarterly revenue grew eleven percent\ndriven by the hardware unit (Europe)",
        "Page two discusses hiring\nand the new office lease"]


@pytest.mark.parametrize("kw", [dict(), dict(flate=True), dict(flate=True, hex_font=True), dict(encrypt="rc4"),
                                dict(encrypt="aes128", flate=True),
                                dict(encrypt="aes256", flate=True, user_pw="s3cret")])
def test_pdf_text_extraction(kw):
    raw = make_pdf(PAGES, **kw)
    assert PDFParser().extract_pages(raw, kw.get("user_pw", "")) == WANT


def test_pdf_passwords_and_ingest():
    raw = make_pdf(PAGES, encrypt="aes256", user_pw="s3cret", flate=True)
    with pytest.raises(PDFError):
        PDFParser().extract_pages(raw, "")
    with pytest.raises(PDFError):
        PDFParser().extract_pages(raw, "nope")
    assert PDFParser().extract_pages(raw, "owner") == WANT           # the owner password opens it too
    assert PDFParser().extract_pages(make_pdf(PAGES, encrypt="rc4", user_pw="u"), "owner") == WANT
    eng = RAGEngine()
    assert "error" in eng.ingest("report.pdf", raw)
    res = eng.ingest("report.pdf", raw, pdf_password="s3cret")
    assert res["doc_type"] == "pdf" and res["chunk_count"] == 2
    hit = eng.search("office lease", top_k=1)[0]
    assert hit["metadata"]["page"] == 2 and "pdf_password" not in json.dumps(hit["metadata"])
    with pytest.raises(PDFError):
        PDFParser().extract_pages(b"hello", "")


def test_pdf_ocr_hook_is_used_for_image_only_pages():
    raw = make_pdf([[]])            # a page without text
    calls = []
    pages = PDFParser().extract_pages(raw, "", ocr_fn=lambda data, hint: calls.append(hint) or "scanned text")
    assert pages == [""] and calls == []          # no images on the page: nothing to hand to the hook


def test_reference_named_crypto_and_format_helpers(tmp_path):
    """Function names of the reference's rag / format / cache modules that callers may import directly."""
    import numpy as np
    from helpers.make_pdf import make_pdf
    from zse_b200.cache.attention_metadata import build_attention_metadata
    from zse_b200.format import fast_quant
    from zse_b200.format.spec import align_offset
    from zse_b200.rag import pdf_crypto as pc
    from zse_b200.rag.dense import dense_cosine
    from zse_b200.rag.zpf import compress_csv, decompress_zpf
    key, iv = bytes(range(16)), bytes(range(16, 32))
    ct = pc.aes128_cbc_encrypt(key, iv, b"attack at dawn")
    assert pc.aes128_cbc_decrypt(key, iv + ct) == b"attack at dawn"
    k32 = bytes(range(32))
    assert pc.aes256_cbc_decrypt(k32, pc.aes256_cbc_encrypt(k32, iv, b"x" * 40), iv=iv) == b"x" * 40
    plain = make_pdf([["hello"]])
    assert pc.detect_encryption(plain) is None
    locked = make_pdf([["secret text"]], encrypt="aes128", user_pw="pw", owner_pw="own")
    enc = pc.detect_encryption(locked)
    assert enc is not None and enc.supported and enc.uses_aes_for_streams and enc.file_key is None
    assert not enc.derive_file_key(b"nope") and enc.derive_file_key(b"pw") and enc.file_key
    assert pc.find_stream_object_numbers(plain)
    a = np.array([1.0, 0.0, 1.0], np.float32)
    assert abs(dense_cosine(a.tobytes(), a.tobytes()) - 1.0) < 1e-6
    assert abs(dense_cosine(a.astype(np.float16).tobytes(), a.astype(np.float16).tobytes(), np.float16) - 1.0) < 1e-3
    doc = compress_csv("city,temp\nParis,20\nParis,21\nParis,19\nRome,25\n")
    assert "Paris" in decompress_zpf(doc.compressed)
    md = build_attention_metadata([[3, 4], [7]], [20, 5], 16)
    assert md.num_seqs == 2 and md.max_blocks_per_seq == 2 and md.block_tables_nbytes == 16
    assert align_offset(4097, 4096) == 8192
    w = (np.arange(256) / 100.0).astype(np.float32)
    p, s, z = fast_quant.quantize_tensor_fast(w.tobytes(), "F32", 256)
    assert len(p) == 128 and len(s) == 4 and len(z) == 4

"""Retrieval-augmented generation on top of the serving engine: parsers (text, JSON, JSONL, CSV, PDF incl. encrypted),
ZPF token-saving compression, BM25 + TF-IDF + dense retrieval with rank fusion, LLM reranking, SQLite store."""
from .embeddings import BM25Scorer, TokenEmbedder
from .engine import RAGEngine
from .parser import Chunk, CSVParser, JSONLParser, JSONParser, TextParser, get_parser
from .store import InvertedIndex, RAGStore, SearchResult

__all__ = ["RAGEngine", "RAGStore", "InvertedIndex", "SearchResult", "TokenEmbedder", "BM25Scorer", "Chunk",
           "TextParser", "JSONParser", "JSONLParser", "CSVParser", "get_parser"]

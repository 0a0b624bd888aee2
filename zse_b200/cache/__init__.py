from .attention_metadata import AttentionMetadata, build_attention_metadata
from .block_pool import Block, BlockPool
from .cache_manager import CacheStats, KVCacheHandle, KVCacheManager
from .dedup import BlockDedup
from .evictor import EvictionCandidate, Evictor
from .page_table import PageTable, SequenceEntry

__all__ = ["AttentionMetadata", "Block", "BlockPool", "CacheStats", "KVCacheHandle", "KVCacheManager", "BlockDedup",
           "Evictor", "EvictionCandidate", "PageTable", "SequenceEntry", "build_attention_metadata"]

"""The ``.zse`` model container: reader, writer, quantisers, tokenizer, converters."""
from .config import ModelConfig, QuantConfig
from .header import FileHeader, SectionEntry
from .loader import ZSELoader
from .spec import MAGIC, VERSION, Flags, QuantMethod, SectionType, should_quantize
from .tokenizer import BPETokenizer, SpecialTokens
from .weight_index import WeightEntry, WeightIndex
from .writer import ZSEWriter

__all__ = ["ModelConfig", "QuantConfig", "FileHeader", "SectionEntry", "ZSELoader", "ZSEWriter", "MAGIC", "VERSION",
           "Flags", "QuantMethod", "SectionType", "should_quantize", "BPETokenizer", "SpecialTokens", "WeightEntry",
           "WeightIndex"]

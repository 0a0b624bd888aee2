"""The ``.zse`` model container: reader, writer, quantisers, tokenizer, converters."""
from .config import ModelConfig, QuantConfig
from .header import FileHeader, SectionEntry, read_header_and_sections
from .loader import ZSELoader
from .quantize import dequantize_tensor, quantize_tensor
from .spec import MAGIC, VERSION, Flags, QuantMethod, SectionType, should_quantize
from .tokenizer import BPETokenizer, SpecialTokens
from .weight_index import WeightEntry, WeightIndex
from .writer import ZSEWriter

__all__ = ["ModelConfig", "QuantConfig", "FileHeader", "SectionEntry", "ZSELoader", "ZSEWriter", "MAGIC", "VERSION",
           "Flags", "QuantMethod", "SectionType", "should_quantize", "BPETokenizer", "SpecialTokens", "WeightEntry",
           "WeightIndex", "read_header_and_sections", "quantize_tensor", "dequantize_tensor"]

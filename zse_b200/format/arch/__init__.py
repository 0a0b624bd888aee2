from .base import ArchAdapter, detect_architecture, get_adapter, register_adapter, supported_architectures
from . import llama, qwen2, phi3, gemma2, gemma4  # noqa: F401  (registration)

__all__ = ["ArchAdapter", "detect_architecture", "get_adapter", "register_adapter", "supported_architectures"]

from .manager import LoRAManager
from .weights import LoRAAdapter, LoRAWeight, LoRAWeightStore

__all__ = ["LoRAManager", "LoRAAdapter", "LoRAWeight", "LoRAWeightStore"]

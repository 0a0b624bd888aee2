"""LoRA adapter bookkeeping (zse-engine/zse_engine/orchestrator/lora_weights.py:22-167).

An adapter holds, per (layer, module), ``A [rank, in]`` and ``B [out, rank]``; the update is
``y += (alpha/rank) * B (A x)``.  Tensors live wherever the manager put them (CPU for tests, CUDA when serving).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass
class LoRAWeight:
    layer_name: str
    rank: int
    in_features: int
    out_features: int
    a: Any = None            # tensor [rank, in]
    b: Any = None            # tensor [out, rank]

    @property
    def nbytes(self) -> int:
        return 2 * self.rank * (self.in_features + self.out_features)

    @property
    def loaded(self) -> bool:
        return self.a is not None and self.b is not None

    # the reference's names (zse-engine/zse_engine/orchestrator/lora_weights.py:36-60)
    @property
    def total_gpu_bytes(self) -> int:
        return self.nbytes

    @property
    def a_shape(self) -> Tuple[int, int]:
        return (self.rank, self.in_features)

    @property
    def b_shape(self) -> Tuple[int, int]:
        return (self.out_features, self.rank)

    @staticmethod
    def _ptr(t) -> int:
        return int(t.data_ptr()) if t is not None and hasattr(t, "data_ptr") else 0

    @staticmethod
    def _nbytes(t) -> int:
        return int(t.numel() * t.element_size()) if t is not None and hasattr(t, "numel") else 0

    a_ptr = property(lambda self: self._ptr(self.a))
    b_ptr = property(lambda self: self._ptr(self.b))
    a_nbytes = property(lambda self: self._nbytes(self.a))
    b_nbytes = property(lambda self: self._nbytes(self.b))

    def make_a_tensor(self):
        return self.a

    def make_b_tensor(self):
        return self.b


@dataclass
class LoRAAdapter:
    adapter_id: str
    rank: int
    alpha: float
    target_modules: List[str]
    num_layers: int
    weights: Dict[Tuple[int, str], LoRAWeight] = field(default_factory=dict)
    slot: int = -1           # index in the batched weight tables (-1 = not resident)
    base_model: str = ""     # free-form metadata, as in the reference's record
    description: str = ""
    generation: int = 0      # load counter of the manager when this adapter became resident

    @property
    def scaling(self) -> float:
        return float(self.alpha) / float(self.rank) if self.rank else 0.0

    def add_weight(self, layer_idx: int, module_name: str, weight: LoRAWeight) -> None:
        self.weights[(layer_idx, module_name)] = weight

    def get_weight(self, layer_idx: int, module_name: str) -> Optional[LoRAWeight]:
        return self.weights.get((layer_idx, module_name))

    def has_module(self, module: str) -> bool:
        return module in self.target_modules

    def has_weight(self, layer_idx: int, module_name: str) -> bool:
        return (layer_idx, module_name) in self.weights

    @property
    def num_weight_pairs(self) -> int:
        return len(self.weights)

    @property
    def total_bytes(self) -> int:
        return sum(w.nbytes for w in self.weights.values())

    @property
    def total_gpu_bytes(self) -> int:
        return self.total_bytes

    def summary(self) -> str:
        return (f"LoRA adapter '{self.adapter_id}': rank {self.rank}, alpha {self.alpha:g} (scaling "
                f"{self.scaling:.3f}), {self.num_layers} layers x {', '.join(self.target_modules)}, "
                f"{self.num_weight_pairs} weight pairs, {self.total_bytes / 2 ** 20:.2f} MiB")


class LoRAWeightStore:
    """Adapters by id, with a byte budget."""

    def __init__(self, max_bytes: int = 0):
        self._adapters: Dict[str, LoRAAdapter] = {}
        self.max_bytes = max_bytes

    def add(self, adapter: LoRAAdapter) -> None:
        if adapter.adapter_id in self._adapters:
            raise ValueError(f"adapter '{adapter.adapter_id}' is already loaded")
        if self.max_bytes and self.total_bytes + adapter.total_bytes > self.max_bytes:
            raise MemoryError(f"adapter '{adapter.adapter_id}' does not fit the LoRA budget")
        self._adapters[adapter.adapter_id] = adapter

    def remove(self, adapter_id: str) -> Optional[LoRAAdapter]:
        return self._adapters.pop(adapter_id, None)

    def get(self, adapter_id: str) -> Optional[LoRAAdapter]:
        return self._adapters.get(adapter_id)

    def list_ids(self) -> List[str]:
        return list(self._adapters)

    def __contains__(self, adapter_id: str) -> bool:
        return adapter_id in self._adapters

    def __len__(self) -> int:
        return len(self._adapters)

    @property
    def total_bytes(self) -> int:
        return sum(a.total_bytes for a in self._adapters.values())

    # the reference's names (zse-engine/zse_engine/orchestrator/lora_weights.py:133-167)
    def has(self, adapter_id: str) -> bool:
        return adapter_id in self._adapters

    @property
    def num_adapters(self) -> int:
        return len(self._adapters)

    @property
    def total_gpu_bytes(self) -> int:
        return self.total_bytes

    def list_adapters(self) -> List[str]:
        return list(self._adapters)

    def summary(self) -> str:
        lines = [f"LoRA store: {len(self._adapters)} adapters, {self.total_bytes / 2 ** 20:.2f} MiB"]
        lines += ["  " + a.summary() for a in self._adapters.values()]
        return "\n".join(lines)


def random_adapter_file(path: str, config, rank: int = 8, alpha: float = 16.0,
                        target_modules: Optional[List[str]] = None, seed: int = 0, std: float = 0.05) -> LoRAAdapter:
    """Writes a ``.zse-lora`` file with random A/B matrices for a model config (tests, benchmarks, smoke runs)."""
    import numpy as np

    from ..format.lora_format import module_shapes, save_lora
    targets = list(target_modules or ["q_proj", "k_proj", "v_proj"])
    shapes = module_shapes(config.hidden_size, config.intermediate_size, config.num_heads, config.num_kv_heads,
                           config.head_dim)
    rng = np.random.default_rng(seed)
    ad = LoRAAdapter("", rank, alpha, targets, config.num_layers)
    data = {}
    for layer in range(config.num_layers):
        for t in targets:
            fin, fout = shapes[t]
            data[(layer, t)] = ((rng.standard_normal((rank, fin)) * std).astype(np.float16),
                                (rng.standard_normal((fout, rank)) * std).astype(np.float16))
            ad.add_weight(layer, t, LoRAWeight(f"model.layers.{layer}.{t}", rank, fin, fout))
    save_lora(path, ad, data)
    return ad

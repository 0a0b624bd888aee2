"""LoRA adapters resident on the device, hot-swappable while serving
(zse-engine/zse_engine/orchestrator/lora_manager.py:37-396).

All loaded adapters of one rank share padded weight tables per (layer, module): ``A [slots, rank, in]`` and
``B [slots, out, rank]``; a request's adapter is a slot index carried per token, so a decode batch mixing adapters
runs in one launch pair per projection (``ops.lora_apply``).  Targets, as in the reference
(zse-engine/zse_engine/orchestrator/model_runner.py:1000-1109): ``q_proj``, ``k_proj``, ``v_proj`` (added to the fused
QKV output before RoPE), ``o_proj`` and ``down_proj`` (their update is an fp16 addend of the fused residual + RMSNorm
kernel that follows the projection), ``gate_proj`` and ``up_proj`` (the MLP then runs without the fused SwiGLU
epilogue: projection, updates, activation).  Under tensor parallelism ``A`` is replicated and ``B`` is row-sharded like
the base weight for the column-parallel targets; for the row-parallel ones (``o_proj``, ``down_proj``) ``A`` is sharded by
columns like the projection's input and ``B`` is whole, so that every rank's update is a partial sum that the
projection's own all-reduce completes (no extra exchange).
"""
from __future__ import annotations

import threading
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from ..format.lora_format import load_lora, module_shapes
from .weights import LoRAAdapter, LoRAWeight, LoRAWeightStore

QKV_TARGETS = ("q_proj", "k_proj", "v_proj")
ROW_PARALLEL_TARGETS = ("o_proj", "down_proj")
MLP_IN_TARGETS = ("gate_proj", "up_proj")
SUPPORTED_TARGETS = QKV_TARGETS + ROW_PARALLEL_TARGETS + MLP_IN_TARGETS


class LoRAManager:
    def __init__(self, model, device, max_adapters: int = 32, max_rank: int = 64):
        self._model = model
        self._device = torch.device(device)
        self._lock = threading.Lock()
        self._store = LoRAWeightStore()
        self._max_adapters, self._max_rank = max_adapters, max_rank
        self._slots: List[Optional[str]] = [None] * max_adapters
        self._rank = 0                                   # common (padded) rank of the tables
        self._a: Dict[Tuple[int, str], torch.Tensor] = {}
        self._b: Dict[Tuple[int, str], torch.Tensor] = {}
        self._scales = torch.zeros(max_adapters, dtype=torch.float32, device=self._device)
        self._loads = self._unloads = 0

    # ---- geometry -----------------------------------------------------------------------------------------
    def _a_columns(self, module: str) -> Tuple[int, int]:
        """Column range of ``A`` this rank holds: all of it, except for the row-parallel projections, whose input is
        sharded (o_proj reads this rank's heads, down_proj this rank's slice of the intermediate dimension).  There the
        rank's update B (A[:, cols] x[cols]) is a partial sum like the projection's own output, and the same
        all-reduce completes both."""
        c, p = self._model.config, self._model.plan
        if module == "o_proj":
            return tuple(p.q_rows) if p.tp_size > 1 else (0, c.q_dim)
        if module == "down_proj":
            return tuple(p.inter) if p.tp_size > 1 else (0, c.intermediate_size)
        return (0, c.hidden_size)

    def _module_geometry(self, module: str):
        """(in_features, full out_features, local row range of B, column offset inside the fused qkv output)."""
        c, p = self._model.config, self._model.plan
        if module == "o_proj":
            return c.q_dim, c.hidden_size, (0, c.hidden_size), 0
        if module == "down_proj":
            return c.intermediate_size, c.hidden_size, (0, c.hidden_size), 0
        if module in MLP_IN_TARGETS:
            return c.hidden_size, c.intermediate_size, p.inter, 0
        if module == "q_proj":
            return c.hidden_size, c.q_dim, p.q_rows, 0
        if module == "k_proj":
            return c.hidden_size, c.kv_dim, p.kv_rows, p.q_dim
        if module == "v_proj":
            return c.hidden_size, c.kv_dim, p.kv_rows, p.q_dim + p.kv_dim
        raise KeyError(module)

    def weight_shapes(self) -> Dict[str, Tuple[int, int]]:
        c = self._model.config
        return module_shapes(c.hidden_size, c.intermediate_size, c.num_heads, c.num_kv_heads, c.head_dim)

    # ---- load / unload --------------------------------------------------------------------------------------
    def load_adapter(self, adapter_id: str, path: str) -> LoRAAdapter:
        adapter, data = load_lora(path, self.weight_shapes())
        adapter.adapter_id = adapter_id
        arrays = {}
        for (layer, mod), (a_bytes, b_bytes) in data.items():
            w = adapter.get_weight(layer, mod)
            arrays[(layer, mod)] = (np.frombuffer(a_bytes, np.float16).reshape(w.rank, w.in_features),
                                    np.frombuffer(b_bytes, np.float16).reshape(w.out_features, w.rank))
        return self.load_adapter_from_arrays(adapter_id, adapter.rank, adapter.alpha, adapter.target_modules,
                                             adapter.num_layers, arrays)

    def load_adapter_from_arrays(self, adapter_id: str, rank: int, alpha: float, target_modules: List[str],
                                 num_layers: int, arrays: Dict[Tuple[int, str], tuple]) -> LoRAAdapter:
        """``arrays[(layer, module)] = (A [rank, in], B [out, rank])`` as numpy / torch tensors (full, unsharded)."""
        unsupported = [t for t in target_modules if t not in SUPPORTED_TARGETS]
        if unsupported:
            raise ValueError(f"LoRA targets {unsupported} are not supported (supported: {SUPPORTED_TARGETS})")
        if rank > self._max_rank or rank % 2:
            raise ValueError(f"LoRA rank {rank} must be even and <= {self._max_rank}")
        if type(self._model).__name__ != "DecoderModel":
            raise ValueError("adapters are wired for the Llama / Mistral / Qwen2 / Phi-3 decoder only")
        with self._lock:
            if adapter_id in self._store:
                raise ValueError(f"adapter '{adapter_id}' is already loaded")
            try:
                slot = self._slots.index(None)
            except ValueError:
                raise MemoryError(f"all {self._max_adapters} adapter slots are in use") from None
            if rank > self._rank:
                self._grow_rank(rank)
            ad = LoRAAdapter(adapter_id, rank, alpha, list(target_modules), num_layers)
            for (layer, mod), (a, b) in arrays.items():
                fin, fout, rows, _ = self._module_geometry(mod)
                a_t = (a if isinstance(a, torch.Tensor) else torch.from_numpy(np.array(a))).to(torch.float16)
                b_t = (b if isinstance(b, torch.Tensor) else torch.from_numpy(np.array(b))).to(torch.float16)
                if tuple(a_t.shape) != (rank, fin) or tuple(b_t.shape) != (fout, rank):
                    raise ValueError(f"bad LoRA shapes for layer {layer} {mod}: A {tuple(a_t.shape)}, "
                                     f"B {tuple(b_t.shape)}")
                ta, tb = self._tables(layer, mod)
                ta[slot].zero_()
                tb[slot].zero_()
                cols = self._a_columns(mod)
                ta[slot, :rank].copy_(a_t[:, cols[0]:cols[1]].to(self._device))
                tb[slot, :, :rank].copy_(b_t[rows[0]:rows[1]].to(self._device))
                ad.add_weight(layer, mod, LoRAWeight(f"model.layers.{layer}.{mod}", rank, cols[1] - cols[0], fout, ta[slot],
                                                            tb[slot]))
            ad.slot = slot
            self._slots[slot] = adapter_id
            self._scales[slot] = ad.scaling
            self._store.add(ad)
            self._loads += 1
            ad.generation = self._loads            # tells a re-loaded adapter from the one that had this name before
            self._model.lora = self
            return ad

    def _tables(self, layer: int, mod: str):
        key = (layer, mod)
        if key not in self._a:
            _, _, rows, _ = self._module_geometry(mod)
            cols = self._a_columns(mod)
            self._a[key] = torch.zeros(self._max_adapters, self._rank, cols[1] - cols[0], dtype=torch.float16,
                                       device=self._device)
            self._b[key] = torch.zeros(self._max_adapters, rows[1] - rows[0], self._rank, dtype=torch.float16,
                                       device=self._device)
        return self._a[key], self._b[key]

    def _grow_rank(self, rank: int) -> None:
        for key in list(self._a):
            a, b = self._a[key], self._b[key]
            na = torch.zeros(a.shape[0], rank, a.shape[2], dtype=a.dtype, device=a.device)
            nb = torch.zeros(b.shape[0], b.shape[1], rank, dtype=b.dtype, device=b.device)
            na[:, : a.shape[1]] = a
            nb[:, :, : b.shape[2]] = b
            self._a[key], self._b[key] = na, nb
        self._rank = rank

    def unload_adapter(self, adapter_id: str) -> bool:
        with self._lock:
            ad = self._store.remove(adapter_id)
            if ad is None:
                return False
            self._slots[ad.slot] = None
            self._scales[ad.slot] = 0.0
            for (layer, mod) in ad.weights:
                if (layer, mod) in self._a:
                    self._a[(layer, mod)][ad.slot].zero_()
                    self._b[(layer, mod)][ad.slot].zero_()
            self._unloads += 1
            if len(self._store) == 0:
                self._model.lora = None
            return True

    # ---- the reference's entry points (zse-engine/zse_engine/orchestrator/lora_manager.py:88-246) -----------------
    def load_adapter_from_file(self, adapter_id: str, path: str, weight_shapes=None) -> LoRAAdapter:
        """``weight_shapes`` is accepted for compatibility; the shapes come from the model."""
        return self.load_adapter(adapter_id, path)

    def load_adapter_from_dict(self, adapter_id: str, rank: int, alpha: float, num_layers: int,
                               target_modules: List[str], weights_data: Dict[Tuple[int, str], tuple],
                               weight_shapes=None) -> LoRAAdapter:
        """``weights_data[(layer, module)] = (A, B)`` as fp16 bytes, numpy arrays or tensors."""
        shapes = self.weight_shapes()
        arrays = {}
        for (layer, mod), (a, b) in weights_data.items():
            fin, fout = shapes[mod]
            if isinstance(a, (bytes, bytearray, memoryview)):
                a = np.frombuffer(a, np.float16).reshape(rank, fin)
            if isinstance(b, (bytes, bytearray, memoryview)):
                b = np.frombuffer(b, np.float16).reshape(fout, rank)
            arrays[(layer, mod)] = (a, b)
        return self.load_adapter_from_arrays(adapter_id, rank, alpha, list(target_modules), num_layers, arrays)

    def load_adapter_random(self, adapter_id: str, rank: int = 8, alpha: float = 16.0, num_layers: int = 0,
                            target_modules: Optional[List[str]] = None, seed: int = 0, std: float = 0.02,
                            **_ignored) -> LoRAAdapter:
        """An adapter with random matrices (tests and benchmarks); model dimensions come from the model."""
        shapes = self.weight_shapes()
        rng = np.random.default_rng(seed)
        targets = list(target_modules or ["q_proj", "v_proj"])
        layers = num_layers or self._model.config.num_layers
        arrays = {(l, t): ((rng.standard_normal((rank, shapes[t][0])) * std).astype(np.float16),
                           (rng.standard_normal((shapes[t][1], rank)) * std).astype(np.float16))
                  for l in range(layers) for t in targets}
        return self.load_adapter_from_arrays(adapter_id, rank, alpha, targets, layers, arrays)

    def get_adapter(self, adapter_id: str) -> Optional[LoRAAdapter]:
        return self._store.get(adapter_id)

    def has_adapter(self, adapter_id: str) -> bool:
        return adapter_id in self._store

    @property
    def num_adapters(self) -> int:
        return len(self._store)

    def summary(self) -> str:
        lines = [f"LoRA adapters: {len(self._store)} of {self._max_adapters} slots, table rank {self._rank}"]
        for a in self.list_adapters():
            lines.append(f"  {a['adapter_id']}: rank {a['rank']}, alpha {a['alpha']:g}, "
                         f"{', '.join(a['target_modules'])}, {a['bytes'] / 2 ** 20:.1f} MiB, slot {a['slot']}")
        return "\n".join(lines)

    # ---- queries --------------------------------------------------------------------------------------------
    def is_loaded(self, adapter_id: str) -> bool:
        return adapter_id in self._store

    def slot_of(self, adapter_id: Optional[str]) -> int:
        ad = self._store.get(adapter_id) if adapter_id else None
        return -1 if ad is None else ad.slot

    def cache_salt(self, adapter_id: Optional[str]) -> int:
        """Non-zero value that names the loaded adapter in the prefix cache (0: base model).  Keys and values written
        under one adapter must never be reused by a sequence that runs with another one or with none; the load
        counter keeps blocks of an unloaded adapter from matching a later adapter of the same name.  The value is
        the same in every tensor-parallel worker (no per-process hash)."""
        ad = self._store.get(adapter_id) if adapter_id else None
        if ad is None:
            return 0
        import zlib
        return ((zlib.crc32(adapter_id.encode("utf-8")) << 24) ^ (int(getattr(ad, "generation", 0)) << 1) | 1) \
            & 0xFFFFFFFFFFFFFFFF

    def list_adapters(self) -> List[dict]:
        return [{"adapter_id": i, "rank": a.rank, "alpha": a.alpha, "target_modules": a.target_modules,
                 "num_layers": a.num_layers, "bytes": a.total_bytes, "slot": a.slot}
                for i, a in ((i, self._store.get(i)) for i in self._store.list_ids())]

    def stats(self) -> dict:
        return {"num_adapters": len(self._store), "max_adapters": self._max_adapters, "table_rank": self._rank,
                "total_bytes": self._store.total_bytes, "loads": self._loads, "unloads": self._unloads,
                "table_bytes": sum(t.numel() * 2 for t in list(self._a.values()) + list(self._b.values()))}

    # ---- hot path -------------------------------------------------------------------------------------------
    def has(self, layer: int, module: str) -> bool:
        return (layer, module) in self._a

    def _scratch(self, b, name: str, width: int) -> torch.Tensor:
        """A [max_tokens, width] fp16 buffer that lives with the step buffers ``b`` (made on first use)."""
        t = getattr(b, name, None)
        if t is None or t.shape[1] != width:
            t = torch.zeros(b.max_tokens, width, dtype=torch.float16, device=self._device)
            setattr(b, name, t)
        return t

    def delta(self, layer: int, module: str, x: torch.Tensor, b, M: int) -> Optional[torch.Tensor]:
        """fp16 ``[>= M, out]`` with the summed update of every resident adapter for ``module`` of ``layer`` applied
        to ``x`` (rows of tokens without an adapter stay zero), or None when no adapter touches the module."""
        key = (layer, module)
        if key not in self._a:
            return None
        _, _, rows, _ = self._module_geometry(module)
        cols = self._a_columns(module)
        fin = cols[1] - cols[0]
        n_out = rows[1] - rows[0]
        out = self._scratch(b, "lora_delta_" + ("h" if module in ROW_PARALLEL_TARGETS else module), n_out)
        out[:M].zero_()
        self._model.ops.lora_apply(x, self._a[key], self._b[key], b.adapter_ids, self._scales, out, M, fin, n_out,
                                   self._rank, tmp=b.lora_tmp)
        return out

    def apply_lora(self, out: torch.Tensor, inp: torch.Tensor, adapter, layer_idx: int, module_name: str, M: int,
                   N: Optional[int] = None, K: Optional[int] = None) -> bool:
        """``out[:M, :N] += (alpha / rank) * (inp[:M, :K] A^T) B^T`` for ONE adapter, on whatever device the tensors
        live (zse-engine/zse_engine/orchestrator/lora_manager.py:255-330).  ``adapter``: a ``LoRAAdapter`` or its id.
        For callers that apply an adapter to a projection themselves; the engine's passes use the batched tables
        (``apply_qkv`` / ``delta``: one shrink and one expand launch for every adapter in the batch).  Returns False
        when the adapter has no weights for the module."""
        if isinstance(adapter, str):
            adapter = self._store.get(adapter)
        w = adapter.get_weight(layer_idx, module_name) if adapter is not None else None
        if w is None or not w.loaded:
            return False
        N = w.out_features if N is None else N
        K = w.in_features if K is None else K
        if (N, K) != (w.out_features, w.in_features):
            raise ValueError(f"{module_name} of layer {layer_idx} is [{w.out_features}, {w.in_features}], not [{N}, {K}]")
        a, b_ = w.a.to(inp.device), w.b.to(inp.device)
        tmp = inp[:M, :K].float() @ a.float().t()
        # the resident tables are padded to the table rank (zeros) and, on a sharded model, hold this rank's rows
        out[:M, : b_.shape[0]] += (adapter.scaling * (tmp @ b_.float().t())).to(out.dtype)
        return True

    def apply_qkv(self, layer: int, b, M: int) -> None:
        """Adds every resident adapter's update to the fused QKV output of ``layer`` for the first ``M`` tokens."""
        ops = self._model.ops
        for mod in QKV_TARGETS:
            key = (layer, mod)
            if key not in self._a:
                continue
            fin, _, rows, col0 = self._module_geometry(mod)
            ops.lora_apply(b.xnorm, self._a[key], self._b[key], b.adapter_ids, self._scales, b.qkv, M, fin,
                           rows[1] - rows[0], self._rank, tmp=b.lora_tmp, y_col0=col0)

    def destroy(self) -> None:
        with self._lock:
            self._a.clear()
            self._b.clear()

"""``.zse-lora`` adapter files.

Layout (zse-engine/zse_engine/format/lora_format.py:1-156): 32-byte header ``"ZLRA"``, u32 version (1), u32 rank,
f32 alpha, u32 num_layers, u32 num_targets, u64 total weight bytes; then one 64-byte NUL-padded name per target
module; then for every layer, for every target in header order: ``A [rank, in]`` fp16 followed by
``B [out, rank]`` fp16.
"""
from __future__ import annotations

import struct
from typing import Dict, List, Tuple

import numpy as np

LORA_MAGIC = b"ZLRA"
LORA_VERSION = 1
TARGET_NAME_SIZE = 64
_HDR = struct.Struct("<4sIIfIIQ")


def _bytes(x) -> bytes:
    if isinstance(x, (bytes, bytearray, memoryview)):
        return bytes(x)
    if isinstance(x, np.ndarray):
        return np.ascontiguousarray(x, dtype=np.float16).tobytes()
    return x.detach().to("cpu").contiguous().numpy().astype(np.float16).tobytes()  # torch tensor


def save_lora(path: str, adapter, weight_data: Dict[Tuple[int, str], tuple]) -> None:
    """``adapter`` needs ``rank``, ``alpha``, ``num_layers``, ``target_modules``; ``weight_data`` maps
    ``(layer, module)`` to ``(A, B)`` given as bytes, numpy arrays or torch tensors."""
    targets: List[str] = list(adapter.target_modules)
    blobs = {k: (_bytes(a), _bytes(b)) for k, (a, b) in weight_data.items()}
    total = sum(len(a) + len(b) for a, b in blobs.values())
    with open(path, "wb") as f:
        f.write(_HDR.pack(LORA_MAGIC, LORA_VERSION, adapter.rank, float(adapter.alpha), adapter.num_layers,
                          len(targets), total))
        for t in targets:
            f.write(t.encode("utf-8")[:TARGET_NAME_SIZE - 1].ljust(TARGET_NAME_SIZE, b"\x00"))
        for layer in range(adapter.num_layers):
            for t in targets:
                if (layer, t) in blobs:
                    a, b = blobs[(layer, t)]
                    f.write(a)
                    f.write(b)


def read_lora_header(path: str) -> dict:
    with open(path, "rb") as f:
        raw = f.read(_HDR.size)
        if len(raw) < _HDR.size or raw[:4] != LORA_MAGIC:
            raise ValueError(f"invalid .zse-lora file: bad magic {raw[:4]!r}")
        _, version, rank, alpha, layers, ntargets, total = _HDR.unpack(raw)
        if version != LORA_VERSION:
            raise ValueError(f"unsupported .zse-lora version {version}")
        targets = [f.read(TARGET_NAME_SIZE).split(b"\x00", 1)[0].decode("utf-8") for _ in range(ntargets)]
    return {"rank": rank, "alpha": alpha, "num_layers": layers, "targets": targets, "total_bytes": total,
            "data_offset": _HDR.size + ntargets * TARGET_NAME_SIZE}


def load_lora(path: str, weight_shapes: Dict[str, Tuple[int, int]]):
    """``weight_shapes``: module name -> ``(in_features, out_features)``.  Returns ``(adapter, weight_data)`` with
    ``weight_data[(layer, module)] = (a_bytes, b_bytes)``; targets absent from ``weight_shapes`` are skipped
    (their bytes cannot be sized, as in the reference, so they must come last or be known)."""
    from ..lora.weights import LoRAAdapter, LoRAWeight
    h = read_lora_header(path)
    adapter = LoRAAdapter(adapter_id="", rank=h["rank"], alpha=h["alpha"], target_modules=h["targets"],
                          num_layers=h["num_layers"])
    data = {}
    with open(path, "rb") as f:
        f.seek(h["data_offset"])
        for layer in range(h["num_layers"]):
            for t in h["targets"]:
                if t not in weight_shapes:
                    continue
                fin, fout = weight_shapes[t]
                a = f.read(h["rank"] * fin * 2)
                b = f.read(fout * h["rank"] * 2)
                if len(a) != h["rank"] * fin * 2 or len(b) != fout * h["rank"] * 2:
                    raise ValueError(f"truncated .zse-lora at layer {layer}, {t}")
                data[(layer, t)] = (a, b)
                adapter.add_weight(layer, t, LoRAWeight(f"model.layers.{layer}.{t}", h["rank"], fin, fout))
    return adapter, data


def module_shapes(hidden_size: int, intermediate_size: int = 0, num_heads: int = 32, num_kv_heads: int = 32,
                  head_dim: int = 128) -> Dict[str, Tuple[int, int]]:
    s = {"q_proj": (hidden_size, num_heads * head_dim), "k_proj": (hidden_size, num_kv_heads * head_dim),
         "v_proj": (hidden_size, num_kv_heads * head_dim), "o_proj": (num_heads * head_dim, hidden_size)}
    if intermediate_size > 0:
        s.update({"gate_proj": (hidden_size, intermediate_size), "up_proj": (hidden_size, intermediate_size),
                  "down_proj": (intermediate_size, hidden_size)})
    return s


def estimate_lora_size(rank: int, num_layers: int, target_modules: List[str], hidden_size: int,
                       intermediate_size: int = 0, num_heads: int = 32, num_kv_heads: int = 32,
                       head_dim: int = 128) -> int:
    shapes = module_shapes(hidden_size, intermediate_size, num_heads, num_kv_heads, head_dim)
    per_layer = sum(rank * shapes[t][0] * 2 + shapes[t][1] * rank * 2 for t in target_modules if t in shapes)
    return per_layer * num_layers

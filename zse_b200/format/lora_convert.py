"""HuggingFace PEFT LoRA adapters -> ``.zse-lora``.

A PEFT adapter directory holds ``adapter_config.json`` (``r``, ``lora_alpha``, ``target_modules``) and
``adapter_model.safetensors`` with tensors named ``...layers.<n>.<block>.<module>.lora_A.weight`` ``[r, in]`` and
``...lora_B.weight`` ``[out, r]``.  The ``.zse-lora`` layout wants the same two matrices per layer and target in a
fixed order (zse-engine/zse_engine/format/lora_format.py:35-193); the reference ships the file format and a loader
but no importer, so adapters trained with the usual tools could not be served.  Every layer must carry every target
(the file has no per-layer directory); rank patterns that differ between modules are refused.
"""
from __future__ import annotations

import json
import os
import re
from typing import Dict, List, Optional, Tuple

import numpy as np

from .convert import build_tensor_map, read_safetensors_tensor
from .lora_format import save_lora

SERVED_MODULES = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")
_NAME = re.compile(r"layers\.(\d+)\.(?:self_attn|mlp)\.([a-z_]+)\.lora_([AB])(?:\.[^.]+)?\.weight$")


class _Meta:
    def __init__(self, rank: int, alpha: float, num_layers: int, targets: List[str]):
        self.rank, self.alpha, self.num_layers, self.target_modules = rank, alpha, num_layers, targets


def convert_peft_to_zse_lora(adapter_dir: str, output_path: str, modules: Optional[List[str]] = None) -> dict:
    """Writes ``output_path``; returns ``{rank, alpha, num_layers, targets, skipped}``.  ``modules`` restricts the
    targets (default: every served projection the adapter has)."""
    with open(os.path.join(adapter_dir, "adapter_config.json"), "r", encoding="utf-8") as f:
        cfg = json.load(f)
    rank, alpha = int(cfg["r"]), float(cfg.get("lora_alpha", cfg["r"]))
    if cfg.get("rank_pattern") or cfg.get("alpha_pattern"):
        raise ValueError("adapters with per-module rank or alpha patterns cannot be stored in a .zse-lora file")
    if cfg.get("use_dora"):
        raise ValueError("DoRA adapters are not LoRA adapters: they cannot be served as A/B pairs")
    files = [os.path.join(adapter_dir, n) for n in sorted(os.listdir(adapter_dir)) if n.endswith(".safetensors")]
    if not files:
        raise FileNotFoundError(f"no .safetensors file in {adapter_dir}")
    found: Dict[Tuple[int, str], Dict[str, np.ndarray]] = {}
    skipped: List[str] = []
    for name, (path, info, base) in build_tensor_map(files).items():
        m = _NAME.search(name)
        if not m:
            if "lora_" in name:
                skipped.append(name)
            continue
        layer, module, which = int(m.group(1)), m.group(2), m.group(3)
        if module not in SERVED_MODULES or (modules and module not in modules):
            skipped.append(name)
            continue
        values, shape = read_safetensors_tensor(path, info, base)
        arr = np.asarray(values, dtype=np.float32).reshape(shape)
        found.setdefault((layer, module), {})[which] = arr
    if not found:
        raise ValueError("no LoRA matrices for the attention or MLP projections in this adapter")
    num_layers = max(layer for layer, _ in found) + 1
    targets = [t for t in SERVED_MODULES if any(mod == t for _, mod in found)]
    data = {}
    for layer in range(num_layers):
        for t in targets:
            pair = found.get((layer, t))
            if pair is None or "A" not in pair or "B" not in pair:
                raise ValueError(f"layer {layer} has no complete LoRA pair for {t}: a .zse-lora file needs every target "
                                 f"in every layer (restrict the targets with `modules`)")
            a, b = pair["A"], pair["B"]
            if a.shape[0] != rank or b.shape[1] != rank:
                raise ValueError(f"layer {layer} {t}: A {a.shape} / B {b.shape} do not have rank {rank}")
            data[(layer, t)] = (a.astype(np.float16), b.astype(np.float16))
    if cfg.get("use_rslora"):                   # rank-stabilised scaling alpha/sqrt(r): fold it into alpha (alpha/r)
        alpha = alpha * (rank ** 0.5)
    save_lora(output_path, _Meta(rank, alpha, num_layers, targets), data)
    return {"rank": rank, "alpha": alpha, "num_layers": num_layers, "targets": targets, "skipped": skipped}

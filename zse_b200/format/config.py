"""Model and quantisation metadata stored in the CONFIG section.

Field names and defaults follow zse-engine/zse_engine/format/config.py:10-135 so that
files written by either implementation load in the other.  Unknown keys are ignored on
load; this build adds ``quant.int4_layout`` (``"rowmajor"`` or ``"tiled64x8"``), which the
reference loader skips because it filters the quant dict by known keys.
"""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional

from . import serializer
from .spec import DEFAULT_GROUP_SIZE, DEFAULT_QUANT_BITS, QuantMethod


@dataclass
class QuantConfig:
    method: int = int(QuantMethod.INT4_ASYM)
    bits: int = DEFAULT_QUANT_BITS
    group_size: int = DEFAULT_GROUP_SIZE
    scale_dtype: str = "float16"
    tiled_weights: bool = True          # kept for wire compatibility; does not describe the bytes
    int4_layout: Optional[str] = None   # "rowmajor" | "tiled64x8" | None (= not recorded)

    def to_dict(self) -> dict:
        d = {"method": int(self.method), "bits": self.bits, "group_size": self.group_size,
             "scale_dtype": self.scale_dtype, "tiled_weights": self.tiled_weights}
        if self.int4_layout is not None:
            d["int4_layout"] = self.int4_layout
        return d

    @classmethod
    def from_dict(cls, d: dict) -> "QuantConfig":
        names = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in names})


@dataclass
class LayerSpec:
    head_dim: int
    num_kv_heads: int
    rope_theta: float
    rotary_dim: int          # leading pairs (i, i + head_dim/2), i < rotary_dim/2, rotate; the rest pass through
    window: int              # 0 = full causal attention
    k_is_v: bool             # no v_proj: V is the k_proj output before its norm
    scale: float
    softcap: float           # 0 = none
    qk_norm: bool            # per-head RMSNorm of q and k (learned weight) and of v (no weight)


@dataclass
class ModelConfig:
    arch: str = "llama"
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 32
    head_dim: int = 128
    hidden_size: int = 4096
    intermediate_size: int = 11008
    vocab_size: int = 32000
    max_seq_len: int = 4096
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-5
    rope_scaling: Optional[Dict[str, Any]] = None
    sliding_window: Optional[int] = None
    tie_word_embeddings: bool = False
    # Gemma-family extensions (None/False = not applicable)
    layer_types: Optional[List[str]] = None
    global_head_dim: Optional[int] = None
    global_num_kv_heads: Optional[int] = None
    global_rope_theta: Optional[float] = None
    partial_rotary_factor: Optional[float] = None
    hidden_activation: Optional[str] = None
    final_logit_softcapping: Optional[float] = None
    attn_logit_softcapping: Optional[float] = None
    query_pre_attn_scalar: Optional[float] = None
    attention_k_eq_v: bool = False
    embed_scale: bool = False
    multimodal: Optional[Dict[str, Any]] = None
    quant: QuantConfig = field(default_factory=QuantConfig)

    # ---- (de)serialisation -------------------------------------------------------
    def to_dict(self) -> dict:
        d: Dict[str, Any] = {}
        for f in fields(self):
            v = getattr(self, f.name)
            if f.name == "quant":
                d["quant"] = self.quant.to_dict()
            elif v is not None:
                d[f.name] = v
        return d

    @classmethod
    def from_dict(cls, d: dict) -> "ModelConfig":
        d = dict(d)
        quant = d.pop("quant", None)
        names = {f.name for f in fields(cls)}
        cfg = cls(**{k: v for k, v in d.items() if k in names})
        if quant:
            cfg.quant = QuantConfig.from_dict(quant)
        return cfg

    def serialize(self) -> bytes:
        return serializer.encode(self.to_dict())

    @classmethod
    def deserialize(cls, data) -> "ModelConfig":
        return cls.from_dict(serializer.decode(data))

    # ---- derived sizes -----------------------------------------------------------
    @property
    def q_dim(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def kv_head_dim(self) -> int:
        return self.head_dim

    @property
    def kv_cache_bytes_per_token(self) -> int:
        """fp16 K and V of one token in one layer (of the widest layer when layers differ)."""
        n, d = self.kv_pool_dims()
        return 2 * n * d * 2

    @property
    def total_kv_cache_bytes_per_token(self) -> int:
        return self.kv_cache_bytes_per_token * self.num_layers

    # ---- per-layer attention geometry (Gemma-family models mix layer kinds) -----------------------
    @property
    def is_gemma(self) -> bool:
        return self.arch.startswith("gemma")

    @property
    def norm_weight_offset(self) -> float:
        """Gemma-2 stores RMSNorm weights as ``w - 1`` (the norm multiplies by ``1 + w``); Gemma-4 and everything
        else multiply by the stored weight (zse-engine/zse_engine/orchestrator/kernels.py:1475-1478)."""
        return 1.0 if self.arch == "gemma2" else 0.0

    def layer_kind(self, i: int) -> str:
        if self.layer_types and i < len(self.layer_types):
            return self.layer_types[i]
        return "full_attention"

    def layer_spec(self, i: int) -> "LayerSpec":
        """Attention geometry of layer ``i`` (zse-engine/zse_engine/orchestrator/model_runner.py:132-152)."""
        sliding = self.layer_kind(i) == "sliding_attention"
        hd, nkv, theta, rot = self.head_dim, self.num_kv_heads, self.rope_theta, self.head_dim
        shares = False
        if self.arch == "gemma4" and not sliding:
            hd = self.global_head_dim or self.head_dim
            shares = bool(self.attention_k_eq_v)
            nkv = (self.global_num_kv_heads or self.num_kv_heads) if shares else self.num_kv_heads
            theta = self.global_rope_theta or self.rope_theta
            rot = 2 * int((self.partial_rotary_factor or 1.0) * hd // 2)
        if self.arch == "gemma4":
            scale = 1.0                         # q/k norms carry the scaling
        elif self.query_pre_attn_scalar:
            scale = float(self.query_pre_attn_scalar) ** -0.5
        else:
            scale = float(hd) ** -0.5
        window = int(self.sliding_window or 0) if (sliding or not self.layer_types) else 0
        return LayerSpec(hd, nkv, float(theta), rot, window, shares, scale,
                         float(self.attn_logit_softcapping or 0.0), self.arch == "gemma4")

    def kv_pool_dims(self, num_kv_heads: Optional[int] = None):
        """(kv_heads, head_dim) the KV pool is allocated with; ``num_kv_heads`` = this rank's share of
        ``self.num_kv_heads`` under tensor parallelism.  Models whose layers differ get rows of the widest layer
        (``1 x max(kv_heads * head_dim)`` of the local heads); each layer lays its heads out inside that row."""
        local = num_kv_heads or self.num_kv_heads
        tp = max(1, self.num_kv_heads // max(1, local))
        specs = {(s.num_kv_heads, s.head_dim) for s in (self.layer_spec(i) for i in range(self.num_layers))}
        if len(specs) <= 1:
            return local, self.head_dim
        return 1, max(max(1, n // tp) * d for n, d in specs)

    def linear_param_count(self) -> int:
        per_layer = (self.hidden_size * self.q_dim + 2 * self.hidden_size * self.kv_dim
                     + self.q_dim * self.hidden_size + 3 * self.hidden_size * self.intermediate_size)
        return per_layer * self.num_layers

    def estimate_model_size_bytes(self) -> int:
        params = self.linear_param_count()
        fp16 = self.vocab_size * self.hidden_size * 2 * (1 if self.tie_word_embeddings else 2)
        fp16 += self.num_layers * self.hidden_size * 2 * 2
        if self.quant.method == QuantMethod.NONE:
            return params * 2 + fp16
        groups = params // max(1, self.quant.group_size)
        per_group = 4 if self.quant.method == QuantMethod.INT4_ASYM else 2
        return params * self.quant.bits // 8 + groups * per_group + fp16

"""Architecture adapters: HuggingFace ``config.json`` -> ``ModelConfig`` and tensor-name mapping.

Capabilities of zse-engine/zse_engine/format/arch/base.py:15-123: a registry keyed by architecture
name, detection from ``architectures`` / ``model_type``, ``model.`` prefix stripping, the fp16
keep-list, name-sorted load order and basic shape sanity warnings.
"""
from __future__ import annotations

from typing import Dict, List, Type

from ..config import ModelConfig
from ..spec import should_quantize as _default_should_quantize

_REGISTRY: Dict[str, Type["ArchAdapter"]] = {}


def register_adapter(cls):
    _REGISTRY[cls.ARCH_NAME] = cls
    return cls


def get_adapter(arch_name: str) -> "ArchAdapter":
    try:
        return _REGISTRY[arch_name]()
    except KeyError:
        raise ValueError(f"unknown architecture '{arch_name}'; supported: {', '.join(sorted(_REGISTRY))}") from None


def supported_architectures() -> List[str]:
    return sorted(_REGISTRY)


# checked in this order; the first substring hit on an `architectures` entry wins
_DETECT = (("llama", "llama"), ("mistral", "mistral"), ("qwen", "qwen2"), ("phi", "phi3"),
           ("gemma4", "gemma4"), ("gemma_4", "gemma4"), ("gemma", "gemma2"))


def detect_architecture(hf_config: dict) -> str:
    for name in hf_config.get("architectures") or []:
        low = name.lower()
        for needle, arch in _DETECT:
            if needle in low:
                return arch
    mt = str(hf_config.get("model_type", "")).lower()
    if mt in _REGISTRY:
        return mt
    raise ValueError(f"cannot detect the architecture (architectures={hf_config.get('architectures')}, "
                     f"model_type={hf_config.get('model_type')})")


def rope_settings(hf: dict, default_theta: float):
    """(theta, scaling dict or None) from either spelling of a HuggingFace config: the older top-level
    ``rope_theta`` / ``rope_scaling`` keys, or ``rope_parameters`` (transformers 5 writes the base and the scaling
    parameters together there; ``rope_type: default`` means no scaling)."""
    rp = hf.get("rope_parameters")
    theta, scaling = hf.get("rope_theta"), hf.get("rope_scaling")
    if isinstance(rp, dict) and ("rope_theta" in rp or "rope_type" in rp or "type" in rp):
        theta = rp.get("rope_theta", theta)
        if scaling is None:
            scaling = {k: v for k, v in rp.items() if k != "rope_theta"}
    if isinstance(scaling, dict):
        kind = scaling.get("rope_type", scaling.get("type"))
        if kind in (None, "default"):
            scaling = None
    return float(theta if theta is not None else default_theta), scaling


class ArchAdapter:
    ARCH_NAME = "unknown"
    #: tensors every layer must have; subclasses extend
    LAYER_TENSORS = ("self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight",
                     "self_attn.o_proj.weight", "mlp.gate_proj.weight", "mlp.up_proj.weight",
                     "mlp.down_proj.weight", "input_layernorm.weight", "post_attention_layernorm.weight")

    def config_from_hf(self, hf_config: dict) -> ModelConfig:
        hf = hf_config
        raise NotImplementedError

    def _common(self, hf: dict, arch: str, *, max_seq: int, theta: float, eps: float, tie: bool,
                explicit_head_dim: bool) -> ModelConfig:
        h, nh = hf["hidden_size"], hf["num_attention_heads"]
        hd = hf.get("head_dim") if explicit_head_dim else None
        rope_theta, rope_scaling = rope_settings(hf, theta)
        return ModelConfig(arch=arch, num_layers=hf["num_hidden_layers"], num_heads=nh,
                           num_kv_heads=hf.get("num_key_value_heads", nh), head_dim=hd or h // nh,
                           hidden_size=h, intermediate_size=hf["intermediate_size"], vocab_size=hf["vocab_size"],
                           max_seq_len=hf.get("max_position_embeddings", max_seq),
                           rope_theta=rope_theta,
                           rms_norm_eps=float(hf.get("rms_norm_eps", eps)),
                           rope_scaling=rope_scaling, sliding_window=hf.get("sliding_window"),
                           tie_word_embeddings=bool(hf.get("tie_word_embeddings", tie)))

    #: explicit renames (HF name -> stored name) applied before the ``model.`` prefix is stripped
    TENSOR_NAME_MAP: Dict[str, str] = {}

    def map_tensor_name(self, hf_name: str) -> str:
        hf_name = self.TENSOR_NAME_MAP.get(hf_name, hf_name)
        return hf_name[6:] if hf_name.startswith("model.") else hf_name

    def should_quantize(self, tensor_name: str) -> bool:
        return _default_should_quantize(tensor_name)

    def tensor_load_order(self, tensor_names: List[str]) -> List[str]:
        names = tensor_names
        return sorted(names)

    def layer_tensors(self, config: ModelConfig, layer: int) -> List[str]:
        return list(self.LAYER_TENSORS)

    def expected_tensors(self, config: ModelConfig) -> List[str]:
        out = ["embed_tokens.weight"]
        for i in range(config.num_layers):
            out += [f"layers.{i}.{t}" for t in self.layer_tensors(config, i)]
        out.append("norm.weight")
        if not config.tie_word_embeddings:
            out.append("lm_head.weight")
        return out

    def validate_config(self, config: ModelConfig) -> List[str]:
        c = config
        w = []
        if c.hidden_size % c.num_heads:
            w.append(f"hidden_size ({c.hidden_size}) not divisible by num_heads ({c.num_heads})")
        if c.num_heads % c.num_kv_heads:
            w.append(f"num_heads ({c.num_heads}) not divisible by num_kv_heads ({c.num_kv_heads})")
        kind = (c.rope_scaling or {}).get("rope_type", (c.rope_scaling or {}).get("type"))
        if kind not in (None, "default", "linear", "llama3"):
            w.append(f"rope scaling of type '{kind}' is not applied by the runtime (linear and llama3 are): positions "
                     f"beyond the original context length will be rotated with the unscaled frequencies")
        return w

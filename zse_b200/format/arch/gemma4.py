"""Gemma-4 unified text backbone (zse-engine/zse_engine/format/arch/gemma4.py:40-234).

The language model sits under ``text_config``; sliding and full-attention layers have different
head_dim / kv heads / RoPE (``layer_types``, ``global_*``, ``partial_rotary_factor``); full-attention layers
share K and V (no ``v_proj``); every layer has q/k norms, four layer norms and a ``layer_scalar``.  Modality
projections are renamed to ``vision.*`` / ``audio.*`` and never quantised.
"""
from .base import ArchAdapter, register_adapter
from ..config import ModelConfig

_VISION_KEYS = ("patch_size", "model_patch_size", "mm_embed_dim", "mm_posemb_size", "num_soft_tokens",
                "output_proj_dims", "pooling_kernel_size", "rms_norm_eps")
_AUDIO_KEYS = ("audio_embed_dim", "audio_samples_per_token", "output_proj_dims", "rms_norm_eps")


@register_adapter
class Gemma4Adapter(ArchAdapter):
    ARCH_NAME = "gemma4"

    def config_from_hf(self, hf_config):
        hf = hf_config
        tc = hf.get("text_config", hf)
        rope = tc.get("rope_parameters", {}) or {}
        sliding, full = rope.get("sliding_attention", {}) or {}, rope.get("full_attention", {}) or {}
        mm = {}
        if hf.get("vision_config"):
            mm["vision"] = {k: hf["vision_config"].get(k) for k in _VISION_KEYS}
            mm["vision"]["image_token_id"] = hf.get("image_token_id")
        if hf.get("audio_config"):
            mm["audio"] = {k: hf["audio_config"].get(k) for k in _AUDIO_KEYS}
            mm["audio"]["audio_token_id"] = hf.get("audio_token_id")
        h, nh = tc["hidden_size"], tc["num_attention_heads"]
        return ModelConfig(
            arch="gemma4", num_layers=tc["num_hidden_layers"], num_heads=nh,
            num_kv_heads=tc.get("num_key_value_heads", nh), head_dim=tc.get("head_dim", h // nh), hidden_size=h,
            intermediate_size=tc["intermediate_size"], vocab_size=tc["vocab_size"],
            max_seq_len=tc.get("max_position_embeddings", 262144),
            rope_theta=float(sliding.get("rope_theta", tc.get("rope_theta", 10000.0))),
            rms_norm_eps=float(tc.get("rms_norm_eps", 1e-6)), sliding_window=tc.get("sliding_window"),
            tie_word_embeddings=bool(tc.get("tie_word_embeddings", hf.get("tie_word_embeddings", True))),
            layer_types=tc.get("layer_types"), global_head_dim=tc.get("global_head_dim"),
            global_num_kv_heads=tc.get("num_global_key_value_heads"), global_rope_theta=full.get("rope_theta"),
            partial_rotary_factor=full.get("partial_rotary_factor"), hidden_activation=tc.get("hidden_activation"),
            final_logit_softcapping=tc.get("final_logit_softcapping"),
            attn_logit_softcapping=tc.get("attn_logit_softcapping"),
            query_pre_attn_scalar=tc.get("query_pre_attn_scalar"),
            attention_k_eq_v=bool(tc.get("attention_k_eq_v", False)), embed_scale=True, multimodal=mm or None)

    def map_tensor_name(self, hf_name):
        name = hf_name[6:] if hf_name.startswith("model.") else hf_name
        if name.startswith("language_model."):
            name = name[len("language_model."):]
            return name[6:] if name.startswith("model.") else name
        for src, dst in (("vision_embedder.", "vision."), ("embed_vision.", "vision.proj."),
                         ("embed_audio.", "audio.proj."), ("audio_embedder.", "audio.")):
            if name.startswith(src):
                return dst + name[len(src):]
        return name

    def should_quantize(self, tensor_name):
        if tensor_name.startswith(("vision.", "audio.")) or "layer_scalar" in tensor_name:
            return False
        return super().should_quantize(tensor_name)

    def _shares_kv(self, c, i):
        return bool(c.attention_k_eq_v and c.layer_types and i < len(c.layer_types)
                    and c.layer_types[i] == "full_attention")

    def layer_tensors(self, c, i):
        t = ["self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.o_proj.weight",
             "self_attn.q_norm.weight", "self_attn.k_norm.weight", "mlp.gate_proj.weight", "mlp.up_proj.weight",
             "mlp.down_proj.weight", "input_layernorm.weight", "post_attention_layernorm.weight",
             "pre_feedforward_layernorm.weight", "post_feedforward_layernorm.weight", "layer_scalar"]
        if not self._shares_kv(c, i):
            t.append("self_attn.v_proj.weight")
        return t

    def validate_config(self, config):
        c = config
        w = super().validate_config(c)
        if c.global_head_dim and c.global_head_dim != c.head_dim:
            w.append(f"mixed head_dim: sliding {c.head_dim}, full-attention {c.global_head_dim}")
        if c.partial_rotary_factor:
            w.append(f"full-attention layers rotate only {c.partial_rotary_factor:.0%} of each head")
        return w

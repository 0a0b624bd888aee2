"""Phi-3 (zse-engine/zse_engine/format/arch/phi3.py): fused ``qkv_proj`` and ``gate_up_proj`` tensors are
stored under their fused names; the runtime splits them when the model is built."""
from .base import ArchAdapter, register_adapter


@register_adapter
class Phi3Adapter(ArchAdapter):
    ARCH_NAME = "phi3"
    LAYER_TENSORS = ("self_attn.qkv_proj.weight", "self_attn.o_proj.weight", "mlp.gate_up_proj.weight",
                     "mlp.down_proj.weight", "input_layernorm.weight", "post_attention_layernorm.weight")

    def config_from_hf(self, hf_config):
        hf = hf_config
        c = self._common(hf, "phi3", max_seq=4096, theta=10000.0, eps=1e-5, tie=False, explicit_head_dim=False)
        # Phi-4-mini rotates only the leading part of each head (pairs (i, i + rot/2) inside that part)
        f = hf.get("partial_rotary_factor", (hf.get("rope_parameters") or {}).get("partial_rotary_factor"))
        if f is not None and float(f) < 1.0:
            c.partial_rotary_factor = float(f)
        if isinstance(c.rope_scaling, dict):
            c.rope_scaling = {k: v for k, v in c.rope_scaling.items() if k != "partial_rotary_factor"} or None
            if c.rope_scaling and c.rope_scaling.get("rope_type", c.rope_scaling.get("type")) in (None, "default"):
                c.rope_scaling = None
        return c

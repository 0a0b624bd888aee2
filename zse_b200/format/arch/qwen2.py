"""Qwen2 / Qwen2.5 (zse-engine/zse_engine/format/arch/qwen2.py): Llama layout plus q/k/v biases,
rope_theta 1e6, eps 1e-6, head_dim always hidden/heads, embeddings tied unless the config says otherwise."""
from .base import ArchAdapter, register_adapter


@register_adapter
class Qwen2Adapter(ArchAdapter):
    ARCH_NAME = "qwen2"
    LAYER_TENSORS = ArchAdapter.LAYER_TENSORS + ("self_attn.q_proj.bias", "self_attn.k_proj.bias",
                                                 "self_attn.v_proj.bias")

    def config_from_hf(self, hf_config):
        hf = hf_config
        c = self._common(hf, "qwen2", max_seq=32768, theta=1000000.0, eps=1e-6, tie=True, explicit_head_dim=False)
        if not hf.get("use_sliding_window", False):      # the window in Qwen2 configs is inert unless switched on
            c.sliding_window = None
        return c

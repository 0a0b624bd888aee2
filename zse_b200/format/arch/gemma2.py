"""Gemma-2 (zse-engine/zse_engine/format/arch/gemma2.py): explicit head_dim, four norms per layer, GeGLU,
soft-capping, tied embeddings by default."""
from .base import ArchAdapter, register_adapter


@register_adapter
class Gemma2Adapter(ArchAdapter):
    ARCH_NAME = "gemma2"
    LAYER_TENSORS = ArchAdapter.LAYER_TENSORS + ("pre_feedforward_layernorm.weight",
                                                 "post_feedforward_layernorm.weight")

    def config_from_hf(self, hf_config):
        hf = hf_config
        c = self._common(hf, "gemma2", max_seq=8192, theta=10000.0, eps=1e-6, tie=True, explicit_head_dim=True)
        c.rope_scaling = None
        c.hidden_activation = hf.get("hidden_activation", "gelu_pytorch_tanh")
        c.final_logit_softcapping = hf.get("final_logit_softcapping")
        c.attn_logit_softcapping = hf.get("attn_logit_softcapping")
        c.query_pre_attn_scalar = hf.get("query_pre_attn_scalar")
        c.embed_scale = True
        # local (sliding-window) and global attention alternate, starting with a local layer
        c.layer_types = hf.get("layer_types") or ["sliding_attention" if (i + 1) % 2 else "full_attention"
                                                  for i in range(c.num_layers)]
        c.sliding_window = hf.get("sliding_window", 4096)
        return c

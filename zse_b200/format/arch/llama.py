"""Llama and Mistral (zse-engine/zse_engine/format/arch/llama.py): RMSNorm, SwiGLU, RoPE, optional GQA."""
from .base import ArchAdapter, register_adapter


@register_adapter
class LlamaAdapter(ArchAdapter):
    ARCH_NAME = "llama"

    def config_from_hf(self, hf_config):
        hf = hf_config
        return self._common(hf, self.ARCH_NAME, max_seq=4096, theta=10000.0, eps=1e-5, tie=False,
                            explicit_head_dim=True)


@register_adapter
class MistralAdapter(LlamaAdapter):
    ARCH_NAME = "mistral"

    def config_from_hf(self, hf_config):
        hf = hf_config
        c = super().config_from_hf(hf)
        if c.sliding_window is None:
            c.sliding_window = 4096
        return c

"""Logit parity of the fp32 oracle (and so of the converter, the arch adapters and the name maps) with HuggingFace
transformers on tiny random models of every supported family.  The models are built on the CPU from a config,
saved as safetensors, converted to an fp16 ``.zse`` file and run through ``OracleModel``; the logits must agree
to rounding (the reference gates Gemma-4 the same way: argmax, top-5 and cosine > 0.99 against HF,
zse-engine/tests/test_modal_gemma4_parity.py)."""
import os

import numpy as np
import pytest
import torch

transformers = pytest.importorskip("transformers")

from zse_b200.format.convert import convert_hf_to_zse
from zse_b200.format.loader import ZSELoader
from zse_b200.format.spec import QuantMethod
from zse_b200.models.oracle import OracleModel

COMMON = dict(vocab_size=320, hidden_size=64, intermediate_size=160, num_hidden_layers=3, num_attention_heads=4,
              num_key_value_heads=2, max_position_embeddings=256)


def _llama():
    from transformers import LlamaConfig, LlamaForCausalLM
    return LlamaForCausalLM(LlamaConfig(**COMMON, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False))


def _llama3_scaled():
    from transformers import LlamaConfig, LlamaForCausalLM
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 16}
    # a base that is not the adapter's default either: it must be read from wherever this transformers puts it
    return LlamaForCausalLM(LlamaConfig(**COMMON, rms_norm_eps=1e-5, rope_theta=500000.0, rope_scaling=scaling,
                                        tie_word_embeddings=False))


def _llama_linear():
    from transformers import LlamaConfig, LlamaForCausalLM
    return LlamaForCausalLM(LlamaConfig(**COMMON, rms_norm_eps=1e-5, rope_theta=10000.0,
                                        rope_scaling={"rope_type": "linear", "factor": 4.0},
                                        tie_word_embeddings=False))


def _mistral():
    from transformers import MistralConfig, MistralForCausalLM
    return MistralForCausalLM(MistralConfig(**COMMON, sliding_window=None, head_dim=16, tie_word_embeddings=False))


def _mistral_window():
    from transformers import MistralConfig, MistralForCausalLM
    return MistralForCausalLM(MistralConfig(**COMMON, sliding_window=8, head_dim=16, tie_word_embeddings=False,
                                            attn_implementation="eager"))


def _qwen2():
    from transformers import Qwen2Config, Qwen2ForCausalLM
    return Qwen2ForCausalLM(Qwen2Config(**COMMON, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True))


def _phi3():
    from transformers import Phi3Config, Phi3ForCausalLM
    return Phi3ForCausalLM(Phi3Config(**COMMON, rms_norm_eps=1e-5, rope_theta=10000.0, pad_token_id=0,
                                      tie_word_embeddings=False))


def _phi3_partial():
    from transformers import Phi3Config, Phi3ForCausalLM
    return Phi3ForCausalLM(Phi3Config(**COMMON, rms_norm_eps=1e-5, rope_theta=10000.0, pad_token_id=0,
                                      partial_rotary_factor=0.5, tie_word_embeddings=False))


def _gemma2():
    from transformers import Gemma2Config, Gemma2ForCausalLM
    return Gemma2ForCausalLM(Gemma2Config(**COMMON, head_dim=32, sliding_window=8, query_pre_attn_scalar=24,
                                          attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
                                          attn_implementation="eager"))


def _gemma4(k_eq_v=False):
    from transformers import Gemma4ForCausalLM, Gemma4TextConfig
    kind = ["sliding_attention", "sliding_attention", "full_attention"]
    cfg = Gemma4TextConfig(**COMMON, head_dim=16, global_head_dim=32, layer_types=kind, sliding_window=8,
                           hidden_size_per_layer_input=0, vocab_size_per_layer_input=320, enable_moe_block=False,
                           num_kv_shared_layers=0, attention_k_eq_v=k_eq_v,
                           num_global_key_value_heads=1 if k_eq_v else None, final_logit_softcapping=30.0,
                           attn_implementation="eager")
    return Gemma4ForCausalLM(cfg)


def _randomise(model, seed):
    """Random values everywhere, norm weights and the Gemma-4 layer scalars included, so that no term is trivial."""
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in list(model.named_parameters()) + list(model.named_buffers()):
            if "inv_freq" in name or "embed_scale" in name:
                continue
            if name.endswith("layer_scalar"):
                p.copy_(0.5 + torch.rand(p.shape, generator=g))
            elif "norm" in name:
                p.copy_(0.3 * torch.randn(p.shape, generator=g) + (0.0 if "gemma2" in type(model).__name__.lower()
                                                                   else 1.0))
            elif p.dtype.is_floating_point:
                p.copy_(0.08 * torch.randn(p.shape, generator=g))


@pytest.mark.parametrize("family", ["llama", "llama_rope3", "llama_ropelinear", "mistral", "mistral_window", "qwen2", "phi3", "phi3_partial", "gemma2", "gemma4",
                                    "gemma4_k_eq_v"])
def test_oracle_matches_transformers(tmp_path, family):
    torch.manual_seed(0)
    build = {"llama": _llama, "llama_rope3": _llama3_scaled, "llama_ropelinear": _llama_linear, "mistral": _mistral, "qwen2": _qwen2, "mistral_window": _mistral_window, "phi3": _phi3, "phi3_partial": _phi3_partial, "gemma2": _gemma2, "gemma4": _gemma4,
             "gemma4_k_eq_v": lambda: _gemma4(True)}[family]
    model = build().eval().float()
    _randomise(model, 1)
    if getattr(model.config, "tie_word_embeddings", False):
        model.tie_weights()
    hf_dir = tmp_path / "hf"
    model.save_pretrained(str(hf_dir), safe_serialization=True)
    out = str(tmp_path / "m.zse")
    convert_hf_to_zse(str(hf_dir), out, quant_method=int(QuantMethod.NONE), skip_tokenizer=True)
    loader = ZSELoader(out)
    assert loader.config.arch == family.split("_")[0]
    if family == "phi3_partial":
        assert loader.config.partial_rotary_factor == 0.5
    if family == "llama_rope3":
        assert loader.config.rope_theta == 500000.0 and loader.config.rope_scaling["rope_type"] == "llama3"
    oracle = OracleModel(loader)
    # longer than the sliding window (8), so that local layers really drop tokens
    ids = torch.randint(0, COMMON["vocab_size"], (1, 21), generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        want = model(input_ids=ids).logits[0].float()
    got = oracle.forward(ids[0].tolist())
    # the file stores fp16 weights: compare against HF running the same rounded weights
    with torch.no_grad():
        for p in model.parameters():
            p.copy_(p.half().float())
        for name, b in model.named_buffers():
            if name.endswith("layer_scalar"):
                b.copy_(b.half().float())
        want = model(input_ids=ids).logits[0].float()
    cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
    assert float(cos.min()) > 0.9999, (family, float(cos.min()))
    assert torch.equal(got.argmax(-1), want.argmax(-1))
    assert float((got - want).abs().max()) < 2e-3 * max(1.0, float(want.abs().max()))
    loader.close()

"""Synthetic models: random weights of a given architecture written as a ``.zse`` file.

``write_random_model`` draws every linear weight from N(0, std), quantises it (INT4 group-128 by default) and
streams it into the file; norms are 1, biases N(0, std).  ``fast=True`` skips the float stage and writes random
nibbles with plausible scales/zeros directly, which is what the benchmarks use for multi-GB shapes (the bytes are
statistically the same as quantised N(0, std) weights and cost no quantisation time).
"""
from __future__ import annotations

from typing import Optional

import numpy as np

from .config import ModelConfig, QuantConfig
from .spec import QuantMethod
from .tokenizer import BPETokenizer, BYTE_ENCODER, SpecialTokens
from .writer import ZSEWriter

SHAPES = {
    "tiny": dict(num_layers=2, hidden_size=256, num_heads=4, num_kv_heads=2, head_dim=64, intermediate_size=688,
                 vocab_size=1024, rms_norm_eps=1e-6, rope_theta=10000.0, arch="llama", max_seq_len=2048),
    "tiny-aligned": dict(num_layers=2, hidden_size=256, num_heads=4, num_kv_heads=2, head_dim=64,
                         intermediate_size=768, vocab_size=1024, rms_norm_eps=1e-6, rope_theta=10000.0, arch="qwen2",
                         max_seq_len=2048),
    "tiny-phi3": dict(num_layers=2, hidden_size=256, num_heads=4, num_kv_heads=2, head_dim=64, intermediate_size=768,
                      vocab_size=1024, rms_norm_eps=1e-5, rope_theta=10000.0, arch="phi3", max_seq_len=2048),
    "small-128": dict(num_layers=2, hidden_size=512, num_heads=4, num_kv_heads=2, head_dim=128,
                      intermediate_size=1024, vocab_size=2048, rms_norm_eps=1e-6, rope_theta=1e6, arch="qwen2",
                      max_seq_len=4096),
    # an intermediate size whose 128-column groups (15) do not divide evenly over 2, 4 or 8 ranks, and 8 kv heads so
    # that every rank count up to 8 gets whole heads: the small analogue of a 13824-wide MLP on 8 GPUs
    "small-uneven": dict(num_layers=2, hidden_size=1024, num_heads=8, num_kv_heads=8, head_dim=128,
                         intermediate_size=1920, vocab_size=2048, rms_norm_eps=1e-6, rope_theta=1e6, arch="qwen2",
                         max_seq_len=4096),
    # Gemma-2 block: four norms, GeGLU, soft-capped scores and logits, local/global layers alternate
    "tiny-gemma2": dict(num_layers=4, hidden_size=256, num_heads=4, num_kv_heads=2, head_dim=64,
                        intermediate_size=768, vocab_size=1024, rms_norm_eps=1e-6, rope_theta=10000.0, arch="gemma2",
                        max_seq_len=2048, sliding_window=24, query_pre_attn_scalar=64.0, attn_logit_softcapping=50.0,
                        final_logit_softcapping=30.0, hidden_activation="gelu_pytorch_tanh", embed_scale=True,
                        tie_word_embeddings=True,
                        layer_types=["sliding_attention", "full_attention"] * 2),
    # Gemma-4 block: q/k/v head norms, local layers (head_dim 64) and global layers (head_dim 128, a quarter of it
    # rotated, V = K projection, one kv head), learned layer scalars
    "tiny-gemma4": dict(num_layers=3, hidden_size=256, num_heads=4, num_kv_heads=2, head_dim=64,
                        intermediate_size=768, vocab_size=1024, rms_norm_eps=1e-6, rope_theta=10000.0, arch="gemma4",
                        max_seq_len=2048, sliding_window=24, global_head_dim=128, global_num_kv_heads=1,
                        global_rope_theta=1e6, partial_rotary_factor=0.25, attention_k_eq_v=True,
                        final_logit_softcapping=30.0, hidden_activation="gelu_pytorch_tanh", embed_scale=True,
                        tie_word_embeddings=True,
                        layer_types=["sliding_attention", "sliding_attention", "full_attention"]),
    "gemma2-9b": dict(num_layers=42, hidden_size=3584, num_heads=16, num_kv_heads=8, head_dim=256,
                      intermediate_size=14336, vocab_size=256000, rms_norm_eps=1e-6, rope_theta=10000.0,
                      arch="gemma2", max_seq_len=8192, sliding_window=4096, query_pre_attn_scalar=256.0,
                      attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
                      hidden_activation="gelu_pytorch_tanh", embed_scale=True, tie_word_embeddings=True,
                      layer_types=["sliding_attention", "full_attention"] * 21),
    "qwen2.5-7b": dict(num_layers=28, hidden_size=3584, num_heads=28, num_kv_heads=4, head_dim=128,
                       intermediate_size=18944, vocab_size=152064, rms_norm_eps=1e-6, rope_theta=1e6, arch="qwen2",
                       max_seq_len=32768),
    "qwen2.5-14b": dict(num_layers=48, hidden_size=5120, num_heads=40, num_kv_heads=8, head_dim=128,
                        intermediate_size=13824, vocab_size=152064, rms_norm_eps=1e-6, rope_theta=1e6, arch="qwen2",
                        max_seq_len=32768),
    "qwen2.5-32b": dict(num_layers=64, hidden_size=5120, num_heads=40, num_kv_heads=8, head_dim=128,
                        intermediate_size=27648, vocab_size=152064, rms_norm_eps=1e-6, rope_theta=1e6, arch="qwen2",
                        max_seq_len=32768),
    "qwen2.5-72b": dict(num_layers=80, hidden_size=8192, num_heads=64, num_kv_heads=8, head_dim=128,
                        intermediate_size=29568, vocab_size=152064, rms_norm_eps=1e-6, rope_theta=1e6, arch="qwen2",
                        max_seq_len=32768),
}


def shape_config(name: str, quant: str = "int4", **overrides) -> ModelConfig:
    kw = dict(SHAPES[name])
    kw.update(overrides)
    method = {"int4": QuantMethod.INT4_ASYM, "int8": QuantMethod.INT8_SYM, "fp16": QuantMethod.NONE}[quant]
    bits = {"int4": 4, "int8": 8, "fp16": 16}[quant]
    return ModelConfig(quant=QuantConfig(method=int(method), bits=bits, group_size=128), **kw)


def byte_tokenizer(vocab_size: int = 1024) -> BPETokenizer:
    """A real (if dull) byte-level BPE tokenizer: 256 byte symbols, a few merges, ChatML markers."""
    vocab = {BYTE_ENCODER[b]: b for b in range(256)}
    merges = []
    for a, b in (("t", "h"), ("i", "n"), ("th", "e"), ("Ġ", "t"), ("Ġ", "a"), ("e", "r"), ("a", "n"), ("o", "n")):
        if a + b not in vocab and len(vocab) < vocab_size - 8:
            vocab[a + b] = len(vocab)
            merges.append((a, b))
    nxt = len(vocab)
    added = {"<|endoftext|>": nxt, "<|im_start|>": nxt + 1, "<|im_end|>": nxt + 2}
    return BPETokenizer(vocab=vocab, merges=merges, added_tokens=added,
                        special_tokens=SpecialTokens(bos_id=nxt, eos_id=nxt, pad_id=nxt, unk_id=0))


def layer_weight_shapes(c: ModelConfig, layer: int = 0):
    sp = c.layer_spec(layer) if c.is_gemma else None
    q_dim = c.num_heads * sp.head_dim if sp else c.q_dim
    kv_dim = sp.num_kv_heads * sp.head_dim if sp else c.kv_dim
    if c.arch == "phi3":        # [q; k; v] and [gate; up] are stored stacked
        return [("self_attn.qkv_proj", q_dim + 2 * kv_dim, c.hidden_size), ("self_attn.o_proj", c.hidden_size, q_dim),
                ("mlp.gate_up_proj", 2 * c.intermediate_size, c.hidden_size),
                ("mlp.down_proj", c.hidden_size, c.intermediate_size)]
    out = [("self_attn.q_proj", q_dim, c.hidden_size), ("self_attn.k_proj", kv_dim, c.hidden_size)]
    if not (sp and sp.k_is_v):
        out.append(("self_attn.v_proj", kv_dim, c.hidden_size))
    return out + [("self_attn.o_proj", c.hidden_size, q_dim), ("mlp.gate_proj", c.intermediate_size, c.hidden_size),
                  ("mlp.up_proj", c.intermediate_size, c.hidden_size),
                  ("mlp.down_proj", c.hidden_size, c.intermediate_size)]


def write_random_model(path: str, config: ModelConfig, seed: int = 0, std: float = 0.02, fast: bool = False,
                       with_tokenizer: bool = True, qkv_bias: Optional[bool] = None) -> None:
    rng = np.random.default_rng(seed)
    c = config
    qkv_bias = (c.arch == "qwen2") if qkv_bias is None else qkv_bias
    gs = c.quant.group_size
    w = ZSEWriter(path)
    w.set_config(c)
    if with_tokenizer:
        w.set_tokenizer(byte_tokenizer(c.vocab_size).serialize())
    w.begin_weights()

    def linear(name, n, k):
        if c.quant.method == QuantMethod.NONE:
            w.add_weight_raw_fp16(name, (n, k), (rng.standard_normal((n, k), dtype=np.float32) * std).astype(np.float16))
        elif fast and c.quant.method == QuantMethod.INT4_ASYM:
            total = n * k
            groups = (total + gs - 1) // gs
            packed = np.frombuffer(rng.bytes(groups * gs // 2), dtype=np.uint8)
            # range of 128 N(0,std) samples is about 5.2 std wide, centred near 0
            half = (2.6 + 0.35 * rng.standard_normal(groups, dtype=np.float32)).clip(1.5, 4.0) * std
            w.add_weight_raw(name, (n, k), packed, (2 * half / 15).astype(np.float16), (-half).astype(np.float16), gs)
        else:
            w.add_weight(name, rng.standard_normal((n, k), dtype=np.float32) * std, (n, k), quantize=True)

    def fp16(name, shape, values):
        w.add_weight_raw_fp16(name, shape, np.asarray(values, dtype=np.float16))

    def big_fp16(name, n, k):
        if fast:  # one random block of rows, repeated: N(0, std) entries, a fraction of the generation time
            rows = min(n, 4096)
            block = (rng.standard_normal((rows, k), dtype=np.float32) * std).astype(np.float16)
            fp16(name, (n, k), np.tile(block, ((n + rows - 1) // rows, 1))[:n])
        else:
            fp16(name, (n, k), rng.standard_normal((n, k), dtype=np.float32) * std)

    # stored norm weights: Gemma-2 files hold w - 1
    norm_mean = 1.0 - c.norm_weight_offset

    def norm(name, n):
        fp16(name, (n,), norm_mean + 0.1 * rng.standard_normal(n))

    big_fp16("embed_tokens.weight", c.vocab_size, c.hidden_size)
    for i in range(c.num_layers):
        p = f"layers.{i}"
        fp16(f"{p}.input_layernorm.weight", (c.hidden_size,), norm_mean + 0.1 * rng.standard_normal(c.hidden_size))
        if c.is_gemma:
            norm(f"{p}.pre_feedforward_layernorm.weight", c.hidden_size)
            norm(f"{p}.post_feedforward_layernorm.weight", c.hidden_size)
            sp = c.layer_spec(i)
            if sp.qk_norm:
                norm(f"{p}.self_attn.q_norm.weight", sp.head_dim)
                norm(f"{p}.self_attn.k_norm.weight", sp.head_dim)
                fp16(f"{p}.layer_scalar", (1,), [0.8 + 0.4 * rng.random()])
        for name, n, k in layer_weight_shapes(c, i):
            linear(f"{p}.{name}.weight", n, k)
            if qkv_bias and name.split(".")[-1] in ("q_proj", "k_proj", "v_proj"):
                fp16(f"{p}.{name}.bias", (n,), rng.standard_normal(n) * std)
        fp16(f"{p}.post_attention_layernorm.weight", (c.hidden_size,),
             norm_mean + 0.1 * rng.standard_normal(c.hidden_size))
    fp16("norm.weight", (c.hidden_size,), norm_mean + 0.1 * rng.standard_normal(c.hidden_size))
    if not c.tie_word_embeddings:
        big_fp16("lm_head.weight", c.vocab_size, c.hidden_size)
    w.finalize()

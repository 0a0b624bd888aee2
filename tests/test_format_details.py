"""More of the format layer, piece by piece: architecture detection and the adapter registry, both spellings of the RoPE
settings in HuggingFace configs, what gets quantised, the tensors a layer must have, config-derived sizes, the
safetensors reader the converter is built on, and the section checksum (the reference's tests/test_zse_format.py and
test_convert_pipeline.py cover the same ground on its side)."""
import json
import struct
import zlib

import numpy as np
import pytest

from zse_b200.format import synth
from zse_b200.format.arch.base import (ArchAdapter, detect_architecture, get_adapter, register_adapter, rope_settings,
                                       supported_architectures)
from zse_b200.format.convert import (build_tensor_map, find_safetensor_files, read_safetensors_metadata,
                                     read_safetensors_tensor, read_safetensors_tensor_raw, write_safetensors)
from zse_b200.format.header import compute_crc32


# ---- architecture detection and registry ------------------------------------------------------------------------
@pytest.mark.parametrize("architectures,model_type,want", [
    (["LlamaForCausalLM"], "llama", "llama"),
    (["MistralForCausalLM"], "mistral", "mistral"),
    (["Qwen2ForCausalLM"], "qwen2", "qwen2"),
    (["Phi3ForCausalLM"], "phi3", "phi3"),
    (["Gemma2ForCausalLM"], "gemma2", "gemma2"),
    (["Gemma4ForConditionalGeneration"], "gemma4", "gemma4"),       # "gemma4" is tested before the plain "gemma"
    (None, "qwen2", "qwen2"),                                       # no class name: the model type decides
    ([], "llama", "llama"),
])
def test_architecture_is_detected_from_class_name_or_model_type(architectures, model_type, want):
    assert detect_architecture({"architectures": architectures, "model_type": model_type}) == want


def test_unknown_architectures_are_refused_with_what_was_seen():
    with pytest.raises(ValueError, match="cannot detect the architecture.*BertModel.*bert"):
        detect_architecture({"architectures": ["BertModel"], "model_type": "bert"})
    with pytest.raises(ValueError, match="unknown architecture 'bert'; supported: .*llama"):
        get_adapter("bert")
    assert {"llama", "mistral", "qwen2", "phi3", "gemma2", "gemma4"} <= set(supported_architectures())
    assert supported_architectures() == sorted(supported_architectures())
    assert get_adapter("qwen2").ARCH_NAME == "qwen2"


def test_an_adapter_registered_by_a_user_is_found(monkeypatch):
    from zse_b200.format.arch import base
    monkeypatch.setattr(base, "_REGISTRY", dict(base._REGISTRY))           # leave the real registry alone

    @register_adapter
    class Mine(ArchAdapter):
        ARCH_NAME = "my-arch"

    assert "my-arch" in supported_architectures() and isinstance(get_adapter("my-arch"), Mine)
    assert detect_architecture({"model_type": "my-arch"}) == "my-arch"


# ---- RoPE settings ----------------------------------------------------------------------------------------------
def test_rope_settings_in_both_spellings():
    assert rope_settings({}, 10000.0) == (10000.0, None)
    assert rope_settings({"rope_theta": 1e6}, 10000.0) == (1e6, None)
    llama3 = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
              "original_max_position_embeddings": 8192}
    theta, scaling = rope_settings({"rope_theta": 5e5, "rope_scaling": llama3}, 10000.0)
    assert theta == 5e5 and scaling == llama3
    # transformers 5: base and scaling parameters together under rope_parameters
    theta, scaling = rope_settings({"rope_parameters": {"rope_theta": 5e5, **llama3}}, 10000.0)
    assert theta == 5e5 and scaling == llama3
    assert rope_settings({"rope_parameters": {"rope_theta": 1e6, "rope_type": "default"}}, 1.0) == (1e6, None)
    assert rope_settings({"rope_scaling": {"type": "linear", "factor": 2.0}}, 7.0) == (7.0, {"type": "linear", "factor": 2.0})
    assert rope_settings({"rope_scaling": {"type": "default"}}, 7.0) == (7.0, None)


# ---- tensor names, quantisation, load order ---------------------------------------------------------------------
def test_tensor_names_lose_their_model_prefix_and_norms_stay_fp16():
    a = get_adapter("llama")
    assert a.map_tensor_name("model.layers.3.self_attn.q_proj.weight") == "layers.3.self_attn.q_proj.weight"
    assert a.map_tensor_name("lm_head.weight") == "lm_head.weight"
    assert a.should_quantize("layers.0.self_attn.q_proj.weight") and a.should_quantize("layers.0.mlp.down_proj.weight")
    for keep in ("embed_tokens.weight", "norm.weight", "layers.0.input_layernorm.weight",
                 "layers.0.self_attn.q_proj.bias"):
        assert not a.should_quantize(keep), keep
    assert a.tensor_load_order(["b", "a", "c"]) == ["a", "b", "c"]
    assert a.tensor_load_order(tensor_names=["z", "y"]) == ["y", "z"]


def test_expected_tensors_follow_the_config():
    c = synth.shape_config("tiny")
    a = get_adapter(c.arch)
    names = a.expected_tensors(c)
    assert names[0] == "embed_tokens.weight" and "norm.weight" in names
    assert ("lm_head.weight" in names) == (not c.tie_word_embeddings)
    per_layer = a.layer_tensors(c, 0)
    assert {"self_attn.q_proj.weight", "self_attn.o_proj.weight", "mlp.gate_proj.weight", "mlp.down_proj.weight",
            "input_layernorm.weight"} <= set(per_layer)
    assert sum(n.startswith("layers.1.") for n in names) == len(per_layer)
    g4 = synth.shape_config("tiny-gemma4")
    ga = get_adapter("gemma4")
    assert not ga.should_quantize("layers.0.self_attn.q_norm.weight")
    assert any("q_norm" in t for t in ga.layer_tensors(g4, 0))


def test_config_validation_warns_instead_of_failing():
    import dataclasses
    c = synth.shape_config("tiny")
    a = get_adapter(c.arch)
    assert a.validate_config(c) == [] and a.validate_config(config=c) == []
    odd = dataclasses.replace(c, num_heads=c.num_heads + 1)
    w = a.validate_config(odd)
    assert any("not divisible by num_heads" in x for x in w) and any("not divisible by num_kv_heads" in x for x in w)
    yarn = dataclasses.replace(c, rope_scaling={"rope_type": "yarn", "factor": 4.0})
    assert any("'yarn' is not applied" in x for x in a.validate_config(yarn))
    for kind in ("linear", "llama3", "default"):
        assert a.validate_config(dataclasses.replace(c, rope_scaling={"rope_type": kind, "factor": 2.0})) == []


# ---- config-derived sizes ---------------------------------------------------------------------------------------
def test_cache_bytes_and_parameter_counts_of_the_7b_shape():
    c = synth.shape_config("qwen2.5-7b")
    assert c.kv_head_dim == c.head_dim == 128 and not c.is_gemma and c.layer_kind(5) == "full_attention"
    assert c.kv_cache_bytes_per_token == 2 * c.num_kv_heads * 128 * 2 == 2048
    assert c.total_kv_cache_bytes_per_token == 2048 * c.num_layers
    q, kv, H, I = c.num_heads * 128, c.num_kv_heads * 128, c.hidden_size, c.intermediate_size
    assert c.linear_param_count() == c.num_layers * (H * q + 2 * H * kv + q * H + 3 * H * I)
    size = c.estimate_model_size_bytes()
    params = c.linear_param_count()
    # INT4 with groups of 128: half a byte per weight + 4 bytes of scale and zero per group + fp16 embeddings and norms
    assert size == params // 2 + (params // 128) * 4 + c.vocab_size * H * 2 * (1 if c.tie_word_embeddings else 2) \
        + c.num_layers * H * 2 * 2
    assert 4.5e9 < size < 6.5e9                                                 # ~5.5 GB: the published file size
    g = synth.shape_config("tiny-gemma2")
    assert g.is_gemma and {g.layer_kind(i) for i in range(g.num_layers)} <= {"full_attention", "sliding_attention"}


# ---- the safetensors reader -------------------------------------------------------------------------------------
def test_safetensors_round_trip_in_three_element_types(tmp_path):
    rng = np.random.default_rng(0)
    a32 = rng.standard_normal((4, 6)).astype(np.float32)
    a16 = rng.standard_normal((3, 5)).astype(np.float16)
    path = str(tmp_path / "m.safetensors")
    write_safetensors(path, {"a32": a32, "a16": a16})
    meta, base = read_safetensors_metadata(path)
    (n,) = struct.unpack("<Q", open(path, "rb").read(8))
    assert base == 8 + n and set(meta) - {"__metadata__"} == {"a32", "a16"}
    assert meta["a32"]["dtype"] == "F32" and meta["a32"]["shape"] == [4, 6] and meta["a16"]["dtype"] == "F16"
    raw, dtype, shape = read_safetensors_tensor_raw(path, meta["a16"], base)
    assert (dtype, shape) == ("F16", (3, 5)) and raw == a16.tobytes()
    got, shape = read_safetensors_tensor(path, meta["a32"], base)
    assert shape == (4, 6) and got.dtype == np.float32 and np.array_equal(got.reshape(4, 6), a32)
    got16, _ = read_safetensors_tensor(path, meta["a16"], base)
    assert np.array_equal(got16.reshape(3, 5), a16.astype(np.float32))
    # bfloat16 files: the upper half of the float32 pattern
    bpath = str(tmp_path / "b.safetensors")
    write_safetensors(bpath, {"w": a32}, bf16=True)
    bmeta, bbase = read_safetensors_metadata(bpath)
    assert bmeta["w"]["dtype"] == "BF16"
    back, _ = read_safetensors_tensor(bpath, bmeta["w"], bbase)
    assert np.abs(back.reshape(4, 6) - a32).max() < 0.02 and np.all((back.view(np.uint32) & 0xFFFF) == 0)
    with pytest.raises(ValueError, match="unsupported safetensors dtype"):
        read_safetensors_tensor(path, {**meta["a32"], "dtype": "F8_E4M3"}, base)


def test_shards_are_found_in_order_and_mapped_by_tensor_name(tmp_path):
    with pytest.raises(FileNotFoundError, match="no .safetensors files"):
        find_safetensor_files(str(tmp_path))
    one = np.ones((2, 2), dtype=np.float32)
    write_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), {"b": one * 2})
    write_safetensors(str(tmp_path / "model-00001-of-00002.safetensors"), {"a": one, "c": one * 3})
    (tmp_path / "config.json").write_text("{}")
    files = find_safetensor_files(str(tmp_path))
    assert [f.rsplit("/", 1)[1] for f in files] == ["model-00001-of-00002.safetensors", "model-00002-of-00002.safetensors"]
    tmap = build_tensor_map(files)
    assert set(tmap) == {"a", "b", "c"} and tmap["b"][0] == files[1] and tmap["c"][0] == files[0]
    path, info, base = tmap["c"]
    got, shape = read_safetensors_tensor(path, info, base)
    assert shape == (2, 2) and np.all(got == 3.0)


# ---- checksums --------------------------------------------------------------------------------------------------
def test_section_checksum_is_crc32():
    assert compute_crc32(b"") == 0
    assert compute_crc32(b"123456789") == 0xCBF43926                            # the standard check value
    data = bytes(range(256)) * 10
    assert compute_crc32(data) == zlib.crc32(data) & 0xFFFFFFFF == compute_crc32(memoryview(data))


# ---- raw-bytes quantiser entry points and alignment helpers ---------------------------------------------------------
def test_raw_bytes_entry_points_follow_the_array_quantiser():
    import numpy as np
    from zse_b200.format import fast_quant
    from zse_b200.format import quantize as Q
    rng = np.random.default_rng(3)
    w = rng.standard_normal(300).astype(np.float32)                               # 2 full groups and a tail of 44
    vals, scales = fast_quant.quantize_tensor_int8_fast(w.tobytes() + b"junk-after-the-tensor", "F32", 300)
    v2, s2 = Q.quantize_int8_arrays(w, 128)
    assert vals == np.asarray(v2).tobytes() and scales == np.asarray(s2).tobytes()
    back = Q.dequantize_tensor_int8(np.frombuffer(vals, np.int8), np.frombuffer(scales, np.float16), (300,))
    assert np.abs(back - w).max() <= np.abs(w).max() / 127 * 0.51 + 1e-3
    p, s, z = fast_quant.quantize_tensor_fast(w.astype(np.float16).tobytes(), "F16", 300)
    p2, s2, z2 = Q.quantize_int4_arrays(w.astype(np.float16).astype(np.float32), 128)
    assert (p, s, z) == (np.asarray(p2).tobytes(), np.asarray(s2).tobytes(), np.asarray(z2).tobytes())
    assert len(p) == Q.compute_packed_size(300)[0] and len(s) == len(z) == Q.compute_packed_size(300)[1]


def test_fp16_conversion_of_each_source_type():
    import numpy as np
    from zse_b200.format import fast_quant
    from zse_b200.format.quantize import quantize_fp16
    w = np.array([1.0, -2.5, 0.333251953125, 1000.0], dtype=np.float32)           # all exact in fp16 and in bf16's range
    want = w.astype(np.float16).tobytes()
    assert fast_quant.convert_to_fp16_fast(w.tobytes(), "F32", 4) == want == quantize_fp16(w)
    assert fast_quant.convert_to_fp16_fast(w.astype(np.float64).tobytes(), "F64", 4) == want
    assert fast_quant.convert_to_fp16_fast(want + b"\0\0", "F16", 4) == want      # fp16 passes through, cut to size
    bf = (w.view(np.uint32) >> 16).astype(np.uint16)                              # truncated bfloat16
    got = np.frombuffer(fast_quant.convert_to_fp16_fast(bf.tobytes(), "BF16", 4), np.float16)
    assert got.tolist()[:2] == [1.0, -2.5] and got[3] == 1000.0
    assert abs(float(got[2]) - 0.3333) < 2e-3                                     # bf16 kept 8 bits of it
    assert fast_quant.convert_to_fp16_fast(w.tobytes(), "F32", 2) == want[:4]


def test_repack_to_the_64_by_8_tiles_places_each_byte():
    import numpy as np
    from zse_b200.format import fast_quant
    from zse_b200.format.quantize import untile_int4_64x8
    n, k = 70, 48                                                                 # 2 row tiles (one ragged), 3 k tiles
    raw = (np.arange(n * k // 2) % 251).astype(np.uint8)
    t = np.frombuffer(fast_quant.repack_int4_tiled(raw.tobytes(), n, k), np.uint8)
    assert t.size == 2 * 3 * 64 * 8
    tiles = t.reshape(2, 3, 64, 8)
    src = raw.reshape(n, k // 2)
    assert (tiles[0, 1, 5] == src[5, 8:16]).all() and (tiles[1, 2, 3] == src[67, 16:24]).all()
    assert tiles[1, :, 6:].sum() == 0                                             # rows 70..127 are padding
    assert (untile_int4_64x8(t, n, k) == raw).all()


def test_alignment_helpers():
    from zse_b200.format.spec import align_offset, align_up, pad_to_alignment
    assert [align_up(x, 64) for x in (0, 1, 63, 64, 65)] == [0, 64, 64, 64, 128]
    assert align_offset(4097, 4096) == align_up(4097, 4096) == 8192
    assert pad_to_alignment(64, 64) == b"" and pad_to_alignment(60, 64) == b"\0" * 4
    assert len(pad_to_alignment(1, 4096)) == 4095


# ---- writer and loader: raw appends and typed views ------------------------------------------------------------------
def test_raw_appends_come_back_through_the_typed_views(tmp_path):
    import numpy as np
    from zse_b200.format import ZSELoader, ZSEWriter, synth
    from zse_b200.format import quantize as Q
    from zse_b200.format.spec import Flags
    rng = np.random.default_rng(11)
    w4 = rng.standard_normal((8, 128)).astype(np.float32)
    w8 = rng.standard_normal((4, 128)).astype(np.float32)
    wf = rng.standard_normal((3, 5)).astype(np.float16)
    path = str(tmp_path / "raw.zse")
    with ZSEWriter(path) as wr:
        wr.set_config(synth.shape_config("tiny"))
        wr.set_tokenizer(b"")                                                     # an empty tokenizer section is legal
        wr.begin_weights()
        p, s, z = Q.quantize_int4_arrays(w4, 128)
        wr.add_weight_raw("a.weight", w4.shape, p, s, z)
        q8, s8 = Q.quantize_int8_arrays(w8, 128)
        wr.add_weight_raw_int8("b.weight", w8.shape, q8, s8)
        wr.add_weight_raw_fp16("c.weight", wf.shape, wf)
    with ZSELoader(path) as l:
        assert l.header.flags & Flags.HAS_TOKENIZER and l.file_descriptor >= 0
        ea, eb, ec = (l.weight_index.find(n) for n in ("a.weight", "b.weight", "c.weight"))
        assert (ea.dtype, eb.dtype, ec.dtype) == ("int4", "int8", "float16")
        assert all(e.data_offset % 64 == 0 for e in (ea, eb, ec))                 # every tensor starts aligned
        assert ea.end_offset <= eb.data_offset and eb.end_offset <= ec.data_offset
        assert l.view_data(ea).dtype == np.uint8 and (l.view_data(ea) == np.asarray(p).reshape(-1)).all()
        assert (l.int4_rowmajor(ea) == l.view_data(ea)).all()
        assert (l.view_scales(ea) == np.asarray(s)).all() and (l.view_zeros(ea) == np.asarray(z)).all()
        assert l.view_data(eb).dtype == np.int8 and (l.view_data(eb) == np.asarray(q8).reshape(-1)).all()
        assert (l.view_scales(eb) == np.asarray(s8)).all() and l.get_weight_zeros(eb) == b""
        assert l.view_data(ec).shape == (3, 5) and (l.view_data(ec) == wf).all()
        assert l.get_weight_scales(ec) == b"" and l.get_weight_data(ec) == wf.tobytes()
        mm, off = l.get_mmap_pointer_and_offset(ec)
        assert bytes(mm[off:off + ec.data_nbytes]) == wf.tobytes()                # an absolute file offset
        assert off == l.weight_data_section()[0] + ec.data_offset
        assert np.abs(l.get_weight_as_float(ea) - w4).max() < 0.3 and np.abs(l.get_weight_as_float(eb) - w8).max() < 0.03
        assert "int4: 1" in l.summary() and "int8: 1" in l.summary() and "float16: 1" in l.summary()
    assert l.file_descriptor == -1                                                 # closed


def test_an_aborted_writer_leaves_no_readable_file(tmp_path):
    import numpy as np
    from zse_b200.format import ZSELoader, ZSEWriter, synth
    path = str(tmp_path / "cut.zse")
    with pytest.raises(RuntimeError, match="stop"):
        with ZSEWriter(path) as wr:
            wr.set_config(synth.shape_config("tiny"))
            wr.begin_weights()
            wr.add_weight("x.weight", np.ones((2, 128), np.float32), (2, 128))
            raise RuntimeError("stop")
    wr.finalize()                                                                  # after abort: nothing more is written
    with pytest.raises(ValueError):
        ZSELoader(path)                                                            # the header was never filled in
    with pytest.raises(ValueError, match="set_config"):
        ZSEWriter(str(tmp_path / "early.zse")).begin_weights()
    (tmp_path / "empty.zse").write_bytes(b"")
    with pytest.raises(ValueError, match="empty"):
        ZSELoader(str(tmp_path / "empty.zse"))

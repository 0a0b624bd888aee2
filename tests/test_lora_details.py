"""Unit tests of the LoRA bookkeeping and of the ``.zse-lora`` file format (the shape of the reference's
tests/test_lora.py: weights, adapter, store, file round trip).  What an adapter does to a model's outputs is covered by
tests/test_convert_tp_lora.py."""
import struct

import numpy as np
import pytest
import torch

from zse_b200.format import synth
from zse_b200.format.lora_format import (LORA_MAGIC, LORA_VERSION, TARGET_NAME_SIZE, estimate_lora_size, load_lora,
                                         module_shapes, read_lora_header, save_lora)
from zse_b200.lora.weights import LoRAAdapter, LoRAWeight, LoRAWeightStore, random_adapter_file


# ---- one weight pair --------------------------------------------------------------------------------------------
def test_weight_pair_geometry_and_sizes():
    w = LoRAWeight("model.layers.0.q_proj", rank=8, in_features=64, out_features=96)
    assert w.a_shape == (8, 64) and w.b_shape == (96, 8)
    assert w.nbytes == 2 * 8 * (64 + 96) == w.total_gpu_bytes
    assert not w.loaded and w.a_ptr == 0 and w.b_ptr == 0 and w.a_nbytes == 0 and w.b_nbytes == 0
    w.a = torch.zeros(8, 64, dtype=torch.float16)
    assert not w.loaded                                   # both halves are needed
    w.b = torch.zeros(96, 8, dtype=torch.float16)
    assert w.loaded and w.a_ptr == w.a.data_ptr() and w.b_ptr == w.b.data_ptr()
    assert w.a_nbytes == 8 * 64 * 2 and w.b_nbytes == 96 * 8 * 2 and w.a_nbytes + w.b_nbytes == w.nbytes
    assert w.make_a_tensor() is w.a and w.make_b_tensor() is w.b


# ---- an adapter -------------------------------------------------------------------------------------------------
def _adapter(aid="ad", rank=4, layers=2, targets=("q_proj", "v_proj"), fin=32, fout=48):
    ad = LoRAAdapter(aid, rank, 8.0, list(targets), layers)
    for layer in range(layers):
        for t in targets:
            ad.add_weight(layer, t, LoRAWeight(f"model.layers.{layer}.{t}", rank, fin, fout))
    return ad


def test_adapter_lookup_scaling_and_totals():
    ad = _adapter()
    assert ad.scaling == 2.0 and LoRAAdapter("z", 0, 8.0, [], 0).scaling == 0.0
    assert ad.has_module("q_proj") and not ad.has_module("o_proj")
    assert ad.has_weight(1, "v_proj") and not ad.has_weight(2, "v_proj") and not ad.has_weight(0, "k_proj")
    assert ad.get_weight(0, "q_proj").layer_name == "model.layers.0.q_proj" and ad.get_weight(5, "q_proj") is None
    assert ad.num_weight_pairs == 4
    assert ad.total_bytes == 4 * 2 * 4 * (32 + 48) == ad.total_gpu_bytes
    assert ad.slot == -1 and ad.generation == 0 and ad.base_model == "" and ad.description == ""
    s = ad.summary()
    assert "'ad'" in s and "rank 4" in s and "q_proj, v_proj" in s and "4 weight pairs" in s and "2.000" in s
    ad.add_weight(0, "q_proj", LoRAWeight("again", 4, 32, 48))           # replacing a pair does not add one
    assert ad.num_weight_pairs == 4 and ad.get_weight(0, "q_proj").layer_name == "again"


# ---- the store --------------------------------------------------------------------------------------------------
def test_store_add_get_remove_and_names():
    st = LoRAWeightStore()
    a, b = _adapter("a"), _adapter("b", rank=8)
    st.add(a)
    st.add(b)
    assert len(st) == 2 == st.num_adapters and "a" in st and st.has("b") and not st.has("c") and "c" not in st
    assert st.get("a") is a and st.get("c") is None
    assert st.list_ids() == ["a", "b"] == st.list_adapters()
    assert st.total_bytes == a.total_bytes + b.total_bytes == st.total_gpu_bytes
    with pytest.raises(ValueError):
        st.add(_adapter("a"))                                              # ids are unique
    assert st.remove("a") is a and st.remove("a") is None
    assert st.list_ids() == ["b"] and st.total_bytes == b.total_bytes
    text = st.summary()
    assert text.splitlines()[0].startswith("LoRA store: 1 adapters") and "'b'" in text
    assert LoRAWeightStore().summary().startswith("LoRA store: 0 adapters")


def test_store_budget():
    one = _adapter("x").total_bytes
    st = LoRAWeightStore(max_bytes=2 * one)
    st.add(_adapter("x"))
    st.add(_adapter("y"))
    with pytest.raises(MemoryError):
        st.add(_adapter("z"))
    assert st.list_ids() == ["x", "y"]                                      # the refused adapter left no trace
    st.remove("x")
    st.add(_adapter("z"))
    assert LoRAWeightStore(max_bytes=0).max_bytes == 0                      # 0 = no budget
    big = LoRAWeightStore()
    for i in range(40):
        big.add(_adapter(f"a{i}"))
    assert len(big) == 40


# ---- shapes and size estimates ----------------------------------------------------------------------------------
def test_module_shapes_follow_the_attention_geometry():
    s = module_shapes(hidden_size=512, intermediate_size=1024, num_heads=8, num_kv_heads=2, head_dim=64)
    assert s["q_proj"] == (512, 512) and s["k_proj"] == (512, 128) == s["v_proj"] and s["o_proj"] == (512, 512)
    assert s["gate_proj"] == (512, 1024) == s["up_proj"] and s["down_proj"] == (1024, 512)
    assert set(module_shapes(512)) == {"q_proj", "k_proj", "v_proj", "o_proj"}         # no MLP without its width
    wide = module_shapes(hidden_size=256, num_heads=4, num_kv_heads=4, head_dim=128)   # heads wider than hidden / heads
    assert wide["q_proj"] == (256, 512) and wide["o_proj"] == (512, 256)


def test_size_estimate_equals_what_a_file_holds(tmp_path):
    cfg = synth.shape_config("tiny")
    targets = ["q_proj", "o_proj", "down_proj"]
    path = str(tmp_path / "a.zse-lora")
    ad = random_adapter_file(path, cfg, rank=4, alpha=8.0, target_modules=targets, seed=1)
    want = estimate_lora_size(4, cfg.num_layers, targets, cfg.hidden_size, cfg.intermediate_size, cfg.num_heads,
                              cfg.num_kv_heads, cfg.head_dim)
    h = read_lora_header(path)
    assert h["total_bytes"] == want == ad.total_bytes
    assert estimate_lora_size(4, 2, ["not_a_module"], 64) == 0
    assert estimate_lora_size(8, 3, ["q_proj"], 64, num_heads=2, num_kv_heads=2, head_dim=32) == 3 * 8 * (64 + 64) * 2


# ---- the file format --------------------------------------------------------------------------------------------
def _save(tmp_path, rank=4, layers=2, targets=("q_proj", "v_proj"), shapes=None, seed=0, name="x.zse-lora"):
    shapes = shapes or {"q_proj": (32, 48), "v_proj": (32, 16)}
    rng = np.random.default_rng(seed)
    ad = LoRAAdapter("", rank, 6.0, list(targets), layers)
    data = {}
    for layer in range(layers):
        for t in targets:
            fin, fout = shapes[t]
            data[(layer, t)] = (rng.standard_normal((rank, fin)).astype(np.float16),
                                rng.standard_normal((fout, rank)).astype(np.float16))
    path = str(tmp_path / name)
    save_lora(path, ad, data)
    return path, ad, data, shapes


def test_header_layout_on_disk(tmp_path):
    path, ad, data, shapes = _save(tmp_path)
    raw = open(path, "rb").read()
    magic, version, rank, alpha, layers, ntargets, total = struct.unpack_from("<4sIIfIIQ", raw, 0)
    assert (magic, version, rank, alpha, layers, ntargets) == (LORA_MAGIC, LORA_VERSION, 4, 6.0, 2, 2)
    assert struct.calcsize("<4sIIfIIQ") == 32
    names = [raw[32 + i * TARGET_NAME_SIZE: 32 + (i + 1) * TARGET_NAME_SIZE] for i in range(2)]
    assert names[0] == b"q_proj".ljust(64, b"\x00") and names[1].rstrip(b"\x00") == b"v_proj"
    body = len(raw) - 32 - 2 * 64
    assert total == body == sum(a.nbytes + b.nbytes for a, b in data.values())
    # weights follow in layer order, targets in header order, A before B
    first_a = np.frombuffer(raw, dtype=np.float16, count=4 * 32, offset=32 + 128).reshape(4, 32)
    assert np.array_equal(first_a, data[(0, "q_proj")][0])


def test_round_trip_returns_the_same_bytes(tmp_path):
    path, _, data, shapes = _save(tmp_path, seed=3)
    h = read_lora_header(path)
    assert h == {"rank": 4, "alpha": 6.0, "num_layers": 2, "targets": ["q_proj", "v_proj"],
                 "total_bytes": h["total_bytes"], "data_offset": 32 + 2 * 64}
    ad, got = load_lora(path, shapes)
    assert ad.rank == 4 and ad.alpha == 6.0 and ad.num_layers == 2 and ad.target_modules == ["q_proj", "v_proj"]
    assert ad.adapter_id == "" and ad.num_weight_pairs == 4 and set(got) == set(data)
    for key, (a, b) in data.items():
        assert got[key] == (a.tobytes(), b.tobytes())
        w = ad.get_weight(*key)
        assert (w.in_features, w.out_features) == shapes[key[1]] and w.rank == 4
        assert w.layer_name == f"model.layers.{key[0]}.{key[1]}"


def test_save_accepts_bytes_arrays_and_tensors(tmp_path):
    a = np.arange(4 * 8, dtype=np.float32).reshape(4, 8) / 8
    b = np.arange(6 * 4, dtype=np.float32).reshape(6, 4) / 4
    ad = LoRAAdapter("", 4, 4.0, ["q_proj"], 3)
    forms = {(0, "q_proj"): (a.astype(np.float16).tobytes(), b.astype(np.float16).tobytes()),
             (1, "q_proj"): (a, b),                                                     # fp32 arrays are narrowed
             (2, "q_proj"): (torch.from_numpy(a).double(), torch.from_numpy(b).half())}
    path = str(tmp_path / "forms.zse-lora")
    save_lora(path, ad, forms)
    _, got = load_lora(path, {"q_proj": (8, 6)})
    want = (a.astype(np.float16).tobytes(), b.astype(np.float16).tobytes())
    assert got[(0, "q_proj")] == got[(1, "q_proj")] == got[(2, "q_proj")] == want


def test_long_and_unicode_target_names_are_cut_to_their_field(tmp_path):
    long_name = "m" * 80
    ad = LoRAAdapter("", 2, 2.0, [long_name], 1)
    path = str(tmp_path / "n.zse-lora")
    save_lora(path, ad, {})
    assert read_lora_header(path)["targets"] == ["m" * 63]                              # 63 bytes + the terminating NUL


def test_bad_files_are_refused(tmp_path):
    path, _, data, shapes = _save(tmp_path)
    raw = open(path, "rb").read()
    bad_magic = tmp_path / "magic.zse-lora"
    bad_magic.write_bytes(b"NOPE" + raw[4:])
    with pytest.raises(ValueError, match="bad magic"):
        read_lora_header(str(bad_magic))
    bad_version = tmp_path / "version.zse-lora"
    bad_version.write_bytes(raw[:4] + struct.pack("<I", 9) + raw[8:])
    with pytest.raises(ValueError, match="version 9"):
        read_lora_header(str(bad_version))
    short = tmp_path / "short.zse-lora"
    short.write_bytes(raw[:10])
    with pytest.raises(ValueError):
        read_lora_header(str(short))
    cut = tmp_path / "cut.zse-lora"
    cut.write_bytes(raw[:-10])
    with pytest.raises(ValueError, match="truncated .zse-lora at layer 1, v_proj"):
        load_lora(str(cut), shapes)
    with pytest.raises(FileNotFoundError):
        read_lora_header(str(tmp_path / "missing.zse-lora"))


def test_targets_the_model_does_not_have_are_skipped(tmp_path):
    path, _, data, shapes = _save(tmp_path, targets=("q_proj",), shapes={"q_proj": (32, 48)})
    ad, got = load_lora(path, {"k_proj": (32, 16)})
    assert got == {} and ad.num_weight_pairs == 0 and ad.target_modules == ["q_proj"]


def test_random_adapter_file_is_deterministic_and_shaped_by_the_model(tmp_path):
    cfg = synth.shape_config("tiny")
    p1, p2, p3 = (str(tmp_path / n) for n in ("a", "b", "c"))
    ad = random_adapter_file(p1, cfg, rank=8, alpha=16.0, seed=5)
    random_adapter_file(p2, cfg, rank=8, alpha=16.0, seed=5)
    random_adapter_file(p3, cfg, rank=8, alpha=16.0, seed=6)
    assert open(p1, "rb").read() == open(p2, "rb").read() != open(p3, "rb").read()
    assert ad.target_modules == ["q_proj", "k_proj", "v_proj"] and ad.num_layers == cfg.num_layers
    shapes = module_shapes(cfg.hidden_size, cfg.intermediate_size, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim)
    loaded, got = load_lora(p1, shapes)
    assert loaded.num_weight_pairs == 3 * cfg.num_layers
    a, b = got[(0, "k_proj")]
    A = np.frombuffer(a, dtype=np.float16).reshape(8, shapes["k_proj"][0]).astype(np.float32)
    assert 0.02 < A.std() < 0.08 and len(b) == shapes["k_proj"][1] * 8 * 2                 # N(0, 0.05)

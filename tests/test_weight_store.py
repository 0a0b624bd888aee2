"""Name-based weight stores (whole model and per-rank shards), the kernel registry, scratch-buffer and memory
accounting, and the graph wrapper: the reference's orchestrator classes that callers may use directly."""
import numpy as np
import pytest
import torch

from zse_b200.format.loader import ZSELoader
from zse_b200.format.synth import shape_config, write_random_model
from zse_b200.parallel.shard_plan import make_plan
from zse_b200.parallel.tp_weight_loader import TPWeightLoader
from zse_b200.runtime.weight_stream import GPUWeight, WeightLoader, WeightStore


def _model(tmp_path, shape, **kw):
    path = str(tmp_path / f"{shape}.zse")
    write_random_model(path, shape_config(shape, **kw), seed=3)
    return ZSELoader(path)


def test_weight_loader_mirrors_every_tensor(tmp_path):
    loader = _model(tmp_path, "tiny")
    seen = []
    wl = WeightLoader(loader, "cpu")
    store = wl.load_all(lambda name, i, n: seen.append((name, i, n)))
    assert isinstance(store, WeightStore) and store.num_weights == len(loader.weight_index) == len(seen)
    assert seen[-1][1] == seen[-1][2] == store.num_weights
    total = 0
    for e in loader.weight_index:
        w = store.get(e.name)
        assert isinstance(w, GPUWeight) and store.has("model." + e.name) and e.name in store
        assert (w.data_nbytes, w.scales_nbytes, w.zeros_nbytes) == (e.data_nbytes, e.scale_nbytes, e.zeros_nbytes)
        assert w.data_ptr != 0 and w.num_elements == e.num_elements
        total += w.total_gpu_bytes
        np.testing.assert_allclose(w.to_float().numpy(), loader.get_weight_as_float(e).reshape(e.shape), atol=1e-6)
    assert store.total_bytes == total and store.find("nope") is None
    assert "tensors" in store.summary()
    with pytest.raises(KeyError):
        store.get("nope")
    store.destroy()
    assert store.num_weights == 0 and store.total_bytes == 0


@pytest.mark.parametrize("shape", ["tiny", "tiny-aligned", "tiny-phi3", "tiny-gemma2"])
def test_tp_weight_loader_shards_reassemble(tmp_path, shape):
    try:
        loader = _model(tmp_path, shape)
    except (KeyError, ValueError):
        pytest.skip(f"no synthetic shape {shape}")
    c = loader.config
    tp = 2
    stores = [TPWeightLoader(loader, "cpu", make_plan(c, tp, r)).load_all() for r in range(tp)]
    tpl = [TPWeightLoader(loader, "cpu", make_plan(c, tp, r)) for r in range(tp)]
    checked = 0
    for e in loader.weight_index:
        full = torch.from_numpy(np.asarray(loader.get_weight_as_float(e), np.float32).reshape(e.shape))
        shards = [s.get(e.name).to_float() for s in stores]
        stacked = tpl[0].stacked_row_ranges(e.name)
        rows, cols = tpl[0].shard_ranges(e.name)
        if stacked is not None:
            for r in range(tp):
                want = torch.cat([full[a:b] for a, b in tpl[r].stacked_row_ranges(e.name)])
                torch.testing.assert_close(shards[r], want, atol=2e-3, rtol=0)
            checked += 1
        elif rows is not None:
            torch.testing.assert_close(torch.cat(shards, 0), full, atol=2e-3, rtol=0)
            checked += 1
        elif cols is not None:
            torch.testing.assert_close(torch.cat(shards, 1), full, atol=2e-3, rtol=0)
            checked += 1
        else:
            for s in shards:
                torch.testing.assert_close(s, full, atol=2e-3, rtol=0)
    assert checked >= 4 * c.num_layers - 1
    assert stores[0].total_bytes < WeightLoader(loader, "cpu").load_all().total_bytes


def test_kernel_registry_names():
    from zse_b200.ops import native
    from zse_b200.ops.registry import ESSENTIAL, KERNEL_TABLE, InferenceKernels
    k = InferenceKernels()
    assert len(k.kernel_names) == len(KERNEL_TABLE) >= 32
    for name, (entry, _) in KERNEL_TABLE.items():
        assert callable(getattr(native, entry)), (name, entry)
    for names in ESSENTIAL.values():
        assert set(names) <= set(KERNEL_TABLE)
    assert not k.is_compiled("paged_attention")
    assert k.get("paged_attention") is native.attn_decode and k.is_compiled("paged_attention")
    assert k.num_compiled == 1 and "attn_decode" in k.describe("paged_attention")
    with pytest.raises(KeyError):
        k.get("no_such_kernel")
    with pytest.raises(ValueError):
        InferenceKernels("rocm")
    # a launch geometry cannot be imposed on entry points that plan their own: refused, not ignored
    with pytest.raises(ValueError):
        k.launch("paged_attention", (8, 1, 1), (128, 1, 1))
    assert "mma.sync" in k.describe("paged_attention") and "tcgen05.st" in k.describe("tiled_dequant_matmul_int4")


def test_vram_accounting_and_scratch():
    from zse_b200.runtime.vram import GB, ScratchBuffers, VRAMAllocator
    c = shape_config("tiny")
    a = VRAMAllocator(180 * GB)
    assert a.CUDA_CONTEXT_BYTES == 400 << 20 and a.SAFETY_MARGIN_PCT == 0.05
    a.track_weight_upload(1000)
    a.track_weight_upload(24)
    assert a.weight_bytes == 1024 and a.allocated_bytes == 1024
    s = a.allocate_scratch(c, max_seq_len=32)
    assert isinstance(s, ScratchBuffers)
    assert tuple(s.hidden.shape) == (32, c.hidden_size) and s.hidden_f32.dtype == torch.float32
    assert tuple(s.logits.shape) == (32, c.vocab_size)
    assert tuple(s.qkv.shape) == (32, (c.num_heads + 2 * c.num_kv_heads) * c.head_dim)
    assert s.total_bytes == sum(getattr(s, f).numel() * getattr(s, f).element_size() for f in s.FIELDS)
    assert a.allocated_bytes == 1024 + s.total_bytes
    u = a.utilization()
    assert u["weight_bytes"] == 1024 and u["used_bytes"] == a.allocated_bytes
    plan = a.plan_allocation(c, weight_bytes=1 * GB, scratch_bytes=1 * GB, block_size=16, max_seq_len=256,
                             max_batch_seqs=4)
    assert plan.total_vram == 180 * GB and plan.available_vram == 180 * GB - (400 << 20)
    assert plan.max_batch_tokens == plan.kv_blocks * 16 and 0 < plan.utilization_pct < 100
    assert plan.reserved_bytes > 0
    g4 = shape_config("tiny-gemma4")
    widths = VRAMAllocator.scratch_shapes(g4, 8)
    assert widths["attn_out"][0][1] >= max(g4.num_heads * g4.layer_spec(i).head_dim for i in range(g4.num_layers))
    s.destroy()
    assert s.hidden is None


def test_graph_runner_without_gpu():
    from zse_b200.runtime.graph import CUDAGraphRunner
    g = CUDAGraphRunner()
    assert not g.is_captured
    with pytest.raises(RuntimeError):
        g.replay()
    with pytest.raises(RuntimeError):
        g.end_capture()
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            g.begin_capture()
    g.sync()
    g.destroy()


def test_runner_reference_call_forms(tmp_path):
    """decode_step / batched_decode / gpu_argmax / *_graph in the reference's form: the runner extends the cache and
    returns fp16 logits bytes (or the greedy token)."""
    from zse_b200.cache.cache_manager import KVCacheManager
    from zse_b200.models.decoder import DecoderModel
    from zse_b200.models.oracle import OracleModel
    from zse_b200.runtime.runner import ModelRunner, TPModelRunner
    from zse_b200.runtime.step_driver import FastDecoder, NativeStep
    assert FastDecoder is not NativeStep and all(hasattr(FastDecoder, m) for m in ("compile", "available", "setup", "decode_step"))
    loader = _model(tmp_path, "tiny")
    c = loader.config
    oracle = OracleModel(loader)
    model = DecoderModel.from_loader(loader, torch.device("cpu"))
    cache = KVCacheManager(c, num_blocks=32, block_size=16, device=torch.device("cpu"))
    r = TPModelRunner(model, cache, max_batch_seqs=4, max_tokens_per_pass=64, max_seq_len=128)
    assert (r.hidden_size, r.vocab_size, r.tp_size, r.tp_rank) == (c.hidden_size, c.vocab_size, 1, 0)
    r.init_graph(128)
    with pytest.raises(ValueError):
        r.init_graph(100000)
    prompts = {1: [5, 9, 200, 31], 2: [7, 7, 3]}
    for sid, p in prompts.items():
        cache.allocate_sequence(sid, num_tokens=len(p))
    first = r.prefill([(sid, p, 0) for sid, p in prompts.items()])
    want = {sid: oracle.greedy(p, 4) for sid, p in prompts.items()}
    assert [int(t) for t in first] == [want[1][0], want[2][0]]
    # one batched step: logits come back as fp16 bytes, the argmax is the oracle's next token
    rows = r.batched_decode([want[1][0], want[2][0]], [1, 2], [len(prompts[1]), len(prompts[2])])
    assert len(rows) == 2 and all(len(b) == 2 * c.vocab_size for b in rows)
    got = [int(np.frombuffer(b, np.float16).argmax()) for b in rows]
    assert got == [want[1][1], want[2][1]] == [r.gpu_argmax(0), r.gpu_argmax(1)]
    assert cache.num_tokens(1) == len(prompts[1]) + 1
    with pytest.raises(ValueError):
        r.batched_decode([0], [1], [0])                 # a stale position is refused before the cache is touched
    assert cache.num_tokens(1) == len(prompts[1]) + 1
    assert r.batched_decode_graph([want[1][1], want[2][1]], [1, 2]) == [want[1][2], want[2][2]]
    assert r.decode_step_graph(want[1][2], 1, len(prompts[1]) + 2) == want[1][3]
    lg = r.decode_step(want[2][2], 2)
    assert int(np.frombuffer(lg, np.float16).argmax()) == want[2][3]
    assert r.decode_step(want[2][3], 2, skip_logits_download=True) is None
    assert r.precapture_batched_graphs((1, 2)) == 0      # no graphs on the CPU path
    r.destroy_graph()


def test_small_reference_named_accessors(tmp_path):
    """Field and method names of the reference on cache, LoRA, RAG, server and format records."""
    from zse_b200.cache.block_pool import BlockPool
    from zse_b200.cache.cache_manager import KVCacheManager
    from zse_b200.format.arch.base import ArchAdapter, get_adapter
    from zse_b200.lora.manager import LoRAManager
    from zse_b200.models.decoder import DecoderModel
    from zse_b200.rag.store import SearchResult, StoredChunk
    from zse_b200.rag.zpf import compress_csv, compress_json, compress_text
    from zse_b200.server.database import ServerDatabase, UsageRecord
    from zse_b200.server.router import Request, Route
    # block pool addresses follow the layer-major slab
    pool = BlockPool(8, 16, 3, 2, 64, device=torch.device("cpu"))
    a, b = pool.alloc(), pool.alloc()
    per_layer = 2 * 2 * 16 * 64 * 2
    assert pool.layer_block_bytes == per_layer and b.gpu_offset == b.block_id * per_layer
    base = pool.slab.data_ptr()
    assert pool.gpu_ptr_for_block(a) == base + a.block_id * per_layer
    assert pool.gpu_ptr_for_block_layer(b, 2) == pool.slab[2, b.block_id].data_ptr()
    assert pool.gpu_ptr_for_kv(b, 1, True) == pool.slab[1, b.block_id, 1].data_ptr()
    assert pool.is_uniform_kv and pool.layer_kv_elems(0) == 128 and pool.layer_byte_offset(1) == 8 * per_layer
    # attention metadata with device copies
    loader = _model(tmp_path, "tiny")
    c = loader.config
    cache = KVCacheManager(c, num_blocks=16, block_size=16, device=torch.device("cpu"))
    cache.allocate_sequence(1, num_tokens=20)
    md = cache.get_attention_metadata([1], True)
    assert md.block_tables_gpu_ptr != 0 and md.seq_lengths_gpu.tolist() == [20]
    assert cache.get_attention_metadata([1]).block_tables_gpu_ptr == 0
    # LoRA: single-adapter application against the merged update
    model = DecoderModel.from_loader(loader, torch.device("cpu"))
    mgr = LoRAManager(model, torch.device("cpu"))
    ad = mgr.load_adapter_random("r", rank=4, alpha=8.0, target_modules=["q_proj"], seed=1)
    ad.base_model, ad.description = "tiny", "test"
    w = ad.get_weight(0, "q_proj")
    assert w.a_ptr and w.b_ptr and w.a_nbytes > 0 and w.b_nbytes > 0
    x = torch.randn(3, c.hidden_size, dtype=torch.float16)
    out = torch.zeros(3, c.num_heads * c.head_dim, dtype=torch.float16)
    assert mgr.apply_lora(out, x, "r", 0, "q_proj", 3)
    want = 2.0 * (x.float() @ w.a.float().t()) @ w.b.float().t()
    torch.testing.assert_close(out.float(), want, atol=2e-2, rtol=2e-2)
    assert not mgr.apply_lora(out, x, "r", 0, "k_proj", 3)
    # RAG records
    r = SearchResult(1, 2, "d", "text", "text", 0.5, {"chunk_index": 3}, {"bm25": 1.5, "tfidf": 0.25, "dense": 0.75})
    assert (r.bm25_score, r.cosine_score, r.dense_score, r.rerank_score) == (1.5, 0.25, 0.75, None)
    assert isinstance(r.chunk, StoredChunk) and r.chunk.chunk_index == 3 and r.chunk.token_count == 0
    assert compress_text("a  b").doc_type == "text" and compress_json({"a": 1}).doc_type == "json"
    d = compress_csv("a,b\n1,2\n1,3\n1,4\n")
    assert d.doc_type == "csv" and d.original_text.startswith("a,b") and d.compressed_text == d.compressed
    # server records
    db = ServerDatabase(str(tmp_path / "s.db"))
    _, key = db.create_key("k")
    db.record_usage(key.id, 5, 7, "m", None, "req-1", 12.5)
    rec = db.recent_usage(key.id)[0]
    assert isinstance(rec, UsageRecord) and (rec.prompt_tokens, rec.total_tokens, rec.request_id) == (5, 12, "req-1")
    db.close()
    rt = Route("get", "/v1/doc/{id}", None)
    assert rt.match("GET", "/v1/doc/42") == {"id": "42"} and rt.match("POST", "/v1/doc/42") is None
    assert Route("*", "/x", None).match("DELETE", "/x") == {}
    req = Request("GET", "/x", query={"a": "1"}, params={"id": "2"})
    req.api_key = "K"
    assert (req.query_params, req.path_params, req.api_key, req.context["api_key"]) == ({"a": "1"}, {"id": "2"}, "K", "K")
    # arch adapters
    class Renaming(ArchAdapter):
        TENSOR_NAME_MAP = {"transformer.wte.weight": "model.embed_tokens.weight"}
    assert Renaming().map_tensor_name("transformer.wte.weight") == "embed_tokens.weight"
    assert "layers.0.self_attn.qkv_proj.weight" in get_adapter("phi3").expected_tensors(
        shape_config("tiny-phi3"))


def test_package_level_names():
    """What the reference exports from its sub-packages is reachable from the matching ones here."""
    import importlib
    wanted = {
        "zse_b200.format": ["MAGIC", "VERSION", "SectionType", "Flags", "QuantMethod", "FileHeader", "SectionEntry",
                            "read_header_and_sections", "ModelConfig", "QuantConfig", "WeightIndex", "WeightEntry",
                            "quantize_tensor", "dequantize_tensor", "BPETokenizer", "ZSEWriter"],
        "zse_b200.cache": ["BlockPool", "Block", "PageTable", "SequenceEntry", "Evictor", "EvictionCandidate",
                           "BlockDedup", "KVCacheManager", "KVCacheHandle", "CacheStats", "AttentionMetadata",
                           "build_attention_metadata"],
        "zse_b200.sched": ["ZStreamerEngine", "SchedulerConfig", "Scheduler", "MemoryBudget", "RequestQueue",
                           "BatchRunner", "InferenceRequest", "RequestOutput", "GenerationParams", "RequestState",
                           "FinishReason"],
        "zse_b200.server": ["ZSEServer", "ServerDatabase", "AuthManager"],
        "zse_b200.runtime": ["ZSEEngine", "VRAMAllocator", "WeightLoader", "InferenceKernels", "ModelRunner",
                             "CUDAGraphRunner", "FastDecoder"],
        "zse_b200.parallel": ["TensorParallelGroup", "TPConfig", "tp_launch", "TPEngine", "TPWeightLoader",
                              "NcclCommunicator"],
    }
    for mod, names in wanted.items():
        m = importlib.import_module(mod)
        assert not [n for n in names if not hasattr(m, n)], mod
    with pytest.raises(AttributeError):
        importlib.import_module("zse_b200.runtime").NoSuchThing


def test_top_level_names_are_lazy():
    """`import zse_b200` stays cheap (no torch); the main classes resolve on first use."""
    import os
    import subprocess
    import sys
    code = ("import sys, zse_b200; assert 'torch' not in sys.modules; "
            "assert zse_b200.ZSEEngine.__name__ == 'ZSEEngine' and zse_b200.ZStreamerEngine and zse_b200.EngineConfig; "
            "assert 'ZSEServer' in dir(zse_b200)\n"
            "try:\n    zse_b200.not_a_name\nexcept AttributeError:\n    print('ok')")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=240,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0 and r.stdout.strip() == "ok", r.stderr[-1500:]


def test_streamed_load_falls_back_and_says_why(monkeypatch, capsys, tmp_path):
    """`open_mirror`: off for CPU devices and when switched off; a failure of the streamed pass (made up here: the
    mirror's constructor raises) yields None - the caller copies tensor by tensor - with the reason in the load
    statistics, and with ZSE_DEBUG_LOAD=1 also on stderr with the traceback."""
    from zse_b200.runtime import weight_stream as ws
    loader = _model(tmp_path, "tiny")
    assert ws.open_mirror(loader, "cpu") is None
    made = []

    class Broken:
        def __init__(self, loader, device):
            made.append(str(device))
            raise OSError("cannot lock 512 MB of host memory")

    monkeypatch.setattr(ws, "DeviceMirror", Broken)
    monkeypatch.setenv("ZSE_STREAM_WEIGHTS", "0")
    assert ws.open_mirror(loader, "cuda:0") is None and made == []                  # switched off: not even tried
    monkeypatch.setenv("ZSE_STREAM_WEIGHTS", "1")
    stats = {}
    assert ws.open_mirror(loader, "cuda:0", stats) is None and made == ["cuda:0"]
    assert stats == {"stream_error": "cannot lock 512 MB of host memory"}
    assert capsys.readouterr().err == ""                                             # quiet by default
    monkeypatch.setenv("ZSE_DEBUG_LOAD", "1")
    assert ws.open_mirror(loader, "cuda:0") is None
    err = capsys.readouterr().err
    assert "Traceback" in err and "streamed weight load failed (OSError" in err and "tensor by tensor" in err

    class Fine:
        seconds, size = 0.5, 10 ** 9

        def __init__(self, loader, device):
            pass

    monkeypatch.setattr(ws, "DeviceMirror", Fine)
    stats = {}
    assert isinstance(ws.open_mirror(loader, "cuda:0", stats), Fine) and stats == {"stream_s": 0.5, "stream_gbs": 2.0}

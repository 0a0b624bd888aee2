"""Kernel language: parsing, typing, CUDA text (compiled for sm_100a with nvcc, which needs no GPU), fusion, launch
configuration, and the CPU emulation of launches checked against plain torch.  The reference tests its compiler by
generating source for sample kernels (zse-compiler/tests/test_compiler.py, test_gaps.py, test_tier*.py); the emulator
lets these tests check what the kernels compute as well."""
import os

import numpy as np
import pytest
import torch

import zse_b200.dsl as zse

BLOCK = 64


@zse.kernel
def vector_add(a: zse.Tensor, b: zse.Tensor, out: zse.Tensor, n: int):
    i = zse.global_id(0)
    if i < n:
        out[i] = a[i] + b[i]


@zse.kernel
def rmsnorm(x: zse.Tensor, w: zse.Tensor, out: zse.Tensor, n: int, eps: float):
    """One block per row; strided partial sums, then a block reduction every thread receives."""
    row = zse.block_id(0)
    tid = zse.thread_id(0)
    acc = 0.0
    for i in range(tid, n, zse.block_dim(0)):
        v = x[row * n + i]
        acc += v * v
    total = zse.block_reduce_sum(acc)
    scale = zse.rsqrt(total / float(n) + eps)
    for i in range(tid, n, zse.block_dim(0)):
        out[row * n + i] = x[row * n + i] * scale * w[i]


@zse.kernel
def softmax_warp(x: zse.Tensor, out: zse.Tensor, n: int):
    """One warp per row of up to 32 values."""
    row = zse.block_id(0)
    lane = zse.lane_id()
    v = x[row * n + lane] if lane < n else -1e30
    m = zse.warp_reduce_max(v)
    e = zse.exp(v - m) if lane < n else 0.0
    s = zse.warp_reduce_sum(e)
    if lane < n:
        out[row * n + lane] = e / s


@zse.kernel
def shuffles(x: zse.Tensor[zse.int32], out: zse.Tensor[zse.int32]):
    lane = zse.lane_id()
    v = x[lane]
    out[lane] = zse.warp_shuffle_down(v, 1)
    out[32 + lane] = zse.warp_shuffle_xor(v, 3)
    out[64 + lane] = zse.warp_shuffle(v, 5)
    out[96 + lane] = zse.warp_ballot(v % 2 == 0) & 0xFFFF
    out[128 + lane] = 1 if zse.warp_any(v > 30) else 0
    out[160 + lane] = 1 if zse.warp_all(v >= 0) else 0
    out[192 + lane] = zse.warp_shuffle_up(v, 2)


@zse.kernel
def dequant_rows(packed: zse.Tensor[zse.uint8], scales: zse.Tensor[zse.float16], zeros: zse.Tensor[zse.float16],
                 out: zse.Tensor[zse.float16], groups: int):
    """INT4 asymmetric groups of 128 -> fp16: a thread expands one 32-bit word (8 values)."""
    w = zse.global_id(0)
    if w < groups * 16:
        words = zse.reinterpret(packed, zse.uint32)
        buf = zse.local_array(8, zse.int32)
        zse.unpack_uint4(words[w], buf, 0)
        g = w // 16
        for j in range(8):
            out[w * 8 + j] = buf[j] * scales[g] + zeros[g]


@zse.kernel
def transpose_tile(src: zse.Tensor, dst: zse.Tensor, rows: int, cols: int):
    tile = zse.shared_memory((16, 16), zse.float32)
    flipped = zse.shared_memory(256, zse.float32)
    zse.tile_load(src, zse.block_id(1), zse.block_id(0), 16, tile, rows, cols)
    for e in range(zse.thread_id(0), 256, zse.block_dim(0)):
        flipped[(e % 16) * 16 + e // 16] = tile[e]
    zse.tile_store(flipped, dst, zse.block_id(0), zse.block_id(1), 16, cols, rows)


@zse.kernel
def histogram(x: zse.Tensor[zse.int32], bins: zse.Tensor[zse.int32], n: int):
    i = zse.global_id(0)
    if i < n:
        zse.atomic_add(bins[x[i] % 8], 1)


@zse.kernel
def add_bias(x: zse.Tensor, bias: zse.Tensor, out: zse.Tensor, n: int, width: int):
    i = zse.global_id(0)
    if i >= n:
        return
    out[i] = x[i] + bias[i % width]


@zse.kernel
def silu(x: zse.Tensor, out: zse.Tensor, n: int):
    i = zse.global_id(0)
    if i >= n:
        return
    v = x[i]
    out[i] = v / (1.0 + zse.exp(-v))


@zse.kernel
def vec4_scale(x: zse.Tensor, out: zse.Tensor, alpha: float):
    i = zse.global_id(0)
    v = zse.load_float4(x, i)
    zse.store_float4(out, i, v.x * alpha, v.y * alpha, v[2] * alpha, v[3] * alpha)


def _blocks(n, b=BLOCK):
    return ((n + b - 1) // b,)


# ---- what the kernels compute (CPU emulation against torch) -----------------------------------------------------------
def test_vector_add_emulated_for_three_element_types():
    g = torch.Generator().manual_seed(0)
    for dt, tol in ((torch.float32, 0), (torch.float16, 1e-3), (torch.bfloat16, 1e-2)):
        a, b = torch.randn(150, generator=g).to(dt), torch.randn(150, generator=g).to(dt)
        out = torch.zeros(150, dtype=dt)
        vector_add.emulate(_blocks(150), (BLOCK,), (a, b, out, 150))
        torch.testing.assert_close(out.float(), (a.float() + b.float()).to(dt).float(), atol=tol, rtol=0)


def test_rmsnorm_block_reduction():
    g = torch.Generator().manual_seed(1)
    x, w = torch.randn(3, 200, generator=g), torch.rand(200, generator=g) + 0.5
    out = torch.zeros_like(x)
    rmsnorm.emulate((3,), (BLOCK,), (x, w, out, 200, 1e-6))
    want = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-6) * w
    torch.testing.assert_close(out, want, atol=1e-5, rtol=1e-5)


def test_softmax_with_warp_reductions():
    x = torch.randn(4, 20, generator=torch.Generator().manual_seed(2))
    out = torch.zeros_like(x)
    softmax_warp.emulate((4,), (32,), (x, out, 20))
    torch.testing.assert_close(out, torch.softmax(x, -1), atol=1e-6, rtol=1e-5)


def test_warp_shuffles_and_votes():
    x = torch.arange(32, dtype=torch.int32)
    out = torch.zeros(224, dtype=torch.int32)
    shuffles.emulate((1,), (32,), (x, out))
    lanes = np.arange(32)
    o = out.numpy()
    assert (o[:32] == np.where(lanes + 1 < 32, lanes + 1, lanes)).all()
    assert (o[32:64] == (lanes ^ 3)).all() and (o[64:96] == 5).all()
    assert (o[96:128] == (0x55555555 & 0xFFFF)).all()
    assert (o[128:160] == 1).all() and (o[160:192] == 1).all()
    assert (o[192:224] == np.where(lanes - 2 >= 0, lanes - 2, lanes)).all()


def test_int4_dequant_matches_the_format_oracle():
    from zse_b200.format import quantize as q
    w = np.random.default_rng(3).standard_normal(4 * 128).astype(np.float32)
    packed, scales, zeros = q.quantize_int4_arrays(w, 128)
    want = q.dequantize_int4_arrays(packed, scales, zeros, w.size, 128)
    out = torch.zeros(w.size, dtype=torch.float16)
    args = (torch.from_numpy(packed.copy()), torch.from_numpy(scales.copy()), torch.from_numpy(zeros.copy()), out, 4)
    dequant_rows.emulate(_blocks(4 * 16), (BLOCK,), args)
    np.testing.assert_allclose(out.float().numpy(), want, atol=2e-3)


def test_tile_load_store_with_ragged_edges():
    src = torch.randn(20, 37, generator=torch.Generator().manual_seed(4))
    dst = torch.zeros(37, 20)
    transpose_tile.emulate((3, 2), (BLOCK,), (src, dst, 20, 37))
    torch.testing.assert_close(dst, src.t().contiguous())


def test_atomics_and_vector_access():
    x = torch.randint(0, 100, (300,), dtype=torch.int32, generator=torch.Generator().manual_seed(5))
    bins = torch.zeros(8, dtype=torch.int32)
    histogram.emulate(_blocks(300), (BLOCK,), (x, bins, 300))
    assert bins.tolist() == torch.bincount(x % 8, minlength=8).tolist()
    v = torch.arange(64, dtype=torch.float32)
    out = torch.zeros(64)
    vec4_scale.emulate((1,), (16,), (v, out, 0.5))
    torch.testing.assert_close(out, v * 0.5)


def test_fused_kernels_skip_the_intermediate_tensor():
    fused = zse.fuse([add_bias, silu], name="add_bias_silu")
    assert [p.name for p in fused.params] == ["x", "bias", "n", "width", "out"]
    src = fused.source()
    assert "_fused_0" in src and src.count("__global__") == 1
    x, bias = torch.randn(100, generator=torch.Generator().manual_seed(6)), torch.randn(10)
    out = torch.zeros(100)
    fused.emulate(_blocks(100), (BLOCK,), (x, bias, 100, 10, out))
    torch.testing.assert_close(out, torch.nn.functional.silu(x + bias.repeat(10)), atol=1e-6, rtol=1e-5)
    three = zse.fuse([add_bias, silu, vector_add], chain=["x", "a"])
    res, extra = torch.zeros(100), torch.ones(100)
    three.emulate(_blocks(100), (BLOCK,), (x, bias, 100, 10, extra, res))
    torch.testing.assert_close(res, torch.nn.functional.silu(x + bias.repeat(10)) + 1, atol=1e-6, rtol=1e-5)
    with pytest.raises(zse.KernelSyntaxError, match="chain"):
        zse.fuse([silu, vector_add])                 # two readable tensors: ambiguous without chain=
    with pytest.raises(zse.KernelSyntaxError, match="element-wise"):
        zse.fuse([silu, rmsnorm], chain=["x"])


# ---- text and binaries ------------------------------------------------------------------------------------------------
ALL_KERNELS = [vector_add, rmsnorm, softmax_warp, shuffles, dequant_rows, transpose_tile, histogram, add_bias, silu,
               vec4_scale]


def test_source_is_specialised_by_element_type():
    src32 = vector_add.source()
    assert 'extern "C" __global__ void vector_add(float* a, float* b, float* out, int n)' in src32
    src16 = vector_add.source(dtypes={"a": zse.float16, "b": "float16", "out": zse.bfloat16})
    assert "__half* a, __half* b, __nv_bfloat16* out" in src16
    assert "__half2float(a[i])" in src16 and "__float2bfloat16" in src16
    assert "#line" not in src32 and "#line" in vector_add.source(line_info=True)
    assert vector_add.ir.name == "vector_add" and [p.kind for p in vector_add.params] == ["tensor"] * 3 + ["int"]
    text = rmsnorm.source()
    assert "zse_block_sum_float" in text and "__shfl_xor_sync(0xffffffffu" in text and "rsqrtf" in text
    assert "__shared__ float tile[256];" in transpose_tile.source()
    assert "atomicAdd(&bins[" in histogram.source()
    assert "reinterpret_cast<unsigned int*>(packed)" in dequant_rows.source()
    with pytest.raises(ValueError):
        vector_add.source("rocm")
    with pytest.raises(RuntimeError, match="launch"):
        vector_add(1, 2, 3, 4)


@pytest.mark.timeout(600)
def test_every_kernel_compiles_for_sm_100a(tmp_path, monkeypatch):
    """nvcc cross-compiles the generated text into a cubin; a second request is served from the cache."""
    monkeypatch.setenv("ZSE_KERNEL_CACHE", str(tmp_path))
    comp = zse.RuntimeCompiler()
    fused = zse.fuse([add_bias, silu])
    for k in ALL_KERNELS + [fused]:
        ck = comp.compile(k.source(line_info=True), k.name)
        assert ck.cubin[:4] == b"\x7fELF" and not ck.from_cache, k.name
    assert comp.stats["compiled"] == len(ALL_KERNELS) + 1
    half = comp.compile(vector_add.source(dtypes={"a": "float16", "b": "float16", "out": "float16"}), "vector_add")
    assert half.key != comp.compile(vector_add.source(line_info=True), "vector_add").key
    assert comp.stats["memory_hits"] == 1
    again = zse.RuntimeCompiler().compile(silu.source(line_info=True), "silu")
    assert again.from_cache and len(os.listdir(tmp_path)) == len(ALL_KERNELS) + 2
    with pytest.raises(zse.KernelCompileError) as err:
        comp.compile('extern "C" __global__ void broken() { int x = ; }', "broken")
    assert "error" in err.value.log
    with pytest.raises(ValueError):
        comp.compile("", "x", backend="metal")


# ---- what is refused ----------------------------------------------------------------------------------------------------
def _bad_try(x: zse.Tensor):
    try:
        x[0] = 1.0
    except Exception:
        pass


def _bad_comprehension(x: zse.Tensor):
    x[0] = sum([i for i in range(4)])


def _bad_return(x: zse.Tensor):
    return x[0]


def _bad_unknown(x: zse.Tensor):
    x[0] = undefined_function(1.0)      # noqa: F821


def _bad_read_before_write(x: zse.Tensor):
    x[0] = y                             # noqa: F821


def _bad_bits(x: zse.Tensor):
    x[0] = x[1] & 3


def _bad_atomic(x: zse.Tensor[zse.float16]):
    zse.atomic_add(x[0], 1.0)


def _bad_axis(x: zse.Tensor, a: int):
    x[0] = zse.thread_id(a)


def test_errors_name_the_python_line():
    for fn, exc, word in ((_bad_try, zse.KernelSyntaxError, "try/except"),
                          (_bad_comprehension, zse.KernelSyntaxError, "comprehensions"),
                          (_bad_return, zse.KernelSyntaxError, "returns nothing"),
                          (_bad_unknown, zse.KernelSyntaxError, "undefined_function"),
                          (_bad_read_before_write, zse.KernelSyntaxError, "'y'"),
                          (_bad_axis, zse.KernelSyntaxError, "axis")):
        with pytest.raises(exc, match=word) as err:
            zse.kernel(fn)
        assert "test_dsl.py" in str(err.value) and err.value.lineno > 0
    for fn, word in ((_bad_bits, "integers"), (_bad_atomic, "atomic_add works on")):
        k = zse.kernel(fn)
        with pytest.raises(zse.KernelTypeError, match=word):
            k.source()
    with pytest.raises(RuntimeError, match="only be used inside"):
        zse.thread_id(0)


@zse.kernel
def _divergent_barrier(x: zse.Tensor):
    if zse.thread_id(0) < 16:
        zse.syncthreads()
    x[zse.thread_id(0)] = 1.0


def test_launch_configuration_and_emulator_checks():
    cfg = zse.LaunchConfig((4,), (16, 8))
    assert cfg.grid == (4, 1, 1) and cfg.block == (16, 8, 1) and cfg.threads_per_block == 128
    assert cfg.total_threads == 512
    for grid, block, smem in (((1,), (2048,), 0), ((1,), (32, 64), 0), ((1, 70000), (32,), 0), ((0,), (32,), 0),
                              ((1,), (32,), 300 * 1024)):
        with pytest.raises(zse.KernelLaunchError):
            zse.LaunchConfig(grid, block, smem)
    x = torch.zeros(64)
    with pytest.raises(zse.KernelLaunchError, match="multiple of 32"):
        rmsnorm.emulate((1,), (48,), (x, x, x, 64, 1e-6))
    with pytest.raises(zse.KernelLaunchError, match="returned while"):
        _divergent_barrier.emulate((1,), (32,), (x,))
    with pytest.raises(zse.KernelTypeError, match="takes 4 arguments"):
        vector_add.emulate((1,), (32,), (x, x, x))
    with pytest.raises(zse.KernelTypeError, match="declared"):
        histogram.emulate((1,), (32,), (x, x, 4))
    with pytest.raises(IndexError, match="outside"):
        vec4_scale.emulate((1,), (32,), (x, x, 1.0))        # 32 threads x 4 floats > 64 elements
    if not torch.cuda.is_available():
        with pytest.raises(zse.KernelLaunchError, match="emulate"):
            vector_add.launch((1,), (32,), (x, x, x, 64))


def test_tensors_and_memory_on_the_host():
    t = zse.Tensor(shape=(1024,), dtype=zse.float32)
    assert (t.numel, t.nbytes, t.ndim, t.data_ptr) == (1024, 4096, 1, 0)
    assert zse.Tensor((32, 64), zse.float16).nbytes == 4096 and zse.Tensor((1024,), zse.int4).nbytes == 512
    mem = zse.GPUMemory("cpu")
    a = mem.zeros((8,), zse.float32)
    b = mem.allocate((8,), zse.float32)
    assert mem.allocated_bytes == 64 and a.data_ptr != 0
    mem.copy_host_to_device(np.arange(8, dtype=np.float32), a)
    mem.copy_device_to_device(a, b)
    assert np.frombuffer(mem.copy_device_to_host(b), np.float32).tolist() == list(range(8))
    out = mem.zeros((8,), zse.float32)
    vector_add.emulate((1,), (32,), (a, b, out, 8))
    assert mem.to_numpy(out).tolist() == [2.0 * i for i in range(8)]
    mem.memset(out, 0)
    assert mem.to_numpy(out).sum() == 0
    packed = mem.zeros((64,), zse.int4)
    assert packed.data.numel() == 32 and packed.data.dtype == torch.uint8
    mem.free(a)
    assert mem.allocated_bytes == 64 + 32 + 32 - 32 and mem.peak_bytes >= 128
    assert mem.allocate_pinned(16).numel() == 16 and mem.get_total_memory() == 0
    assert zse.detect_backend() in ("cuda", "cpu") and isinstance(zse.get_devices(), list)


def test_autotune_sweeps_block_sizes_with_a_stub_timer():
    """The sweep logic without a GPU: a stand-in profiler 'times' each candidate from its block size."""
    from zse_b200.runtime.profiler import AutoTuner, ProfileResult

    class Stub:
        def __init__(self):
            self.seen = []

        def time(self, name, fn, nbytes=0, flops=0, **extra):
            b = int(name.split("[")[1].rstrip("]"))
            self.seen.append(b)
            return ProfileResult(name, abs(b - 128) + 1.0, 1.0, 1, nbytes, flops, {})

    stub = Stub()
    res = rmsnorm.autotune(1000, (), block_sizes=(16, 48, 64, 128, 256), tuner=AutoTuner(stub))
    assert stub.seen == [64, 128, 256] and res["best"] == 128      # 16 and 48 are not whole warps


@zse.kernel
def wmma_matmul(a: zse.Tensor[zse.float16], b: zse.Tensor[zse.float16], c: zse.Tensor, n: int, k: int):
    """One warp per 16x16 tile of C = A [m, k] @ B [k, n] (row-major), fp16 inputs, fp32 accumulation."""
    acc = zse.wmma_fill(0.0)
    for kk in range(0, k, 16):
        fa = zse.wmma_load_a(a, zse.block_id(1) * 16, kk, k)
        fb = zse.wmma_load_b(b, kk, zse.block_id(0) * 16, n)
        acc = zse.wmma_mma(fa, fb, acc)
    zse.wmma_store(c, zse.block_id(1) * 16, zse.block_id(0) * 16, n, acc)


def test_tensor_core_tiles_through_wmma(tmp_path, monkeypatch):
    g = torch.Generator().manual_seed(7)
    a, b = torch.randn(32, 48, generator=g).half(), torch.randn(48, 16, generator=g).half()
    c = torch.zeros(32, 16)
    wmma_matmul.emulate((1, 2), (32,), (a, b, c, 16, 48))
    torch.testing.assert_close(c, a.float() @ b.float(), atol=1e-4, rtol=1e-4)
    src = wmma_matmul.source()
    assert "#include <mma.h>" in src and "nvcuda::wmma::mma_sync(acc, fa, fb, acc);" in src
    with pytest.raises(zse.KernelLaunchError, match="multiple of 32"):
        wmma_matmul.emulate((1, 2), (16,), (a, b, c, 16, 48))
    monkeypatch.setenv("ZSE_KERNEL_CACHE", str(tmp_path))
    assert zse.RuntimeCompiler().compile(wmma_matmul.source(line_info=True), "wmma_matmul").cubin[:4] == b"\x7fELF"


def test_prepacked_arguments_keep_their_storage():
    x = torch.zeros(8)
    pre = vector_add.prepack((x, x, x, 8))
    addr, first = pre.address, pre.values[3].value
    pre.set(3, 5)
    y = torch.ones(8)
    pre.set(0, y)
    assert (first, pre.values[3].value, pre.address, len(pre)) == (8, 5, addr, 4)
    assert pre.values[0].value == y.data_ptr() and pre.values[1].value == x.data_ptr()
    with pytest.raises(zse.KernelTypeError):
        pre.set(0, torch.zeros(8, dtype=torch.float16))
    from zse_b200.dsl.dtypes import from_string
    assert from_string("fp16") is zse.float16 and from_string("bfloat16") is zse.bfloat16
    assert zse.infer_types(vector_add.ir).var_types["i"] == "int"


def test_resource_report():
    r = rmsnorm.resources({"x": "float16", "w": "float16", "out": "float16"})
    assert 0 < r["registers"] <= 64 and r["spill_stores"] == r["spill_loads"] == 0 and r["shared_bytes"] >= 128
    from zse_b200.dsl import report
    assert any(k.name == "wmma_matmul" for _, k in report.kernels_of(__file__))


# ---- race detection in the emulator -------------------------------------------------------------------------------------
@zse.kernel
def _racy_sum(x: zse.Tensor, out: zse.Tensor, n: int):
    i = zse.global_id(0)
    if i < n:
        out[0] = out[0] + x[i]                 # every thread reads and writes out[0] without an atomic


@zse.kernel
def _racy_shared(x: zse.Tensor, out: zse.Tensor):
    buf = zse.shared_memory(64, zse.float32)
    t = zse.thread_id(0)
    buf[t] = x[t]
    out[t] = buf[63 - t]                       # reads a neighbour's slot with no barrier in between


@zse.kernel
def _ordered_shared(x: zse.Tensor, out: zse.Tensor):
    buf = zse.shared_memory(64, zse.float32)
    t = zse.thread_id(0)
    buf[t] = x[t]
    zse.syncthreads()
    out[t] = buf[63 - t]
    zse.syncthreads()
    buf[63 - t] = 0.0                          # reuse after a second barrier is fine


def test_emulator_finds_data_races():
    x, out = torch.arange(64, dtype=torch.float32), torch.zeros(64)
    with pytest.raises(zse.KernelRaceError) as err:
        _racy_sum.emulate((2,), (32,), (x, out, 64), check_races=True)
    assert any("out[0]" in r for r in err.value.races) and "line" in err.value.races[0]
    with pytest.raises(zse.KernelRaceError, match="read-after-write race on buf"):
        _racy_shared.emulate((1,), (64,), (x, out), check_races=True)
    _ordered_shared.emulate((1,), (64,), (x, out), check_races=True)
    assert out.tolist() == list(range(63, -1, -1))
    # the kernels above that are meant to be correct are race free: atomics, reductions, tiles, tensor-core tiles
    bins = torch.zeros(8, dtype=torch.int32)
    histogram.emulate((2,), (32,), (torch.arange(64, dtype=torch.int32), bins, 64), check_races=True)
    xs, w, o = torch.randn(2, 96), torch.ones(96), torch.zeros(2, 96)
    rmsnorm.emulate((2,), (32,), (xs, w, o, 96, 1e-6), check_races=True)
    src, dst = torch.randn(20, 37), torch.zeros(37, 20)
    transpose_tile.emulate((3, 2), (64,), (src, dst, 20, 37), check_races=True)
    a, b, c = torch.randn(16, 16).half(), torch.randn(16, 16).half(), torch.zeros(16, 16)
    wmma_matmul.emulate((1, 1), (32,), (a, b, c, 16, 16), check_races=True)
    torch.testing.assert_close(c, a.float() @ b.float(), atol=1e-4, rtol=1e-4)


@zse.kernel
def layernorm(x: zse.Tensor, weight: zse.Tensor, out: zse.Tensor, n: int):
    """Two block reductions in a row (mean, then variance): the reduction's scratch is reused safely."""
    tid = zse.thread_id(0)
    idx = zse.block_id(0) * n + tid
    val = x[idx] if tid < n else 0.0
    mean = zse.block_reduce_sum(val) / float(n)
    diff = val - mean if tid < n else 0.0
    var = zse.block_reduce_sum(diff * diff) / float(n)
    if tid < n:
        out[idx] = weight[tid] * (diff * zse.rsqrt(var + 0.00001))


def test_layernorm_with_two_reductions():
    x, w = torch.randn(3, 50, generator=torch.Generator().manual_seed(8)), torch.rand(50) + 0.5
    out = torch.zeros_like(x)
    layernorm.emulate((3,), (64,), (x, w, out, 50), check_races=True)
    want = torch.nn.functional.layer_norm(x, (50,), eps=1e-5) * w
    torch.testing.assert_close(out, want, atol=1e-5, rtol=1e-4)
    assert layernorm.source().count("zse_block_sum_float(") >= 3       # the helper and its two call sites

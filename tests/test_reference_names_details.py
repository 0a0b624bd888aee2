"""Reference-named accessors that thin code written against the reference relies on - element-type and tensor
descriptors, device facts, pre-packed kernel arguments, raw device and pinned addresses, the compiled-kernel profiler
and tuner, the C-launcher handle - each checked for what it returns, not merely for existing.  No GPU is involved: raw
"device" memory is host memory here, and the profiler is driven with a stand-in launcher."""
import ctypes
import time

import pytest
import torch

import zse_b200.dsl as zse
from zse_b200.runtime.device import DeviceInfo
from zse_b200.runtime.profiler import AutoTuner, KernelProfile, KernelProfiler, TuneResult


@zse.kernel
def fill_one(a: zse.Tensor, n: int):
    i = zse.global_id(0)
    if i < n:
        a[i] = 1.0


# ---- element types and tensor descriptors -----------------------------------------------------------------------
def test_element_sizes_round_up_to_whole_bytes():
    assert [d.size_bytes() for d in (zse.float32, zse.float16, zse.bfloat16, zse.int8, zse.int4, zse.uint4)] == \
        [4, 2, 2, 1, 1, 1]
    assert zse.int4.size_bits == 4 and zse.int4.nbytes == 0.5


def test_tensor_descriptor_reshape_device_and_strides():
    t = zse.Tensor((4, 6), zse.float16)
    assert t.device == "cpu" and t.is_contiguous() and t.strides == (6, 1) and t.data_ptr == 0
    r = t.reshape(3, 8)
    assert r.shape == (3, 8) and r.dtype is zse.float16 and r.numel == t.numel
    assert t.reshape((2, 12)).shape == (2, 12)
    with pytest.raises(ValueError, match="Cannot reshape"):
        t.reshape(5, 5)
    real = zse.zeros((2, 3, 4), zse.float32, device="cpu")
    view = real.reshape(6, 4)
    assert view.data_ptr == real.data_ptr and tuple(view.data.shape) == (6, 4) and real.strides == (12, 4, 1)
    packed = zse.zeros((16,), zse.int4, device="cpu")            # raw bytes underneath: the description changes only
    assert packed.reshape(4, 4).data is packed.data


def test_device_info_in_gigabytes():
    d = DeviceInfo(0, "B200", (10, 0), 180 * 1024 ** 3, 90 * 1024 ** 3, 148, 232448)
    assert d.vram_total_gb == 180.0 and d.vram_free_gb == 90.0 and d.vram_total_bytes == 180 * 1024 ** 3
    assert d.backend == "cuda" and d.num_sms == 148 and d.is_blackwell and d.warp_size == 32


# ---- pre-packed arguments ---------------------------------------------------------------------------------------
def test_prepacked_arguments_from_values_and_in_place_updates():
    x = torch.zeros(8)
    pa = zse.PrepackedArgs.from_args(x, zse.Tensor((4,), zse.float32), 5, 2.5, 1 << 20)
    assert len(pa) == 5
    assert pa.values[0].value == x.data_ptr() and pa.values[1].value in (0, None)
    assert (pa.values[2].value, pa.values[3].value, pa.values[4].value) == (5, 2.5, 1 << 20)
    addr, first = pa.address, ctypes.addressof(pa.values[2])
    pa.set_int(2, 7)
    pa.set_float(3, -1.5)
    pa.set_ptr(1, 4096)
    assert (pa.values[2].value, pa.values[3].value, pa.values[1].value) == (7, -1.5, 4096)
    assert pa.address == addr and ctypes.addressof(pa.values[2]) == first          # nothing was reallocated
    assert pa.arg_array is pa.array and pa.arg_array[2] == first                   # the array points at the slots
    with pytest.raises(TypeError, match="Unsupported arg type"):
        zse.PrepackedArgs.from_args("text")
    zse.KernelLauncher().sync()                                                    # nothing to wait for on a CPU box


# ---- raw addresses ----------------------------------------------------------------------------------------------
def test_raw_device_and_pinned_addresses():
    m = zse.GPUMemory("cpu")
    assert m.malloc_raw(0) == 0 and m.pinned_alloc(0) == 0
    p = m.malloc_raw(64)
    assert p != 0 and m.allocated_bytes == 64 and m.peak_bytes >= 64
    m.copy_host_to_device_raw(bytes(range(16)), p + 8, 16)
    h = m.pinned_alloc(32)
    host = (ctypes.c_ubyte * 32).from_address(h)
    for i in range(32):
        host[i] = 100 + i
    m.copy_host_to_device_raw_ptr(h, p + 24, 8)
    stream = m.create_stream()
    m.copy_host_to_device_async_raw_ptr(h + 8, p + 32, 8, stream)
    m.synchronize_stream(stream)
    got = bytes((ctypes.c_ubyte * 64).from_address(p))
    assert got[8:24] == bytes(range(16)) and got[24:32] == bytes(range(100, 108)) and got[32:40] == bytes(range(108, 116))
    with pytest.raises(ValueError, match="not inside an allocation"):
        m.copy_host_to_device_raw(b"x" * 8, p + 60, 8)
    with pytest.raises(ValueError):
        m.copy_host_to_device_raw_ptr(h, 12345, 4)
    m.copy_host_to_device_raw(b"", p, 0)                                           # nothing to do
    m.destroy_stream(stream)
    m.pinned_free(h)
    m.pinned_free(h)
    m.free_raw(p)
    m.free_raw(p)
    assert m.allocated_bytes == 0


# ---- profiler and tuner of compiled kernels ---------------------------------------------------------------------
class _Compiled:
    name = "stub"


class _Launcher:
    """Pretends that blocks of 128 threads are the fastest."""

    def __init__(self):
        self.blocks = []

    def launch_prepacked(self, compiled, config, packed):
        self.blocks.append(config.block)
        time.sleep(0.0004 * (1 + abs(config.block[0] - 128) / 64))


def test_profile_record_and_its_derived_figures():
    prof = KernelProfiler(device="cpu", warmup=3, iters=3, flush_l2=False)
    launcher = _Launcher()
    r = prof.profile(_Compiled(), zse.LaunchConfig((4,), (64,)), (1, 2.0), warmup_runs=2, profile_runs=3,
                     launcher=launcher)
    assert isinstance(r, KernelProfile) and r.kernel_name == "stub" and r.backend == "host"
    assert r.grid == (4, 1, 1) and r.block == (64, 1, 1) and r.num_runs == 3 and len(launcher.blocks) == 5
    assert 0.3 < r.elapsed_ms < 50 and r.throughput_gflops is None
    assert r.bandwidth_gb_s(10 ** 6) == pytest.approx(1e-3 / (r.elapsed_ms / 1e3))
    r.total_flops = 2 * 10 ** 6
    assert r.throughput_gflops == pytest.approx(2 * 10 ** 6 / (r.elapsed_ms * 1e6))
    assert KernelProfile("k", "cuda", 0.0, (1,), (1,)).bandwidth_gb_s(100) == 0.0
    assert "stub" in repr(r) and "block=(64, 1, 1)" in repr(r)
    packed = zse.PrepackedArgs.from_args(3, 4.0)                                   # pre-packed arguments pass through
    assert prof.profile(_Compiled(), zse.LaunchConfig((1,), (32,)), packed, 0, 1, launcher).num_runs == 1


def test_one_dimensional_sweep_keeps_the_fastest_divisor():
    tuner = AutoTuner(KernelProfiler(device="cpu", warmup=3, iters=3, flush_l2=False))
    launcher = _Launcher()
    t = tuner.tune_1d(_Compiled(), (1, 2.0), 1024, launcher=launcher)
    assert isinstance(t, TuneResult) and t.kernel_name == "stub" and len(t.all_results) == 6
    assert t.best_config.block == (128, 1, 1) and t.best_config.grid == (8, 1, 1)
    assert t.best_time_ms == min(r.elapsed_ms for r in t.all_results)
    text = t.summary()
    assert text.startswith("Auto-tune results for 'stub':") and "<- best" in text and text.count("block=") == 6
    # only block sizes that divide the thread count are tried; none -> an error that says so
    t = tuner.tune_1d(_Compiled(), (1,), 96, launcher=_Launcher())
    assert sorted(r.block[0] for r in t.all_results) == [32]
    with pytest.raises(RuntimeError, match="No valid configurations found for 50 threads"):
        tuner.tune_1d(_Compiled(), (1,), 50, launcher=_Launcher())


def test_two_dimensional_sweep_skips_blocks_the_device_cannot_run():
    tuner = AutoTuner(KernelProfiler(device="cpu", warmup=3, iters=3, flush_l2=False))
    t = tuner.tune_2d(_Compiled(), (1,), (100, 60), block_sizes=[(8, 8), (16, 16), (64, 64)], launcher=_Launcher())
    assert {r.block[:2] for r in t.all_results} == {(8, 8), (16, 16)}              # 64 x 64 = 4096 threads: refused
    by_block = {r.block[:2]: r.grid for r in t.all_results}
    assert by_block[(8, 8)] == (8, 13, 1) and by_block[(16, 16)] == (4, 7, 1)      # x covers the 60 columns
    assert len(tuner.tune_2d(_Compiled(), (1,), (64, 64), launcher=_Launcher()).all_results) == 9


# ---- generator objects, error locations, ids --------------------------------------------------------------------
def test_generator_objects_and_error_locations():
    assert zse.CUDACodegen().generate(fill_one) == fill_one.source()
    assert "#line" in zse.BaseCodegen(line_info=True).generate(fill_one.typed(None))
    assert zse.CUDACodegen.backend == "cuda" and issubclass(zse.CUDACodegen, zse.BaseCodegen)
    err = zse.KernelSyntaxError("bad thing", "kernels.py", 12, "    x = undefined()")
    loc = err.location
    assert isinstance(loc, zse.SourceLocation) and (loc.file, loc.line, loc.col) == ("kernels.py", 12, 0)
    assert str(loc) == "kernels.py:12\n  x = undefined()"
    assert zse.KernelSyntaxError("no line known").location is None
    assert str(zse.SourceLocation("a.py", 3)) == "a.py:3"


def test_parse_error_formatting_shows_the_line_in_context():
    from zse_b200.dsl.errors import format_parse_error, get_kernel_source_lines
    lines = get_kernel_source_lines(fill_one)
    assert lines[0].startswith("@zse.kernel") and lines[1].startswith("def fill_one(") and "a[i] = 1.0" in lines[4]
    assert get_kernel_source_lines(fill_one._func) == lines and get_kernel_source_lines(len) == []
    text = format_parse_error(fill_one, 4, "something is wrong here")
    rows = text.split("\n")
    assert rows[0] == "Parse error in 'fill_one', line 4:" and rows[-1] == "  Error: something is wrong here"
    marked = [r for r in rows if r.startswith("  >>")]
    assert len(marked) == 1 and "  4|" in marked[0] and "if i < n" in marked[0]
    assert len(rows) == 2 + 5                                      # two lines of context on either side
    assert format_parse_error(fill_one, 0, "m") == "Parse error in 'fill_one': m"
    assert format_parse_error(len, 3, "m") == "Parse error in 'len': m"


def test_unique_id_record_carries_the_rendezvous_address():
    from zse_b200.parallel.tensor_parallel import NCCL_UNIQUE_ID_BYTES, NcclUniqueId, get_unique_id
    uid = get_unique_id("cpu")
    rec = NcclUniqueId.from_address_string(uid)
    assert ctypes.sizeof(rec) == NCCL_UNIQUE_ID_BYTES == 128 and rec.address == uid and uid.startswith(b"127.0.0.1:")
    assert NcclUniqueId.from_address_string("host:1").address == b"host:1"
    with pytest.raises(ValueError):
        NcclUniqueId.from_address_string("x" * 200)


def test_one_process_communicator_setup_is_refused_with_a_pointer():
    from zse_b200.parallel.tensor_parallel import comm_init_all
    with pytest.raises(RuntimeError, match="tp_launch"):
        comm_init_all(2)


# ---- the C-launcher handle --------------------------------------------------------------------------------------
def test_fast_decoder_lifecycle_without_a_gpu(tmp_path):
    from zse_b200.format import ZSELoader, synth
    from zse_b200.models.decoder import DecoderModel
    from zse_b200.runtime import FastDecoder
    fd = FastDecoder()
    assert fd.available is False and fd.decode_step(None, 1) == -1
    assert fd.compile() in (True, False)                                            # loads the library where it exists
    path = str(tmp_path / "tiny.zse")
    synth.write_random_model(path, synth.shape_config("tiny"), seed=0)
    model = DecoderModel.from_loader(ZSELoader(path), "cpu")
    assert fd.setup(model, buffers=None) is False                                   # the driver is for CUDA models
    assert fd.setup(model, object()) is False and fd.available is False
    with pytest.raises(RuntimeError, match="not available"):
        fd.forward(None, 1, True, 1, 1, 1, 1)


# ---- roofline arithmetic of a timing record -------------------------------------------------------------------------
def test_profile_rows_divide_by_the_given_peaks():
    from zse_b200.runtime.profiler import ProfileResult, measured_peaks
    r = ProfileResult("copy", ms=0.5, ms_min=0.4, launches=10, bytes=2_000_000_000, flops=0, extra={"ctas": 148})
    assert r.gbs == pytest.approx(4000.0) and r.tflops == 0.0
    row = r.row({"hbm_gbs": 8000.0, "tflops": 1000.0})
    assert row == {"name": "copy", "us": 500.0, "us_min": 400.0, "GB/s": 4000.0, "TFLOP/s": 0.0, "frac_hbm": 0.5,
                   "frac_tensor": None, "ctas": 148}
    g = ProfileResult("gemm", ms=2.0, ms_min=2.0, launches=1, bytes=0, flops=1_000_000_000_000)
    assert g.tflops == pytest.approx(500.0) and g.row({"hbm_gbs": 8000.0, "tflops": 1000.0})["frac_tensor"] == 0.5
    assert "frac_hbm" not in g.row()
    assert ProfileResult("none", 0.0, 0.0, 0, 10, 10).gbs == 0.0                  # no time, no rate
    p = measured_peaks()
    assert p["source"] in ("measured", "fallback") and 3000 < p["hbm_gbs"] < 9000 and 500 < p["tflops"] < 2500
    assert p["tflops_sustained"] <= p["tflops"] * 1.05

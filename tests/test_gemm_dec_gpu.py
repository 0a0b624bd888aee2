"""The persistent decode GEMM (csrc/gemm_w4_dec.cu) against the fp32 restatement: both work plans (stream / split),
odd tile counts, every token count bucket, all epilogues, and replays from a CUDA graph."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from zse_b200.format import quantize as Q
from zse_b200.ops import native
from zse_b200.ops import reference as ref


@pytest.fixture(scope="module")
def ops():
    from zse_b200.ops.backend import CudaOps
    o = CudaOps("cuda")
    yield o
    o.check()


@pytest.fixture(scope="module")
def ws(ops):
    return native.gemm_w4_dec_workspace(ops.device, ops.sm_count)


def _parts(N, K, seed, std=0.02):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((N, K)) * std).astype(np.float32)
    p, s, z = Q.quantize_int4_arrays(w, 128)
    deq = Q.dequantize_int4_arrays(p, s, z, N * K, 128).reshape(N, K)
    part = {"dtype": "int4", "data": p.reshape(N, K // 2), "scales": s.reshape(N, K // 128),
            "zeros": z.reshape(N, K // 128), "shape": (N, K)}
    return part, torch.from_numpy(deq).cuda()


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


# (M, N, K): split plans with 1..8 segments, odd tile counts (N = 128 * odd), a stream plan (more than 74 tile pairs)
SHAPES = [(1, 256, 256), (5, 128, 512), (16, 384, 1024), (17, 640, 2048), (33, 896, 5120), (64, 1024, 4096),
          (64, 5120, 640), (48, 2560, 1792), (64, 19456, 384), (31, 20480, 256), (64, 200, 256), (8, 19328, 640),
          (7, 1024, 128), (64, 384, 128), (4, 20480, 128)]        # a single K stage: shards of narrow layers at TP8


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_dec_fp16_and_fp32_epilogues(ops, ws, M, N, K):
    part, wd = _parts(N, K, seed=M * 7 + N)
    bias = (np.random.default_rng(1).standard_normal(N) * 0.1).astype(np.float16)
    w = ops.make_linear([part], K, 128, bias)
    assert w.kind == "w4t" and native.gemm_w4_dec_supported(M, N, K, 0)
    x = (torch.randn(M + 3, K, device="cuda") * 0.5).half()
    out = torch.full((M + 3, N), 7.0, dtype=torch.float16, device="cuda")
    native.gemm_w4_dec(w.data, x, x.shape[0], w.bias, out, M, N, K, out.stride(0), 0, ws, ops.status.ptr)
    out32 = torch.full((M + 3, N), 7.0, dtype=torch.float32, device="cuda")
    native.gemm_w4_dec(w.data, x, x.shape[0], None, out32, M, N, K, out32.stride(0), 2, ws, ops.status.ptr)
    torch.cuda.synchronize()
    ops.check()
    want = ref.linear(x[:M], wd, torch.from_numpy(bias).cuda())
    assert _rel(out[:M], want) < 2e-3, _rel(out[:M], want)
    assert _rel(out32[:M], x[:M].float() @ wd.T) < 2e-3
    assert torch.all(out[M:] == 7.0) and torch.all(out32[M:] == 7.0)        # rows past M untouched


@pytest.mark.parametrize("M,I,K", [(1, 128, 256), (9, 192, 512), (64, 1024, 1024), (40, 1728, 5120), (64, 9600, 256),
                                   (23, 9664, 384), (5, 256, 128)])
def test_dec_swiglu(ops, ws, M, I, K):
    g, gd = _parts(I, K, 3)
    u, ud = _parts(I, K, 4)
    w = ops.make_linear([g, u], K, 128, swiglu=True)
    x = (torch.randn(M, K, device="cuda")).half()
    out = torch.zeros(M, I, dtype=torch.float16, device="cuda")
    native.gemm_w4_dec(w.data, x, M, None, out, M, w.N, K, out.stride(0), 1, ws, ops.status.ptr)
    torch.cuda.synchronize()
    ops.check()
    want = ref.swiglu(x.float() @ gd.T, x.float() @ ud.T)
    assert _rel(out, want) < 3e-3, _rel(out, want)


@pytest.mark.parametrize("M,nh,nkv,K,bs", [(1, 4, 1, 512, 16), (7, 5, 1, 640, 16), (64, 8, 2, 1024, 32),
                                           (33, 40, 8, 256, 16), (4, 1, 1, 128, 16)])
def test_dec_qkv_rope_kv_write(ops, ws, M, nh, nkv, K, bs):
    hd = 128
    N = (nh + 2 * nkv) * hd
    part, wd = _parts(N, K, 21)
    bias = (np.random.default_rng(2).standard_normal(N) * 0.1).astype(np.float16)
    w = ops.make_linear([part], K, 128, bias)
    x = (torch.randn(M, K, device="cuda") * 0.5).half()
    max_pos = 4096
    inv = ref.inv_freq(hd, 1e6)
    ang = torch.arange(max_pos, dtype=torch.float32)[:, None] * inv[None, :]
    cos_sin = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).contiguous().cuda()       # [max_pos, 64, 2]
    positions = torch.randint(0, max_pos, (M,), dtype=torch.int32, device="cuda")
    blocks = M + 2
    perm = torch.randperm(blocks * bs, device="cuda")[:M].long()
    slots = perm.clone()
    if M > 2:
        slots[1] = -1                                         # a token that must not be stored
    kv = torch.zeros(blocks, 2, nkv, bs, hd, dtype=torch.float16, device="cuda")
    qkv = torch.zeros(M, N, dtype=torch.float16, device="cuda")
    native.gemm_w4_dec_qkv_rope(w.data, x, M, w.bias, qkv, qkv.stride(0), M, K, nh, nkv, kv, bs, positions, slots,
                                cos_sin, max_pos, ws, ops.status.ptr)
    torch.cuda.synchronize()
    ops.check()
    full = ref.linear(x, wd, torch.from_numpy(bias).cuda()).float()
    want_qkv = full.clone()
    want_kv = torch.zeros_like(kv)
    ref.rope_kv_write(want_qkv, want_kv, positions, slots, inv.cuda(), nh, nkv, hd, bs)
    assert _rel(qkv[:, : nh * hd], want_qkv[:, : nh * hd]) < 3e-3
    assert _rel(kv, want_kv) < 3e-3
    stored = slots >= 0
    assert float(kv.float().abs().sum()) > 0 and bool(stored.any())


def test_dec_graph_replay_and_back_to_back(ops, ws):
    """The launch epoch lives in device memory: a captured launch replays unchanged, and calls of different shapes that
    follow each other on one stream share the workspace."""
    shapes = [(64, 1024, 4096, 0), (64, 2560, 1792, 0), (64, 3456, 1024, 1), (16, 19456, 384, 0)]
    cases = []
    for M, N, K, epi in shapes:
        if epi == 1:
            g, gd = _parts(N // 2, K, 5)
            u, ud = _parts(N // 2, K, 6)
            w = ops.make_linear([g, u], K, 128, swiglu=True)
            x = torch.randn(M, K, device="cuda").half()
            want = ref.swiglu(x.float() @ gd.T, x.float() @ ud.T)
            out = torch.zeros(M, N // 2, dtype=torch.float16, device="cuda")
        else:
            part, wd = _parts(N, K, 9)
            w = ops.make_linear([part], K, 128)
            x = torch.randn(M, K, device="cuda").half()
            want = x.float() @ wd.T
            out = torch.zeros(M, N, dtype=torch.float16, device="cuda")
        cases.append((w, x, out, want, M, N, K, epi))

    def run_all():
        for w, x, out, want, M, N, K, epi in cases:
            native.gemm_w4_dec(w.data, x, M, None, out, M, N, K, out.stride(0), epi, ws, ops.status.ptr)

    for _ in range(3):
        run_all()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        run_all()
        with torch.cuda.graph(g, stream=s):
            run_all()
    torch.cuda.current_stream().wait_stream(s)
    for _ in range(3):
        for c in cases:
            c[2].zero_()
        g.replay()
        torch.cuda.synchronize()
        ops.check()
        for w, x, out, want, M, N, K, epi in cases:
            assert _rel(out, want) < 3e-3


def _parts8(N, K, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    q, s = Q.quantize_int8_arrays(w, 128)
    deq = (q.reshape(N, K // 128, 128).astype(np.float32) * s.reshape(N, K // 128, 1).astype(np.float32)).reshape(N, K)
    part = {"dtype": "int8", "data": q.reshape(N, K), "scales": s.reshape(N, K // 128), "shape": (N, K)}
    return part, torch.from_numpy(deq).cuda()


@pytest.mark.parametrize("M,N,K", [(1, 256, 256), (17, 640, 2048), (64, 1024, 4096), (48, 2560, 1792),
                                   (64, 19456, 384), (64, 200, 256), (200, 512, 1024)])
def test_int8_weights_stay_eight_bits_wide(ops, ws, M, N, K):
    """INT8 layers: tiled 8-bit chunks on the device (a little over one byte per weight), expanded in registers by the
    decode kernel; passes of more than 64 tokens expand into the shared fp16 scratch and take the fp16 GEMM."""
    part, wd = _parts8(N, K, seed=N + M)
    bias = (np.random.default_rng(1).standard_normal(N) * 0.1).astype(np.float16)
    w = ops.make_linear([part], K, 128, bias)
    assert w.kind == "w8t" and w.data.numel() == ((N + 127) // 128) * (K // 128) * 16640
    x = (torch.randn(M + 3, K, device="cuda") * 0.5).half()
    out = torch.full((M + 3, N), 7.0, dtype=torch.float16, device="cuda")
    ops.linear(w, x, M, out)
    planes = torch.zeros(8, M, N, dtype=torch.float32, device="cuda")
    n_planes = ops.linear_partial(w, x, M, planes)
    torch.cuda.synchronize()
    ops.check()
    want = ref.linear(x[:M], wd, torch.from_numpy(bias).cuda())
    assert _rel(out[:M], want) < 2e-3, _rel(out[:M], want)
    assert torch.all(out[M:] == 7.0)
    got = planes.view(-1)[: n_planes * M * N].view(n_planes, M, N).sum(0)
    assert _rel(got, x[:M].float() @ wd.T) < 2e-3


@pytest.mark.parametrize("M,I,K", [(9, 192, 512), (64, 1728, 1024), (150, 320, 256)])
def test_int8_gate_up_with_swiglu(ops, ws, M, I, K):
    g, gd = _parts8(I, K, 3)
    u, ud = _parts8(I, K, 4)
    w = ops.make_linear([g, u], K, 128, swiglu=True)
    assert w.kind == "w8t"
    x = (torch.randn(M, K, device="cuda")).half()
    out = torch.zeros(M, I, dtype=torch.float16, device="cuda")
    ops.linear_swiglu(w, x, M, out)
    torch.cuda.synchronize()
    ops.check()
    want = ref.swiglu(x.float() @ gd.T, x.float() @ ud.T)
    assert _rel(out, want) < 3e-3, _rel(out, want)

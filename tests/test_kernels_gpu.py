"""Numerics of every CUDA kernel against the plain-PyTorch fp32 restatement in ops/reference.py."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from zse_b200.format import quantize as Q
from zse_b200.ops import reference as ref


@pytest.fixture(scope="module")
def ops():
    from zse_b200.ops.backend import CudaOps
    o = CudaOps("cuda")
    yield o
    o.check()


def _w4_parts(N, K, seed, std=0.02):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((N, K)) * std).astype(np.float32)
    p, s, z = Q.quantize_int4_arrays(w, 128)
    deq = Q.dequantize_int4_arrays(p, s, z, N * K, 128).reshape(N, K)
    part = {"dtype": "int4", "data": p.reshape(N, K // 2), "scales": s.reshape(N, K // 128),
            "zeros": z.reshape(N, K // 128), "shape": (N, K)}
    return part, torch.from_numpy(deq).cuda()


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


@pytest.mark.parametrize("M,N,K", [(1, 128, 128), (7, 256, 512), (16, 384, 1024), (17, 128, 256), (33, 640, 512),
                                   (64, 1024, 2048), (100, 256, 384), (130, 128, 640), (300, 512, 256),
                                   (5, 200, 256)])
def test_gemm_w4_fp16_epilogue(ops, M, N, K):
    part, wd = _w4_parts(N, K, seed=M * 7 + N)
    bias = (np.random.default_rng(1).standard_normal(N) * 0.1).astype(np.float16)
    w = ops.make_linear([part], K, 128, bias)
    assert w.kind == "w4t"
    x = (torch.randn(M + 3, K, device="cuda") * 0.5).half()
    out = torch.full((M + 3, N), 7.0, dtype=torch.float16, device="cuda")
    ops.linear(w, x, M, out)
    torch.cuda.synchronize()
    ops.check()
    want = ref.linear(x[:M], wd, torch.from_numpy(bias).cuda())
    assert _rel(out[:M], want) < 2e-3, _rel(out[:M], want)
    assert torch.all(out[M:] == 7.0)            # rows past M untouched


@pytest.mark.parametrize("M,I,K", [(1, 128, 256), (9, 192, 512), (64, 1024, 1024), (150, 320, 256)])
def test_gemm_w4_swiglu(ops, M, I, K):
    g, gd = _w4_parts(I, K, 3)
    u, ud = _w4_parts(I, K, 4)
    w = ops.make_linear([g, u], K, 128, swiglu=True)
    x = (torch.randn(M, K, device="cuda")).half()
    out = torch.zeros(M, I, dtype=torch.float16, device="cuda")
    ops.linear_swiglu(w, x, M, out)
    torch.cuda.synchronize()
    ops.check()
    want = ref.swiglu(x.float() @ gd.T, x.float() @ ud.T)
    assert _rel(out, want) < 3e-3, _rel(out, want)


@pytest.mark.parametrize("M,N,K,ks", [(1, 256, 2048, 4), (8, 128, 1024, 3), (64, 512, 4096, 8), (40, 256, 128, 4)])
def test_gemm_w4_splitk_partials_and_add_rmsnorm(ops, M, N, K, ks):
    part, wd = _w4_parts(N, K, 11)
    w = ops.make_linear([part], K, 128)
    x = torch.randn(M, K, device="cuda").half()
    partials = torch.zeros(8, M, N, dtype=torch.float32, device="cuda")
    planes = ops.linear_partial(w, x, M, partials, k_split=ks)
    torch.cuda.synchronize()
    ops.check()
    assert 1 <= planes <= ks
    want = x.float() @ wd.T
    got = partials[:planes].sum(0)
    assert _rel(got, want) < 2e-3
    # the reduction fused with residual add + RMSNorm
    resid = torch.randn(M, N, device="cuda")
    r0 = resid.clone()
    wn = (1 + 0.1 * torch.randn(N, device="cuda")).half()
    out = torch.zeros(M, N, dtype=torch.float16, device="cuda")
    ops.add_rmsnorm(resid, partials, planes, None, wn, out, M, 1e-6)
    torch.cuda.synchronize()
    assert torch.allclose(resid, r0 + got, atol=1e-5, rtol=1e-5)
    assert _rel(out, ref.rmsnorm(r0 + got, wn, 1e-6)) < 2e-3


def _w4_parts_gpu(N, K, seed):
    """Large shapes: weights are drawn and quantised on the device (native quantiser), dequantised by the oracle."""
    from zse_b200.ops import native
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).half()
    packed = torch.zeros(N, K // 2, dtype=torch.uint8, device="cuda")
    sc = torch.zeros(N, K // 128, dtype=torch.float16, device="cuda")
    zr = torch.zeros(N, K // 128, dtype=torch.float16, device="cuda")
    native.quantize_w4(w, packed, sc, zr, N * K // 128)
    torch.cuda.synchronize()
    deq = ref.dequant_int4(packed, sc, zr, (N, K), 128)
    return {"dtype": "int4", "data": packed, "scales": sc, "zeros": zr, "shape": (N, K)}, deq


@pytest.mark.parametrize("M,N,K,epi", [(64, 7168, 5120, "f16"), (64, 5120, 5120, "partial"), (64, 5120, 13824, "partial"),
                                       (64, 13824, 5120, "swiglu"), (1, 3584, 18944, "partial"),
                                       (256, 8192, 8192, "f16"), (700, 2048, 1024, "swiglu"), (2048, 1024, 2048, "f16"),
                                       (300, 1280, 1024, "partial"), (16, 18944, 3584, "swiglu")])
def test_gemm_w4_model_shapes(ops, M, N, K, epi):
    """Shapes of the served models: cluster split-K, two weight tiles per CTA, several token tiles."""
    x = (torch.randn(M, K, device="cuda") * 0.5).half()
    if epi == "swiglu":
        g, gd = _w4_parts_gpu(N, K, 1)
        u, ud = _w4_parts_gpu(N, K, 2)
        w = ops.make_linear([g, u], K, 128, swiglu=True)
        out = torch.zeros(M, N, dtype=torch.float16, device="cuda")
        ops.linear_swiglu(w, x, M, out)
        want = ref.swiglu(x.float() @ gd.T, x.float() @ ud.T)
    else:
        p, wd = _w4_parts_gpu(N, K, 3)
        bias = (torch.randn(N, device="cuda") * 0.1).half() if epi == "f16" else None
        w = ops.make_linear([p], K, 128, bias)
        if epi == "f16":
            out = torch.zeros(M, N, dtype=torch.float16, device="cuda")
            ops.linear(w, x, M, out)
            want = ref.linear(x, wd, bias)
        else:
            planes = torch.zeros(8, M, N, dtype=torch.float32, device="cuda")
            n_pl = ops.linear_partial(w, x, M, planes)
            out, want = planes[:n_pl].sum(0), x.float() @ wd.T
    torch.cuda.synchronize()
    ops.check()
    assert _rel(out, want) < 3e-3, _rel(out, want)
    # determinism: the on-chip reduction adds the K splits in a fixed order
    if epi == "partial":
        again = torch.zeros(8, M, N, dtype=torch.float32, device="cuda")
        ops.linear_partial(w, x, M, again)
        torch.cuda.synchronize()
        assert torch.equal(again[:n_pl].sum(0), out)


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("M,N,K,epi", [(64, 5120, 5120, "partial"), (64, 13824, 5120, "swiglu"), (1, 3584, 2048, "f16"),
                                       (17, 1024, 4096, "partial"), (40, 2560, 1024, "swiglu"), (64, 640, 1152, "f16")])
def test_gemm_w4_wide_and_narrow_ctas_agree(ops, mode, M, N, K, epi):
    """Both CTA shapes (one wide CTA per SM / two narrow CTAs per SM) against the oracle, cluster split included."""
    from zse_b200.ops import native
    native.gemm_w4_set_mode(mode)
    try:
        x = (torch.randn(M, K, device="cuda") * 0.5).half()
        if epi == "swiglu":
            g, gd = _w4_parts_gpu(N, K, 11)
            u, ud = _w4_parts_gpu(N, K, 12)
            w = ops.make_linear([g, u], K, 128, swiglu=True)
            out = torch.zeros(M, N, dtype=torch.float16, device="cuda")
            ops.linear_swiglu(w, x, M, out)
            split = torch.zeros(M, N, dtype=torch.float16, device="cuda")
            native.gemm_w4(w.data, x, M, None, split, M, 2 * N, K, N, 1, 2, ops.status.ptr)
            want = ref.swiglu(x.float() @ gd.T, x.float() @ ud.T)
            torch.cuda.synchronize()
            assert _rel(split, want) < 3e-3
        else:
            p, wd = _w4_parts_gpu(N, K, 13)
            bias = (torch.randn(N, device="cuda") * 0.1).half() if epi == "f16" else None
            w = ops.make_linear([p], K, 128, bias)
            if epi == "f16":
                out = torch.zeros(M, N, dtype=torch.float16, device="cuda")
                ops.linear(w, x, M, out)
                want = ref.linear(x, wd, bias)
            else:
                planes = torch.zeros(8, M, N, dtype=torch.float32, device="cuda")
                n_pl = ops.linear_partial(w, x, M, planes)
                out, want = planes[:n_pl].sum(0), x.float() @ wd.T
        torch.cuda.synchronize()
        ops.check()
        assert _rel(out, want) < 3e-3, _rel(out, want)
    finally:
        native.gemm_w4_set_mode(0)


@pytest.mark.parametrize("M,N,K,epi", [(1, 9472, 3584, "swiglu"), (2, 9472, 1024, "swiglu"), (2, 12288, 1024, "f16"),
                                       (1, 3584, 18944, "partial"), (2, 5120, 5120, "partial"),
                                       (1, 152064 // 8, 512, "f16")])
def test_gemv_w4_one_and_two_tokens(ops, M, N, K, epi):
    """CUDA-core GEMV path (taken for one or two tokens) against the oracle and against the tensor-core kernel."""
    from zse_b200.ops import native
    x = (torch.randn(M, K, device="cuda") * 0.5).half()

    def run():
        if epi == "swiglu":
            out = torch.zeros(M, N, dtype=torch.float16, device="cuda")
            ops.linear_swiglu(w, x, M, out)
            return out
        if epi == "f16":
            out = torch.zeros(M, N, dtype=torch.float16, device="cuda")
            ops.linear(w, x, M, out)
            return out
        planes = torch.zeros(8, M, N, dtype=torch.float32, device="cuda")
        n_pl = ops.linear_partial(w, x, M, planes)
        return planes.view(-1)[: n_pl * M * N].view(n_pl, M, N).sum(0)

    if epi == "swiglu":
        g, gd = _w4_parts_gpu(N, K, 21)
        u, ud = _w4_parts_gpu(N, K, 22)
        w = ops.make_linear([g, u], K, 128, swiglu=True)
        want = ref.swiglu(x.float() @ gd.T, x.float() @ ud.T)
    else:
        p, wd = _w4_parts_gpu(N, K, 23)
        bias = (torch.randn(N, device="cuda") * 0.1).half() if epi == "f16" else None
        w = ops.make_linear([p], K, 128, bias)
        want = ref.linear(x, wd, bias) if epi == "f16" else x.float() @ wd.T
    got = run()
    torch.cuda.synchronize()
    ops.check()
    assert _rel(got, want) < 3e-3, _rel(got, want)
    native.gemm_w4_set_mode(4)                  # same call on the tensor cores
    try:
        tc = run()
        torch.cuda.synchronize()
    finally:
        native.gemm_w4_set_mode(0)
    assert _rel(got, tc) < 3e-3


@pytest.mark.parametrize("ks", [2, 3, 4])
def test_gemm_w4_cluster_split_with_fused_epilogues(ops, ks):
    """Explicit K split on an epilogue that needs the whole sum: the CTAs of a cluster add their accumulators through
    distributed shared memory before bias / SwiGLU are applied."""
    from zse_b200.ops import native
    M, N, K = 48, 1024, 2048
    p, wd = _w4_parts_gpu(N, K, 5)
    bias = (torch.randn(N, device="cuda") * 0.1).half()
    w = ops.make_linear([p], K, 128, bias)
    x = (torch.randn(M, K, device="cuda") * 0.5).half()
    out = torch.zeros(M, N, dtype=torch.float16, device="cuda")
    native.gemm_w4(w.data, x, M, w.bias, out, M, N, K, N, 0, ks, ops.status.ptr)
    g, gd = _w4_parts_gpu(N, K, 6)
    u, ud = _w4_parts_gpu(N, K, 7)
    wg = ops.make_linear([g, u], K, 128, swiglu=True)
    act = torch.zeros(M, N, dtype=torch.float16, device="cuda")
    native.gemm_w4(wg.data, x, M, None, act, M, 2 * N, K, N, 1, ks, ops.status.ptr)
    torch.cuda.synchronize()
    ops.check()
    assert _rel(out, ref.linear(x, wd, bias)) < 3e-3
    assert _rel(act, ref.swiglu(x.float() @ gd.T, x.float() @ ud.T)) < 3e-3


def test_rope_kv_write_from_planes(ops):
    """QKV produced as fp32 split-K planes: the RoPE kernel adds the planes and the bias, rotates, stores q as fp16
    and k/v into the cache - same result as the fp16 path."""
    hd, nh, nkv, bs, M, blocks = 128, 6, 2, 16, 19, 8
    ld = (nh + 2 * nkv) * hd
    planes = torch.randn(3, M, ld, device="cuda")
    bias = (torch.randn(ld, device="cuda") * 0.1).half()
    full = (planes.sum(0) + bias.float()).half()
    kv_a = torch.zeros(blocks, 2, nkv, bs, hd, dtype=torch.float16, device="cuda")
    kv_b = kv_a.clone()
    pos = torch.randint(0, 2000, (M,), device="cuda", dtype=torch.int32)
    slots = torch.randperm(blocks * bs, device="cuda")[:M].long()
    freqs = ref.inv_freq(hd, 1e6).cuda()
    want = full.clone()
    ref.rope_kv_write(want, kv_a, pos, slots, freqs, nh, nkv, hd, bs)
    got = torch.zeros(M, ld, dtype=torch.float16, device="cuda")
    ops.rope_kv_write(got, kv_b, pos, slots, freqs, M, nh, nkv, hd, bs, planes=planes, n_planes=3, bias=bias)
    torch.cuda.synchronize()
    assert (got[:, : nh * hd].float() - want[:, : nh * hd].float()).abs().max() < 2e-2
    assert (kv_b.float() - kv_a.float()).abs().max() < 2e-2


@pytest.mark.parametrize("M,N,K", [(1, 1000, 256), (20, 128, 688), (64, 4096, 512), (200, 300, 264)])
def test_gemm_f16(ops, M, N, K):
    w32 = torch.randn(N, K, device="cuda") * 0.05
    part = {"dtype": "float16", "data": w32.half().cpu().numpy(), "shape": (N, K)}
    w = ops.make_linear([part], K, 128)
    assert w.kind == "f16"
    x = torch.randn(M, K, device="cuda").half()
    out = torch.zeros(M, N, dtype=torch.float16, device="cuda")
    ops.linear(w, x, M, out)
    partials = torch.zeros(4, M, N, dtype=torch.float32, device="cuda")
    planes = ops.linear_partial(w, x, M, partials, k_split=3)
    torch.cuda.synchronize()
    ops.check()
    want = x.float() @ w32.half().float().T
    assert _rel(out, want) < 2e-3
    assert _rel(partials[:planes].sum(0), want) < 1e-3


def test_odd_k_int4_goes_through_dense_path(ops):
    """K = 688: quantisation groups straddle rows; the weight is dequantised once and served by the fp16 kernel."""
    N, K = 256, 688
    rng = np.random.default_rng(0)
    wf = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    p, s, z = Q.quantize_int4_arrays(wf, 128)
    deq = torch.from_numpy(Q.dequantize_int4_arrays(p, s, z, N * K, 128).reshape(N, K)).cuda()
    part = {"dtype": "int4", "flat_data": p, "flat_scales": s, "flat_zeros": z, "flat_shape": (N, K),
            "rows": (0, N), "cols": (0, K), "shape": (N, K)}
    w = ops.make_linear([part], K, 128)
    assert w.kind == "f16"
    x = torch.randn(5, K, device="cuda").half()
    out = torch.zeros(5, N, dtype=torch.float16, device="cuda")
    ops.linear(w, x, 5, out)
    torch.cuda.synchronize()
    assert _rel(out, x.float() @ deq.T) < 3e-3


def test_repack_dequant_quantize_roundtrip(ops):
    from zse_b200.ops import native
    n = 128 * 300
    w = (torch.randn(n, device="cuda") * 0.02).half()
    packed = torch.zeros(n // 2, dtype=torch.uint8, device="cuda")
    sc = torch.zeros(n // 128, dtype=torch.float16, device="cuda")
    zr = torch.zeros(n // 128, dtype=torch.float16, device="cuda")
    native.quantize_w4(w, packed, sc, zr, n // 128)
    back = torch.zeros(n, dtype=torch.float16, device="cuda")
    native.dequant_w4(packed, sc, zr, back, n, 128)
    torch.cuda.synchronize()
    p, s, z = Q.quantize_int4_arrays(w.float().cpu().numpy(), 128)
    assert (packed.cpu().numpy() != p).mean() < 0.002        # ties at .5 may round differently in fp32
    assert torch.allclose(sc.cpu(), torch.from_numpy(s), atol=1e-6)
    step = (w.float().view(-1, 128).max(1).values - w.float().view(-1, 128).min(1).values) / 15
    assert ((back.float() - w.float()).abs().view(-1, 128).max(1).values <= step * 0.51 + 2e-4).all()


def test_embedding_and_rmsnorm(ops):
    V, H, M = 1000, 512, 37
    table = torch.randn(V, H, device="cuda").half()
    ids = torch.randint(0, V, (M,), device="cuda", dtype=torch.int32)
    out = torch.zeros(M, H, device="cuda")
    ops.embedding(table, ids, out, M, 2.0)
    w = torch.randn(H, device="cuda").half()
    y = torch.zeros(M, H, dtype=torch.float16, device="cuda")
    ops.add_rmsnorm(out, None, 0, None, w, y, M, 1e-5)
    torch.cuda.synchronize()
    assert torch.equal(out, table[ids.long()].float() * 2.0)
    assert _rel(y, ref.rmsnorm(out, w, 1e-5)) < 1e-3


@pytest.mark.parametrize("hd,nh,nkv,bs,M", [(128, 8, 2, 16, 23), (64, 4, 2, 32, 23), (128, 5, 1, 16, 23),
                                            (128, 20, 4, 16, 300), (256, 3, 1, 16, 40), (96, 4, 2, 16, 23)])
def test_rope_kv_write(ops, hd, nh, nkv, bs, M):
    blocks = (M + bs - 1) // bs + 11
    qkv = torch.randn(M, (nh + 2 * nkv) * hd, device="cuda").half()
    kv = torch.zeros(blocks, 2, nkv, bs, hd, dtype=torch.float16, device="cuda")
    pos = torch.randint(0, 3000, (M,), device="cuda", dtype=torch.int32)
    slots = torch.randperm(blocks * bs, device="cuda")[:M].long()
    slots[3] = -1
    freqs = ref.inv_freq(hd, 1e6).cuda()
    q2, kv2 = qkv.clone(), kv.clone()
    ref.rope_kv_write(q2, kv2, pos, slots, freqs, nh, nkv, hd, bs)
    ops.rope_kv_write(qkv, kv, pos, slots, freqs, M, nh, nkv, hd, bs)
    torch.cuda.synchronize()
    assert (qkv.float() - q2.float()).abs().max() < 4e-3
    assert (kv.float() - kv2.float()).abs().max() < 4e-3


def _make_cache(S, lens, nkv, hd, bs, blocks, holes=()):
    kv = (torch.randn(blocks, 2, nkv, bs, hd, device="cuda") * 0.5).half()
    maxb = (max(lens) + bs - 1) // bs + 1
    bt = torch.full((S, maxb), -1, dtype=torch.int32, device="cuda")
    perm = torch.randperm(blocks)
    at = 0
    for s, n in enumerate(lens):
        nb = (n + bs - 1) // bs
        bt[s, :nb] = perm[at:at + nb].int().cuda()
        at += nb
    for s, b in holes:
        bt[s, b] = -1
    return kv, bt


@pytest.mark.parametrize("hd,nh,nkv,bs,splits", [(128, 8, 2, 16, 1), (128, 10, 2, 16, 4), (64, 4, 2, 32, 3),
                                                 (128, 28, 4, 16, 8), (128, 8, 1, 64, 2)])
def test_attn_decode(ops, hd, nh, nkv, bs, splits):
    lens = [1, 15, 16, 17, 200, 333, 64, 5]
    S = len(lens)
    kv, bt = _make_cache(S, lens, nkv, hd, bs, 128, holes=[(4, 2)] if bs == 16 else ())
    q = torch.randn(S, nh * hd + 2 * nkv * hd, device="cuda").half()
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    out = torch.zeros(S, nh * hd, dtype=torch.float16, device="cuda")
    scratch = torch.zeros(S * nh * splits * (hd + 2), device="cuda")
    ops.attn_decode(q, kv, bt, sl, out, S, nh, nkv, hd, bs, 1 / math.sqrt(hd), scratch, splits)
    torch.cuda.synchronize()
    want = ref.attn_decode(q[:, : nh * hd], kv, bt, sl, nh, nkv, hd, bs, 1 / math.sqrt(hd))
    assert (out.float() - want.float()).abs().max() < 3e-3


@pytest.mark.parametrize("hd,nh,nkv,bs", [(128, 4, 2, 16), (64, 4, 1, 32), (128, 5, 1, 16)])
def test_attn_prefill_chunks(ops, hd, nh, nkv, bs):
    # three sequences: fresh prompt, a second chunk on top of 100 cached tokens, a 5-token verify after 37
    q_lens, pos0 = [130, 70, 5], [0, 100, 37]
    S = 3
    totals = [a + b for a, b in zip(q_lens, pos0)]
    kv, bt = _make_cache(S, totals, nkv, hd, bs, 64)
    cu = torch.tensor([0, 130, 200, 205], dtype=torch.int32, device="cuda")
    p0 = torch.tensor(pos0, dtype=torch.int32, device="cuda")
    q = torch.randn(205, (nh + 2 * nkv) * hd, device="cuda").half()
    out = torch.zeros(205, nh * hd, dtype=torch.float16, device="cuda")
    ops.attn_prefill(q, kv, bt, cu, p0, out, S, 205, 130, nh, nkv, hd, bs, 1 / math.sqrt(hd))
    torch.cuda.synchronize()
    want = ref.attn_prefill(q[:, : nh * hd], kv, bt, cu, p0, nh, nkv, hd, bs, 1 / math.sqrt(hd))
    assert (out.float() - want.float()).abs().max() < 3e-3


@pytest.mark.parametrize("nh,nkv,bs,q_lens,pos0,mode", [
    (8, 2, 16, [300, 70, 5, 128], [0, 100, 37, 256], 0),          # long chunks: one CTA per 128 rows of one head
    (5, 1, 32, [300, 70, 5, 128], [0, 100, 37, 256], 0),
    (4, 4, 64, [300, 70, 5, 128], [0, 100, 37, 256], 0),
    (10, 2, 16, [5, 16, 1, 9], [37, 100, 0, 300], 0),              # chunks of <= 16 rows: query heads packed per kv head
    (8, 1, 16, [4, 4, 4], [500, 17, 129], 0),                      # eight query heads on one kv head
    (10, 2, 16, [5, 16, 1, 9], [37, 100, 0, 300], 2),              # the same chunks without packing
])
def test_attn_prefill_on_tcgen05(ops, nh, nkv, bs, q_lens, pos0, mode):
    """The tcgen05 prefill kernel (S = Q K^T and O = P V on the tensor cores, probabilities through TMEM, V as an
    MN-major operand straight from the cache layout) against the fp32 oracle: a fresh prompt longer than two key tiles,
    a chunk on top of cached tokens that starts inside a tile, a short verify chunk, a chunk of exactly one tile; and
    verification-sized chunks, where one CTA serves all query heads of a kv head."""
    from zse_b200.ops import native
    hd = 128
    S = len(q_lens)
    totals = [a + b for a, b in zip(q_lens, pos0)]
    # the second sequence has a hole in its block table (a block the cache dropped): its keys are masked, not read
    kv, bt = _make_cache(S, totals, nkv, hd, bs, 160 * 16 // bs, holes=[(1, 1)] if totals[1] > 2 * bs else ())
    cu = torch.tensor([0] + [int(v) for v in torch.tensor(q_lens).cumsum(0)], dtype=torch.int32, device="cuda")
    p0 = torch.tensor(pos0, dtype=torch.int32, device="cuda")
    total = sum(q_lens)
    q = torch.randn(total, (nh + 2 * nkv) * hd, device="cuda").half()
    out = torch.full((total + 3, nh * hd), 7.0, dtype=torch.float16, device="cuda")
    native.attn_prefill_tc(q, q.stride(0), total, kv, bt, cu, p0, out, out.stride(0), S, max(q_lens), nh, nkv, hd, bs,
                           1 / math.sqrt(hd), ops.status.ptr, mode)
    torch.cuda.synchronize()
    ops.check()
    want = ref.attn_prefill(q[:, : nh * hd], kv, bt, cu, p0, nh, nkv, hd, bs, 1 / math.sqrt(hd))
    assert (out[:total].float() - want.float()).abs().max() < 4e-3
    assert torch.all(out[total:] == 7.0)                       # nothing past the last row is written
    old = torch.zeros(total, nh * hd, dtype=torch.float16, device="cuda")
    ops.attn_prefill(q, kv, bt, cu, p0, old, S, total, max(q_lens), nh, nkv, hd, bs, 1 / math.sqrt(hd))
    torch.cuda.synchronize()
    assert (out[:total].float() - old.float()).abs().max() < 4e-3


def test_argmax_and_sampling_distribution(ops):
    V, M = 5000, 6
    logits = (torch.randn(M, V, device="cuda") * 2).half()
    logits[2, 77] = 30.0
    out = torch.zeros(M, dtype=torch.int32, device="cuda")
    ops.argmax(logits, out, M)
    torch.cuda.synchronize()
    assert torch.equal(out.long().cpu(), logits.float().argmax(-1).cpu())
    # sampling: empirical distribution of row 0 under temperature/top-k/top-p vs the exact filtered distribution
    T, k, p = 0.8, 40, 0.9
    n_draw = 4000
    row = logits[:1].repeat(n_draw, 1).contiguous()
    temp = torch.full((n_draw,), T, device="cuda")
    tk = torch.full((n_draw,), k, dtype=torch.int32, device="cuda")
    tp = torch.full((n_draw,), p, device="cuda")
    seeds = torch.arange(n_draw, dtype=torch.int64, device="cuda")
    draws = torch.zeros(n_draw, dtype=torch.int32, device="cuda")
    ops.sample(row, draws, n_draw, temp, tk, tp, seeds, 5)
    d2 = torch.zeros_like(draws)
    ops.sample(row, d2, n_draw, temp, tk, tp, seeds, 5)
    torch.cuda.synchronize()
    assert torch.equal(draws, d2)                       # same seeds, same step -> same tokens
    want = ref.filtered_probs(logits[0], T, k, p).cpu()
    support = want > 0
    got = torch.bincount(draws.long().cpu(), minlength=V).float() / n_draw
    assert got[~support].sum() == 0                     # nothing outside the kept set
    assert (got - want).abs().max() < 0.03
    # greedy rows inside a sampling launch
    temp[:10] = 0
    ops.sample(row, draws, n_draw, temp, tk, tp, seeds, 6)
    torch.cuda.synchronize()
    assert (draws[:10].long().cpu() == int(logits[0].float().argmax())).all()


def test_repetition_penalty(ops):
    logits = torch.tensor([[2.0, -2.0, 1.0, 0.5]], device="cuda").half().repeat(2, 1).contiguous()
    rows = torch.tensor([0, 0, 1], dtype=torch.int32, device="cuda")
    toks = torch.tensor([0, 1, 2], dtype=torch.int32, device="cuda")
    cnt = torch.tensor([1, 4, 2], dtype=torch.int32, device="cuda")
    pen = torch.tensor([1.5, 2.0], device="cuda")
    ops.apply_repetition_penalty(logits, rows, toks, cnt, 3, pen)
    torch.cuda.synchronize()
    assert abs(float(logits[0, 0]) - 2.0 / 1.5) < 2e-3
    assert abs(float(logits[0, 1]) + 2.0 * 1.5 ** 3) < 1e-2
    assert abs(float(logits[1, 2]) - 1.0 / 2.0 ** 2) < 2e-3 and float(logits[1, 3]) == 0.5


def test_lora_shrink_expand(ops):
    M, K, N, r, A = 9, 512, 384, 16, 3
    x = torch.randn(M, K, device="cuda").half()
    a = (torch.randn(A, r, K, device="cuda") * 0.05).half()
    b = (torch.randn(A, N, r, device="cuda") * 0.05).half()
    ids = torch.tensor([0, 2, -1, 1, 1, 0, -1, 2, 2], dtype=torch.int32, device="cuda")
    scales = torch.tensor([2.0, 0.5, 1.0], device="cuda")
    y = torch.randn(M, N + 64, device="cuda").half()
    y0 = y.clone()
    ops.lora_apply(x, a, b, ids, scales, y, M, K, N, r, y_col0=64)
    torch.cuda.synchronize()
    for t in range(M):
        i = int(ids[t])
        want = y0[t, 64:].float()
        if i >= 0:
            want = want + ref.lora_delta(x[t:t + 1], a[i], b[i], float(scales[i]))[0]
        assert (y[t, 64:].float() - want).abs().max() < 5e-3
        assert torch.equal(y[t, :64], y0[t, :64])


def test_read_probe_runs_and_rejects_bad_arguments(ops):
    """The bandwidth probe of the microbenchmark: a launch over a small buffer completes without touching its sink,
    and sizes it cannot split are refused on the host."""
    from zse_b200.ops import native
    buf = torch.ones(1 << 20, dtype=torch.uint8, device="cuda")
    sink = torch.zeros(1, dtype=torch.int32, device="cuda")
    native.read_probe(buf, buf.numel(), 3, 16, sink)
    torch.cuda.synchronize()
    assert int(sink.item()) == 0
    with pytest.raises(Exception):
        native.read_probe(buf, 1024, 1, 16, sink)          # fewer than 512 loads of 16 bytes
    with pytest.raises(Exception):
        native.read_probe(buf, buf.numel(), 0, 16, sink)

"""The kernel-language library ``zse_b200.dsl.kernels``: every kernel is emulated on the CPU against plain torch, and
every one compiles to a cubin for sm_100a (nvcc needs no GPU).  The GPU launches are in tests/test_dsl_gpu.py."""
import numpy as np
import pytest
import torch

from zse_b200.dsl import kernels as K
from zse_b200.format import quantize as Q
from zse_b200.ops import reference as ref


def _int4(N, Kd, seed=0):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((N, Kd)) * 0.05).astype(np.float32)
    p, s, z = Q.quantize_int4_arrays(w, 128)
    deq = Q.dequantize_int4_arrays(p, s, z, N * Kd, 128).reshape(N, Kd)
    return (torch.from_numpy(p.copy()), torch.from_numpy(s.copy()), torch.from_numpy(z.copy()),
            torch.from_numpy(deq))


def cases():
    """name -> (kernel, grid, block, args, outputs to compare as (tensor, wanted, atol))."""
    g = torch.Generator().manual_seed(3)
    out = {}
    a, b = torch.randn(150, generator=g), torch.randn(150, generator=g)
    o = torch.zeros(150)
    out["vector_add"] = (K.vector_add, (3,), (64,), (a, b, o, 150), [(o, a + b, 0)])
    x, bias = torch.randn(6, 40, generator=g), torch.randn(40, generator=g)
    o = torch.zeros(6, 40)
    out["add_bias"] = (K.add_bias, (4,), (64,), (x, bias, o, 240, 40), [(o, x + bias, 1e-6)])
    o = torch.zeros(240)
    out["silu"] = (K.silu, (4,), (64,), (x.reshape(-1), o, 240), [(o, torch.nn.functional.silu(x.reshape(-1)), 1e-5)])
    up = torch.randn(240, generator=g)
    o = torch.zeros(240)
    out["swiglu"] = (K.swiglu, (4,), (64,), (x.reshape(-1), up, o, 240),
                     [(o, torch.nn.functional.silu(x.reshape(-1)) * up, 1e-5)])
    xs, w = torch.randn(3, 200, generator=g), torch.rand(200, generator=g) + 0.5
    o = torch.zeros(3, 200)
    out["rmsnorm"] = (K.rmsnorm, (3,), (64,), (xs, w, o, 200, 1e-6), [(o, ref.rmsnorm(xs, w, 1e-6).float(), 1e-4)])
    xl, wl = torch.randn(3, 50, generator=g), torch.rand(50, generator=g) + 0.5
    o = torch.zeros(3, 50)
    out["layernorm"] = (K.layernorm, (3,), (64,), (xl, wl, o, 50),
                        [(o, torch.nn.functional.layer_norm(xl, (50,), eps=1e-5) * wl, 1e-4)])
    xm = torch.randn(5, 20, generator=g)
    o = torch.zeros(5, 20)
    out["softmax_warp"] = (K.softmax_warp, (5,), (32,), (xm, o, 20), [(o, torch.softmax(xm, -1), 1e-6)])
    p, s, z, deq = _int4(4, 256)
    o = torch.zeros(4 * 256, dtype=torch.float16)
    out["dequant_rows"] = (K.dequant_rows, (2,), (64,), (p, s, z, o, 8), [(o, deq.reshape(-1), 2e-3)])
    xh = torch.randn(3, 256, generator=g).half()
    p, s, z, deq = _int4(6, 256, seed=1)
    o = torch.zeros(3, 6, dtype=torch.float16)
    out["dequant_matmul_int4"] = (K.dequant_matmul_int4, (1,), (32,), (xh, p, s, z, o, 3, 6, 256),
                                  [(o, xh.float() @ deq.T, 5e-3)])
    q8 = torch.randint(-127, 127, (6, 256), dtype=torch.int8, generator=g)
    sc = (torch.rand(6, 2, generator=g) * 0.01).half()
    w8 = (q8.float().view(6, 2, 128) * sc.float()[:, :, None]).view(6, 256)
    o = torch.zeros(3, 6, dtype=torch.float16)
    out["dequant_matmul_int8"] = (K.dequant_matmul_int8, (1,), (32,), (xh, q8, sc, o, 3, 6, 256, 128),
                                  [(o, xh.float() @ w8.T, 2e-2)])
    o = torch.zeros(6, dtype=torch.float16)
    out["gemv_int4_warp"] = (K.gemv_int4_warp, (3,), (64,), (xh[0].contiguous(), p, s, z, o, 6, 256),
                             [(o, (xh[0].float() @ deq.T), 5e-3)])
    nh, nkv, hd, bs, T = 2, 1, 16, 4, 5
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, generator=g).half()
    cache = torch.zeros(3, 2, nkv, bs, hd, dtype=torch.float16)
    pos = torch.tensor([0, 3, 7, 2, 9], dtype=torch.int32)
    slots = torch.tensor([0, 5, -1, 11, 2], dtype=torch.int32)
    inv = ref.inv_freq(hd, 10000.0)
    want_q, want_c = qkv.clone(), cache.clone()
    ref.rope_kv_write(want_q, want_c, pos, slots.long(), inv, nh, nkv, hd, bs)
    n = T * (nh + 2 * nkv) * (hd // 2)
    out["rope_kv_write"] = (K.rope_kv_write, ((n + 31) // 32,), (32,), (qkv, cache, pos, slots, inv, T, nh, nkv, hd, bs),
                            [(qkv, want_q, 2e-3), (cache, want_c, 2e-3)])
    # decode attention over a paged cache: three sequences (one of them with a dropped block), GQA 4:2, head_dim 64
    nh, nkv, hd, bs, S, mb = 4, 2, 64, 4, 3, 5
    lens = torch.tensor([9, 1, 17], dtype=torch.int32)
    cache = (torch.randn(12, 2, nkv, bs, hd, generator=g) * 0.5).half()
    bt = torch.tensor([[3, 7, 1, -1, -1], [0, -1, -1, -1, -1], [5, -1, 2, 9, 4]], dtype=torch.int32)   # -1 inside: a hole
    ld = (nh + 2 * nkv) * hd
    qkv = torch.randn(S, ld, generator=g).half()
    o = torch.zeros(S, nh * hd, dtype=torch.float16)
    want = torch.zeros(S, nh, hd)
    for sq in range(S):
        for h in range(nh):
            keys, vals = [], []
            for t in range(int(lens[sq])):
                b = int(bt[sq, t // bs])
                if b >= 0:
                    keys.append(cache[b, 0, h // (nh // nkv), t % bs].float())
                    vals.append(cache[b, 1, h // (nh // nkv), t % bs].float())
            kk, vv = torch.stack(keys), torch.stack(vals)
            pr = torch.softmax((kk @ qkv[sq, h * hd:(h + 1) * hd].float()) / 8.0, 0)
            want[sq, h] = pr @ vv
    out["paged_attention"] = (K.paged_attention, (S, nh), (32,),
                              (o, qkv, cache, bt, lens, nh, nkv, hd, bs, mb, ld, 1 / 8.0),
                              [(o, want.reshape(S, nh * hd), 3e-3)])
    # shared-memory tiled INT4 GEMM with ragged edges in M and N
    xm = torch.randn(21, 256, generator=g).half()
    p, s, z, deq = _int4(37, 256, seed=2)
    o = torch.zeros(21, 37, dtype=torch.float16)
    out["tiled_dequant_matmul_int4"] = (K.tiled_dequant_matmul_int4, (3, 2), (16, 16), (xm, p, s, z, o, 21, 37, 256),
                                        [(o, xm.float() @ deq.T, 8e-3)])
    return out


def test_library_covers_the_inference_kernels():
    assert set(cases()) == set(K.ALL)
    assert K.bgemv_int4_wave32 is K.gemv_int4_warp and K.fused_rope_kv_write is K.rope_kv_write
    assert set(K.REFERENCE_NAMES.values()) <= set(K.ALL) and not set(K.REFERENCE_NAMES) & set(K.ALL)


@pytest.mark.parametrize("name", sorted(K.ALL))
def test_kernel_emulated_against_torch(name):
    kern, grid, block, args, checks = cases()[name]
    kern.emulate(grid, block, args, check_races=name not in ("dequant_matmul_int8",))
    for got, want, atol in checks:
        torch.testing.assert_close(got.float(), want.float(), atol=atol, rtol=1e-3)


@pytest.mark.timeout(900)
def test_every_library_kernel_compiles_for_sm_100a(tmp_path, monkeypatch):
    monkeypatch.setenv("ZSE_KERNEL_CACHE", str(tmp_path))
    for name, (kern, grid, block, args, _) in cases().items():
        sig = dict(kern._sig_of_args(args))
        ck = kern.compile("cuda", sig)
        assert ck.cubin and len(ck.cubin) > 512, name

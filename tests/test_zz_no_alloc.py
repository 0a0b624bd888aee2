"""Decode attention with library-owned scratch (csrc/attn_decode_static.h) against the entry point that takes the
caller's scratch.  Collected last on purpose: the fixed array is shared by every call on the device, so the check
also has to hold after everything else in the suite has run, and on two calls in a row."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

ARGS = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
        ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
        ctypes.c_int, ctypes.c_float, ctypes.c_void_p]


@pytest.fixture(scope="module")
def lib():
    from zse_b200.ops import native
    native.load()
    so = ctypes.CDLL(native.lib_path())
    so.zse_attn_decode_static.restype, so.zse_attn_decode_static.argtypes = ctypes.c_int, ARGS
    so.zse_attn_decode_static_setup.restype, so.zse_attn_decode_static_setup.argtypes = ctypes.c_int, []
    so.zse_attn_decode_static_max_floats.restype = ctypes.c_int64
    so.zse_attn_decode_static_max_floats.argtypes = []
    return so


def _case(seed, lens, nh, nkv, hd, bs, blocks):
    g = torch.Generator(device="cuda").manual_seed(seed)
    S = len(lens)
    kv = (torch.randn(blocks, 2, nkv, bs, hd, device="cuda", generator=g) * 0.5).half()
    maxb = (max(lens) + bs - 1) // bs + 1
    bt = torch.full((S, maxb), -1, dtype=torch.int32, device="cuda")
    perm = torch.randperm(blocks, generator=torch.Generator().manual_seed(seed))
    at = 0
    for s, n in enumerate(lens):
        nb = (n + bs - 1) // bs
        bt[s, :nb] = perm[at:at + nb].int().cuda()
        at += nb
    q = torch.randn(S, (nh + 2 * nkv) * hd, device="cuda", generator=g).half()
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    return q, kv, bt, sl


def _static(lib, q, kv, bt, sl, nh, nkv, hd, bs, splits):
    S = q.shape[0]
    out = torch.zeros(S, nh * hd, dtype=torch.float16, device="cuda")
    rc = lib.zse_attn_decode_static(q.data_ptr(), q.stride(0), kv.data_ptr(), bt.data_ptr(), bt.shape[1],
                                    sl.data_ptr(), out.data_ptr(), out.stride(0), S, nh, nkv, hd, bs, splits,
                                    1 / math.sqrt(hd), torch.cuda.current_stream().cuda_stream)
    return rc, out


def _dynamic(q, kv, bt, sl, nh, nkv, hd, bs, splits):
    from zse_b200.ops import native
    S = q.shape[0]
    out = torch.zeros(S, nh * hd, dtype=torch.float16, device="cuda")
    scratch = torch.empty(max(1, native.attn_decode_scratch_floats(S, nh, hd, splits)), device="cuda")
    native.attn_decode(q, q.stride(0), kv, bt, bt.shape[1], sl, out, out.stride(0), scratch, S, nh, nkv, hd, bs,
                       splits, 1 / math.sqrt(hd))
    return out


def test_static_scratch_matches_caller_scratch_twice_in_a_row(lib):
    assert lib.zse_attn_decode_static_setup() == 0
    nh, nkv, hd, bs = 28, 4, 128, 16
    # two different calls back to back: the second reuses the array the first one filled
    for seed, lens, splits in [(1, [1, 15, 16, 17, 200, 333, 64, 5], 8), (2, [700, 3, 129], 5),
                               (3, [40, 41], 1)]:
        q, kv, bt, sl = _case(seed, lens, nh, nkv, hd, bs, 128)
        want = _dynamic(q, kv, bt, sl, nh, nkv, hd, bs, splits)
        rc1, got1 = _static(lib, q, kv, bt, sl, nh, nkv, hd, bs, splits)
        rc2, got2 = _static(lib, q, kv, bt, sl, nh, nkv, hd, bs, splits)
        torch.cuda.synchronize()
        assert rc1 == 0 and rc2 == 0
        assert torch.equal(got1, want) and torch.equal(got2, want)


def test_static_scratch_rejects_oversized_call(lib):
    limit = lib.zse_attn_decode_static_max_floats()
    nh, nkv, hd, bs, splits = 32, 8, 128, 16, 16
    S = limit // (nh * splits * (hd + 2)) + 1
    q, kv, bt, sl = _case(4, [8] * S, nh, nkv, hd, bs, S)
    rc, out = _static(lib, q, kv, bt, sl, nh, nkv, hd, bs, splits)
    torch.cuda.synchronize()
    assert rc == -5                      # ZSE_ERR_LIMIT: nothing was launched
    assert float(out.abs().max()) == 0.0
    rc, _ = _static(lib, q, kv, bt, sl, nh, nkv, hd, bs, 1)   # the same batch without splits needs no scratch
    torch.cuda.synchronize()
    assert rc == 0

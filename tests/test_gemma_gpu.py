"""Gemma-family kernels (csrc/gemma.cu) against their plain-PyTorch fp32 restatement, and the Gemma-2 / Gemma-4
engine path on the GPU against the fp32 oracle model."""
import math
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

from zse_b200.ops import reference as ref


@pytest.fixture(scope="module")
def ops():
    from zse_b200.ops.backend import CudaOps
    o = CudaOps("cuda")
    yield o
    o.check()


def _pool_view(blocks, nkv, bs, hd, width):
    """A layer's [blocks, 2, nkv, bs, hd] view inside pool rows of `width` >= nkv*hd elements per token."""
    pool = torch.zeros(blocks, 2, 1, bs, width, dtype=torch.float16, device="cuda")
    view = pool.as_strided((blocks, 2, nkv, bs, hd), (pool.stride(0), pool.stride(1), bs * hd, hd, 1), 0)
    return pool, view


@pytest.mark.parametrize("hd,nh,nkv,rot,k_is_v,norm,width", [
    (64, 4, 2, 64, False, True, 128), (128, 4, 1, 32, True, True, 128), (256, 8, 4, 256, False, False, 1024),
    (512, 2, 1, 128, True, True, 512), (16, 4, 2, 16, False, True, 32), (96, 3, 1, 48, False, True, 96)])
def test_headnorm_rope_kv_write(ops, hd, nh, nkv, rot, k_is_v, norm, width):
    M, blocks, bs = 19, 8, 16
    ld = (nh + (1 if k_is_v else 2) * nkv) * hd
    qkv = torch.randn(M, ld, device="cuda").half()
    pool, kv = _pool_view(blocks, nkv, bs, hd, width)
    pool2 = pool.clone()
    kv2 = pool2.as_strided(kv.shape, kv.stride(), 0)
    pos = torch.randint(0, 4000, (M,), device="cuda", dtype=torch.int32)
    slots = torch.randperm(blocks * bs, device="cuda")[:M].long()
    slots[5] = -1
    from zse_b200.models.gemma import rope_table
    freqs = rope_table(hd, 1e6, rot).cuda()
    qw = (1 + 0.2 * torch.randn(hd, device="cuda")).half() if norm else None
    kw = (1 + 0.2 * torch.randn(hd, device="cuda")).half() if norm else None
    q2 = qkv.clone()
    ref.headnorm_rope_kv_write(q2, kv2, pos, slots, freqs, qw, kw, norm, k_is_v, 1e-6, nh, nkv, hd, bs)
    ops.headnorm_rope_kv_write(qkv, kv, pos, slots, freqs, qw, kw, norm, k_is_v, 1e-6, M, nh, nkv, hd, bs)
    torch.cuda.synchronize()
    assert (qkv[:, : nh * hd].float() - q2[:, : nh * hd].float()).abs().max() < 6e-3
    assert torch.equal(qkv[:, nh * hd:], q2[:, nh * hd:])      # k and v columns are left as the projection wrote them
    assert (pool.float() - pool2.float()).abs().max() < 6e-3
    assert pool2.abs().sum() > 0


def _cache(S, lens, nkv, hd, bs, blocks, width, holes=()):
    pool, kv = _pool_view(blocks, nkv, bs, hd, width)
    kv.copy_((torch.randn(kv.shape, device="cuda") * 0.5).half())
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


@pytest.mark.parametrize("hd,nh,nkv,softcap,window,width", [
    (64, 4, 2, 50.0, 24, 128), (128, 8, 1, 0.0, 0, 256), (256, 8, 4, 50.0, 100, 1024), (512, 4, 1, 0.0, 0, 512),
    (16, 4, 2, 30.0, 7, 32), (96, 6, 2, 0.0, 40, 192)])
def test_attn_generic_decode(ops, hd, nh, nkv, softcap, window, width):
    lens = [1, 15, 16, 17, 200, 333, 64, 5]
    S, bs = len(lens), 16
    kv, bt = _cache(S, lens, nkv, hd, bs, 64, width, holes=[(4, 2), (5, 20)])
    q = torch.randn(S, (nh + 2 * nkv) * hd, device="cuda").half()
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    out = torch.zeros(S, nh * hd, dtype=torch.float16, device="cuda")
    scale = 1 / math.sqrt(hd)
    want = ref.attn_decode(q[:, : nh * hd], kv, bt, sl, nh, nkv, hd, bs, scale, softcap, window)
    # the dispatching op (tensor-core kernel for head_dim 64/128/256, CUDA-core kernel otherwise), with and without
    # a split of the keys, and the CUDA-core kernel on its own
    for splits in (1, 3):
        out.zero_()
        scratch = torch.zeros(S * nh * splits * (hd + 2), device="cuda")
        ops.attn_decode(q, kv, bt, sl, out, S, nh, nkv, hd, bs, scale, scratch, splits, softcap=softcap, window=window)
        torch.cuda.synchronize()
        assert (out.float() - want.float()).abs().max() < 3e-3, splits
    out.zero_()
    ops.n.attn_generic(q, q.stride(0), kv, bt, sl, None, None, S, out, out.stride(0), S, nh, nkv, hd, bs, scale,
                       softcap, window)
    torch.cuda.synchronize()
    assert (out.float() - want.float()).abs().max() < 3e-3


@pytest.mark.parametrize("hd,nh,nkv,softcap,window,width", [
    (64, 4, 2, 50.0, 24, 128), (128, 4, 1, 0.0, 0, 128), (256, 4, 2, 50.0, 60, 512), (32, 2, 1, 0.0, 9, 64)])
def test_attn_generic_prefill_chunks(ops, hd, nh, nkv, softcap, window, width):
    q_lens, pos0 = [130, 70, 5], [0, 100, 37]
    S, bs = 3, 16
    totals = [a + b for a, b in zip(q_lens, pos0)]
    kv, bt = _cache(S, totals, nkv, hd, bs, 64, width, holes=[(1, 1)])
    cu = torch.tensor([0, 130, 200, 205], dtype=torch.int32, device="cuda")
    p0 = torch.tensor(pos0, dtype=torch.int32, device="cuda")
    q = torch.randn(205, (nh + 2 * nkv) * hd, device="cuda").half()
    out = torch.zeros(205, nh * hd, dtype=torch.float16, device="cuda")
    scale = 1 / math.sqrt(hd)
    want = ref.attn_prefill(q[:, : nh * hd], kv, bt, cu, p0, nh, nkv, hd, bs, scale, softcap, window)
    ops.attn_prefill(q, kv, bt, cu, p0, out, S, 205, 130, nh, nkv, hd, bs, scale, softcap=softcap, window=window)
    torch.cuda.synchronize()
    assert (out.float() - want.float()).abs().max() < 3e-3
    out.zero_()
    ops.n.attn_generic(q, q.stride(0), kv, bt, None, cu, p0, S, out, out.stride(0), 205, nh, nkv, hd, bs, scale,
                       softcap, window)
    torch.cuda.synchronize()
    assert (out.float() - want.float()).abs().max() < 3e-3


@pytest.mark.parametrize("M,H,scalar,has_next", [(1, 256, True, True), (37, 3584, False, True), (64, 5120, True, False),
                                                 (5, 100, True, True)])
def test_norm_add_rmsnorm_glu_and_softcap(ops, M, H, scalar, has_next):
    x = torch.randn(M + 2, H, device="cuda").half()
    res = torch.randn(M + 2, H, device="cuda")
    w_post = (1 + 0.1 * torch.randn(H, device="cuda")).half()
    w_next = (1 + 0.1 * torch.randn(H, device="cuda")).half() if has_next else None
    sc = torch.tensor([0.83], device="cuda").half() if scalar else None
    out = torch.full((M + 2, H), 3.0, dtype=torch.float16, device="cuda")
    res2 = res.clone()
    want = ref.norm_add_rmsnorm(x[:M], w_post, res2[:M], sc, w_next, 1e-6)
    ops.norm_add_rmsnorm(x, w_post, res, sc, w_next, out if has_next else None, M, 1e-6)
    torch.cuda.synchronize()
    assert (res - res2).abs().max() < 1e-4 * max(1.0, float(res2.abs().max()))
    assert torch.equal(res[M:], res2[M:])
    if has_next:
        assert (out[:M].float() - want.float()).abs().max() < 4e-3
        assert torch.all(out[M:] == 3.0)
    # GeGLU on a [M, 2I] projection output and soft-capped logits
    I = 2 * (H // 4)
    gu = torch.randn(M, 2 * I, device="cuda").half()
    act = torch.zeros(M, I, dtype=torch.float16, device="cuda")
    ops.glu(gu, act, M, I, True)
    assert (act.float() - ref.swiglu(gu[:, :I], gu[:, I:], True).float()).abs().max() < 4e-3
    logits = (torch.randn(M, 1000, device="cuda") * 40).half()
    want_l = ref.softcap(logits, 30.0)
    ops.softcap(logits, M, 30.0)
    torch.cuda.synchronize()
    assert (logits.float() - want_l.float()).abs().max() < 3e-2


@pytest.mark.parametrize("shape,quant", [("tiny-gemma2", "fp16"), ("tiny-gemma4", "fp16"), ("tiny-gemma2", "int4"),
                                         ("tiny-gemma4", "int4")])
def test_gemma_engine_matches_oracle(tmp_path, shape, quant):
    """Greedy tokens of the CUDA engine (batched decode with CUDA graphs, chunked prefill past the sliding window)
    against the fp32 oracle; fp16 rounding may flip a near-tie, so a token may differ only where the oracle's own
    top-2 logits are close."""
    from zse_b200.config import EngineConfig
    from zse_b200.engine import ZStreamerEngine
    from zse_b200.format import synth
    from zse_b200.format.loader import ZSELoader
    from zse_b200.models.oracle import OracleModel
    path = str(tmp_path / "m.zse")
    synth.write_random_model(path, synth.shape_config(shape, quant), seed=5, std=0.05)
    oracle = OracleModel(ZSELoader(path))
    eng = ZStreamerEngine(path, config=EngineConfig(device="cuda", max_batch_seqs=8, max_seq_len=256, quiet=True,
                                                    prefill_chunk_size=32, max_batch_tokens=64))
    rng = random.Random(0)
    prompts = [[rng.randrange(1000) for _ in range(rng.randint(3, 70))] for _ in range(5)]
    ids = [eng.add_request_tokens(p, max_tokens=12, temperature=0.0, stop_tokens=[]) for p in prompts]
    eng.run_until_done()
    for p, i in zip(prompts, ids):
        got = eng.get_result(i).output_tokens
        seq = list(p)
        for tok in got:
            logits = oracle.forward(seq)[-1]
            top = torch.topk(logits, 2)
            if tok != int(top.indices[0]):
                assert tok == int(top.indices[1]) and float(top.values[0] - top.values[1]) < 0.05, (shape, quant)
            seq.append(tok)
    eng.destroy()

"""The plain-PyTorch restatement of the device ops (zse_b200/ops/reference.py) is what every CUDA kernel is compared
against, so it gets checked itself: each function against a hand-computed case or an independent scalar loop, on
CPU.  A mistake in the oracle would otherwise be copied into the kernels unnoticed."""
import math

import pytest
import torch

from zse_b200.ops import reference as ref


def test_int4_groups_are_flat_and_low_nibble_first():
    packed = torch.tensor([0x21, 0x43, 0xF0, 0x5A], dtype=torch.uint8)           # values 1,2,3,4 | 0,15,10,5
    scales = torch.tensor([0.5, 2.0], dtype=torch.float16)
    zeros = torch.tensor([-1.0, 1.0], dtype=torch.float16)
    w = ref.dequant_int4(packed, scales, zeros, (2, 4), group_size=4)
    assert w.tolist() == [[-0.5, 0.0, 0.5, 1.0], [1.0, 31.0, 21.0, 11.0]]
    w = ref.dequant_int4(packed, scales, zeros, (7,), group_size=4)              # a tail shorter than its group
    assert w.tolist() == [-0.5, 0.0, 0.5, 1.0, 1.0, 31.0, 21.0]
    w = ref.dequant_int4(packed, scales, zeros, (4, 2), group_size=4)            # groups ignore the row length
    assert w[2].tolist() == [1.0, 31.0]


def test_int8_groups():
    q = torch.tensor([1, -2, 127, -128, 5, 6], dtype=torch.int8)
    w = ref.dequant_int8(q, torch.tensor([0.5, 2.0, 9.0], dtype=torch.float16), (2, 2), group_size=2)
    assert w.tolist() == [[0.5, -1.0], [254.0, -256.0]]


def test_linear_accumulates_in_fp32_and_saturates():
    x = torch.tensor([[1.0, 2.0], [300.0, 300.0]], dtype=torch.float16)
    w = torch.tensor([[3.0, 4.0], [200.0, 200.0]])
    y = ref.linear(x, w, bias=torch.tensor([1.0, 0.0]))
    assert y.dtype == torch.float16
    assert y.tolist() == [[12.0, 600.0], [2100.0, 65504.0]]      # 2101 rounds to even; 120000 is clamped
    assert torch.isfinite(y).all()


def test_swiglu_and_its_gelu_form():
    g = torch.tensor([0.0, 1.0, -2.0], dtype=torch.float16)
    u = torch.tensor([5.0, 2.0, 3.0], dtype=torch.float16)
    want = [0.0, 2.0 / (1 + math.exp(-1.0)), -6.0 / (1 + math.exp(2.0))]
    assert ref.swiglu(g, u).float().tolist() == pytest.approx(want, rel=1e-3)
    gelu = lambda v: 0.5 * v * (1 + math.tanh(math.sqrt(2 / math.pi) * (v + 0.044715 * v ** 3)))
    assert ref.swiglu(g, u, gelu=True).float().tolist() == pytest.approx([0.0, 2 * gelu(1.0), 3 * gelu(-2.0)],
                                                                           rel=2e-3, abs=1e-4)


def test_rmsnorm_hand_case():
    y = ref.rmsnorm(torch.tensor([[3.0, 4.0]]), torch.tensor([1.0, 2.0]), eps=0.0)
    r = math.sqrt(12.5)
    assert y.dtype == torch.float16 and y.float().tolist()[0] == pytest.approx([3 / r, 8 / r], rel=1e-3)
    assert ref.rmsnorm(torch.zeros(1, 4), torch.ones(4), eps=1e-6).abs().sum() == 0       # eps keeps zero rows finite


def test_frequency_table_and_scaling_rules():
    f = ref.inv_freq(8, 10000.0)
    assert f.dtype == torch.float32 and f.tolist() == pytest.approx([1.0, 0.1, 0.01, 0.001], rel=1e-6)
    assert ref.inv_freq(8, 10000.0, {"type": "linear", "factor": 4.0}).tolist() == pytest.approx(
        [0.25, 0.025, 0.0025, 0.00025], rel=1e-6)
    sc = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 8192}
    g = ref.inv_freq(8, 10000.0, sc).tolist()
    assert g[0] == pytest.approx(1.0) and g[1] == pytest.approx(0.1) and g[2] == pytest.approx(0.01)   # short waves stay
    s3 = (8192 * 0.001 / (2 * math.pi) - 1.0) / 3.0                               # wave length 6283: in between
    assert 0 < s3 < 1 and g[3] == pytest.approx(0.001 * (1 - s3) / 8 + 0.001 * s3, rel=1e-5)
    far = ref.inv_freq(8, 1e8, sc).tolist()
    assert far[3] == pytest.approx(1e-6 / 8)                                      # a long wave is slowed by the factor
    assert ref.inv_freq(8, 10000.0, {"rope_type": "default"}).tolist() == f.tolist()


def test_rope_rotates_half_pairs_and_leaves_the_rest():
    x = torch.zeros(2, 1, 6)
    x[:, 0] = torch.tensor([1.0, 2.0, 3.0, 4.0, 7.0, 9.0])
    freqs = torch.tensor([1.0, 0.5])                                              # rotary width 4 of 6
    y = ref.rope_(x, torch.tensor([0, 3]), freqs)
    assert y[0, 0].tolist() == [1.0, 2.0, 3.0, 4.0, 7.0, 9.0]                     # position 0: identity
    c0, s0, c1, s1 = math.cos(3.0), math.sin(3.0), math.cos(1.5), math.sin(1.5)
    want = [1 * c0 - 3 * s0, 2 * c1 - 4 * s1, 3 * c0 + 1 * s0, 4 * c1 + 2 * s1, 7.0, 9.0]
    assert y[1, 0].tolist() == pytest.approx(want, rel=1e-5)
    assert y[1, 0, :4].norm().item() == pytest.approx(x[1, 0, :4].norm().item(), rel=1e-5)   # a rotation


def test_rope_kv_write_scatters_by_slot():
    nh, nkv, hd, bs = 2, 1, 4, 2
    torch.manual_seed(0)
    qkv = torch.randn(3, (nh + 2 * nkv) * hd)
    before = qkv.clone()
    kv = torch.zeros(3, 2, nkv, bs, hd)
    freqs = ref.inv_freq(hd, 10000.0)
    pos = torch.tensor([0, 5, 6])
    ref.rope_kv_write(qkv, kv, pos, torch.tensor([4, -1, 3]), freqs, nh, nkv, hd, bs)
    k_rot = ref.rope_(before[:, nh * hd:(nh + nkv) * hd].view(3, nkv, hd), pos, freqs)
    assert torch.equal(qkv[:, (nh + nkv) * hd:], before[:, (nh + nkv) * hd:])     # v is not rotated
    assert torch.allclose(qkv[:, nh * hd:(nh + nkv) * hd].view(3, nkv, hd), k_rot)
    assert torch.allclose(kv[2, 0, 0, 0], k_rot[0, 0]) and torch.allclose(kv[2, 1, 0, 0], before[0, 12:])   # slot 4
    assert torch.allclose(kv[1, 0, 0, 1], k_rot[2, 0]) and torch.allclose(kv[1, 1, 0, 1], before[2, 12:])   # slot 3
    assert kv[0].abs().sum() == 0 and kv[2, :, :, 1].abs().sum() == 0 and kv[1, :, :, 0].abs().sum() == 0   # -1: nowhere


def test_headnorm_variant_normalises_heads_and_can_share_k_as_v():
    nh, nkv, hd, bs, eps = 1, 1, 4, 2, 1e-6
    qkv = torch.tensor([[2.0, 0, 0, 0, 0, 3.0, 0, 0, 9.0, 9.0, 9.0, 9.0]])
    kv = torch.zeros(1, 2, nkv, bs, hd)
    ref.headnorm_rope_kv_write(qkv, kv, torch.tensor([0]), torch.tensor([1]), torch.zeros(2),
                               torch.full((hd,), 2.0), None, True, True, eps, nh, nkv, hd, bs)
    assert qkv[0, :4].tolist() == pytest.approx([4.0, 0, 0, 0], rel=1e-4)         # unit RMS: 2 -> sqrt(4) = 2, x weight
    assert kv[0, 0, 0, 1].tolist() == [0, 3.0, 0, 0]                              # k without a norm weight: as is
    assert kv[0, 1, 0, 1].tolist() == pytest.approx([0, 2.0, 0, 0], rel=1e-4)     # v = k's projection, normalised


def test_norm_add_rmsnorm_sandwich():
    res = torch.tensor([[1.0, 1.0]])
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float16)
    out = ref.norm_add_rmsnorm(x, torch.tensor([1.0, 1.0]), res, torch.tensor([2.0]), torch.tensor([1.0, 1.0]), 0.0)
    r = math.sqrt(12.5)
    want = [2 * (1 + 3 / r), 2 * (1 + 4 / r)]
    assert res.tolist()[0] == pytest.approx(want, rel=1e-6)                        # the residual is updated in place
    rr = math.sqrt((want[0] ** 2 + want[1] ** 2) / 2)
    assert out.float().tolist()[0] == pytest.approx([want[0] / rr, want[1] / rr], rel=1e-3)
    assert ref.norm_add_rmsnorm(x, torch.ones(2), res, None, None, 0.0) is None


def test_softcap():
    y = ref.softcap(torch.tensor([0.0, 50.0, -1000.0]), 50.0)
    assert y.tolist() == pytest.approx([0.0, 50 * math.tanh(1.0), -50.0], rel=1e-6)


def _cache(n_blocks, nkv, bs, hd, seed=0):
    torch.manual_seed(seed)
    return torch.randn(n_blocks, 2, nkv, bs, hd).to(torch.float16)


def _naive(q_row, kv, table, n, h, nh, nkv, hd, bs, scale, cap=0.0, first=0):
    """One head of one query by scalar loops over cache positions first..n-1."""
    g = h // (nh // nkv)
    scores, vals = [], []
    for t in range(first, n):
        blk = int(table[t // bs])
        if blk < 0:
            continue
        k = kv[blk, 0, g, t % bs].float()
        s = float((q_row[h * hd:(h + 1) * hd].float() * k).sum()) * scale
        scores.append(cap * math.tanh(s / cap) if cap else s)
        vals.append(kv[blk, 1, g, t % bs].float())
    if not scores:
        return torch.zeros(hd)
    m = max(scores)
    w = [math.exp(s - m) for s in scores]
    return sum(wi * v for wi, v in zip(w, vals)) / sum(w)


@pytest.mark.parametrize("cap,window", [(0.0, 0), (30.0, 0), (0.0, 3)])
def test_decode_attention_against_scalar_loops(cap, window):
    nh, nkv, hd, bs = 4, 2, 8, 4
    kv = _cache(6, nkv, bs, hd)
    tables = torch.tensor([[3, 1, 5], [2, -1, 0], [4, 4, 4]], dtype=torch.int32)   # a hole in sequence 1
    lens = torch.tensor([9, 10, 0])
    q = torch.randn(3, nh * hd).to(torch.float16)
    out = ref.attn_decode(q, kv, tables, lens, nh, nkv, hd, bs, 0.3, softcap=cap, window=window)
    assert out.dtype == torch.float16 and out[2].abs().sum() == 0                  # an empty sequence gives zeros
    for s in range(2):
        n = int(lens[s])
        for h in range(nh):
            want = _naive(q[s], kv, tables[s], n, h, nh, nkv, hd, bs, 0.3, cap, max(0, n - window) if window else 0)
            assert torch.allclose(out[s, h * hd:(h + 1) * hd].float(), want, atol=2e-3)


@pytest.mark.parametrize("window", [0, 2])
def test_prefill_attention_is_causal_from_the_cached_prefix(window):
    nh, nkv, hd, bs = 2, 1, 8, 4
    kv = _cache(5, nkv, bs, hd, seed=1)
    tables = torch.tensor([[2, 0, 4], [1, 3, -1]], dtype=torch.int32)
    cu_q = torch.tensor([0, 3, 3, 5])                                              # 3 rows, none, 2 rows
    tables = torch.cat([tables[:1], tables[:1], tables[1:]])
    pos0 = torch.tensor([4, 0, 0])                                                 # sequence 0 has 4 tokens cached
    q = torch.randn(5, nh * hd).to(torch.float16)
    out = ref.attn_prefill(q, kv, tables, cu_q, pos0, nh, nkv, hd, bs, 0.25, window=window)
    for s, (a, b) in enumerate([(0, 3), (3, 3), (3, 5)]):
        for r in range(a, b):
            pos = int(pos0[s]) + r - a
            for h in range(nh):
                want = _naive(q[r], kv, tables[s], pos + 1, h, nh, nkv, hd, bs, 0.25,
                              first=max(0, pos + 1 - window) if window else 0)
                assert torch.allclose(out[r, h * hd:(h + 1) * hd].float(), want, atol=2e-3)


def test_a_row_that_sees_only_holes_is_zero():
    kv = _cache(2, 1, 4, 8)
    out = ref.attn_decode(torch.ones(1, 8, dtype=torch.float16), kv, torch.tensor([[-1]], dtype=torch.int32),
                          torch.tensor([3]), 1, 1, 8, 4, 1.0)
    assert out.abs().sum() == 0 and torch.isfinite(out).all()


def test_repetition_penalty_grows_with_the_count():
    logits = torch.tensor([2.0, -2.0, 4.0, 1.0])
    out = ref.apply_repetition_penalty(logits, {0: 1, 1: 1, 2: 4, 9: 3, 3: 0}, 2.0)
    assert out.tolist() == [1.0, -4.0, 0.5, 1.0]                                   # 2^(1 + log2 4) = 8 for token 2
    assert logits.tolist() == [2.0, -2.0, 4.0, 1.0]                                # the input is not changed


def test_filtered_distribution():
    logits = torch.log(torch.tensor([0.5, 0.25, 0.125, 0.125]))
    assert ref.filtered_probs(logits, 1.0, 0, 1.0).tolist() == pytest.approx([0.5, 0.25, 0.125, 0.125])
    assert ref.filtered_probs(logits, 1.0, 2, 1.0).tolist() == pytest.approx([2 / 3, 1 / 3, 0, 0])
    assert ref.filtered_probs(logits, 1.0, 3, 1.0).tolist() == pytest.approx([0.5, 0.25, 0.125, 0.125])  # a tie stays
    assert ref.filtered_probs(logits, 1.0, 0, 0.7).tolist() == pytest.approx([2 / 3, 1 / 3, 0, 0])       # 0.5 < 0.7
    assert ref.filtered_probs(logits, 1.0, 0, 0.5).tolist() == pytest.approx([1, 0, 0, 0])
    assert ref.filtered_probs(logits, 1.0, 0, 0.8).tolist() == pytest.approx([0.5, 0.25, 0.125, 0.125])  # tie at the cut
    cold = ref.filtered_probs(logits, 0.5, 0, 1.0)                                 # T = 1/2 squares the odds
    assert cold.tolist() == pytest.approx([16 / 22, 4 / 22, 1 / 22, 1 / 22])
    assert ref.filtered_probs(logits, 0.0, 0, 1.0).tolist() == pytest.approx([1, 0, 0, 0])               # T -> 0: argmax


def test_lora_delta_shape_and_value():
    x = torch.tensor([[1.0, 2.0, 3.0]], dtype=torch.float16)
    a = torch.tensor([[1.0, 0.0, 1.0], [0.0, 1.0, 0.0]], dtype=torch.float16)       # r = 2
    b = torch.tensor([[1.0, 1.0], [2.0, 0.0], [0.0, -1.0], [0.5, 0.5]], dtype=torch.float16)
    d = ref.lora_delta(x, a, b, 0.5)
    assert d.dtype == torch.float32 and d.tolist() == [[3.0, 4.0, -1.0, 1.5]]

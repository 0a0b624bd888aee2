"""Per-kernel microbenchmarks with roofline fractions:  ``python -m zse_b200.runtime.microbench --shape qwen2.5-14b
--tokens 64``.

Times the kernels of one decoder layer (plus lm_head and token selection) at the given decode batch, cold-cache, with
CUDA events, and prints achieved GB/s (algorithmic bytes / time) against the measured copy bandwidth."""
from __future__ import annotations

import argparse
import json
import math

import torch

from ..format import synth
from ..ops import native
from ..ops.backend import CudaOps
from ..ops import reference as ref
from .profiler import KernelProfiler, measured_peaks


def _w4(ops, N, K, swiglu=False, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    parts = []
    for i in range(2 if swiglu else 1):
        packed = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device="cuda", generator=g)
        sc = torch.full((N, K // 128), 0.008, dtype=torch.float16, device="cuda")
        zr = torch.full((N, K // 128), -0.06, dtype=torch.float16, device="cuda")
        parts.append({"dtype": "int4", "data": packed, "scales": sc, "zeros": zr, "shape": (N, K)})
    return ops.make_linear(parts, K, 128, swiglu=swiglu)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="qwen2.5-14b")
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=1216, help="cached tokens per sequence for the attention kernel")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--only", default="", help="comma separated kernel names")
    ap.add_argument("--kv-block", type=int, default=16, help="tokens per KV block in the prefill-attention rows")
    ap.add_argument("--json", default="")
    ap.add_argument("--w4-mode", type=int, default=0, help="INT4 GEMM CTA shape: 0 planner, 1 wide, 2 narrow (2 per SM)")
    a = ap.parse_args()
    if a.w4_mode:
        from ..ops import native
        native.gemm_w4_set_mode(a.w4_mode)
    c = synth.shape_config(a.shape)
    ops = CudaOps("cuda")
    prof = KernelProfiler(iters=a.iters)
    peaks = measured_peaks()
    M, H, tp = a.tokens, c.hidden_size, a.tp
    from ..parallel.shard_plan import make_plan
    plan = make_plan(c, tp, 0)              # rank 0's shard: group-aligned, so possibly the larger of two sizes
    nh, nkv, hd = plan.num_heads, plan.num_kv_heads, c.head_dim
    q_dim, kv_dim, I = nh * hd, nkv * hd, plan.inter_size
    only = set(x for x in a.only.split(",") if x)
    rows = []
    x = (torch.randn(M, H, device="cuda") * 0.5).half()
    w4_bytes = lambda N, K: N * K // 2 + N * (K // 128) * 4

    def run(name, fn, nbytes, flops=0):
        if only and name not in only:
            return
        r = prof.time(name, fn, nbytes, flops)
        rows.append(r.row(peaks))
        ops.check()

    def want(*names) -> bool:
        """Whether any of these kernels will run: sections allocate their inputs only then (a capture of one kernel
        under a profiler should hold that kernel's few hundred MB, not the whole set)."""
        return not only or any(n in only for n in names)

    # linear layers
    wqkv = _w4(ops, q_dim + 2 * kv_dim, H)
    qkv = torch.zeros(M, q_dim + 2 * kv_dim, dtype=torch.float16, device="cuda")
    run("qkv_gemm", lambda: ops.linear(wqkv, x, M, qkv), w4_bytes(q_dim + 2 * kv_dim, H) + M * H * 2,
        2 * M * H * (q_dim + 2 * kv_dim))
    planes_q = torch.zeros(8, M, q_dim + 2 * kv_dim, dtype=torch.float32, device="cuda")
    run("qkv_gemm_planes", lambda: ops.linear_partial(wqkv, x, M, planes_q),
        w4_bytes(q_dim + 2 * kv_dim, H) + M * H * 2, 2 * M * H * (q_dim + 2 * kv_dim))
    wo = _w4(ops, H, q_dim)
    xa = (torch.randn(M, q_dim, device="cuda") * 0.5).half()
    planes = torch.zeros(8, M, H, dtype=torch.float32, device="cuda")
    run("o_gemm", lambda: ops.linear_partial(wo, xa, M, planes), w4_bytes(H, q_dim) + M * q_dim * 2, 2 * M * H * q_dim)
    wgu = _w4(ops, I, H, swiglu=True)
    act = torch.zeros(M, I, dtype=torch.float16, device="cuda")
    run("gate_up_gemm", lambda: ops.linear_swiglu(wgu, x, M, act), 2 * w4_bytes(I, H) + M * H * 2, 4 * M * H * I)
    wd = _w4(ops, H, I)
    xi = (torch.randn(M, I, device="cuda") * 0.5).half()
    run("down_gemm", lambda: ops.linear_partial(wd, xi, M, planes), w4_bytes(H, I) + M * I * 2, 2 * M * H * I)
    # norms
    resid = torch.randn(M, H, device="cuda")
    wn = torch.ones(H, dtype=torch.float16, device="cuda")
    xn = torch.zeros(M, H, dtype=torch.float16, device="cuda")
    n_pl = ops.linear_partial(wd, xi, M, planes) if want("add_rmsnorm") else 1
    run("add_rmsnorm", lambda: ops.add_rmsnorm(resid, planes, n_pl, None, wn, xn, M, 1e-6),
        M * H * (4 + 4 + 4 * n_pl + 2))
    # what the memory system delivers to all SMs at once: a 32 MB buffer that stays in L2 read 32 times (each CTA another
    # slice each time), and 1 GB read once from DRAM.  The first is the ceiling of every operand that all CTAs re-read.
    if want("l2_read_32mb", "hbm_read_1gb"):
        from ..ops import native as _nat
        sink = torch.zeros(1, dtype=torch.int32, device="cuda")
        small = torch.ones(32 << 20, dtype=torch.uint8, device="cuda")
        run("l2_read_32mb", lambda: _nat.read_probe(small, small.numel(), 32, 4 * ops.sm_count, sink), 32 * small.numel())
        big = torch.ones(1 << 30, dtype=torch.uint8, device="cuda")
        run("hbm_read_1gb", lambda: _nat.read_probe(big, big.numel(), 1, 4 * ops.sm_count, sink), big.numel())
        del small, big
    # attention over a paged cache
    if want("attn_decode_s1", "attn_decode_s2", "attn_decode_s4", "rope_kv_write"):
        bs = 16
        nblk = (a.ctx + bs - 1) // bs
        kv = (torch.randn(M * nblk + 1, 2, nkv, bs, hd, device="cuda") * 0.3).half()
        bt = torch.randperm(M * nblk, device="cuda").int().view(M, nblk).contiguous()
        lens = torch.full((M,), a.ctx, dtype=torch.int32, device="cuda")
        ao = torch.zeros(M, q_dim, dtype=torch.float16, device="cuda")
        for splits in (1, 2, 4):
            scratch = torch.zeros(M * nh * splits * (hd + 2), device="cuda")
            run(f"attn_decode_s{splits}",
                lambda s=splits, sc=scratch: ops.attn_decode(qkv, kv, bt, lens, ao, M, nh, nkv, hd, bs, 1 / math.sqrt(hd),
                                                              sc, s),
                M * a.ctx * nkv * hd * 2 * 2)
        pos = torch.full((M,), a.ctx - 1, dtype=torch.int32, device="cuda")
        slots = (bt[:, -1].long() * bs + (a.ctx - 1) % bs).contiguous()
        inv = ref.inv_freq(hd, c.rope_theta).cuda()
        run("rope_kv_write", lambda: ops.rope_kv_write(qkv, kv, pos, slots, inv, M, nh, nkv, hd, bs),
            M * (q_dim + 2 * kv_dim) * 2 * 2)
    # chunked-prefill attention: sequences of 2048 tokens (or one shorter one), causal, from position 0
    if want("attn_prefill_tc", "attn_prefill_mma") and hd == 128:
        from ..ops import native as _native
        q_len = min(M, 2048)
        n_seq = max(1, M // q_len)
        pbs = a.kv_block
        nb = (q_len + pbs - 1) // pbs
        kvp = (torch.randn(n_seq * nb + 1, 2, nkv, pbs, hd, device="cuda") * 0.3).half()
        btp = torch.randperm(n_seq * nb, device="cuda").int().view(n_seq, nb).contiguous()
        cu = torch.arange(0, (n_seq + 1) * q_len, q_len, dtype=torch.int32, device="cuda")
        p0 = torch.zeros(n_seq, dtype=torch.int32, device="cuda")
        total = n_seq * q_len
        qp = (torch.randn(total, q_dim + 2 * kv_dim, device="cuda") * 0.5).half()
        op = torch.zeros(total, q_dim, dtype=torch.float16, device="cuda")
        causal_flops = 4 * hd * nh * n_seq * (q_len * (q_len + 1) // 2)
        kv_bytes = n_seq * q_len * nkv * hd * 2 * 2 + total * q_dim * 2 * 2
        run("attn_prefill_tc",
            lambda: _native.attn_prefill_tc(qp, qp.stride(0), total, kvp, btp, cu, p0, op, op.stride(0), n_seq, q_len, nh,
                                            nkv, hd, pbs, 1 / math.sqrt(hd), ops.status.ptr), kv_bytes, causal_flops)
        run("attn_prefill_mma",
            lambda: _native.attn_prefill_ext(qp, qp.stride(0), kvp, btp, cu, p0, op, op.stride(0), n_seq, q_len, nh, nkv,
                                             hd, pbs, 1 / math.sqrt(hd)), kv_bytes, causal_flops)
    # batched LoRA: every token routed to one of 32 rank-16 adapters on a q_proj-sized projection
    if want("lora_apply"):
        n_ad, r_lora = 32, 16
        a_tab = (torch.randn(n_ad, r_lora, H, device="cuda") * 0.01).half()
        b_tab = (torch.randn(n_ad, q_dim, r_lora, device="cuda") * 0.01).half()
        ad_ids = (torch.arange(M, device="cuda", dtype=torch.int32) % n_ad).contiguous()
        ad_scales = torch.full((n_ad,), 2.0, device="cuda")
        y_lora = torch.zeros(M, q_dim, dtype=torch.float16, device="cuda")
        touched = min(M, n_ad) * (r_lora * H + q_dim * r_lora) * 2          # adapter matrices that are read at all
        run("lora_apply", lambda: ops.lora_apply(x, a_tab, b_tab, ad_ids, ad_scales, y_lora, M, H, q_dim, r_lora),
            touched + M * (H + 2 * q_dim) * 2, 2 * M * r_lora * (H + q_dim))
    # lm_head + selection
    if want("lm_head_gemm", "argmax", "sample_topk_topp"):
        V = c.vocab_size // tp
        wl = ops.make_linear([{"dtype": "float16", "data": (torch.randn(V, H, device="cuda") * 0.02).half(),
                               "shape": (V, H)}], H, 128)
        logits = torch.zeros(M, V, dtype=torch.float16, device="cuda")
        run("lm_head_gemm", lambda: ops.linear(wl, x, M, logits), V * H * 2 + M * V * 2, 2 * M * V * H)
        out = torch.zeros(M, dtype=torch.int32, device="cuda")
        run("argmax", lambda: ops.argmax(logits, out, M), M * V * 2)
        temp = torch.full((M,), 0.8, device="cuda")
        tk = torch.full((M,), 50, dtype=torch.int32, device="cuda")
        tpp = torch.full((M,), 0.9, device="cuda")
        seeds = torch.arange(M, dtype=torch.int64, device="cuda")
        run("sample_topk_topp", lambda: ops.sample(logits, out, M, temp, tk, tpp, seeds, 1), M * V * 2 * 6)
    hdr = f"{'kernel':22s} {'us':>9s} {'GB/s':>9s} {'of HBM':>7s} {'TFLOP/s':>9s} {'of tensor':>9s}"
    print(f"shape {a.shape}, tokens {M}, tp {tp}, peaks {peaks}")
    print(hdr)
    for r in rows:
        print(f"{r['name']:22s} {r['us']:9.1f} {r['GB/s']:9.1f} {str(r['frac_hbm']):>7s} {r['TFLOP/s']:9.2f} "
              f"{str(r['frac_tensor']):>9s}")
    if a.json:
        with open(a.json, "w") as f:
            json.dump({"shape": a.shape, "tokens": M, "tp": tp, "peaks": peaks, "rows": rows}, f, indent=1)


if __name__ == "__main__":
    main()

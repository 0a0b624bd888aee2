"""Per-role cycle counters of the decode GEMM (csrc/gemm_w4_dec.cu) and a per-tile timeline of the tcgen05 prefill
attention (csrc/attention_tc.cu) from the instrumented library variant.

The ordinary library carries no instrumentation.  ``python -m zse_b200.ops.build --variant timing`` links the same
sources with ``-DZSE_DEC_TIMING`` into ``zse_b200/_C/libzse_b200.timing.so``; in that build every role of one CTA
(CTA 1) records ``clock64()`` differences into a buffer: the MMA-issuing lanes (waits for the activation stage and the
TMEM slot, cycles spent issuing), the dequantisation groups (wait for the weight chunk, dequantise, wait for the slot,
``tcgen05.st``), and the epilogue warps (accumulators complete, cluster barriers, partial sums pushed, stores finished,
all counters seen, rows normalised).  This module runs one launch per shape with cold caches and prints the table;
it is how the figures in the design notes (cycles per ``tcgen05.mma`` per issuing thread, cost of the cluster barriers,
cost of the tail that follows the last MMA) were taken, and how they can be taken again.

    python -m zse_b200.ops.build --variant timing
    python -m zse_b200.runtime.kernel_counters --shape qwen2.5-14b --tokens 64 --tp 1
    python -m zse_b200.runtime.kernel_counters --kernel attn_prefill_tc --tokens 2048

With ``--kernel attn_prefill_tc`` (built with ``-DZSE_ATTN_TIMING``) the heaviest CTA of a causal chunk stamps, for each
key tile, when its three roles passed each barrier: the loader (K slot free, K issued, V slot free, V issued), the MMA
thread (K landed, P of the previous tile consumed, Q K^T issued, V landed, P ready, P V issued) and the first softmax
warp (S complete, probabilities computed, P published).  The table shows which link of the chain a tile waits on.

There is no counterpart in the reference (its kernels carry no counters).
"""
from __future__ import annotations

import argparse
import ctypes
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--shape", default="qwen2.5-14b")
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--tp", type=int, default=1, help="shard the projections as this tensor-parallel degree would")
    ap.add_argument("--kernel", default="gemm_w4_dec", choices=("gemm_w4_dec", "attn_prefill_tc"))
    ap.add_argument("--kv-block", type=int, default=16, help="tokens per KV block (attn_prefill_tc)")
    a = ap.parse_args(argv)

    from ..ops import build as B
    lib_file = B.variant_path("timing")
    if not os.path.exists(lib_file):
        print(f"{lib_file} is missing: run `python -m zse_b200.ops.build --variant timing`", file=sys.stderr)
        return 2
    os.environ["ZSE_NATIVE_LIB"] = lib_file        # before the library is loaded
    import torch
    from ..format import synth
    from ..ops import native
    from ..ops.backend import CudaOps
    from .microbench import _w4

    ops = CudaOps("cuda")
    lib = native.load()
    if a.kernel == "attn_prefill_tc":
        return _attn_timeline(a, ops, lib, native, synth)
    lib.zse_gemm_w4_dec_set_timing.argtypes = [ctypes.c_void_p]
    tbuf = torch.zeros(25 * 8 + 64, dtype=torch.int64, device="cuda")
    lib.zse_gemm_w4_dec_set_timing(tbuf.data_ptr())
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")     # larger than L2: every launch starts cold
    sh = synth.SHAPES[a.shape]
    H, I, tp, M = sh["hidden_size"], sh["intermediate_size"], a.tp, a.tokens
    hd = sh.get("head_dim", H // sh["num_heads"])
    qkv_n = (sh["num_heads"] + 2 * sh["num_kv_heads"]) * hd // tp
    ws = native.gemm_w4_dec_workspace("cuda", ops.sm_count)
    wn = torch.ones(H, dtype=torch.float16, device="cuda")

    def run(tag, N, K, epi):
        swiglu = epi == 1
        w = _w4(ops, N // 2 if swiglu else N, K, swiglu=swiglu)
        x = (torch.randn(M, K, device="cuda") * 0.5).half()
        out = torch.zeros(M, N, dtype=torch.float32 if epi == 2 else torch.float16, device="cuda")
        res = torch.randn(M, H, device="cuda")
        slot = [0]

        def fn():
            if epi == 4:       # projection + residual add + RMSNorm in the kernel (one-rank context)
                ops.linear_residual_norm(w, x, M, res, wn, out, 1e-6, slot[0])
                slot[0] ^= 1
            else:
                native.gemm_w4_dec(w.data, x, M, None, out, M, N, K, N, epi, ws, ops.status.ptr)

        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ops.check()
        best = 1e9
        for _ in range(5):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) * 1000)
        plan = native.gemm_w4_dec_plan(N, K, epi, ops.sm_count)
        nbytes = N * K // 2 + N * (K // 128) * 4
        print(f"{tag}: M={M} N={N} K={K} plan (CTAs, split)={plan} cold {best:.1f} us "
              f"({nbytes / best / 1e6:.2f} TB/s of weights)")
        tbuf.zero_()
        flush.zero_()
        fn()
        torch.cuda.synchronize()
        t = tbuf.cpu()
        roles = t[:200].view(25, 8)
        k_steps = max(1, (K // 128 * ((N + 255) // 256) + plan[0] - 1) // plan[0])
        for lane in range(4):
            r = roles[lane]
            print(f"  mma lane {lane}: wait activations {int(r[0])}  wait TMEM slot {int(r[1])}  issuing {int(r[2])} "
                  f"(~{int(r[2]) / max(1, 4 * k_steps):.0f} cycles per tcgen05.mma: a lane takes every other step of its tile, "
                  f"eight MMAs each)  loop ends at {int(r[3])}")
        r = roles[5]
        print(f"  dequant warp 5: first weight chunk at {int(r[6])}  wait chunk {int(r[0])}  load+dequant {int(r[1])}  "
              f"wait slot {int(r[2])}  tcgen05.st {int(r[3])}  wait::st {int(r[4])}  total {int(r[7])}")
        r = roles[21]
        if plan[1] > 0:
            print(f"  epilogue warp 21: accumulators complete {int(r[0])}  cluster barrier A {int(r[1])}  partial sums "
                  f"pushed {int(r[2])}  cluster barrier B {int(r[3])}  stores issued {int(r[4])}"
                  + (f"  all counters seen {int(r[5])}  rows normalised {int(r[6])}" if epi == 4 else "")
                  + f"  end {int(r[7])}")
        else:
            print(f"  epilogue warp 21: wait accumulators {int(r[0])}  dump {int(r[1])}  wait flags {int(r[2])}  "
                  f"phase 1 {int(r[3])}  phase 2 {int(r[4])}  end {int(r[7])}")

    run("qkv + rope shape (plain fp16 epilogue)", qkv_n, H, 0)
    run("o_proj -> fp32 plane", H, sh["num_heads"] * hd // tp, 2)
    run("gate/up + SwiGLU", 2 * (I // tp // 128 * 128), H, 1)
    run("down_proj -> fp32 plane", H, I // tp // 128 * 128, 2)
    run("o_proj + residual + RMSNorm in the kernel", H, sh["num_heads"] * hd // tp, 4)
    run("down_proj + residual + RMSNorm in the kernel", H, I // tp // 128 * 128, 4)
    return 0


def _attn_timeline(a, ops, lib, native, synth) -> int:
    """One causal chunk of ``--tokens`` rows from position 0 (``--kv-block`` tokens per block, shuffled block table): stamps of the CTA
    that owns the last query tile of head 0, relative to the moment its first K tile landed."""
    import math
    import torch
    sh = synth.SHAPES[a.shape]
    nh, nkv = sh["num_heads"], sh["num_kv_heads"]
    hd = sh.get("head_dim", sh["hidden_size"] // nh)
    q_len, bs = a.tokens, a.kv_block
    nb = (q_len + bs - 1) // bs
    kv = (torch.randn(nb + 1, 2, nkv, bs, hd, device="cuda") * 0.3).half()
    bt = torch.randperm(nb, device="cuda").int().view(1, nb).contiguous()
    cu = torch.tensor([0, q_len], dtype=torch.int32, device="cuda")
    p0 = torch.zeros(1, dtype=torch.int32, device="cuda")
    q = (torch.randn(q_len, (nh + 2 * nkv) * hd, device="cuda") * 0.5).half()
    out = torch.zeros(q_len, nh * hd, dtype=torch.float16, device="cuda")
    tbuf = torch.zeros(24 * 16, dtype=torch.int64, device="cuda")
    lib.zse_attn_prefill_tc_set_timing.argtypes = [ctypes.c_void_p]

    def fn():
        native.attn_prefill_tc(q, q.stride(0), q_len, kv, bt, cu, p0, out, out.stride(0), 1, q_len, nh, nkv, hd, bs,
                               1 / math.sqrt(hd), ops.status.ptr)

    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ops.check()
    lib.zse_attn_prefill_tc_set_timing(tbuf.data_ptr())
    fn()
    torch.cuda.synchronize()
    lib.zse_attn_prefill_tc_set_timing(None)
    t = tbuf.cpu().view(24, 16)
    base = int(t[0, 0])
    names = ("K landed", "prev P read", "QK^T issued", "V landed", "P ready", "PV issued", "S complete", "probs done",
             "P published", "(two-pass) done", "K slot free", "K issued", "V slot free", "V issued", "loader: tile begins",
             "loader: next lookup issued")
    print("cycles since the first K tile landed; columns: " + " | ".join(f"{i}={n}" for i, n in enumerate(names)))
    for tile in range(min(24, (q_len + 127) // 128)):
        row = [int(t[tile, i]) - base if int(t[tile, i]) else -1 for i in range(16)]
        print(f"tile {tile:2d}: " + " ".join(f"{v:7d}" for v in row))
    return 0


if __name__ == "__main__":
    sys.exit(main())

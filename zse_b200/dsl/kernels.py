"""Inference kernels written in the kernel language (importable, unlike test fixtures): the portable counterparts of
the hand-written library, in the spirit of zse-engine/zse_engine/orchestrator/portable_kernels.py:28-813 (INT4 / INT8
dequantising matmuls, a warp-per-row INT4 GEMV, RoPE with the cache write, plus the small element-wise and
normalisation kernels).  They are not the engine's hot path - that is ``csrc/`` - but every one runs three ways:
``emulate`` on the CPU (the oracle of the tests), ``compile`` to a cubin for sm_100a, and ``launch`` on the GPU.

Conventions: weights are row-major ``[N, K]`` like the ``.zse`` file stores them (INT4: two values per byte, low
nibble first, asymmetric groups of 128 with fp16 scale and zero point; INT8: symmetric groups with an fp16 scale),
activations ``[M, K]``, outputs ``[M, N]``."""
from __future__ import annotations

from . import (Tensor, block_dim, block_id, block_reduce_sum, cos, exp, float16, float32, global_id, int8, int32,
               kernel, lane_id, local_array, max_val, reinterpret, rsqrt, shared_memory, sin, syncthreads, thread_id,
               uint8, uint32, unpack_uint4, warp_reduce_max, warp_reduce_sum)


@kernel
def vector_add(a: Tensor, b: Tensor, out: Tensor, n: int):
    i = global_id(0)
    if i < n:
        out[i] = a[i] + b[i]


@kernel
def add_bias(x: Tensor, bias: Tensor, out: Tensor, n: int, width: int):
    i = global_id(0)
    if i >= n:
        return
    out[i] = x[i] + bias[i % width]


@kernel
def silu(x: Tensor, out: Tensor, n: int):
    i = global_id(0)
    if i >= n:
        return
    v = x[i]
    out[i] = v / (1.0 + exp(-v))


@kernel
def swiglu(gate: Tensor, up: Tensor, out: Tensor, n: int):
    i = global_id(0)
    if i < n:
        g = gate[i]
        out[i] = g / (1.0 + exp(-g)) * up[i]


@kernel
def rmsnorm(x: Tensor, w: Tensor, out: Tensor, n: int, eps: float):
    """One block per row; strided partial sums, then a block reduction every thread receives."""
    row = block_id(0)
    tid = thread_id(0)
    acc = 0.0
    for i in range(tid, n, block_dim(0)):
        v = x[row * n + i]
        acc += v * v
    total = block_reduce_sum(acc)
    scale = rsqrt(total / float(n) + eps)
    for i in range(tid, n, block_dim(0)):
        out[row * n + i] = x[row * n + i] * scale * w[i]


@kernel
def layernorm(x: Tensor, weight: Tensor, out: Tensor, n: int):
    """One block per row of at most block_dim values; two block reductions in a row (mean, then variance)."""
    tid = thread_id(0)
    idx = block_id(0) * n + tid
    val = x[idx] if tid < n else 0.0
    mean = block_reduce_sum(val) / float(n)
    diff = val - mean if tid < n else 0.0
    var = block_reduce_sum(diff * diff) / float(n)
    if tid < n:
        out[idx] = weight[tid] * (diff * rsqrt(var + 0.00001))


@kernel
def softmax_warp(x: Tensor, out: Tensor, n: int):
    """One warp per row of up to 32 values."""
    row = block_id(0)
    lane = lane_id()
    v = x[row * n + lane] if lane < n else -1e30
    m = warp_reduce_max(v)
    e = exp(v - m) if lane < n else 0.0
    s = warp_reduce_sum(e)
    if lane < n:
        out[row * n + lane] = e / s


@kernel
def dequant_rows(packed: Tensor[uint8], scales: Tensor[float16], zeros: Tensor[float16], out: Tensor[float16],
                 groups: int):
    """INT4 asymmetric groups of 128 -> fp16: a thread expands one 32-bit word (8 values)."""
    w = global_id(0)
    if w < groups * 16:
        words = reinterpret(packed, uint32)
        buf = local_array(8, int32)
        unpack_uint4(words[w], buf, 0)
        g = w // 16
        for j in range(8):
            out[w * 8 + j] = buf[j] * scales[g] + zeros[g]


@kernel
def dequant_matmul_int4(x: Tensor[float16], packed: Tensor[uint8], scales: Tensor[float16], zeros: Tensor[float16],
                        out: Tensor[float16], m_rows: int, n_rows: int, k: int):
    """out[m, n] = sum_k x[m, k] * (q[n, k] * scale[n, k/128] + zero[n, k/128]); one thread per output, a 32-bit word
    (eight weights) per step."""
    idx = global_id(0)
    if idx < m_rows * n_rows:
        m = idx // n_rows
        n = idx % n_rows
        words = reinterpret(packed, uint32)
        buf = local_array(8, int32)
        acc = 0.0
        for w in range(k // 8):
            unpack_uint4(words[n * (k // 8) + w], buf, 0)
            g = n * (k // 128) + w // 16
            s = scales[g]
            z = zeros[g]
            for j in range(8):
                acc += x[m * k + w * 8 + j] * (buf[j] * s + z)
        out[idx] = acc


@kernel
def dequant_matmul_int8(x: Tensor[float16], q: Tensor[int8], scales: Tensor[float16], out: Tensor[float16],
                        m_rows: int, n_rows: int, k: int, group: int):
    """out[m, n] = sum_k x[m, k] * q[n, k] * scale[n, k/group]; one thread per output."""
    idx = global_id(0)
    if idx < m_rows * n_rows:
        m = idx // n_rows
        n = idx % n_rows
        acc = 0.0
        for g in range(k // group):
            part = 0.0
            for j in range(group):
                part += x[m * k + g * group + j] * q[n * k + g * group + j]
            acc += part * scales[n * (k // group) + g]
        out[idx] = acc


@kernel
def gemv_int4_warp(x: Tensor[float16], packed: Tensor[uint8], scales: Tensor[float16], zeros: Tensor[float16],
                   out: Tensor[float16], n_rows: int, k: int):
    """Single-token GEMV: one warp per weight row, lanes stride over the row's 32-bit words, butterfly reduction."""
    row = block_id(0) * (block_dim(0) // 32) + thread_id(0) // 32
    lane = lane_id()
    acc = 0.0
    if row < n_rows:
        words = reinterpret(packed, uint32)
        buf = local_array(8, int32)
        for w in range(lane, k // 8, 32):
            unpack_uint4(words[row * (k // 8) + w], buf, 0)
            g = row * (k // 128) + w // 16
            s = scales[g]
            z = zeros[g]
            for j in range(8):
                acc += x[w * 8 + j] * (buf[j] * s + z)
    total = warp_reduce_sum(acc)
    if row < n_rows and lane == 0:
        out[row] = total


@kernel
def rope_kv_write(qkv: Tensor[float16], cache: Tensor[float16], positions: Tensor[int32], slots: Tensor[int32],
                  inv_freq: Tensor, tokens: int, nh: int, nkv: int, hd: int, block_size: int):
    """Rotate-half RoPE on the q and k heads of ``qkv`` [tokens, (nh + 2 nkv) * hd] in place and scatter of k / v into
    the paged cache [blocks, 2, nkv, block_size, hd]; one thread per (token, head, rotation pair)."""
    half = hd // 2
    idx = global_id(0)
    heads = nh + 2 * nkv
    if idx < tokens * heads * half:
        i = idx % half
        head = (idx // half) % heads
        t = idx // (half * heads)
        base = (t * heads + head) * hd
        a = qkv[base + i] * 1.0
        b = qkv[base + i + half] * 1.0
        if head < nh + nkv:
            ang = positions[t] * inv_freq[i]
            c = cos(ang)
            s = sin(ang)
            ra = a * c - b * s
            rb = b * c + a * s
            a = ra
            b = rb
            qkv[base + i] = a
            qkv[base + i + half] = b
        if head >= nh:
            slot = slots[t]
            if slot >= 0:
                is_v = 1 if head >= nh + nkv else 0
                kvh = head - nh - is_v * nkv
                blk = slot // block_size
                off = slot % block_size
                dst = (((blk * 2 + is_v) * nkv + kvh) * block_size + off) * hd
                cache[dst + i] = a
                cache[dst + i + half] = b


@kernel
def paged_attention(out: Tensor[float16], q: Tensor[float16], cache: Tensor[float16], block_table: Tensor[int32],
                    seq_lens: Tensor[int32], nh: int, nkv: int, hd: int, block_size: int, max_blocks: int,
                    ldq: int, scale: float):
    """Decode attention over the paged cache ``[blocks, 2, nkv, block_size, hd]`` of one layer: one warp per (sequence,
    query head), launched as grid (num_seqs, nh) x block 32.  A lane holds ``hd / 32`` elements (hd a multiple of 32, at
    most 256) of the query, of the running output and of each key / value row; the score of a token is a butterfly sum
    over the warp, the softmax runs online (maximum and sum carried along, no score vector anywhere), and a block-table
    entry below zero - a block the cache dropped - is skipped.  ``q`` rows are ``ldq`` elements apart (the fused QKV
    buffer can be passed as it is); ``out`` is ``[num_seqs, nh * hd]``."""
    seq = block_id(0)
    head = block_id(1)
    lane = lane_id()
    per = hd // 32
    kvh = head // (nh // nkv)
    n = seq_lens[seq]
    qv = local_array(8, float32)
    acc = local_array(8, float32)
    for j in range(per):
        qv[j] = q[seq * ldq + head * hd + lane * per + j] * scale
        acc[j] = 0.0
    m = -1e30
    total = 0.0
    for t in range(n):
        blk = block_table[seq * max_blocks + t // block_size]
        row = (((max_val(blk, 0) * 2) * nkv + kvh) * block_size + t % block_size) * hd
        part = 0.0
        for j in range(per):
            part += qv[j] * cache[row + lane * per + j]
        score = warp_reduce_sum(part)             # every lane takes part, whether or not the block exists
        if blk >= 0:
            m_new = max_val(m, score)
            alpha = exp(m - m_new)
            p = exp(score - m_new)
            total = total * alpha + p
            vrow = row + nkv * block_size * hd    # the V half of the block
            for j in range(per):
                acc[j] = acc[j] * alpha + p * cache[vrow + lane * per + j]
            m = m_new
    for j in range(per):
        out[(seq * nh + head) * hd + lane * per + j] = acc[j] / total if total > 0.0 else 0.0


@kernel
def tiled_dequant_matmul_int4(x: Tensor[float16], packed: Tensor[uint8], scales: Tensor[float16],
                              zeros: Tensor[float16], out: Tensor[float16], m_rows: int, n_rows: int, k: int):
    """out[m, n] = sum_k x[m, k] * w[n, k] with 16 x 16 output tiles: a block of 16 x 16 threads stages a 16 x 16 tile
    of activations and a 16 x 16 tile of DEQUANTISED weights in shared memory per step of 16 along K, so every value is
    fetched from global memory once per tile instead of once per output.  Launched as grid (ceil(N / 16), ceil(M / 16))
    x block (16, 16); edges are padded with zeros.  (CUDA cores only: the engine's own INT4 GEMMs are the tcgen05
    kernels of ``csrc/``.)"""
    tx = thread_id(0)
    ty = thread_id(1)
    col = block_id(0) * 16 + tx                   # weight row = output column
    row = block_id(1) * 16 + ty
    xs = shared_memory((16, 16), float32)
    ws = shared_memory((16, 16), float32)
    acc = 0.0
    for k0 in range(0, k, 16):
        # thread (tx, ty) stages x[row, k0 + tx] and w[block's row ty, k0 + tx]
        kk = k0 + tx
        xs[ty * 16 + tx] = x[row * k + kk] * 1.0 if row < m_rows and kk < k else 0.0
        wn = block_id(0) * 16 + ty
        wv = 0.0
        if wn < n_rows and kk < k:
            byte = packed[wn * (k // 2) + kk // 2]
            nib = (byte >> (4 * (kk % 2))) & 15
            g = wn * (k // 128) + kk // 128
            wv = nib * scales[g] + zeros[g]
        ws[ty * 16 + tx] = wv
        syncthreads()
        for i in range(16):
            acc += xs[ty * 16 + i] * ws[tx * 16 + i]
        syncthreads()
    if row < m_rows and col < n_rows:
        out[row * n_rows + col] = acc


def _collect():
    from .kernel import KernelFunction
    return {name: obj for name, obj in globals().items() if isinstance(obj, KernelFunction)}


ALL = _collect()

# The reference's names for kernels that exist here under another one (its wave-64 and MFMA variants are for AMD parts
# and have no counterpart): zse-engine/zse_engine/orchestrator/portable_kernels.py:638, 737.
bgemv_int4_wave32 = gemv_int4_warp
fused_rope_kv_write = rope_kv_write
REFERENCE_NAMES = {"bgemv_int4_wave32": "gemv_int4_warp", "fused_rope_kv_write": "rope_kv_write"}

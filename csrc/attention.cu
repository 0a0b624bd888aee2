// Attention over the paged fp16 KV cache.
//
// Cache layout per layer: [num_blocks][2 (K, V)][nkv][block_size][hd]; block_size is a multiple of 16, so a
// 16-token tile of one kv head is a contiguous hd*32-byte run.  Block id -1 in a block table is a hole left by
// eviction and is skipped, as in the reference (zse-engine/zse_engine/orchestrator/kernels.py:571,653).
//
// attn_decode_kernel  - one query token per sequence.  A CTA owns (kv head, sequence, split): all G = nh/nkv query
//                       heads of the kv head form the 16-row M dimension of m16n8k16 MMAs, so K and V are read once
//                       per kv head (the reference reads them once per query head, kernels.py:524-671).  Each warp
//                       streams its own 16-token tiles through a private 3-stage cp.async ring (no CTA barriers in
//                       the main loop), keeps an online-softmax state in registers, and the four warps merge at the
//                       end.  With num_splits > 1 the CTA writes (O, m, l) to scratch and attn_combine_kernel merges.
// attn_prefill_kernel - causal attention of a chunk of query tokens against everything already in the cache
//                       (earlier chunks included), flash-attention style: 64 query rows per CTA, 64-token KV tiles,
//                       online softmax.  Serves prefill, chunked prefill and speculative verification
//                       (replaces kernels.py:859-957, which only sees the current pass).
#include "api.h"
#include "common.cuh"

namespace zse {

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

constexpr int kDecWarps = 4;
constexpr int kDecStages = 3;
constexpr float kLog2e = 1.4426950408889634f;

// Shared-memory tile: `rows` rows of HD halfs; 16-byte chunk c of row r lives at chunk (c ^ (r & 7)).
template <int HD>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return uint32_t(row * (HD * 2) + ((chunk ^ (row & 7)) << 4));
}

// EXT adds what the Gemma family needs: scores soft-capped as cap*tanh(s/cap) and a sliding window (only the last
// `window` tokens are seen).  The cache is addressed through strides (block, K->V), so a layer may be a view into a
// pool with wider rows.
template <int HD, bool EXT>
__global__ void __launch_bounds__(kDecWarps * 32)
attn_decode_kernel(const __half* __restrict__ q, int ldq, const __half* __restrict__ kv, const int* __restrict__ bt,
                   int max_blocks, const int* __restrict__ seq_lens, __half* __restrict__ out, int ldo,
                   float* __restrict__ scratch, int nh, int nkv, int block_size, int num_splits, float scale_log2,
                   long long blk_stride, long long half_stride, float softcap, int window) {
  constexpr int kTileBytes = 16 * HD * 2;              // one 16-token K (or V) tile
  constexpr int kChunksPerRow = HD / 8;
  constexpr int kKSteps = HD / 16;
  constexpr int kNTilesO = HD / 8;
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int kvh = blockIdx.x, seq = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = nh / nkv;
  const int len = seq_lens[seq];
  const int first_tok = (EXT && window > 0) ? max(0, len - window) : 0;
  const int total_tiles = (len + 15) >> 4;
  const int tile0 = first_tok >> 4;
  const int per_split = (total_tiles - tile0 + num_splits - 1) / num_splits;
  const int tile_begin = tile0 + split * per_split;
  const int tile_end = min(total_tiles, tile_begin + per_split);
  const int my_count = tile_end > tile_begin + warp ? (tile_end - tile_begin - warp + kDecWarps - 1) / kDecWarps : 0;

  uint8_t* ring = smem + warp * (kDecStages * 2 * kTileBytes);
  const int* my_bt = bt + size_t(seq) * max_blocks;
  const size_t kv_head_stride = size_t(block_size) * HD;        // elements between kv heads inside a block half

  // Q fragments: rows = query heads of this kv head (zero beyond G)
  uint32_t qa[kKSteps][4];
  {
    const int g0 = lane >> 2, g1 = g0 + 8, c = (lane & 3) * 2;
    const __half* q0 = q + size_t(seq) * ldq + size_t(kvh * G + g0) * HD;
    const __half* q1 = q + size_t(seq) * ldq + size_t(kvh * G + g1) * HD;
#pragma unroll
    for (int kk = 0; kk < kKSteps; ++kk) {
      qa[kk][0] = g0 < G ? *reinterpret_cast<const uint32_t*>(q0 + kk * 16 + c) : 0u;
      qa[kk][1] = g1 < G ? *reinterpret_cast<const uint32_t*>(q1 + kk * 16 + c) : 0u;
      qa[kk][2] = g0 < G ? *reinterpret_cast<const uint32_t*>(q0 + kk * 16 + 8 + c) : 0u;
      qa[kk][3] = g1 < G ? *reinterpret_cast<const uint32_t*>(q1 + kk * 16 + 8 + c) : 0u;
    }
  }

  auto issue = [&](int i) {       // i-th tile of this warp -> ring slot i % stages; always commits a group
    if (i < my_count) {
      const int tile = tile_begin + warp + i * kDecWarps;
      const int tok = tile << 4;
      const int blk = my_bt[tok / block_size];
      if (blk >= 0) {
        const __half* ksrc = kv + size_t(blk) * blk_stride + size_t(kvh) * kv_head_stride + size_t(tok % block_size) * HD;
        const __half* vsrc = ksrc + half_stride;
        uint8_t* kd = ring + (i % kDecStages) * 2 * kTileBytes;
        uint8_t* vd = kd + kTileBytes;
#pragma unroll
        for (int j = 0; j < kTileBytes / 512; ++j) {
          const int idx = j * 32 + lane;
          const int row = idx / kChunksPerRow, ch = idx % kChunksPerRow;
          cp_async16(kd + tile_off<HD>(row, ch), ksrc + idx * 8);
          cp_async16(vd + tile_off<HD>(row, ch), vsrc + idx * 8);
        }
      }
    }
    cp_async_commit();
  };

  float o[kNTilesO][4];
#pragma unroll
  for (int n = 0; n < kNTilesO; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

#pragma unroll
  for (int i = 0; i < kDecStages - 1; ++i) issue(i);

  for (int i = 0; i < my_count; ++i) {
    cp_async_wait<kDecStages - 2>();
    __syncwarp();
    issue(i + kDecStages - 1);
    const int tile = tile_begin + warp + i * kDecWarps;
    const int tok = tile << 4;
    if (my_bt[tok / block_size] < 0) continue;          // hole
    const uint32_t kbase = smem_u32(ring + (i % kDecStages) * 2 * kTileBytes);
    const uint32_t vbase = kbase + kTileBytes;

    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
      const int m = lane >> 3, rr = lane & 7;
      const int row = (m >> 1) * 8 + rr;
#pragma unroll
      for (int kk = 0; kk < kKSteps; ++kk) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(kbase + tile_off<HD>(row, kk * 2 + (m & 1)), b0, b1, b2, b3);
        mma16816(s[0], qa[kk], b0, b1);
        mma16816(s[1], qa[kk], b2, b3);
      }
    }
    // scale, mask the tail, online softmax (rows lane/4 and lane/4 + 8)
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int t = tok + j * 8 + (lane & 3) * 2 + (e & 1);
        float v = s[j][e] * scale_log2;
        if constexpr (EXT) {
          if (softcap > 0.f) v = softcap * kLog2e * tanhf(v * (1.f / (kLog2e * softcap)));
          if (t < first_tok) v = -INFINITY;
        }
        if (t >= len) v = -INFINITY;
        s[j][e] = v;
        if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    if (__any_sync(0xffffffffu, n0 > m0 || n1 > m1)) {
      const float a0 = m0 == -INFINITY ? 0.f : exp2f(m0 - n0), a1 = m1 == -INFINITY ? 0.f : exp2f(m1 - n1);
      l0 *= a0;
      l1 *= a1;
#pragma unroll
      for (int n = 0; n < kNTilesO; ++n) {
        o[n][0] *= a0; o[n][1] *= a0; o[n][2] *= a1; o[n][3] *= a1;
      }
      m0 = n0;
      m1 = n1;
    }
    uint32_t pa[4];
    {
      const float b0f = m0 == -INFINITY ? 0.f : m0, b1f = m1 == -INFINITY ? 0.f : m1;   // fully masked rows
      const float p00 = exp2f(s[0][0] - b0f), p01 = exp2f(s[0][1] - b0f), p02 = exp2f(s[0][2] - b1f),
                  p03 = exp2f(s[0][3] - b1f);
      const float p10 = exp2f(s[1][0] - b0f), p11 = exp2f(s[1][1] - b0f), p12 = exp2f(s[1][2] - b1f),
                  p13 = exp2f(s[1][3] - b1f);
      l0 += p00 + p01 + p10 + p11;
      l1 += p02 + p03 + p12 + p13;
      pa[0] = pack_h2(p00, p01);
      pa[1] = pack_h2(p02, p03);
      pa[2] = pack_h2(p10, p11);
      pa[3] = pack_h2(p12, p13);
    }
    {
      const int m = lane >> 3, rr = lane & 7;
      const int row = (m & 1) * 8 + rr;
#pragma unroll
      for (int p = 0; p < kNTilesO / 2; ++p) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(vbase + tile_off<HD>(row, p * 2 + (m >> 1)), b0, b1, b2, b3);
        mma16816(o[2 * p], pa, b0, b1);
        mma16816(o[2 * p + 1], pa, b2, b3);
      }
    }
  }
  cp_async_wait<0>();
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  __syncthreads();                                       // every warp is done with its ring

  // merge the four warps: smem as [warp][16 rows][HD] fp32 + [warp][16]{m, l}
  float* mo = reinterpret_cast<float*>(smem);
  float* mm = mo + kDecWarps * 16 * HD;
  float* ml = mm + kDecWarps * 16;
  {
    const int r0 = lane >> 2, c = (lane & 3) * 2;
    float* dst = mo + warp * 16 * HD;
#pragma unroll
    for (int n = 0; n < kNTilesO; ++n) {
      dst[r0 * HD + n * 8 + c] = o[n][0];
      dst[r0 * HD + n * 8 + c + 1] = o[n][1];
      dst[(r0 + 8) * HD + n * 8 + c] = o[n][2];
      dst[(r0 + 8) * HD + n * 8 + c + 1] = o[n][3];
    }
    if ((lane & 3) == 0) {
      mm[warp * 16 + r0] = m0;
      mm[warp * 16 + r0 + 8] = m1;
      ml[warp * 16 + r0] = l0;
      ml[warp * 16 + r0 + 8] = l1;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
    const int g = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) M = fmaxf(M, mm[w * 16 + g]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float mw = mm[w * 16 + g];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
      L += ml[w * 16 + g] * f;
      acc += mo[(w * 16 + g) * HD + d] * f;
    }
    const int head = kvh * G + g;
    if (num_splits == 1) {
      out[size_t(seq) * ldo + size_t(head) * HD + d] = __float2half_rn(L > 0.f ? acc / L : 0.f);
    } else {
      float* dst = scratch + (size_t(seq * nh + head) * num_splits + split) * (HD + 2);
      dst[d] = acc;
      if (d == 0) {
        dst[HD] = M;
        dst[HD + 1] = L;
      }
    }
  }
}

template <int HD>
__global__ void attn_combine_kernel(const float* __restrict__ scratch, __half* __restrict__ out, int ldo, int nh,
                                    int num_splits) {
  pdl_launch_dependents();
  pdl_wait();
  const int head = blockIdx.x, seq = blockIdx.y, d = threadIdx.x;
  const float* src = scratch + size_t(seq * nh + head) * num_splits * (HD + 2);
  float M = -INFINITY;
  for (int s = 0; s < num_splits; ++s) M = fmaxf(M, src[s * (HD + 2) + HD]);
  float L = 0.f, acc = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float ms = src[s * (HD + 2) + HD];
    const float f = ms == -INFINITY ? 0.f : exp2f(ms - M);
    L += src[s * (HD + 2) + HD + 1] * f;
    acc += src[s * (HD + 2) + d] * f;
  }
  out[size_t(seq) * ldo + size_t(head) * HD + d] = __float2half_rn(L > 0.f ? acc / L : 0.f);
}

// ---- prefill / chunked prefill / verify ----------------------------------------------------------------
constexpr int kPfWarps = 4;          // 16 query rows each -> 64 query rows per CTA
constexpr int kPfKvTile = 64;

template <int HD, bool EXT>
__global__ void __launch_bounds__(kPfWarps * 32)
attn_prefill_kernel(const __half* __restrict__ q, int ldq, const __half* __restrict__ kv, const int* __restrict__ bt,
                    int max_blocks, const int* __restrict__ cu_q, const int* __restrict__ q_pos0,
                    __half* __restrict__ out, int ldo, int nh, int nkv, int block_size, float scale_log2,
                    long long blk_stride, long long half_stride, float softcap, int window) {
  constexpr int kChunksPerRow = HD / 8;
  constexpr int kKSteps = HD / 16;
  constexpr int kNTilesO = HD / 8;
  constexpr int kTileBytes = kPfKvTile * HD * 2;
  extern __shared__ __align__(128) uint8_t smem[];       // [2 stages][K tile, V tile]
  const int qt = blockIdx.x, head = blockIdx.y, seq = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_begin = cu_q[seq], q_len = cu_q[seq + 1] - q_begin;
  if (qt * 64 >= q_len) return;
  const int pos0 = q_pos0[seq];
  const int kvh = head / (nh / nkv);
  const int* my_bt = bt + size_t(seq) * max_blocks;
  const size_t kv_head_stride = size_t(block_size) * HD;

  // this warp's 16 query rows
  const int r0 = qt * 64 + warp * 16 + (lane >> 2), r1 = r0 + 8;       // row index inside the sequence's chunk
  uint32_t qa[kKSteps][4];
  {
    const int c = (lane & 3) * 2;
    const __half* q0 = q + size_t(q_begin + r0) * ldq + size_t(head) * HD;
    const __half* q1 = q + size_t(q_begin + r1) * ldq + size_t(head) * HD;
#pragma unroll
    for (int kk = 0; kk < kKSteps; ++kk) {
      qa[kk][0] = r0 < q_len ? *reinterpret_cast<const uint32_t*>(q0 + kk * 16 + c) : 0u;
      qa[kk][1] = r1 < q_len ? *reinterpret_cast<const uint32_t*>(q1 + kk * 16 + c) : 0u;
      qa[kk][2] = r0 < q_len ? *reinterpret_cast<const uint32_t*>(q0 + kk * 16 + 8 + c) : 0u;
      qa[kk][3] = r1 < q_len ? *reinterpret_cast<const uint32_t*>(q1 + kk * 16 + 8 + c) : 0u;
    }
  }
  // keys visible to the last query row of this CTA
  const int last_row = min(q_len, qt * 64 + 64) - 1;
  const int kv_len = pos0 + last_row + 1;
  const int n_tiles = (kv_len + kPfKvTile - 1) / kPfKvTile;

  auto issue = [&](int t) {
    if (t < n_tiles) {
      uint8_t* kd = smem + (t & 1) * 2 * kTileBytes;
      uint8_t* vd = kd + kTileBytes;
      // 64 rows x kChunksPerRow chunks, split over 128 threads
      for (int idx = threadIdx.x; idx < kPfKvTile * kChunksPerRow; idx += kPfWarps * 32) {
        const int row = idx / kChunksPerRow, ch = idx % kChunksPerRow;
        const int tok = t * kPfKvTile + row;
        const int blk = tok < kv_len ? my_bt[tok / block_size] : -1;
        if (blk >= 0) {
          const __half* ksrc = kv + size_t(blk) * blk_stride + size_t(kvh) * kv_head_stride +
                               size_t(tok % block_size) * HD + ch * 8;
          cp_async16(kd + tile_off<HD>(row, ch), ksrc);
          cp_async16(vd + tile_off<HD>(row, ch), ksrc + half_stride);
        } else {
          *reinterpret_cast<uint4*>(kd + tile_off<HD>(row, ch)) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(vd + tile_off<HD>(row, ch)) = make_uint4(0, 0, 0, 0);
        }
      }
    }
    cp_async_commit();
  };

  float o[kNTilesO][4];
#pragma unroll
  for (int n = 0; n < kNTilesO; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const int p0 = pos0 + r0, p1 = pos0 + r1;              // absolute positions of the two rows

  // first tile any row of this CTA can see (its first row's window start)
  const int t_begin = (EXT && window > 0) ? max(0, pos0 + qt * 64 - window + 1) / kPfKvTile : 0;
  issue(t_begin);
  for (int t = t_begin; t < n_tiles; ++t) {
    issue(t + 1);
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t kbase = smem_u32(smem + (t & 1) * 2 * kTileBytes);
    const uint32_t vbase = kbase + kTileBytes;
    const int tok0 = t * kPfKvTile;
    // skip tiles entirely in the future of this warp's rows (warp-uniform)
    const int warp_last_pos = pos0 + qt * 64 + warp * 16 + 15;
    if (tok0 <= warp_last_pos) {
      float s[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      {
        const int m = lane >> 3, rr = lane & 7;
#pragma unroll
        for (int kk = 0; kk < kKSteps; ++kk) {
#pragma unroll
          for (int jp = 0; jp < 4; ++jp) {                 // pairs of 8-token n-tiles
            const int row = jp * 16 + (m >> 1) * 8 + rr;
            uint32_t b0, b1, b2, b3;
            ldsm_x4(kbase + tile_off<HD>(row, kk * 2 + (m & 1)), b0, b1, b2, b3);
            mma16816(s[2 * jp], qa[kk], b0, b1);
            mma16816(s[2 * jp + 1], qa[kk], b2, b3);
          }
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        // an 8-token group never straddles a block (block_size is a multiple of 16)
        const bool hole = my_bt[min(tok0 + j * 8, kv_len - 1) / block_size] < 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tk = tok0 + j * 8 + (lane & 3) * 2 + (e & 1);
          const int pos = e < 2 ? p0 : p1;
          float v = s[j][e] * scale_log2;
          if constexpr (EXT) {
            if (softcap > 0.f) v = softcap * kLog2e * tanhf(v * (1.f / (kLog2e * softcap)));
            if (window > 0 && tk <= pos - window) v = -INFINITY;
          }
          if (tk > pos || hole) v = -INFINITY;
          s[j][e] = v;
          if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
        }
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
      const float a0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - n0), a1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - n1);
      l0 *= a0;
      l1 *= a1;
#pragma unroll
      for (int n = 0; n < kNTilesO; ++n) {
        o[n][0] *= a0; o[n][1] *= a0; o[n][2] *= a1; o[n][3] *= a1;
      }
      m0 = n0;
      m1 = n1;
      const float b0f = m0 == -INFINITY ? 0.f : m0, b1f = m1 == -INFINITY ? 0.f : m1;   // fully masked rows
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {                     // 16 tokens per PV k-step
        uint32_t pa[4];
        const float p00 = exp2f(s[2 * ks][0] - b0f), p01 = exp2f(s[2 * ks][1] - b0f);
        const float p02 = exp2f(s[2 * ks][2] - b1f), p03 = exp2f(s[2 * ks][3] - b1f);
        const float p10 = exp2f(s[2 * ks + 1][0] - b0f), p11 = exp2f(s[2 * ks + 1][1] - b0f);
        const float p12 = exp2f(s[2 * ks + 1][2] - b1f), p13 = exp2f(s[2 * ks + 1][3] - b1f);
        l0 += p00 + p01 + p10 + p11;
        l1 += p02 + p03 + p12 + p13;
        pa[0] = pack_h2(p00, p01);
        pa[1] = pack_h2(p02, p03);
        pa[2] = pack_h2(p10, p11);
        pa[3] = pack_h2(p12, p13);
        const int m = lane >> 3, rr = lane & 7;
        const int row = ks * 16 + (m & 1) * 8 + rr;
#pragma unroll
        for (int p = 0; p < kNTilesO / 2; ++p) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(vbase + tile_off<HD>(row, p * 2 + (m >> 1)), b0, b1, b2, b3);
          mma16816(o[2 * p], pa, b0, b1);
          mma16816(o[2 * p + 1], pa, b2, b3);
        }
      }
    }
    __syncthreads();                                       // tile buffer may be refilled
  }
  cp_async_wait<0>();
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
  const int c = (lane & 3) * 2;
#pragma unroll
  for (int n = 0; n < kNTilesO; ++n) {
    if (r0 < q_len)
      *reinterpret_cast<uint32_t*>(out + size_t(q_begin + r0) * ldo + size_t(head) * HD + n * 8 + c) =
          pack_h2(o[n][0] * i0, o[n][1] * i0);
    if (r1 < q_len)
      *reinterpret_cast<uint32_t*>(out + size_t(q_begin + r1) * ldo + size_t(head) * HD + n * 8 + c) =
          pack_h2(o[n][2] * i1, o[n][3] * i1);
  }
}

}  // namespace zse

using namespace zse;

extern "C" int64_t zse_attn_decode_scratch_floats(int num_seqs, int nh, int hd, int max_splits) {
  return int64_t(num_seqs) * nh * max_splits * (hd + 2);
}

// Shared memory the decode kernel asks for, raised once per device (host work: not a stream operation).
template <int HD, bool EXT>
static int prepare_decode() {
  constexpr int ring = kDecWarps * kDecStages * 2 * 16 * HD * 2;
  constexpr int merge = kDecWarps * 16 * HD * 4 + kDecWarps * 16 * 2 * 4;
  constexpr int smem = ring > merge ? ring : merge;
  static bool attr[kMaxDevices] = {};
  const int dev_slot = current_device_slot();
  if (!attr[dev_slot]) {
    if (cudaFuncSetAttribute(attn_decode_kernel<HD, EXT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
        cudaSuccess)
      return ZSE_ERR_LAUNCH;
    attr[dev_slot] = true;
  }
  return 0;
}

template <int HD, bool EXT>
static int launch_decode(const void* q, int ldq, const void* kv, const void* bt, int max_blocks, const void* lens,
                         void* out, int ldo, void* scratch, int num_seqs, int nh, int nkv, int block_size, int splits,
                         float scale, long long blk_stride, long long half_stride, float softcap, int window,
                         cudaStream_t st) {
  constexpr int ring = kDecWarps * kDecStages * 2 * 16 * HD * 2;
  constexpr int merge = kDecWarps * 16 * HD * 4 + kDecWarps * 16 * 2 * 4;
  constexpr int smem = ring > merge ? ring : merge;
  if (int rc = prepare_decode<HD, EXT>()) return rc;
  dim3 grid(nkv, num_seqs, splits);
  if (launch_pdl(attn_decode_kernel<HD, EXT>, grid, dim3(kDecWarps * 32), smem, st,
                 reinterpret_cast<const __half*>(q), ldq, reinterpret_cast<const __half*>(kv),
                 reinterpret_cast<const int*>(bt), max_blocks, reinterpret_cast<const int*>(lens),
                 reinterpret_cast<__half*>(out), ldo, reinterpret_cast<float*>(scratch), nh, nkv, block_size, splits,
                 scale * kLog2e, blk_stride, half_stride, softcap, window) != cudaSuccess)
    return ZSE_ERR_LAUNCH;
  if (splits > 1) {
    if (launch_pdl(attn_combine_kernel<HD>, dim3(nh, num_seqs), dim3(HD), 0, st,
                   reinterpret_cast<const float*>(scratch), reinterpret_cast<__half*>(out), ldo, nh,
                   splits) != cudaSuccess)
      return ZSE_ERR_LAUNCH;
  }
  return 0;
}

extern "C" int zse_attn_decode_ext(const void* q, int ldq, const void* kv_layer, int64_t blk_stride,
                                   int64_t half_stride, const void* block_tables, int max_blocks, const void* seq_lens,
                                   void* out, int ldo, void* scratch, int num_seqs, int nh, int nkv, int hd,
                                   int block_size, int num_splits, float scale, float softcap, int window,
                                   void* stream) {
  if (num_seqs <= 0) return 0;
  if (nh % nkv || nh / nkv > 16 || block_size % 16 || num_splits < 1 || softcap < 0.f || window < 0)
    return ZSE_ERR_SHAPE;
  if (num_splits > 1 && scratch == nullptr) return ZSE_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(kv_layer) & 15) || (blk_stride & 7) || (half_stride & 7)) return ZSE_ERR_ALIGN;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool ext = softcap > 0.f || window > 0;
#define ZSE_DEC(HD_, EXT_)                                                                                           \
  return launch_decode<HD_, EXT_>(q, ldq, kv_layer, block_tables, max_blocks, seq_lens, out, ldo, scratch, num_seqs, \
                                  nh, nkv, block_size, num_splits, scale, blk_stride, half_stride, softcap, window, st)
  if (hd == 128) { if (ext) ZSE_DEC(128, true); ZSE_DEC(128, false); }
  if (hd == 64) { if (ext) ZSE_DEC(64, true); ZSE_DEC(64, false); }
  if (hd == 256) ZSE_DEC(256, true);
#undef ZSE_DEC
  return ZSE_ERR_SHAPE;
}

extern "C" int zse_attn_decode(const void* q, int ldq, const void* kv_layer, const void* block_tables, int max_blocks,
                               const void* seq_lens, void* out, int ldo, void* scratch, int num_seqs, int nh, int nkv,
                               int hd, int block_size, int num_splits, float scale, void* stream) {
  const int64_t half = int64_t(nkv) * block_size * hd;
  return zse_attn_decode_ext(q, ldq, kv_layer, 2 * half, half, block_tables, max_blocks, seq_lens, out, ldo, scratch,
                             num_seqs, nh, nkv, hd, block_size, num_splits, scale, 0.f, 0, stream);
}

template <int HD, bool EXT>
static int launch_prefill(const void* q, int ldq, const void* kv, const void* bt, int max_blocks, const void* cu_q,
                          const void* pos0, void* out, int ldo, int num_seqs, int max_q_len, int nh, int nkv,
                          int block_size, float scale, long long blk_stride, long long half_stride, float softcap,
                          int window, cudaStream_t st) {
  constexpr int smem = 2 * 2 * kPfKvTile * HD * 2;
  static bool attr[kMaxDevices] = {};
  const int dev_slot = current_device_slot();
  if (!attr[dev_slot]) {
    if (cudaFuncSetAttribute(attn_prefill_kernel<HD, EXT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
        cudaSuccess)
      return ZSE_ERR_LAUNCH;
    attr[dev_slot] = true;
  }
  dim3 grid((max_q_len + 63) / 64, nh, num_seqs);
  attn_prefill_kernel<HD, EXT><<<grid, kPfWarps * 32, smem, st>>>(
      reinterpret_cast<const __half*>(q), ldq, reinterpret_cast<const __half*>(kv), reinterpret_cast<const int*>(bt),
      max_blocks, reinterpret_cast<const int*>(cu_q), reinterpret_cast<const int*>(pos0),
      reinterpret_cast<__half*>(out), ldo, nh, nkv, block_size, scale * kLog2e, blk_stride, half_stride, softcap,
      window);
  return cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

extern "C" int zse_attn_prefill_ext(const void* q, int ldq, const void* kv_layer, int64_t blk_stride,
                                    int64_t half_stride, const void* block_tables, int max_blocks, const void* cu_q,
                                    const void* q_pos0, void* out, int ldo, int num_seqs, int max_q_len, int nh,
                                    int nkv, int hd, int block_size, float scale, float softcap, int window,
                                    void* stream) {
  if (num_seqs <= 0 || max_q_len <= 0) return 0;
  if (nh % nkv || block_size % 16 || softcap < 0.f || window < 0) return ZSE_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(kv_layer) & 15) || (blk_stride & 7) || (half_stride & 7)) return ZSE_ERR_ALIGN;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool ext = softcap > 0.f || window > 0;
#define ZSE_PF(HD_, EXT_)                                                                                            \
  return launch_prefill<HD_, EXT_>(q, ldq, kv_layer, block_tables, max_blocks, cu_q, q_pos0, out, ldo, num_seqs,     \
                                   max_q_len, nh, nkv, block_size, scale, blk_stride, half_stride, softcap, window, st)
  if (hd == 128) { if (ext) ZSE_PF(128, true); ZSE_PF(128, false); }
  if (hd == 64) { if (ext) ZSE_PF(64, true); ZSE_PF(64, false); }
  if (hd == 256) ZSE_PF(256, true);
#undef ZSE_PF
  return ZSE_ERR_SHAPE;
}

extern "C" int zse_attn_prefill(const void* q, int ldq, const void* kv_layer, const void* block_tables, int max_blocks,
                                const void* cu_q, const void* q_pos0, void* out, int ldo, int num_seqs, int max_q_len,
                                int nh, int nkv, int hd, int block_size, float scale, void* stream) {
  const int64_t half = int64_t(nkv) * block_size * hd;
  return zse_attn_prefill_ext(q, ldq, kv_layer, 2 * half, half, block_tables, max_blocks, cu_q, q_pos0, out, ldo,
                              num_seqs, max_q_len, nh, nkv, hd, block_size, scale, 0.f, 0, stream);
}

// ---- decode attention with library-owned scratch (attn_decode_static.h) -------------------------------------------
#include "attn_decode_static.h"

static __device__ __align__(256) float g_attn_static_scratch[ZSE_ATTN_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxStaticDevices = 64;
float* g_static_scratch_ptr[kMaxStaticDevices] = {};

// address of the scratch array on the current device, looked up once per device; nullptr with *err set on failure
float* static_scratch(int* err) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxStaticDevices) {
    *err = ZSE_ERR_DRIVER;
    return nullptr;
  }
  if (g_static_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_attn_static_scratch) != cudaSuccess || p == nullptr) {
      (void)cudaGetLastError();
      *err = ZSE_ERR_DRIVER;
      return nullptr;
    }
    g_static_scratch_ptr[dev] = p;
  }
  *err = 0;
  return g_static_scratch_ptr[dev];
}
}  // namespace

extern "C" int64_t zse_attn_decode_static_max_floats(void) { return ZSE_ATTN_STATIC_SCRATCH_FLOATS; }

extern "C" int zse_attn_decode_static_setup(void) {
  // everything the first call on a device would otherwise do on the host: the address of the scratch array and the
  // shared-memory attribute of the kernels zse_attn_decode_static can reach (head_dim 64 / 128 / 256)
  int err = 0;
  static_scratch(&err);
  if (err) return err;
  if (int rc = prepare_decode<128, false>()) return rc;
  if (int rc = prepare_decode<64, false>()) return rc;
  return prepare_decode<256, true>();
}

extern "C" int zse_attn_decode_static(const void* q, int ldq, const void* kv_layer, const void* block_tables,
                                      int max_blocks, const void* seq_lens, void* out, int ldo, int num_seqs, int nh,
                                      int nkv, int hd, int block_size, int num_splits, float scale, void* stream) {
  if (num_seqs <= 0) return 0;
  if (num_splits < 1 || nh <= 0 || hd <= 0) return ZSE_ERR_SHAPE;
  if (num_splits > 1 &&
      zse_attn_decode_scratch_floats(num_seqs, nh, hd, num_splits) > int64_t(ZSE_ATTN_STATIC_SCRATCH_FLOATS))
    return ZSE_ERR_LIMIT;
  float* scratch = nullptr;
  if (num_splits > 1) {                       // one split needs no scratch: no lookup, nothing that can fail
    int err = 0;
    scratch = static_scratch(&err);
    if (scratch == nullptr) return err;
  }
  return zse_attn_decode(q, ldq, kv_layer, block_tables, max_blocks, seq_lens, out, ldo, scratch, num_seqs, nh, nkv,
                         hd, block_size, num_splits, scale, stream);
}

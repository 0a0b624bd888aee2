// Kernels of the Gemma family (Gemma-2, Gemma-4 text), for sm_100a.
//
// What these layers need beyond the Llama/Qwen2 path (zse-engine/zse_engine/orchestrator/kernels.py:1479-1786 and
// model_runner.py:428-540 in the reference): per-head RMSNorm of q and k (learned weight) and of v (no weight),
// partial rotary embedding with a per-layer base, layers whose head_dim / kv-head count differ from their neighbours,
// V taken from the un-normalised K projection, soft-capped attention scores, sliding-window layers, a norm on each
// sub-layer OUTPUT before it joins the residual, a learned scalar per layer, and soft-capped logits.
//
//   headnorm_rope_kv_write  q/k/v head norms + RoPE + paged-cache write in one pass over the projection output
//   attn_generic            paged attention (decode and chunked prefill) for any even head_dim <= 512, with window,
//                           soft-cap and cache holes; CUDA cores, online softmax, one warp per key, the query heads
//                           of a kv head share its K/V loads
//   norm_add_rmsnorm        residual = (residual + RMSNorm(x) * w_post) * scalar;  out = RMSNorm(residual) * w_next
//   softcap                 x = cap * tanh(x / cap) on fp16 logits
//
// The cache of a layer is addressed with explicit strides (block, K/V half), so layers of different width can share
// one pool whose rows are as wide as the widest layer.
#include "api.h"
#include "common.cuh"

#define ST(s) reinterpret_cast<cudaStream_t>(s)
#define LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH)

namespace zse {
namespace {

constexpr int kGemmaMaxPairsPerLane = 8;   // head_dim <= 512: 256 rotation pairs over 32 lanes

// grid (M, nh + 2*nkv), one warp per (token, head).  Head order: q heads, k heads, v heads.
__global__ void __launch_bounds__(32)
headnorm_rope_kv_write_kernel(__half* __restrict__ qkv, int ld, __half* __restrict__ kv_layer, long long blk_stride,
                              long long half_stride, const int* __restrict__ positions,
                              const long long* __restrict__ slots, const float* __restrict__ freqs,
                              const __half* __restrict__ q_norm_w, const __half* __restrict__ k_norm_w, int norm_v,
                              int k_is_v, float eps, int nh, int nkv, int hd, int block_size) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, head = blockIdx.y, lane = threadIdx.x;
  const bool is_q = head < nh, is_v = head >= nh + nkv;
  const int kvh = is_q ? 0 : (is_v ? head - nh - nkv : head - nh);
  // where the head's input sits in the row: v heads of a layer without v_proj read the k projection
  const int col = is_q ? head * hd : (is_v && !k_is_v ? (nh + nkv + kvh) * hd : (nh + kvh) * hd);
  const __half* src = qkv + size_t(t) * ld + col;
  const int half = hd / 2;
  float a[kGemmaMaxPairsPerLane], b[kGemmaMaxPairsPerLane];
  float ss = 0.f;
#pragma unroll
  for (int r = 0; r < kGemmaMaxPairsPerLane; ++r) {
    const int i = lane + 32 * r;
    a[r] = i < half ? __half2float(src[i]) : 0.f;
    b[r] = i < half ? __half2float(src[i + half]) : 0.f;
    ss += a[r] * a[r] + b[r] * b[r];
  }
  const __half* w = is_q ? q_norm_w : (is_v ? nullptr : k_norm_w);
  const bool normed = is_v ? norm_v != 0 : w != nullptr;
  float inv = 1.f;
  if (normed) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    inv = rsqrtf(ss / float(hd) + eps);
  }
  const float pos = float(positions[t]);
  const long long slot = slots[t];
  __half* dst = nullptr;
  if (is_q) {
    dst = qkv + size_t(t) * ld + col;
  } else if (slot >= 0) {
    const long long blk = slot / block_size, off = slot % block_size;
    dst = kv_layer + blk * blk_stride + (is_v ? half_stride : 0) + (size_t(kvh) * block_size + off) * hd;
  }
  if (dst == nullptr) return;
#pragma unroll
  for (int r = 0; r < kGemmaMaxPairsPerLane; ++r) {
    const int i = lane + 32 * r;
    if (i >= half) break;
    float x = a[r] * inv, y = b[r] * inv;
    if (normed && w != nullptr) {
      x *= __half2float(w[i]);
      y *= __half2float(w[i + half]);
    }
    if (!is_v) {
      const float f = freqs[i];
      if (f != 0.f) {
        float s, c;
        sincosf(pos * f, &s, &c);
        const float rx = x * c - y * s, ry = y * c + x * s;
        x = rx;
        y = ry;
      }
    }
    dst[i] = __float2half_rn(clamp_f16(x));
    dst[i + half] = __float2half_rn(clamp_f16(y));
  }
}

// ---- generic paged attention ------------------------------------------------------------------------------------
constexpr int kGenWarps = 8;

__device__ __forceinline__ void gen_cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void gen_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void gen_cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// grid (T, nkv * ceil(G / GT)), 8 warps.  A CTA serves up to GT query heads of one kv head for one query token, so a
// K/V row is loaded once for all of them.  Query token t: decode (cu_q == nullptr): sequence t, position
// seq_lens[t]-1; prefill: sequence s with cu_q[s] <= t < cu_q[s+1], position q_pos0[s] + t - cu_q[s].
// Warp w takes keys first+w, first+w+8, ... and streams their K and V rows through a private ring of STAGES slots in
// shared memory (cp.async, 16 bytes per lane), so STAGES-1 rows per warp are in flight while one is reduced; no CTA
// barrier in the loop.  Lane l owns the half2 elements l + 32 r of a head.  head_dim must be a multiple of 8.
template <int R, int GT, int STAGES>
__global__ void __launch_bounds__(32 * kGenWarps)
attn_generic_kernel(const __half* __restrict__ q, int ldq, const __half* __restrict__ kv_layer, long long blk_stride,
                    long long half_stride, const int* __restrict__ block_tables, int max_blocks,
                    const int* __restrict__ seq_lens, const int* __restrict__ cu_q, const int* __restrict__ q_pos0,
                    int num_seqs, __half* __restrict__ out, int ldo, int nh, int nkv, int hd, int block_size,
                    float scale, float softcap, int window) {
  pdl_launch_dependents();
  pdl_wait();
  // ring: [kGenWarps][STAGES][K row, V row] halfs; reused as [kGenWarps][GT][hd + 2] floats for the merge
  extern __shared__ __align__(16) uint8_t gen_smem_raw[];
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int G = nh / nkv, gchunks = (G + GT - 1) / GT;
  const int kvh = blockIdx.y / gchunks, g0 = (blockIdx.y % gchunks) * GT;
  const int ng = min(GT, G - g0);
  const int head0 = kvh * G + g0;
  int seq = t, pos;
  if (cu_q != nullptr) {
    int lo = 0, hi = num_seqs - 1;               // last s with cu_q[s] <= t
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (cu_q[mid] <= t) lo = mid; else hi = mid - 1;
    }
    seq = lo;
    pos = q_pos0[seq] + t - cu_q[seq];
  } else {
    pos = seq_lens[seq] - 1;
  }
  const int hd2 = hd / 2;
  float2 qv[GT][R], acc[GT][R];
  float m[GT], l[GT];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    const __half2* qp = reinterpret_cast<const __half2*>(q + size_t(t) * ldq + size_t(head0 + min(g, ng - 1)) * hd);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int e = lane + 32 * r;
      qv[g][r] = (e < hd2 && g < ng) ? __half22float2(qp[e]) : make_float2(0.f, 0.f);
      acc[g][r] = make_float2(0.f, 0.f);
    }
    m[g] = -INFINITY;
    l[g] = 0.f;
  }
  const int first = window > 0 ? max(0, pos + 1 - window) : 0;
  const int* table = block_tables + size_t(seq) * max_blocks;
  const int count = pos >= first + warp ? (pos - first - warp) / kGenWarps + 1 : 0;   // keys of this warp
  __half* ring = reinterpret_cast<__half*>(gen_smem_raw) + size_t(warp) * STAGES * 2 * hd;
  const int chunks = hd / 8;                     // 16-byte pieces per row

  auto row_of = [&](int i) -> const __half* {    // K row of this warp's i-th key, or nullptr (a hole)
    const int j = first + warp + i * kGenWarps;
    const int blk = table[j / block_size];
    if (blk < 0) return nullptr;
    return kv_layer + size_t(blk) * blk_stride + (size_t(kvh) * block_size + j % block_size) * hd;
  };
  auto issue = [&](int i) {                      // always commits a group, so that the wait counts stay aligned
    if (i < count) {
      const __half* kp = row_of(i);
      if (kp != nullptr) {
        __half* dst = ring + size_t(i % STAGES) * 2 * hd;
        for (int c = lane; c < chunks; c += 32) {
          gen_cp_async16(dst + c * 8, kp + c * 8);
          gen_cp_async16(dst + hd + c * 8, kp + half_stride + c * 8);
        }
      }
    }
    gen_cp_async_commit();
  };

#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) issue(i);
  for (int i = 0; i < count; ++i) {
    gen_cp_async_wait<STAGES - 2>();
    __syncwarp();                                // slot (i-1) % STAGES is free for everyone; slot i is visible
    issue(i + STAGES - 1);
    if (row_of(i) == nullptr) continue;          // evicted block: its tokens do not exist
    const __half2* k2 = reinterpret_cast<const __half2*>(ring + size_t(i % STAGES) * 2 * hd);
    const __half2* v2 = k2 + hd2;
    float s[GT];
#pragma unroll
    for (int g = 0; g < GT; ++g) s[g] = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int e = lane + 32 * r;
      const float2 kf = e < hd2 ? __half22float2(k2[e]) : make_float2(0.f, 0.f);
#pragma unroll
      for (int g = 0; g < GT; ++g) s[g] += qv[g][r].x * kf.x + qv[g][r].y * kf.y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int g = 0; g < GT; ++g) s[g] += __shfl_xor_sync(0xffffffffu, s[g], o);
    }
    float p[GT];
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      float sc = s[g] * scale;
      if (softcap > 0.f) sc = softcap * tanhf(sc / softcap);
      const float m_new = fmaxf(m[g], sc);
      const float corr = __expf(m[g] - m_new);
      p[g] = __expf(sc - m_new);
      l[g] = l[g] * corr + p[g];
      m[g] = m_new;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        acc[g][r].x *= corr;
        acc[g][r].y *= corr;
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int e = lane + 32 * r;
      const float2 vf = e < hd2 ? __half22float2(v2[e]) : make_float2(0.f, 0.f);
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        acc[g][r].x += p[g] * vf.x;
        acc[g][r].y += p[g] * vf.y;
      }
    }
  }
  gen_cp_async_wait<0>();
  __syncthreads();                               // every warp is done with its ring

  float* gen_smem = reinterpret_cast<float*>(gen_smem_raw);
  const int stride = hd + 2;
  float* mine = gen_smem + size_t(warp) * GT * stride;
#pragma unroll
  for (int g = 0; g < GT; ++g) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int e = lane + 32 * r;
      if (e < hd2) {
        mine[g * stride + 2 * e] = acc[g][r].x;
        mine[g * stride + 2 * e + 1] = acc[g][r].y;
      }
    }
    if (lane == 0) {
      mine[g * stride + hd] = m[g];
      mine[g * stride + hd + 1] = l[g];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < ng * hd; idx += blockDim.x) {
    const int g = idx / hd, e = idx % hd;
    float m_all = -INFINITY;
#pragma unroll
    for (int w2 = 0; w2 < kGenWarps; ++w2) m_all = fmaxf(m_all, gen_smem[(w2 * GT + g) * stride + hd]);
    float l_all = 0.f, v = 0.f;
#pragma unroll
    for (int w2 = 0; w2 < kGenWarps; ++w2) {
      const float* src = gen_smem + (w2 * GT + g) * stride;
      const float f = src[hd] == -INFINITY ? 0.f : __expf(src[hd] - m_all);
      l_all += f * src[hd + 1];
      v += f * src[e];
    }
    out[size_t(t) * ldo + size_t(head0 + g) * hd + e] = __float2half_rn(l_all > 0.f ? v / l_all : 0.f);
  }
}

// ---- post-norm + residual + next pre-norm ---------------------------------------------------------------------------
constexpr int kPostNormThreads = 256;

__device__ __forceinline__ float cta_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();                                // `red` may still be read from the previous call
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float total = 0.f;
  for (int i = 0; i < (blockDim.x >> 5); ++i) total += red[i];
  return total;
}

// One CTA per row.  Rows of up to kPostNormThreads * kPostNormRegs elements are held in registers (one read of x and
// of the residual, all loads issued before the first reduction); longer rows take the looping version.
constexpr int kPostNormRegs = 32;

template <bool IN_REGS>
__global__ void __launch_bounds__(kPostNormThreads)
norm_add_rmsnorm_kernel(const __half* __restrict__ x, const __half* __restrict__ w_post, float* __restrict__ residual,
                        const __half* __restrict__ scalar, const __half* __restrict__ w_next,
                        __half* __restrict__ out, int H, float eps) {
  pdl_launch_dependents();
  __shared__ float red[32];
  const size_t base = size_t(blockIdx.x) * H;
  const float sc = scalar != nullptr ? __half2float(scalar[0]) : 1.f;     // weights do not depend on earlier kernels
  if constexpr (IN_REGS) {
    float wp[kPostNormRegs];
#pragma unroll
    for (int k = 0; k < kPostNormRegs; ++k) {
      const int i = threadIdx.x + k * kPostNormThreads;
      wp[k] = i < H ? __half2float(w_post[i]) : 0.f;
    }
    pdl_wait();
    float xv[kPostNormRegs], rv[kPostNormRegs];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < kPostNormRegs; ++k) {
      const int i = threadIdx.x + k * kPostNormThreads;
      xv[k] = i < H ? __half2float(x[base + i]) : 0.f;
      rv[k] = i < H ? residual[base + i] : 0.f;
      ss += xv[k] * xv[k];
    }
    const float inv = rsqrtf(cta_sum(ss, red) / float(H) + eps);
    float ss2 = 0.f;
#pragma unroll
    for (int k = 0; k < kPostNormRegs; ++k) {
      const int i = threadIdx.x + k * kPostNormThreads;
      rv[k] = (rv[k] + xv[k] * inv * wp[k]) * sc;
      if (i < H) residual[base + i] = rv[k];
      ss2 += rv[k] * rv[k];
    }
    if (out == nullptr) return;
    const float inv2 = rsqrtf(cta_sum(ss2, red) / float(H) + eps);
#pragma unroll
    for (int k = 0; k < kPostNormRegs; ++k) {
      const int i = threadIdx.x + k * kPostNormThreads;
      if (i < H) out[base + i] = __float2half_rn(clamp_f16(rv[k] * inv2 * __half2float(w_next[i])));
    }
  } else {
    pdl_wait();
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float f = __half2float(x[base + i]);
      ss += f * f;
    }
    const float inv = rsqrtf(cta_sum(ss, red) / float(H) + eps);
    float ss2 = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float y = __half2float(x[base + i]) * inv * __half2float(w_post[i]);
      const float r = (residual[base + i] + y) * sc;
      residual[base + i] = r;
      ss2 += r * r;
    }
    if (out == nullptr) return;
    const float inv2 = rsqrtf(cta_sum(ss2, red) / float(H) + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x)      // each thread re-reads what it wrote itself
      out[base + i] = __float2half_rn(clamp_f16(residual[base + i] * inv2 * __half2float(w_next[i])));
  }
}

__global__ void softcap_kernel(__half* __restrict__ x, int ld, int V, float cap) {
  const size_t row = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < V) {
    __half* p = x + row * ld + i;
    *p = __float2half_rn(cap * tanhf(__half2float(*p) / cap));
  }
}

}  // namespace
}  // namespace zse

using namespace zse;

extern "C" int zse_headnorm_rope_kv_write(void* qkv, int ld, void* kv_layer, int64_t blk_stride, int64_t half_stride,
                                          const void* positions, const void* slots, const void* freqs,
                                          const void* q_norm_w, const void* k_norm_w, int norm_v, int k_is_v,
                                          float eps, int M, int nh, int nkv, int hd, int block_size, void* stream) {
  if (M <= 0) return 0;
  if (hd % 2 || hd > 64 * kGemmaMaxPairsPerLane || nh <= 0 || nkv <= 0) return ZSE_ERR_SHAPE;
  dim3 grid(M, nh + 2 * nkv);
  return launch_pdl(headnorm_rope_kv_write_kernel, grid, dim3(32), 0, ST(stream), reinterpret_cast<__half*>(qkv), ld,
                    reinterpret_cast<__half*>(kv_layer), (long long)blk_stride, (long long)half_stride,
                    reinterpret_cast<const int*>(positions), reinterpret_cast<const long long*>(slots),
                    reinterpret_cast<const float*>(freqs), reinterpret_cast<const __half*>(q_norm_w),
                    reinterpret_cast<const __half*>(k_norm_w), norm_v, k_is_v, eps, nh, nkv, hd,
                    block_size) == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

template <int R, int GT, int STAGES>
static int launch_attn_generic(const void* q, int ldq, const void* kv_layer, int64_t blk_stride, int64_t half_stride,
                               const void* block_tables, int max_blocks, const void* seq_lens, const void* cu_q,
                               const void* q_pos0, int num_seqs, void* out, int ldo, int T, int nh, int nkv, int hd,
                               int block_size, float scale, float softcap, int window, void* stream) {
  const int G = nh / nkv;
  dim3 grid(T, nkv * ((G + GT - 1) / GT));
  const size_t ring = size_t(kGenWarps) * STAGES * 2 * hd * sizeof(__half);       // at most 64 KB
  const size_t merge = size_t(kGenWarps) * GT * (hd + 2) * sizeof(float);         // at most 33 KB
  const size_t smem = ring > merge ? ring : merge;
  static bool configured = false;                 // per instantiation; the attribute is per kernel, any device
  auto kern = attn_generic_kernel<R, GT, STAGES>;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024) != cudaSuccess)
      return ZSE_ERR_DRIVER;
    configured = true;
  }
  return launch_pdl(kern, grid, dim3(32 * kGenWarps), smem, ST(stream), reinterpret_cast<const __half*>(q), ldq,
                    reinterpret_cast<const __half*>(kv_layer), (long long)blk_stride, (long long)half_stride,
                    reinterpret_cast<const int*>(block_tables), max_blocks, reinterpret_cast<const int*>(seq_lens),
                    reinterpret_cast<const int*>(cu_q), reinterpret_cast<const int*>(q_pos0), num_seqs,
                    reinterpret_cast<__half*>(out), ldo, nh, nkv, hd, block_size, scale, softcap,
                    window) == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

extern "C" int zse_attn_generic(const void* q, int ldq, const void* kv_layer, int64_t blk_stride, int64_t half_stride,
                                const void* block_tables, int max_blocks, const void* seq_lens, const void* cu_q,
                                const void* q_pos0, int num_seqs, void* out, int ldo, int T, int nh, int nkv, int hd,
                                int block_size, float scale, float softcap, int window, void* stream) {
  if (T <= 0) return 0;
  if (hd % 8 || hd > 512 || nkv <= 0 || nh % nkv || (cu_q == nullptr) != (q_pos0 == nullptr)) return ZSE_ERR_SHAPE;
  if (cu_q == nullptr && seq_lens == nullptr) return ZSE_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(kv_layer) & 15) || (reinterpret_cast<uintptr_t>(q) & 3) || (ldq & 1) ||
      (blk_stride & 7) || (half_stride & 7))
    return ZSE_ERR_ALIGN;
  const int G = nh / nkv;
#define ZSE_GEN(R, GT, ST_)                                                                                           \
  return launch_attn_generic<R, GT, ST_>(q, ldq, kv_layer, blk_stride, half_stride, block_tables, max_blocks,         \
                                         seq_lens, cu_q, q_pos0, num_seqs, out, ldo, T, nh, nkv, hd, block_size,      \
                                         scale, softcap, window, stream)
  // heads per CTA: as many of the kv head's group as the registers allow; ring depth: 8 rows per warp in flight
  // (4 at head_dim 512, where a K+V row pair is 2 KB)
  if (hd <= 64) { if (G == 1) ZSE_GEN(1, 1, 8); if (G == 2) ZSE_GEN(1, 2, 8); ZSE_GEN(1, 4, 8); }
  if (hd <= 128) { if (G == 1) ZSE_GEN(2, 1, 8); if (G == 2) ZSE_GEN(2, 2, 8); ZSE_GEN(2, 4, 8); }
  if (hd <= 256) { if (G == 1) ZSE_GEN(4, 1, 8); if (G == 2) ZSE_GEN(4, 2, 8); ZSE_GEN(4, 4, 8); }
  if (G == 1) ZSE_GEN(8, 1, 4);
  ZSE_GEN(8, 2, 4);
#undef ZSE_GEN
}

extern "C" int zse_norm_add_rmsnorm(const void* x, const void* w_post, void* residual, const void* scalar,
                                    const void* w_next, void* out, int M, int H, float eps, void* stream) {
  if (M <= 0) return 0;
  if (H <= 0 || (out != nullptr && w_next == nullptr)) return ZSE_ERR_SHAPE;
  auto kern = H <= kPostNormThreads * kPostNormRegs ? norm_add_rmsnorm_kernel<true> : norm_add_rmsnorm_kernel<false>;
  return launch_pdl(kern, dim3(M), dim3(kPostNormThreads), 0, ST(stream), reinterpret_cast<const __half*>(x),
                    reinterpret_cast<const __half*>(w_post), reinterpret_cast<float*>(residual),
                    reinterpret_cast<const __half*>(scalar), reinterpret_cast<const __half*>(w_next),
                    reinterpret_cast<__half*>(out), H, eps) == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

extern "C" int zse_softcap_f16(void* x, int ld, int M, int V, float cap, void* stream) {
  if (M <= 0 || V <= 0) return 0;
  if (!(cap > 0.f)) return ZSE_ERR_SHAPE;
  softcap_kernel<<<dim3((V + 255) / 256, M), 256, 0, ST(stream)>>>(reinterpret_cast<__half*>(x), ld, V, cap);
  return LAUNCH_OK();
}

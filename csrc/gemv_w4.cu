// INT4 group-128 weight x one or two token vectors on the CUDA cores.
//
// With one or two tokens the tensor-core kernel (gemm_w4.cu) pays its whole pipeline - TMA, TMEM stores, one
// tcgen05.mma issue slot per 16 K - for a matrix product that is really a stream of dot products, and ends up issue
// bound.  Here a thread owns one weight row of a 128-row tile and walks over K chunks: four 16-byte loads bring the
// row's 128 nibbles of a chunk straight from global memory (a warp reads 512 contiguous bytes per load, so the tiled
// layout built for TMA coalesces as it is), nibbles become fp16 integers with lop3 + one half2 op per pair, and
// the group's scale and minimum are applied once per chunk:
//     y += scale * sum_k(q_k x_k) + zero * sum_k(x_k)
// sum_k(x_k) per group is computed once per CTA when the activations are staged in shared memory.  Products are
// accumulated in half2 over 8 terms (exact integers 0..15 times fp16 activations), then in fp32.
// A CTA is 128 rows x 4 K-slices (512 threads); the slices are added through shared memory.  Epilogues are those of
// the GEMM: fp16 (+bias), SwiGLU (rows 0..63 gate, 64..127 up of the same outputs), fp32 split-K planes.
//
// Replaces the scalar GEMV kernels of the reference for batch 1 (zse-engine/zse_engine/orchestrator/kernels.py:
// 1129-1192 gemv_int4, 1906-2003 batched variants).
#include "gemm_common.cuh"

namespace zse {

constexpr int kGemvSlices = 4;
constexpr int kGemvThreads = 128 * kGemvSlices;
constexpr int kGemvMaxSmem = 96 * 1024;

struct GemvArgs {
  const uint8_t* w;        // tiled chunks [n_tiles][k_chunks][8704]
  const __half* x;         // [M, K] row-major
  const __half* bias;
  void* out;
  int M, N, K, ldo;
  int k_chunks;            // K / 128
  int chunks_per_split;
};

// q pairs of one 32-bit word as fp16 integers: out[i] = (q_{2i}, q_{2i+1}) for the word's 8 consecutive K elements.
__device__ __forceinline__ void unpack_word(uint32_t w, __half2* out) {
  const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
  const __half2 k16th = __half2half2(__ushort_as_half(0x2C00));   // 1/16
  const __half2 kNeg64 = __half2half2(__ushort_as_half(0xD400));  // -64
  uint32_t t0, t1, t2, t3;
  const uint32_t w8 = w >> 8;
  asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xEA;" : "=r"(t0) : "r"(w));
  asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xEA;" : "=r"(t1) : "r"(w));
  asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xEA;" : "=r"(t2) : "r"(w8));
  asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xEA;" : "=r"(t3) : "r"(w8));
  out[0] = __hsub2(*reinterpret_cast<__half2*>(&t0), k1024);
  out[1] = __hfma2(*reinterpret_cast<__half2*>(&t1), k16th, kNeg64);
  out[2] = __hsub2(*reinterpret_cast<__half2*>(&t2), k1024);
  out[3] = __hfma2(*reinterpret_cast<__half2*>(&t3), k16th, kNeg64);
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

template <int MT, int EPI>
__global__ void __launch_bounds__(kGemvThreads, 2)
gemv_w4_kernel(const GemvArgs a) {
  extern __shared__ __align__(16) uint8_t gsm[];
  pdl_launch_dependents();
  const int tile = blockIdx.x;
  const int c0 = blockIdx.z * a.chunks_per_split;
  const int c1 = min(a.k_chunks, c0 + a.chunks_per_split);
  const int n_c = max(0, c1 - c0);
  const int krange = n_c * 128;
  __half* xs = reinterpret_cast<__half*>(gsm);                                  // [MT][krange]
  float* sumx = reinterpret_cast<float*>(gsm + size_t(MT) * krange * 2);        // [MT][n_c]
  float* red = sumx + MT * n_c;                                                 // [slices][128][MT]
  const int row = threadIdx.x & 127, slice = threadIdx.x >> 7;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- weight stream: constant data, so the first requests go out before the previous kernel has finished; two
  // chunks per thread are in flight (more would cost the second CTA per SM its registers)
  const uint8_t* wt = a.w + (size_t(tile) * a.k_chunks + c0) * kW4ChunkBytes;
  uint4 nx1[4];
  __half2 ns1 = __half2half2(__ushort_as_half(0));
  auto fetch = [&](int c, uint4* dst, __half2& sz) {
    if (c < n_c) {
      const uint8_t* chunk = wt + size_t(c) * kW4ChunkBytes;
#pragma unroll
      for (int p4 = 0; p4 < 4; ++p4) dst[p4] = ldg_stream(chunk + (p4 * 128 + row) * 16);
      sz = __ldg(reinterpret_cast<const __half2*>(chunk + 8192 + row * 4));
    }
  };
  fetch(slice, nx1, ns1);

  pdl_wait();                                        // the activations come from the previous kernel
  // ---- stage the activations of this K range, and their sums per quantisation group
  for (int m = 0; m < MT; ++m) {
    const bool live = m < a.M;
    const uint4* src = reinterpret_cast<const uint4*>(a.x + size_t(live ? m : 0) * a.K + size_t(c0) * 128);
    uint4* dst = reinterpret_cast<uint4*>(xs + size_t(m) * krange);
    for (int i = threadIdx.x; i < krange / 8; i += kGemvThreads) dst[i] = live ? src[i] : make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
  for (int g = warp; g < MT * n_c; g += kGemvThreads / 32) {
    const int m = g / n_c, c = g % n_c;
    const uint2 v = reinterpret_cast<const uint2*>(xs + size_t(m) * krange + c * 128)[lane];
    const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
    const float2 q = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
    const float s = warp_sum(p.x + p.y + q.x + q.y);
    if (lane == 0) sumx[g] = s;
  }
  __syncthreads();

  // ---- main loop: this thread's row, chunks slice, slice + 4, ...
  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m] = 0.f;
  for (int c = slice; c < n_c; c += kGemvSlices) {
    uint4 pk[4];
#pragma unroll
    for (int p4 = 0; p4 < 4; ++p4) pk[p4] = nx1[p4];
    const __half2 sz = ns1;
    fetch(c + kGemvSlices, nx1, ns1);
    float qx[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) qx[m] = 0.f;
#pragma unroll
    for (int p4 = 0; p4 < 4; ++p4) {
      const uint32_t words[4] = {pk[p4].x, pk[p4].y, pk[p4].z, pk[p4].w};
#pragma unroll
      for (int wd = 0; wd < 4; ++wd) {
        __half2 q[4];
        unpack_word(words[wd], q);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          // 8 consecutive activations; every lane reads the same address (shared-memory broadcast)
          const uint4 xv = *reinterpret_cast<const uint4*>(xs + size_t(m) * krange + c * 128 + p4 * 32 + wd * 8);
          const __half2* xh = reinterpret_cast<const __half2*>(&xv);
          __half2 s = __hmul2(q[0], xh[0]);
          s = __hfma2(q[1], xh[1], s);
          s = __hfma2(q[2], xh[2], s);
          s = __hfma2(q[3], xh[3], s);
          const float2 f = __half22float2(s);
          qx[m] += f.x + f.y;
        }
      }
    }
    const float sc = __low2float(sz), zr = __high2float(sz);
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] += sc * qx[m] + zr * sumx[m * n_c + c];
  }
  // ---- add the K slices, epilogue
#pragma unroll
  for (int m = 0; m < MT; ++m) red[(slice * 128 + row) * MT + m] = acc[m];
  __syncthreads();
  if (slice != 0) return;
  float v[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    v[m] = 0.f;
#pragma unroll
    for (int s = 0; s < kGemvSlices; ++s) v[m] += red[(s * 128 + row) * MT + m];
  }
  if (EPI == kEpiSwiGLU) {
    // rows 64..127 hold `up`: pass them to the thread that holds the matching `gate` row
    __shared__ float up[64 * MT];
    if (row >= 64) {
#pragma unroll
      for (int m = 0; m < MT; ++m) up[(row - 64) * MT + m] = v[m];
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (row < 64) {
      const int n = tile * 64 + row;
      __half* out = reinterpret_cast<__half*>(a.out);
#pragma unroll
      for (int m = 0; m < MT; ++m)
        if (m < a.M && n < a.N / 2)
          out[size_t(m) * a.ldo + n] = __float2half_rn(clamp_f16(silu_f(v[m]) * up[row * MT + m]));
    }
  } else {
    const int n = tile * kTileN + row;
    if (n < a.N) {
      float bias = 0.f;
      if (EPI == kEpiF16 && a.bias != nullptr) bias = __half2float(a.bias[n]);
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (m < a.M) {
          if (EPI == kEpiF16)
            reinterpret_cast<__half*>(a.out)[size_t(m) * a.ldo + n] = __float2half_rn(clamp_f16(v[m] + bias));
          else
            reinterpret_cast<float*>(a.out)[(size_t(blockIdx.z) * a.M + m) * a.ldo + n] = v[m];
        }
      }
    }
  }
}

static size_t gemv_smem(int MT, int chunks) {
  return size_t(MT) * chunks * 128 * 2 + size_t(MT) * chunks * 4 + size_t(kGemvSlices) * 128 * MT * 4 + 16;
}

// K splits for a GEMV launch, or 0 when this kernel should not be used (too many tokens, or too few tiles to fill the
// GPU with an epilogue that cannot be split over K).
int gemv_w4_plan(int M, int N, int K, int epilogue, int sm_count, int want_split) {
  if (M < 1 || M > 2 || K % 128) return 0;
  const int n_tiles = epilogue == kEpiSwiGLU ? (N / 2 + 63) / 64 : (N + kTileN - 1) / kTileN;
  const int k_chunks = K / 128;
  int ks = 1;
  if (epilogue == kEpiPartialF32) {
    const int target = 2 * sm_count;
    ks = want_split > 0 ? want_split : (target + n_tiles - 1) / n_tiles;
    ks = max(1, min(ks, min(8, max(1, k_chunks / (2 * kGemvSlices)))));
  } else if (n_tiles < sm_count / 2) {
    return 0;                                        // the tensor-core kernel splits K inside a cluster instead
  }
  int cps = (k_chunks + ks - 1) / ks;
  while (gemv_smem(2, cps) > size_t(kGemvMaxSmem)) {
    if (epilogue != kEpiPartialF32 || ks >= 8) return 0;
    ++ks;
    cps = (k_chunks + ks - 1) / ks;
  }
  return (k_chunks + cps - 1) / cps;                 // no empty split
}

template <int MT, int EPI>
static int launch_gemv(const GemvArgs& a, dim3 grid, size_t smem, cudaStream_t st) {
  auto kern = gemv_w4_kernel<MT, EPI>;
  static bool attr_done[kMaxDevices] = {};
  const int dev_slot = current_device_slot();
  if (!attr_done[dev_slot]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvMaxSmem) != cudaSuccess)
      return ZSE_ERR_LAUNCH;
    attr_done[dev_slot] = true;
  }
  return launch_pdl(kern, grid, dim3(kGemvThreads), smem, st, a) == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

int gemv_w4_launch(const void* w_tiled, const void* x, const void* bias, void* out, int M, int N, int K, int ldo,
                   int epilogue, int ks, cudaStream_t st) {
  const int n_tiles = epilogue == kEpiSwiGLU ? (N / 2 + 63) / 64 : (N + kTileN - 1) / kTileN;
  const int k_chunks = K / 128;
  const int cps = (k_chunks + ks - 1) / ks;
  GemvArgs a{reinterpret_cast<const uint8_t*>(w_tiled), reinterpret_cast<const __half*>(x),
             reinterpret_cast<const __half*>(bias), out, M, N, K, ldo, k_chunks, cps};
  dim3 grid(n_tiles, 1, ks);
  const int MT = M <= 1 ? 1 : 2;
  const size_t smem = gemv_smem(MT, cps);
#define ZSE_GEMV_EPI(MTV)                                                                     \
  switch (epilogue) {                                                                         \
    case kEpiF16: return launch_gemv<MTV, kEpiF16>(a, grid, smem, st);                        \
    case kEpiSwiGLU: return launch_gemv<MTV, kEpiSwiGLU>(a, grid, smem, st);                  \
    case kEpiPartialF32: return launch_gemv<MTV, kEpiPartialF32>(a, grid, smem, st);          \
    default: return ZSE_ERR_SHAPE;                                                            \
  }
  if (MT == 1) {
    ZSE_GEMV_EPI(1)
  }
  ZSE_GEMV_EPI(2)
#undef ZSE_GEMV_EPI
}

}  // namespace zse

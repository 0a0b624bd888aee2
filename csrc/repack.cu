// Load-time weight transforms: row-major .zse INT4 -> the tiled chunk stream gemm_w4_kernel consumes, plain
// dequantisation to fp16 (shapes the tiled kernel does not take) and device-side group quantisation.
//
// Chunk (n_tile, k_stage) = 8704 bytes:
//   [h:2][part:2][row:128][16 B]   nibbles of K values k_stage*128 + h*64 + part*32 + (0..31) of tile row `row`;
//                                  inside each 32-bit word the eight values sit at nibble positions
//                                  e0,e2,e4,e6,e1,e3,e5,e7
//   [row:128]{scale fp16, zero fp16}
// Rows past N are zero with scale = zero = 0.  The reference's counterpart is the 64x8 WMMA re-tiling
// (zse-engine/zse_engine/orchestrator/kernels.py:2421-2450, format/fast_quant.py:193-225).
#include "api.h"
#include "common.cuh"

namespace zse {

__global__ void repack_w4_kernel(const uint8_t* __restrict__ packed, const __half* __restrict__ scales,
                                 const __half* __restrict__ zeros, uint8_t* __restrict__ out, int N, int K,
                                 int interleave_rows) {
  const int ks = blockIdx.x, nt = blockIdx.y;
  const int k_stages = K / 128;
  const int r = threadIdx.x & 127, h = threadIdx.x >> 7;
  int src_row;
  bool valid;
  if (interleave_rows > 0) {
    const int local = nt * 64 + (r & 63);
    valid = local < interleave_rows;
    src_row = (r < 64 ? 0 : interleave_rows) + local;
  } else {
    src_row = nt * 128 + r;
    valid = src_row < N;
  }
  uint8_t* chunk = out + (size_t(nt) * k_stages + ks) * 8704;
  uint32_t words[8];
  if (valid) {
    const uint4* src = reinterpret_cast<const uint4*>(packed + size_t(src_row) * (K / 2) + ks * 64 + h * 32);
    const uint4 a = src[0], b = src[1];
    const uint32_t in[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t w = in[j];
      // source nibble i holds element e_i
      uint32_t o = 0;
      o |= ((w >> 0) & 0xF) << 0;    // e0
      o |= ((w >> 8) & 0xF) << 4;    // e2
      o |= ((w >> 16) & 0xF) << 8;   // e4
      o |= ((w >> 24) & 0xF) << 12;  // e6
      o |= ((w >> 4) & 0xF) << 16;   // e1
      o |= ((w >> 12) & 0xF) << 20;  // e3
      o |= ((w >> 20) & 0xF) << 24;  // e5
      o |= ((w >> 28) & 0xF) << 28;  // e7
      words[j] = o;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) words[j] = 0;
  }
  *reinterpret_cast<uint4*>(chunk + ((h * 2 + 0) * 128 + r) * 16) = make_uint4(words[0], words[1], words[2], words[3]);
  *reinterpret_cast<uint4*>(chunk + ((h * 2 + 1) * 128 + r) * 16) = make_uint4(words[4], words[5], words[6], words[7]);
  if (h == 0) {
    __half2 sz = __halves2half2(__ushort_as_half(0), __ushort_as_half(0));
    if (valid) sz = __halves2half2(scales[size_t(src_row) * k_stages + ks], zeros[size_t(src_row) * k_stages + ks]);
    *reinterpret_cast<__half2*>(chunk + 8192 + r * 4) = sz;
  }
}

__global__ void dequant_w4_kernel(const uint8_t* __restrict__ packed, const __half* __restrict__ scales,
                                  const __half* __restrict__ zeros, __half* __restrict__ out, int64_t n, int gs) {
  const int64_t i = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) * 2;
  if (i >= n) return;
  const uint8_t b = packed[i >> 1];
  const int64_t g0 = i / gs, g1 = (i + 1) / gs;
  out[i] = __float2half_rn(float(b & 0xF) * __half2float(scales[g0]) + __half2float(zeros[g0]));
  if (i + 1 < n) out[i + 1] = __float2half_rn(float(b >> 4) * __half2float(scales[g1]) + __half2float(zeros[g1]));
}

__global__ void dequant_w8_kernel(const int8_t* __restrict__ q, const __half* __restrict__ scales,
                                  __half* __restrict__ out, int64_t n, int gs) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2half_rn(float(q[i]) * __half2float(scales[i / gs]));
}

// ---- INT8 (symmetric, groups of 128 along K, fp16 scale) -----------------------------------------------------
// Tiled chunk (n_tile, k_stage) = 16640 bytes:
//   [part:8][row:128][16 B]   int8 values of K = k_stage*128 + part*16 + (0..15) of tile row `row`
//   [row:128] scale fp16
// Rows past N are zero with scale 0.  interleave_rows as for INT4 (64 gate rows + 64 up rows per tile).
__global__ void repack_w8_kernel(const int8_t* __restrict__ q, const __half* __restrict__ scales,
                                 uint8_t* __restrict__ out, int N, int K, int interleave_rows) {
  const int ks = blockIdx.x, nt = blockIdx.y;
  const int k_stages = K / 128;
  const int r = threadIdx.x & 127, h = threadIdx.x >> 7;       // h: parts 4h .. 4h+3
  int src_row;
  bool valid;
  if (interleave_rows > 0) {
    const int local = nt * 64 + (r & 63);
    valid = local < interleave_rows;
    src_row = (r < 64 ? 0 : interleave_rows) + local;
  } else {
    src_row = nt * 128 + r;
    valid = src_row < N;
  }
  uint8_t* chunk = out + (size_t(nt) * k_stages + ks) * 16640;
  const uint4* src = reinterpret_cast<const uint4*>(q + size_t(src_row) * K + ks * 128) + h * 4;
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const uint4 v = valid ? src[p] : make_uint4(0, 0, 0, 0);
    *reinterpret_cast<uint4*>(chunk + ((h * 4 + p) * 128 + r) * 16) = v;
  }
  if (h == 0)
    *reinterpret_cast<__half*>(chunk + 16384 + r * 2) =
        valid ? scales[size_t(src_row) * k_stages + ks] : __ushort_as_half(0);
}

// Tiled INT8 chunks -> dense fp16 [N, K] row-major (gate rows then up rows for an interleaved tensor): what a pass of
// more than 64 tokens runs through the fp16 GEMM, into a scratch buffer that every layer shares.
__global__ void dequant_w8_tiled_kernel(const uint8_t* __restrict__ tiled, __half* __restrict__ out, int N, int K,
                                        int interleave_rows) {
  const int ks = blockIdx.x, nt = blockIdx.y;
  const int k_stages = K / 128;
  const int r = threadIdx.x & 127, h = threadIdx.x >> 7;
  int dst_row;
  bool valid;
  if (interleave_rows > 0) {
    const int local = nt * 64 + (r & 63);
    valid = local < interleave_rows;
    dst_row = (r < 64 ? 0 : interleave_rows) + local;
  } else {
    dst_row = nt * 128 + r;
    valid = dst_row < N;
  }
  if (!valid) return;
  const uint8_t* chunk = tiled + (size_t(nt) * k_stages + ks) * 16640;
  const float s = __half2float(*reinterpret_cast<const __half*>(chunk + 16384 + r * 2));
  __half* dst = out + size_t(dst_row) * K + ks * 128 + h * 64;
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const uint4 v = *reinterpret_cast<const uint4*>(chunk + ((h * 4 + p) * 128 + r) * 16);
    const int8_t* b = reinterpret_cast<const int8_t*>(&v);
    uint4 lo, hi;
    uint32_t* l = reinterpret_cast<uint32_t*>(&lo);
    uint32_t* u = reinterpret_cast<uint32_t*>(&hi);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      l[i] = pack_half2(float(b[2 * i]) * s, float(b[2 * i + 1]) * s);
      u[i] = pack_half2(float(b[8 + 2 * i]) * s, float(b[8 + 2 * i + 1]) * s);
    }
    reinterpret_cast<uint4*>(dst + p * 16)[0] = lo;
    reinterpret_cast<uint4*>(dst + p * 16)[1] = hi;
  }
}

// One warp per group of 128 fp16 values -> 64 bytes + scale + zero (round to nearest, like the python writer).
__global__ void quantize_w4_kernel(const __half* __restrict__ w, uint8_t* __restrict__ packed,
                                   __half* __restrict__ scales, __half* __restrict__ zeros, int64_t n_groups) {
  const int64_t g = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (g >= n_groups) return;
  const int lane = threadIdx.x & 31;
  const __half2* src = reinterpret_cast<const __half2*>(w + g * 128) + lane * 2;
  const float2 a = __half22float2(src[0]), b = __half22float2(src[1]);
  float mn = fminf(fminf(a.x, a.y), fminf(b.x, b.y)), mx = fmaxf(fmaxf(a.x, a.y), fmaxf(b.x, b.y));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  const float range = mx - mn;
  const float scale = range < 1e-10f ? 1.0f : range / 15.0f;
  const float inv = 1.0f / scale;
  auto qz = [&](float v) { return uint32_t(min(15, max(0, __float2int_rn((v - mn) * inv)))); };
  const uint32_t q0 = qz(a.x), q1 = qz(a.y), q2 = qz(b.x), q3 = qz(b.y);
  reinterpret_cast<uint16_t*>(packed + g * 64)[lane] = uint16_t(q0 | (q1 << 4) | (q2 << 8) | (q3 << 12));
  if (lane == 0) {
    scales[g] = __float2half_rn(scale);
    zeros[g] = __float2half_rn(mn);
  }
}

}  // namespace zse

using namespace zse;

extern "C" int64_t zse_w4_tiled_bytes(int N, int K) {
  return int64_t((N + 127) / 128) * (K / 128) * 8704;
}

extern "C" int zse_repack_w4(const void* packed, const void* scales, const void* zeros, void* out_tiled, int N, int K,
                             int interleave_rows, void* stream) {
  if (K % 128 != 0 || N <= 0) return ZSE_ERR_SHAPE;
  if (interleave_rows > 0 && N != 2 * interleave_rows) return ZSE_ERR_SHAPE;
  const int n_tiles = interleave_rows > 0 ? (interleave_rows + 63) / 64 : (N + 127) / 128;
  dim3 grid(K / 128, n_tiles);
  repack_w4_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint8_t*>(packed), reinterpret_cast<const __half*>(scales),
      reinterpret_cast<const __half*>(zeros), reinterpret_cast<uint8_t*>(out_tiled), N, K, interleave_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

extern "C" int64_t zse_w8_tiled_bytes(int N, int K) {
  return int64_t((N + 127) / 128) * (K / 128) * 16640;
}

// Row-major INT8 [N, K] + fp16 scales [N, K/128] -> tiled chunks (interleave_rows as in zse_repack_w4).
extern "C" int zse_repack_w8(const void* q, const void* scales, void* out_tiled, int N, int K, int interleave_rows,
                             void* stream) {
  if (K % 128 != 0 || N <= 0) return ZSE_ERR_SHAPE;
  if (interleave_rows > 0 && N != 2 * interleave_rows) return ZSE_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out_tiled) & 15)) return ZSE_ERR_ALIGN;
  const int n_tiles = interleave_rows > 0 ? (interleave_rows + 63) / 64 : (N + 127) / 128;
  dim3 grid(K / 128, n_tiles);
  repack_w8_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const int8_t*>(q), reinterpret_cast<const __half*>(scales),
      reinterpret_cast<uint8_t*>(out_tiled), N, K, interleave_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

// Tiled INT8 chunks -> fp16 [N, K] row-major.
extern "C" int zse_dequant_w8_tiled(const void* tiled, void* out_f16, int N, int K, int interleave_rows,
                                    void* stream) {
  if (K % 128 != 0 || N <= 0) return ZSE_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(out_f16) & 15) return ZSE_ERR_ALIGN;
  const int n_tiles = interleave_rows > 0 ? (interleave_rows + 63) / 64 : (N + 127) / 128;
  dim3 grid(K / 128, n_tiles);
  dequant_w8_tiled_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint8_t*>(tiled), reinterpret_cast<__half*>(out_f16), N, K, interleave_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

extern "C" int zse_dequant_w4(const void* packed, const void* scales, const void* zeros, void* out_f16,
                              int64_t n_elements, int group_size, void* stream) {
  const int64_t threads = (n_elements + 1) / 2;
  dequant_w4_kernel<<<unsigned((threads + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint8_t*>(packed), reinterpret_cast<const __half*>(scales),
      reinterpret_cast<const __half*>(zeros), reinterpret_cast<__half*>(out_f16), n_elements, group_size);
  return cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

extern "C" int zse_dequant_w8(const void* q, const void* scales, void* out_f16, int64_t n_elements, int group_size,
                              void* stream) {
  dequant_w8_kernel<<<unsigned((n_elements + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const int8_t*>(q), reinterpret_cast<const __half*>(scales), reinterpret_cast<__half*>(out_f16),
      n_elements, group_size);
  return cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

extern "C" int zse_quantize_w4(const void* w_f16, void* packed, void* scales, void* zeros, int64_t n_groups,
                               void* stream) {
  quantize_w4_kernel<<<unsigned((n_groups + 7) / 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __half*>(w_f16), reinterpret_cast<uint8_t*>(packed), reinterpret_cast<__half*>(scales),
      reinterpret_cast<__half*>(zeros), n_groups);
  return cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

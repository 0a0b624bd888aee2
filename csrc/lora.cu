// Batched multi-adapter LoRA: every token carries its own adapter index, so one launch pair serves a decode batch
// whose requests use different adapters (the reference splits the batch by adapter and runs three tiled-matmul
// launches per projection, zse-engine/zse_engine/orchestrator/lora_manager.py:281-361).
//   shrink: tmp[t, r]  = sum_k x[t, k] * A[a_t][r, k]
//   expand: y[t, n]   += scale[a_t] * sum_r tmp[t, r] * B[a_t][n, r]
// Tokens with adapter index -1 are untouched.
#include "api.h"
#include "common.cuh"

namespace zse {

// grid (rank, M), one warp-group of 128 threads per (token, rank row)
__global__ void __launch_bounds__(128)
lora_shrink_kernel(const __half* __restrict__ x, int ldx, const __half* __restrict__ A, const int* __restrict__ ids,
                   float* __restrict__ tmp, int K, int rank) {
  __shared__ float red[4];
  const int r = blockIdx.x, t = blockIdx.y;
  const int a = ids[t];
  if (a < 0) {
    if (threadIdx.x == 0) tmp[size_t(t) * rank + r] = 0.f;
    return;
  }
  const uint4* xr = reinterpret_cast<const uint4*>(x + size_t(t) * ldx);
  const uint4* ar = reinterpret_cast<const uint4*>(A + (size_t(a) * rank + r) * K);
  float acc = 0.f;
  for (int i = threadIdx.x; i < K / 8; i += blockDim.x) {
    const uint4 xv = xr[i], av = ar[i];
    const __half2* xh = reinterpret_cast<const __half2*>(&xv);
    const __half2* ah = reinterpret_cast<const __half2*>(&av);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 xf = __half22float2(xh[j]), af = __half22float2(ah[j]);
      acc += xf.x * af.x + xf.y * af.y;
    }
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) tmp[size_t(t) * rank + r] = red[0] + red[1] + red[2] + red[3];
}

// grid (ceil(N/256), M)
__global__ void __launch_bounds__(256)
lora_expand_kernel(const float* __restrict__ tmp, const __half* __restrict__ B, const int* __restrict__ ids,
                   const float* __restrict__ scales, __half* __restrict__ y, int ldy, int N, int rank) {
  extern __shared__ float tv[];
  const int t = blockIdx.y;
  const int a = ids[t];
  if (a < 0) return;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) tv[i] = tmp[size_t(t) * rank + i];
  __syncthreads();
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const __half* b = B + (size_t(a) * N + n) * rank;
  float acc = 0.f;
  for (int r = 0; r < rank; r += 2) {
    const float2 bf = __half22float2(*reinterpret_cast<const __half2*>(b + r));
    acc += bf.x * tv[r] + bf.y * tv[r + 1];
  }
  __half* dst = y + size_t(t) * ldy + n;
  *dst = __float2half_rn(clamp_f16(__half2float(*dst) + scales[a] * acc));
}


// Shrink and expand in ONE launch, one CTA per token: the activation row is staged in shared memory once, the warps
// take the rank rows of A in turn (16-byte loads, fp32 accumulation, one warp reduction per row), and after a barrier
// every thread adds scale * (t . B[n, :]) to its output columns.  A [rank, K] and B [N, rank] of the token's adapter
// are read once per token, from L2 when several tokens share an adapter; nothing goes through global memory in
// between.  The two-launch pair above re-read the activation row once per rank row.
__global__ void __launch_bounds__(256)
lora_apply_kernel(const __half* __restrict__ x, int ldx, const __half* __restrict__ A, const __half* __restrict__ B,
                  const int* __restrict__ ids, const float* __restrict__ scales, __half* __restrict__ y, int ldy, int K,
                  int N, int rank) {
  extern __shared__ __align__(16) unsigned char lora_smem[];
  float* tv = reinterpret_cast<float*>(lora_smem);                       // [64]
  uint4* xs = reinterpret_cast<uint4*>(lora_smem + 256);                  // [K / 8]
  const int t = blockIdx.x;
  const int a = ids[t];
  if (a < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint4* xr = reinterpret_cast<const uint4*>(x + size_t(t) * ldx);
  for (int i = threadIdx.x; i < K / 8; i += blockDim.x) xs[i] = xr[i];
  __syncthreads();
  for (int r = warp; r < rank; r += 8) {
    const uint4* ar = reinterpret_cast<const uint4*>(A + (size_t(a) * rank + r) * K);
    float acc = 0.f;
    for (int i = lane; i < K / 8; i += 32) {
      const uint4 xv = xs[i], av = ar[i];
      const __half2* xh = reinterpret_cast<const __half2*>(&xv);
      const __half2* ah = reinterpret_cast<const __half2*>(&av);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 xf = __half22float2(xh[j]), af = __half22float2(ah[j]);
        acc += xf.x * af.x + xf.y * af.y;
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) tv[r] = acc;
  }
  __syncthreads();
  const float scale = scales[a];
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    const __half* b = B + (size_t(a) * N + n) * rank;
    float acc = 0.f;
    for (int r = 0; r < rank; r += 2) {
      const float2 bf = __half22float2(*reinterpret_cast<const __half2*>(b + r));
      acc += bf.x * tv[r] + bf.y * tv[r + 1];
    }
    __half* dst = y + size_t(t) * ldy + n;
    *dst = __float2half_rn(clamp_f16(__half2float(*dst) + scale * acc));
  }
}

}  // namespace zse

using namespace zse;

extern "C" int zse_lora_shrink(const void* x, int ldx, const void* a, const void* ids, void* tmp, int M, int K,
                               int rank, void* stream) {
  if (M <= 0) return 0;
  if (K % 8 || rank <= 0 || ldx % 8) return ZSE_ERR_SHAPE;
  lora_shrink_kernel<<<dim3(rank, M), 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __half*>(x), ldx, reinterpret_cast<const __half*>(a), reinterpret_cast<const int*>(ids),
      reinterpret_cast<float*>(tmp), K, rank);
  return cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

extern "C" int zse_lora_expand(const void* tmp, const void* b, const void* ids, const void* scales, void* y, int ldy,
                               int M, int N, int rank, void* stream) {
  if (M <= 0) return 0;
  if (rank % 2 || rank <= 0) return ZSE_ERR_SHAPE;
  lora_expand_kernel<<<dim3((N + 255) / 256, M), 256, rank * sizeof(float), reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float*>(tmp), reinterpret_cast<const __half*>(b), reinterpret_cast<const int*>(ids),
      reinterpret_cast<const float*>(scales), reinterpret_cast<__half*>(y), ldy, N, rank);
  return cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

// y[t, :N] += scale[a_t] * (x[t, :K] A[a_t]^T) B[a_t]^T for every token with an adapter, one launch
// (lora_apply_kernel).  rank even and <= 64, K a multiple of 8 with K * 2 + 256 bytes of shared memory available.
extern "C" int zse_lora_apply(const void* x, int ldx, const void* a, const void* b, const void* ids, const void* scales,
                              void* y, int ldy, int M, int K, int N, int rank, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 8 || ldx % 8 || rank <= 0 || rank % 2 || rank > 64) return ZSE_ERR_SHAPE;
  const size_t smem = 256 + size_t(K) * 2;
  if (smem > 200 * 1024) return ZSE_ERR_SHAPE;
  static size_t raised[kMaxDevices] = {};
  const int dev_slot = current_device_slot();
  if (smem > 48 * 1024 && smem > raised[dev_slot]) {
    if (cudaFuncSetAttribute(lora_apply_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
      return ZSE_ERR_LAUNCH;
    raised[dev_slot] = 200 * 1024;
  }
  lora_apply_kernel<<<M, 256, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __half*>(x), ldx, reinterpret_cast<const __half*>(a), reinterpret_cast<const __half*>(b),
      reinterpret_cast<const int*>(ids), reinterpret_cast<const float*>(scales), reinterpret_cast<__half*>(y), ldy, K, N,
      rank);
  return cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

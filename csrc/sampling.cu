// Token selection on the device: logits never travel to the host.
//
// The reference samples on the CPU after downloading fp16 logits (zse-engine/zse_engine/orchestrator/sampler.py:33-213:
// repetition penalty, temperature, top-k, top-p, categorical) and has single-CTA argmax kernels
// (kernels.py:2307-2397).  Here one CTA per row does all of it.  fp16 logits map to order-preserving 16-bit keys, so
// the k-th largest value and the top-p cut are found exactly with two 256-bin histogram passes each (high byte,
// then low byte) instead of a sort.  Ties at the cut value are all kept.
#include "api.h"
#include "common.cuh"

namespace zse {

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ uint32_t key_of(__half h) {
  const uint32_t b = __half_as_ushort(h);
  return (b & 0x8000u) ? (~b & 0xFFFFu) : (b | 0x8000u);
}
__device__ __forceinline__ float value_of_key(uint32_t k) {
  const uint32_t b = (k & 0x8000u) ? (k & 0x7FFFu) : (~k & 0xFFFFu);
  return __half2float(__ushort_as_half((unsigned short)b));
}

__device__ __forceinline__ unsigned long long block_max_u64(unsigned long long v, unsigned long long* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
    v = other > v ? other : v;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    unsigned long long t = lane < (blockDim.x >> 5) ? red[lane] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, t, o);
      t = other > t ? other : t;
    }
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  const unsigned long long r = red[0];
  __syncthreads();
  return r;
}

// (key, lowest index) of the row maximum; 16-byte loads when the row is 16-byte aligned
__device__ __forceinline__ unsigned long long row_argmax(const __half* row, int V, unsigned long long* red) {
  unsigned long long best = 0ull;
  auto consider = [&](__half h, int i) {
    const unsigned long long cand = ((unsigned long long)key_of(h) << 32) | (0xFFFFFFFFu - (unsigned)i);
    best = cand > best ? cand : best;
  };
  if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const int nvec = V / 8;
    const uint4* rv = reinterpret_cast<const uint4*>(row);
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      const uint4 v = rv[i];
      const __half* h = reinterpret_cast<const __half*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) consider(h[j], i * 8 + j);
    }
    for (int i = nvec * 8 + threadIdx.x; i < V; i += blockDim.x) consider(row[i], i);
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) consider(row[i], i);
  }
  return block_max_u64(best, red);
}

__global__ void __launch_bounds__(kSampleThreads)
argmax_kernel(const __half* __restrict__ logits, int ld, int* __restrict__ out, int V) {
  __shared__ unsigned long long red[32];
  pdl_launch_dependents();
  pdl_wait();
  const unsigned long long b = row_argmax(logits + size_t(blockIdx.x) * ld, V, red);
  if (threadIdx.x == 0) out[blockIdx.x] = int(0xFFFFFFFFu - unsigned(b & 0xFFFFFFFFull));
}

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// Scan a 256-bin histogram from the top; returns the bin where the running total first reaches `target` and the
// total of the bins above it.  Executed by thread 0.
template <typename T>
__device__ __forceinline__ int find_bin(const T* hist, T target, T* above) {
  T run = 0;
  for (int b = 255; b >= 0; --b) {
    if (run + hist[b] >= target) {
      *above = run;
      return b;
    }
    run += hist[b];
  }
  *above = run;
  return 0;
}

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const __half* __restrict__ logits, int ld, int* __restrict__ out, int V,
              const float* __restrict__ temperature, const int* __restrict__ top_k, const float* __restrict__ top_p,
              const unsigned long long* __restrict__ seeds, unsigned long long step) {
  __shared__ unsigned long long red[32];
  __shared__ int hist_i[256];
  __shared__ float hist_f[256];
  __shared__ float scan[kSampleThreads / 32];
  __shared__ int sh_bin;
  __shared__ int sh_rem_i;
  __shared__ float sh_rem_f;
  __shared__ float sh_total;
  __shared__ int sh_choice;
  const int rowi = blockIdx.x;
  const __half* row = logits + size_t(rowi) * ld;
  const float T = temperature ? temperature[rowi] : 1.f;
  const int k = top_k ? top_k[rowi] : 0;
  const float p = top_p ? top_p[rowi] : 1.f;

  const unsigned long long best = row_argmax(row, V, red);
  const int best_idx = int(0xFFFFFFFFu - unsigned(best & 0xFFFFFFFFull));
  if (T <= 0.f || k == 1) {
    if (threadIdx.x == 0) out[rowi] = best_idx;
    return;
  }
  const float mx = value_of_key(uint32_t(best >> 32));
  const float inv_t = 1.f / T;
  const int tid = threadIdx.x;

  // ---- top-k: key of the k-th largest logit ------------------------------------------------------------
  uint32_t kth_key = 0;
  if (k > 0 && k < V) {
    if (tid < 256) hist_i[tid] = 0;
    __syncthreads();
    for (int i = tid; i < V; i += blockDim.x) atomicAdd(&hist_i[key_of(row[i]) >> 8], 1);
    __syncthreads();
    if (tid == 0) {
      int above;
      sh_bin = find_bin<int>(hist_i, k, &above);
      sh_rem_i = k - above;
    }
    __syncthreads();
    const int hi = sh_bin, rem = sh_rem_i;
    __syncthreads();
    if (tid < 256) hist_i[tid] = 0;
    __syncthreads();
    for (int i = tid; i < V; i += blockDim.x) {
      const uint32_t key = key_of(row[i]);
      if (int(key >> 8) == hi) atomicAdd(&hist_i[key & 0xFF], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int above;
      sh_bin = find_bin<int>(hist_i, rem, &above);
    }
    __syncthreads();
    kth_key = (uint32_t(hi) << 8) | uint32_t(sh_bin);
    __syncthreads();
  }

  // ---- top-p over the softmax of what survived top-k ----------------------------------------------------
  uint32_t thr_key = kth_key;
  if (p < 1.f) {
    if (tid < 256) hist_f[tid] = 0.f;
    __syncthreads();
    for (int i = tid; i < V; i += blockDim.x) {
      const uint32_t key = key_of(row[i]);
      if (key >= kth_key) atomicAdd(&hist_f[key >> 8], __expf((__half2float(row[i]) - mx) * inv_t));
    }
    __syncthreads();
    if (tid == 0) {
      float z = 0.f;
      for (int b = 0; b < 256; ++b) z += hist_f[b];
      float above;
      sh_bin = find_bin<float>(hist_f, p * z, &above);
      sh_rem_f = p * z - above;
    }
    __syncthreads();
    const int hi = sh_bin;
    const float rem = sh_rem_f;
    __syncthreads();
    if (tid < 256) hist_f[tid] = 0.f;
    __syncthreads();
    for (int i = tid; i < V; i += blockDim.x) {
      const uint32_t key = key_of(row[i]);
      if (key >= kth_key && int(key >> 8) == hi)
        atomicAdd(&hist_f[key & 0xFF], __expf((__half2float(row[i]) - mx) * inv_t));
    }
    __syncthreads();
    if (tid == 0) {
      float above;
      sh_bin = find_bin<float>(hist_f, rem, &above);
    }
    __syncthreads();
    const uint32_t p_key = (uint32_t(hi) << 8) | uint32_t(sh_bin);
    thr_key = p_key > kth_key ? p_key : kth_key;
    __syncthreads();
  }

  // ---- categorical draw over the kept set, in index order -------------------------------------------------
  const int chunk = (V + blockDim.x - 1) / blockDim.x;
  const int lo = tid * chunk, hi_idx = min(V, lo + chunk);
  float mine = 0.f;
  for (int i = lo; i < hi_idx; ++i)
    if (key_of(row[i]) >= thr_key) mine += __expf((__half2float(row[i]) - mx) * inv_t);
  // block exclusive scan
  float incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, incl, o);
    if ((tid & 31) >= o) incl += n;
  }
  if ((tid & 31) == 31) scan[tid >> 5] = incl;
  if (tid == 0) sh_choice = -1;
  __syncthreads();
  if (tid < 32) {
    float v = tid < (blockDim.x >> 5) ? scan[tid] : 0.f;
    float inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, inc, o);
      if (tid >= o) inc += n;
    }
    if (tid < (blockDim.x >> 5)) scan[tid] = inc - v;      // exclusive warp offsets
    if (tid == 31) sh_total = inc;
  }
  __syncthreads();
  const float excl = scan[tid >> 5] + incl - mine;
  const float total = sh_total;
  // a row that brings its own seed draws from that seed alone: the token does not depend on which row of the batch
  // the request happens to sit in; rows without seeds are told apart by their index
  const uint64_t r = seeds ? splitmix64(seeds[rowi] ^ splitmix64(step * 0x2545F4914F6CDD1Dull))
                           : splitmix64(splitmix64(step * 0x2545F4914F6CDD1Dull + rowi));
  const float u = float(r >> 40) * (1.0f / 16777216.0f) * total;
  if (mine > 0.f && u >= excl && u < excl + mine) {
    float run = excl;
    int pick = -1, last = -1;
    for (int i = lo; i < hi_idx; ++i) {
      if (key_of(row[i]) >= thr_key) {
        last = i;
        run += __expf((__half2float(row[i]) - mx) * inv_t);
        if (run > u) {
          pick = i;
          break;
        }
      }
    }
    atomicMax(&sh_choice, pick >= 0 ? pick : last);
  }
  __syncthreads();
  if (tid == 0) out[rowi] = sh_choice >= 0 ? sh_choice : best_idx;
}

// logit <- logit / f (positive) or logit * f (negative), f = penalty^(1 + log2(count))
__global__ void repetition_penalty_kernel(__half* __restrict__ logits, int ld, const int* __restrict__ rows,
                                          const int* __restrict__ tokens, const int* __restrict__ counts, int n,
                                          const float* __restrict__ penalty, int V) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int r = rows[i], t = tokens[i], c = counts[i];
  const float pen = penalty[r];
  if (c <= 0 || pen == 1.f || t < 0 || t >= V) return;
  const float f = powf(pen, 1.f + log2f(float(c)));
  __half* p = logits + size_t(r) * ld + t;
  const float v = __half2float(*p);
  *p = __float2half_rn(v > 0.f ? v / f : v * f);
}

}  // namespace zse

using namespace zse;

extern "C" int zse_argmax(const void* logits, int ld, void* out, int M, int V, void* stream) {
  if (M <= 0) return 0;
  return launch_pdl(argmax_kernel, dim3(M), dim3(kSampleThreads), 0, reinterpret_cast<cudaStream_t>(stream),
                    reinterpret_cast<const __half*>(logits), ld, reinterpret_cast<int*>(out), V) == cudaSuccess
             ? 0
             : ZSE_ERR_LAUNCH;
}

extern "C" int zse_sample(const void* logits, int ld, void* out, int M, int V, const void* temperature,
                          const void* top_k, const void* top_p, const void* seeds, uint64_t step, void* stream) {
  if (M <= 0) return 0;
  sample_kernel<<<M, kSampleThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __half*>(logits), ld, reinterpret_cast<int*>(out), V,
      reinterpret_cast<const float*>(temperature), reinterpret_cast<const int*>(top_k),
      reinterpret_cast<const float*>(top_p), reinterpret_cast<const unsigned long long*>(seeds), step);
  return cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

extern "C" int zse_apply_repetition_penalty(void* logits, int ld, const void* rows, const void* tokens,
                                            const void* counts, int n, const void* penalty, int V, void* stream) {
  if (n <= 0) return 0;
  repetition_penalty_kernel<<<(n + 255) / 256, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__half*>(logits), ld, reinterpret_cast<const int*>(rows), reinterpret_cast<const int*>(tokens),
      reinterpret_cast<const int*>(counts), n, reinterpret_cast<const float*>(penalty), V);
  return cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

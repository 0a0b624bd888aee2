// Dense fp16-weight linear layers on the 5th-generation tensor cores (lm_head, tensors the INT4 kernel does not
// take, int8 models expanded at load).
//
//   Y[t, n] = sum_k X[t, k] * W[n, k]          X fp16 [M, K] row-major, W fp16 [N, K] row-major
//
// The product is computed transposed ("swap AB"): the UMMA M dimension (128) runs over weight rows n, the UMMA N
// dimension (16..256) over tokens t, so a decode step with a handful of tokens still fills the 128 TMEM lanes and W
// is read exactly once.  Both operands arrive by tiled TMA with the 128-byte swizzle and are consumed from shared
// memory by tcgen05.mma; the accumulator lives in TMEM.  Epilogues: fp16 store (+bias) or fp32 split-K planes.
// Replaces the reference's fp16 GEMV / tiled fp16 matmul (zse-engine/zse_engine/orchestrator/kernels.py:1075-1126,
// 2077-2107).  The INT4 kernel is in gemm_w4.cu.
#include <mutex>
#include <unordered_map>

#include "gemm_common.cuh"

namespace zse {

struct PipeBars {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t a_ready[8];
  uint64_t acc_ready;
  uint32_t tmem_base;
  int abort_flag;
};

// ---- epilogue shared by both kernels ---------------------------------------------------------------
// Warps 2..9: quarter q = warp % 4 owns TMEM lanes [32q, 32q+32); half ch = (warp-2)/4 owns the columns
// [ch*NT/2, (ch+1)*NT/2) (for NT == 16 only ch == 0 works).
template <int NT, int EPI>
__device__ __forceinline__ void epilogue(const GemmArgs& a, uint32_t tmem_acc, int warp, int lane, float* stage_smem,
                                         bool valid) {
  const int q = warp & 3;
  const int ch = (warp - 2) >> 2;
  constexpr int kColsPerHalf = NT >= 32 ? NT / 2 : NT;
  // A warp with nothing to do (no columns, or an aborted main loop) still meets its partner at the pair barrier.
  if ((NT < 32 && ch != 0) || !valid) {
    if (EPI == kEpiSwiGLU) asm volatile("bar.sync %0, 64;" ::"r"(1 + ((q & 1) + 2 * ch)) : "memory");
    return;
  }
  const int col0 = ch * kColsPerHalf;
  const int n_tile = blockIdx.x, t0 = blockIdx.y * NT;
  const uint32_t taddr = tmem_acc + (uint32_t(q * 32) << 16) + col0;

  if (EPI == kEpiSwiGLU) {
    // up rows (q = 2, 3) park their values in shared memory; gate rows (q = 0, 1) combine.
    float* park = stage_smem + ((q & 1) + 2 * ch) * (32 * kColsPerHalf);
    const int bar_id = 1 + ((q & 1) + 2 * ch);
    if (q >= 2) {
#pragma unroll 1
      for (int c = 0; c < kColsPerHalf; c += 16) {
        uint32_t r[16];
        ZSE_TMEM_LD_X16(r, taddr + c);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i) park[(c + i) * 32 + lane] = __uint_as_float(r[i]);
      }
      asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");
    } else {
      asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");
      const int n_out = n_tile * 64 + q * 32 + lane;
      __half* out = reinterpret_cast<__half*>(a.out);
#pragma unroll 1
      for (int c = 0; c < kColsPerHalf; c += 16) {
        uint32_t r[16];
        ZSE_TMEM_LD_X16(r, taddr + c);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int t = t0 + col0 + c + i;
          if (t < a.M && n_out < a.N / 2) {
            const float g = __uint_as_float(r[i]);
            const float u = park[(c + i) * 32 + lane];
            out[size_t(t) * a.ldo + n_out] = __float2half_rn(clamp_f16(silu_f(g) * u));
          }
        }
      }
    }
    return;
  }

  const int n = n_tile * kTileN + q * 32 + lane;
  const bool n_ok = n < a.N;
  float bias = 0.f;
  if (EPI == kEpiF16 && a.bias != nullptr && n_ok) bias = __half2float(a.bias[n]);
#pragma unroll 1
  for (int c = 0; c < kColsPerHalf; c += 16) {
    uint32_t r[16];
    ZSE_TMEM_LD_X16(r, taddr + c);
    tc_wait_ld();
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int t = t0 + col0 + c + i;
      if (t < a.M && n_ok) {
        const float v = __uint_as_float(r[i]);
        if (EPI == kEpiF16) {
          reinterpret_cast<__half*>(a.out)[size_t(t) * a.ldo + n] = __float2half_rn(clamp_f16(v + bias));
        } else {
          reinterpret_cast<float*>(a.out)[(size_t(blockIdx.z) * a.M + t) * a.ldo + n] = v;
        }
      }
    }
  }
}

// ---- fp16 weights ------------------------------------------------------------------------------------
template <int NT>
struct F16Cfg {
  static constexpr int kStageK = 64;
  static constexpr int kABytes = kTileN * 128;
  static constexpr int kXBytes = NT * 128;
  static constexpr int kStageBytes = kABytes + kXBytes;
  static constexpr int kStages = NT <= 64 ? 4 : (NT == 128 ? 6 : 4);
  static constexpr int kTmemCols = NT < 32 ? 32 : NT;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
  static constexpr int kMinBlocks = NT <= 64 ? 2 : 1;
};

template <int NT, int EPI>
__global__ void __launch_bounds__(kGemmThreads, F16Cfg<NT>::kMinBlocks)
gemm_f16_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                const GemmArgs a) {
  using Cfg = F16Cfg<NT>;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  PipeBars* bars = reinterpret_cast<PipeBars*>(smem + S * Cfg::kStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  const int s_begin = blockIdx.z * a.stages_per_split;
  const int n_iter = min(a.k_stages, s_begin + a.stages_per_split) - s_begin;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&bars->full[i], 1);
      mbar_init(&bars->empty[i], 1);
    }
    mbar_init(&bars->acc_ready, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmap_w);
    prefetch_tmap(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;
  volatile int* abort_flag = &bars->abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      int issued = 0;
      pdl_wait();                                        // the activations come from the previous kernel
      for (int it = 0; it < n_iter; ++it) {
        const int s = it % S;
        if (it >= S && !mbar_wait(&bars->empty[s], ((it / S) - 1) & 1, abort_flag, a.status, 11, it)) break;
        uint8_t* st = smem + s * Cfg::kStageBytes;
        mbar_arrive_expect_tx(&bars->full[s], Cfg::kStageBytes);
        const int k0 = (s_begin + it) * Cfg::kStageK;
        tma_load_2d(st, &tmap_w, k0, blockIdx.x * kTileN, &bars->full[s]);
        tma_load_2d(st + Cfg::kABytes, &tmap_x, k0, blockIdx.y * NT, &bars->full[s]);
        issued = it + 1;
      }
      if (*abort_flag) {
        for (int it = max(0, issued - S); it < issued; ++it) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&bars->full[it % S], (it / S) & 1) && globaltimer_ns() - t0 < kWaitLimitNs) {
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(kTileN, NT);
      for (int it = 0; it < n_iter; ++it) {
        const int s = it % S;
        if (!mbar_wait(&bars->full[s], (it / S) & 1, abort_flag, a.status, 12, it)) break;
        tc_fence_after_sync();
        const uint32_t ab = smem_u32(smem + s * Cfg::kStageBytes);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          umma_ss(tmem, make_desc_sw128(ab + j * 32), make_desc_sw128(ab + Cfg::kABytes + j * 32), idesc,
                  (it | j) != 0);
        tc_commit(&bars->empty[s]);
      }
      tc_commit(&bars->acc_ready);
    }
  } else {
    const bool ok = mbar_wait(&bars->acc_ready, 0, abort_flag, a.status, 15, 0);
    tc_fence_after_sync();
    epilogue<NT, EPI>(a, tmem, warp, lane, reinterpret_cast<float*>(smem), ok);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, Cfg::kTmemCols);
}

// ---- host side ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  uint64_t rows, cols;
  uint32_t box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.ptr) ^ (k.rows * 1000003u) ^ (k.cols * 7919u) ^ (uint64_t(k.box_rows) << 48);
  }
};

// fp16 [rows, cols] row-major, box = 64 columns x box_rows rows, 128-byte swizzle, zero fill out of bounds.
int get_tmap(const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows, CUtensorMap* out) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  MapKey key{ptr, rows, cols, box_rows};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return 0;
  }
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return ZSE_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (cols * 2) % 16) return ZSE_ERR_ALIGN;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return ZSE_ERR_DRIVER;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return 0;
}

template <int NT, int EPI>
static int launch_f16(const CUtensorMap& tw, const CUtensorMap& tx, const GemmArgs& a, dim3 grid, cudaStream_t st) {
  auto kern = gemm_f16_kernel<NT, EPI>;
  static bool attr_done[kMaxDevices] = {};
  const int dev_slot = current_device_slot();
  if (!attr_done[dev_slot]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, F16Cfg<NT>::kSmemBytes) !=
        cudaSuccess)
      return ZSE_ERR_LAUNCH;
    attr_done[dev_slot] = true;
  }
  return launch_pdl(kern, grid, dim3(kGemmThreads), size_t(F16Cfg<NT>::kSmemBytes), st, tw, tx, a) == cudaSuccess
             ? 0
             : ZSE_ERR_LAUNCH;
}

}  // namespace zse

using namespace zse;

extern "C" int zse_gemm_f16(const void* w, int w_rows_cap, const void* x, int x_rows_cap, const void* bias, void* out,
                            int M, int N, int K, int ldo, int epilogue, int k_split, void* status, void* stream) {
  if (M <= 0) return 0;
  if (K % 8 != 0 || N <= 0 || epilogue == kEpiSwiGLU) return ZSE_ERR_SHAPE;
  if (epilogue != kEpiPartialF32) k_split = 1;
  const int k_stages = (K + 63) / 64;
  k_split = max(1, min(k_split, k_stages));
  const int spp = (k_stages + k_split - 1) / k_split;
  k_split = (k_stages + spp - 1) / spp;
  const int nt = pick_nt(M);
  CUtensorMap tw, tx;
  if (int rc = get_tmap(w, uint64_t(max(w_rows_cap, N)), uint64_t(K), uint32_t(kTileN), &tw)) return rc;
  if (int rc = get_tmap(x, uint64_t(max(x_rows_cap, M)), uint64_t(K), uint32_t(nt), &tx)) return rc;
  GemmArgs a{nullptr, reinterpret_cast<const __half*>(bias), out, M, N, K, ldo, k_stages, spp,
             reinterpret_cast<Status*>(status)};
  dim3 grid((N + kTileN - 1) / kTileN, (M + nt - 1) / nt, k_split);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int rc = ZSE_ERR_SHAPE;
  if (epilogue == kEpiF16) {
    ZSE_DISPATCH_NT(nt, rc = (launch_f16<NT, kEpiF16>(tw, tx, a, grid, st)))
  } else {
    ZSE_DISPATCH_NT(nt, rc = (launch_f16<NT, kEpiPartialF32>(tw, tx, a, grid, st)))
  }
  return rc;
}

extern "C" int zse_gemm_f16_splits(int M, int N, int K, int k_split) {
  const int k_stages = (K + 63) / 64;
  k_split = max(1, min(k_split, max(1, k_stages)));
  const int spp = (k_stages + k_split - 1) / k_split;
  return (k_stages + spp - 1) / max(1, spp);
}

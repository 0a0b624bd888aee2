// Linear layers on the 5th-generation tensor cores.
//
//   Y[t, n] = sum_k X[t, k] * W[n, k]          X fp16 [M, K] row-major, W is [N, K]
//
// Both kernels compute the transposed product on the hardware ("swap AB"): the UMMA M dimension (128)
// runs over weight rows n, the UMMA N dimension (16..256) over tokens t, so that a decode step with a
// handful of tokens still fills the 128 TMEM lanes and the weight stream is read exactly once.
//
// gemm_w4_kernel  - INT4 group-128 weights (w = nibble*scale + zero).  Per K stage of 128 one 8704-byte chunk
//                   (8192 B of nibbles + 128 x {scale, zero}) arrives by a 1-D bulk TMA copy; eight warps turn it
//                   into fp16 in registers and write it with tcgen05.st straight into TMEM, from where
//                   tcgen05.mma takes it as the A operand (no shared-memory round trip for the dequantised
//                   weights).  The activations arrive by tiled TMA with the 128-byte swizzle and are the B operand.
// gemm_f16_kernel - fp16 weights (lm_head, LoRA-free dense tensors, odd shapes): both operands from shared memory.
//
// Epilogues: fp16 store (+bias), SwiGLU (tile rows 0..63 = gate, 64..127 = up of the same 64 outputs), fp32 split-K
// partials for the row-parallel projections (reduced by add_rmsnorm together with the residual).
//
// Replaces the scalar dequant GEMV / 32x32 tiled matmul kernels of the reference
// (zse-engine/zse_engine/orchestrator/kernels.py:1129-1192,1906-2073,2114-2203).
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "api.h"
#include "common.cuh"

namespace zse {

constexpr int kTileN = 128;          // weight rows per CTA (UMMA M)
constexpr int kW4StageK = 128;       // K per pipeline stage of the INT4 kernel (= quantisation group)
constexpr int kW4ChunkBytes = 8704;  // 8192 nibble bytes + 512 bytes of {scale, zero}
constexpr int kGemmThreads = 320;    // warp 0 producer, warp 1 MMA issuer, warps 2..9 dequant + epilogue

enum Epilogue : int { kEpiF16 = 0, kEpiSwiGLU = 1, kEpiPartialF32 = 2 };

struct GemmArgs {
  const uint8_t* w;        // W4: tiled chunks [n_tiles][k_stages][8704]; F16: unused (tensor map)
  const __half* bias;      // [N] or null (kEpiF16 only)
  void* out;               // fp16 [M, ldo] / fp32 [k_split][M, ldo]
  int M, N, K;
  int ldo;                 // output row stride in elements
  int k_stages;            // total K stages
  int stages_per_split;
  Status* status;
};

template <int NT>
struct W4Cfg {
  static constexpr int kStages = NT <= 64 ? 3 : (NT == 128 ? 5 : 3);
  static constexpr int kTmemCols = NT <= 64 ? 256 : 512;
  static constexpr int kACol0 = NT;                       // A ring starts after the accumulator
  static constexpr int kXBytes = NT * 128;                // one 64-wide K sub-tile of X
  static constexpr int kStageBytes = 2 * kXBytes + kW4ChunkBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
  static constexpr int kMinBlocks = NT <= 64 ? 2 : 1;
};

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

// ---- INT4 weights ------------------------------------------------------------------------------------
// Nibble order inside every 32-bit word of a chunk (fixed by repack_w4): positions 0..7 hold the K elements
// e0,e2,e4,e6,e1,e3,e5,e7 so that masking with 0x000f000f yields the adjacent pair (e0,e1) as a half2.
__device__ __forceinline__ void dequant_word(uint32_t w, __half2 s2, __half2 z2, uint32_t* out4) {
  const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
  const __half2 k16th = __half2half2(__ushort_as_half(0x2C00));   // 1/16
  const __half2 kNeg64 = __half2half2(__ushort_as_half(0xD400));  // -64
  uint32_t t0, t1, t2, t3;
  const uint32_t w8 = w >> 8;
  asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xEA;" : "=r"(t0) : "r"(w));
  asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xEA;" : "=r"(t1) : "r"(w));
  asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xEA;" : "=r"(t2) : "r"(w8));
  asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xEA;" : "=r"(t3) : "r"(w8));
  __half2 e0 = __hsub2(*reinterpret_cast<__half2*>(&t0), k1024);
  __half2 e1 = __hfma2(*reinterpret_cast<__half2*>(&t1), k16th, kNeg64);
  __half2 e2 = __hsub2(*reinterpret_cast<__half2*>(&t2), k1024);
  __half2 e3 = __hfma2(*reinterpret_cast<__half2*>(&t3), k16th, kNeg64);
  e0 = __hfma2(e0, s2, z2);
  e1 = __hfma2(e1, s2, z2);
  e2 = __hfma2(e2, s2, z2);
  e3 = __hfma2(e3, s2, z2);
  out4[0] = *reinterpret_cast<uint32_t*>(&e0);
  out4[1] = *reinterpret_cast<uint32_t*>(&e1);
  out4[2] = *reinterpret_cast<uint32_t*>(&e2);
  out4[3] = *reinterpret_cast<uint32_t*>(&e3);
}

template <int NT, int EPI>
__global__ void __launch_bounds__(kGemmThreads, W4Cfg<NT>::kMinBlocks)
gemm_w4_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmArgs a) {
  using Cfg = W4Cfg<NT>;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* x_tiles = smem;                                   // [S][2][NT*128]
  uint8_t* w_chunks = smem + S * 2 * Cfg::kXBytes;           // [S][8704]
  PipeBars* bars = reinterpret_cast<PipeBars*>(w_chunks + S * kW4ChunkBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x;
  const int s_begin = blockIdx.z * a.stages_per_split;
  const int s_end = min(a.k_stages, s_begin + a.stages_per_split);
  const int n_iter = s_end - s_begin;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&bars->full[i], 1);
      mbar_init(&bars->empty[i], 1);
      mbar_init(&bars->a_ready[i], 8);
    }
    mbar_init(&bars->acc_ready, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
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
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      const uint8_t* wsrc = a.w + (size_t(n_tile) * a.k_stages + s_begin) * kW4ChunkBytes;
      int issued = 0;
      for (int it = 0; it < n_iter; ++it) {
        const int s = it % S;
        if (it >= S && !mbar_wait(&bars->empty[s], ((it / S) - 1) & 1, abort_flag, a.status, 1, it)) break;
        mbar_arrive_expect_tx(&bars->full[s], Cfg::kStageBytes);
        bulk_g2s(w_chunks + s * kW4ChunkBytes, wsrc + size_t(it) * kW4ChunkBytes, kW4ChunkBytes, &bars->full[s]);
        const int k0 = (s_begin + it) * kW4StageK;
        tma_load_2d(x_tiles + (s * 2 + 0) * Cfg::kXBytes, &tmap_x, k0, blockIdx.y * NT, &bars->full[s]);
        tma_load_2d(x_tiles + (s * 2 + 1) * Cfg::kXBytes, &tmap_x, k0 + 64, blockIdx.y * NT, &bars->full[s]);
        issued = it + 1;
      }
      if (*abort_flag) {
        // drain: every copy that was issued must land before the CTA may exit
        for (int it = max(0, issued - S); it < issued; ++it) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&bars->full[it % S], (it / S) & 1) && globaltimer_ns() - t0 < kWaitLimitNs) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(kTileN, NT);
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int s = it % S;
        const uint32_t ph = (it / S) & 1;
        ok = mbar_wait(&bars->full[s], ph, abort_flag, a.status, 2, it) &&
             mbar_wait(&bars->a_ready[s], ph, abort_flag, a.status, 3, it);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t xb = smem_u32(x_tiles + s * 2 * Cfg::kXBytes);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint64_t bdesc = make_desc_sw128(xb + (j >> 2) * Cfg::kXBytes + (j & 3) * 32);
          umma_ts(tmem, tmem + Cfg::kACol0 + s * 64 + j * 8, bdesc, idesc, (it | j) != 0);
        }
        tc_commit(&bars->empty[s]);
      }
      tc_commit(&bars->acc_ready);
    }
  } else {
    // ------------------------------------------------------------------ dequant: chunk -> fp16 -> TMEM
    const int q = warp & 3;              // TMEM lane quarter this warp may touch
    const int h = (warp - 2) >> 2;       // which 64 of the 128 K values of a stage
    const int r = q * 32 + lane;         // weight row inside the tile
    for (int it = 0; it < n_iter; ++it) {
      const int s = it % S;
      if (!mbar_wait(&bars->full[s], (it / S) & 1, abort_flag, a.status, 4, it)) break;
      const uint8_t* chunk = w_chunks + s * kW4ChunkBytes;
      const __half2 sz = *reinterpret_cast<const __half2*>(chunk + 8192 + r * 4);
      const __half2 s2 = __half2half2(__low2half(sz)), z2 = __half2half2(__high2half(sz));
      const uint32_t tdst = tmem + (uint32_t(q * 32) << 16) + Cfg::kACol0 + s * 64 + h * 32;
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        const uint4 pk = *reinterpret_cast<const uint4*>(chunk + ((h * 2 + part) * 128 + r) * 16);
        uint32_t o[16];
        dequant_word(pk.x, s2, z2, o + 0);
        dequant_word(pk.y, s2, z2, o + 4);
        dequant_word(pk.z, s2, z2, o + 8);
        dequant_word(pk.w, s2, z2, o + 12);
        ZSE_TMEM_ST_X16(tdst + part * 16, o);
      }
      tc_wait_st();
      tc_fence_before_sync();
      if (lane == 0) mbar_arrive(&bars->a_ready[s]);
    }
    // ---------------------------------------------------------------- epilogue
    const bool ok = mbar_wait(&bars->acc_ready, 0, abort_flag, a.status, 5, 0);
    tc_fence_after_sync();
    epilogue<NT, EPI>(a, tmem, warp, lane, reinterpret_cast<float*>(smem), ok);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, Cfg::kTmemCols);
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
static int get_tmap(const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows, CUtensorMap* out) {
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

static int pick_nt(int M) {
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128) return 128;
  return 256;
}

template <int NT, int EPI>
static int launch_w4(const CUtensorMap& tx, const GemmArgs& a, dim3 grid, cudaStream_t st) {
  auto kern = gemm_w4_kernel<NT, EPI>;
  static bool attr_done = false;
  if (!attr_done) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, W4Cfg<NT>::kSmemBytes) != cudaSuccess)
      return ZSE_ERR_LAUNCH;
    attr_done = true;
  }
  kern<<<grid, kGemmThreads, W4Cfg<NT>::kSmemBytes, st>>>(tx, a);
  return cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

template <int NT, int EPI>
static int launch_f16(const CUtensorMap& tw, const CUtensorMap& tx, const GemmArgs& a, dim3 grid, cudaStream_t st) {
  auto kern = gemm_f16_kernel<NT, EPI>;
  static bool attr_done = false;
  if (!attr_done) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, F16Cfg<NT>::kSmemBytes) !=
        cudaSuccess)
      return ZSE_ERR_LAUNCH;
    attr_done = true;
  }
  kern<<<grid, kGemmThreads, F16Cfg<NT>::kSmemBytes, st>>>(tw, tx, a);
  return cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

#define ZSE_DISPATCH_NT(nt, CALL)   \
  switch (nt) {                     \
    case 16: { constexpr int NT = 16; CALL; } break;   \
    case 32: { constexpr int NT = 32; CALL; } break;   \
    case 64: { constexpr int NT = 64; CALL; } break;   \
    case 128: { constexpr int NT = 128; CALL; } break; \
    default: { constexpr int NT = 256; CALL; } break;  \
  }

}  // namespace zse

using namespace zse;

extern "C" int zse_gemm_w4(const void* w_tiled, const void* x, int x_rows_cap, const void* bias, void* out, int M,
                           int N, int K, int ldo, int epilogue, int k_split, void* status, void* stream) {
  if (M <= 0) return 0;
  if (K % kW4StageK != 0 || N <= 0) return ZSE_ERR_SHAPE;
  if (epilogue != kEpiPartialF32) k_split = 1;
  const int k_stages = K / kW4StageK;
  k_split = max(1, min(k_split, k_stages));
  const int spp = (k_stages + k_split - 1) / k_split;
  k_split = (k_stages + spp - 1) / spp;
  const int nt = pick_nt(M);
  CUtensorMap tx;
  if (int rc = get_tmap(x, uint64_t(max(x_rows_cap, M)), uint64_t(K), uint32_t(nt), &tx)) return rc;
  GemmArgs a{reinterpret_cast<const uint8_t*>(w_tiled), reinterpret_cast<const __half*>(bias), out, M, N, K, ldo,
             k_stages, spp, reinterpret_cast<Status*>(status)};
  dim3 grid((N + kTileN - 1) / kTileN, (M + nt - 1) / nt, k_split);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int rc = ZSE_ERR_SHAPE;
  if (epilogue == kEpiF16) {
    ZSE_DISPATCH_NT(nt, rc = (launch_w4<NT, kEpiF16>(tx, a, grid, st)))
  } else if (epilogue == kEpiSwiGLU) {
    ZSE_DISPATCH_NT(nt, rc = (launch_w4<NT, kEpiSwiGLU>(tx, a, grid, st)))
  } else if (epilogue == kEpiPartialF32) {
    ZSE_DISPATCH_NT(nt, rc = (launch_w4<NT, kEpiPartialF32>(tx, a, grid, st)))
  }
  return rc;
}

extern "C" int zse_gemm_w4_splits(int M, int N, int K, int k_split) {
  // the number of fp32 partial planes zse_gemm_w4 / zse_gemm_f16 will actually write for this request
  const int k_stages = K / kW4StageK;
  k_split = max(1, min(k_split, max(1, k_stages)));
  const int spp = (k_stages + k_split - 1) / k_split;
  return (k_stages + spp - 1) / max(1, spp);
}

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

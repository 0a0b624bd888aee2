// INT4 group-128 weight GEMM for decode-sized passes (1..64 tokens): one persistent CTA per SM.
//
//   Y[t, n] = sum_k X[t, k] * (nibble[n, k] * scale[n, k/128] + zero[n, k/128])       (swap-AB, as in gemm_w4.cu)
//
// What a decode step needs from this GEMM is not FLOPs but an even weight stream over all SMs and a small fixed cost,
// so the kernel is organised around the stream:
//
//  * Work is the linear space (tile pair, K stage): a "step" is one 128-wide K stage of two adjacent 128-row weight
//    tiles.  Each CTA takes one contiguous range of steps (balanced to +-1 step), so every SM reads the same number
//    of bytes whatever the shape.  Two plans:
//      stream  (many tile pairs)  range c = [c*T/n, (c+1)*T/n): a pair may start in one CTA and end in the next;
//      split   (few tile pairs)   every pair is cut into S equal K segments, one CTA each.
//  * Inside a CTA two pipelines run side by side, one per tile of the pair, and share every activation stage:
//      warp 0      bulk-TMA producer of the weight chunks (one ring per pipeline),
//      warp 1      tiled-TMA producer of the activation stages,
//      warps 2,3   MMA issuers (tcgen05.mma, A = dequantised weights in TMEM, B = activations in shared memory),
//      warps 4-19  dequant: four groups of four warps; a group owns ONE TMEM operand slot, two groups alternate on
//                  the chunks of a pipeline, so dequantising chunk c+1 overlaps the MMAs of chunk c,
//      warps 20-23 epilogue: accumulators are double-buffered in TMEM, so the epilogue of one tile pair runs while
//                  the pipelines already work on the next.
//  * Partial sums of a tile pair that was cut meet in a workspace in global memory (it stays in L2):
//      stream plan: the CTA that holds K stage 0 of the pair owns it; the others dump their fp32 partials first thing
//                   (their piece of that pair is the head of their range) and the owner, which reaches the pair last,
//                   adds them;
//      split plan:  all S CTAs of a pair finish together; each dumps what it does not own and finishes the token
//                   columns it owns (column granule g belongs to segment g mod S), so the fix-up itself is parallel.
//    Flags carry a launch epoch kept in device memory, so nothing has to be reset and a CUDA graph can replay the
//    launch unchanged.
//  * Epilogues work on finished sums staged in shared memory and store 16 bytes per thread: fp16 (+bias), fp32,
//    SwiGLU (tile rows 0..63 gate, 64..127 up), and the fused QKV epilogue (bias + rotate-half RoPE from a cos/sin
//    table + K/V rows written straight into the paged cache).
//
// Replaces, for decode-sized passes, the scalar dequant GEMV / tiled matmul kernels and the separate RoPE + cache-write
// launches of the reference (zse-engine/zse_engine/orchestrator/kernels.py:1129-1192,1906-2073,2114-2203 and
// orchestrator/model_runner.py:1299-1474).
//
// Every wait is bounded and reports through the status word; all CTAs of a launch are resident (grid <= SM count, one
// CTA per SM by shared-memory footprint), which is what makes the waits on other CTAs legitimate.
#include <stdlib.h>

#include "gemm_common.cuh"

namespace zse {

constexpr int kDecWarps = 24;
constexpr int kDecThreads = kDecWarps * 32;
constexpr int kDecSX = 5;            // activation stages
constexpr int kDecSW = 6;            // weight chunks per pipeline ring
constexpr int kDecEpiWarp0 = 20;
constexpr int kDecStageBytes = 64 * 128 * 4;     // finished sums of one tile: [token column][128 rows] fp32

enum DecEpilogue : int { kDecF16 = 0, kDecSwiGLU = 1, kDecF32 = 2, kDecQkvRope = 3, kDecAllReduceNorm = 4 };

struct DecBars {
  uint64_t w_full[2][kDecSW], w_empty[2][kDecSW];
  uint64_t x_full[kDecSX], x_empty[kDecSX];
  uint64_t a_ready[2][2], slot_free[2][2];
  uint64_t acc_full[2][2], acc_empty[2][2];
  uint32_t tmem_base;
  int abort_flag;
};

template <int NT>
struct DecCfg {
  static constexpr int kXBytes = NT * 128;                  // one 64-wide K sub-tile of X
  static constexpr int kXStage = 2 * kXBytes;
  static constexpr int kXRing = ((kDecSX * kXStage + 1023) / 1024) * 1024;
  static constexpr int kWRing = 2 * kDecSW * kW4ChunkBytes;
  static constexpr int kStageOff = kXRing + ((kWRing + 127) / 128) * 128;
  static constexpr int kBarsOff = kStageOff + kDecStageBytes;
  static constexpr int kSmemBytes = kBarsOff + 1024 + 1024;   // barriers + alignment slack
  static constexpr int kGranules = NT / 8;                    // 8-column granules of the token dimension
  static_assert(kSmemBytes <= 232448, "shared memory budget");
};

struct DecRope {
  const int* positions;        // [M]
  const long long* slots;      // [M] cache slot = block * block_size + offset; -1 = do not store
  const float2* cos_sin;       // [max_position][64] {cos, sin} of position * inv_freq[i]
  __half* kv_layer;            // [blocks][2][nkv][block_size][128]
  int nh, nkv, block_size, max_position;
};

struct DecArgs {
  const uint8_t* w;            // tiled chunks [n_tiles][k_stages][8704]
  const __half* bias;          // [N] or null
  void* out;
  int M, N, ldo;
  int k_stages, n_tiles, n_pairs;
  int total_steps;             // n_pairs * k_stages
  int split;                   // 0: stream plan; S >= 1: split plan with S segments per pair
  float* ws;                   // workspace: [grid][2][NT][128] fp32 partial sums
  uint32_t* sync;              // [0] launch epoch, [1] exit ticket, [8 + cta] partial-ready flags
  Status* status;
  DecRope rope;
};

__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

#define ZSE_TMEM_LD_X8(r, taddr)                                                                               \
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"                         \
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) \
               : "r"(taddr)                                                                                    \
               : "memory")

// Nibble order inside every 32-bit word of a chunk (fixed by repack_w4): positions 0..7 hold the K elements
// e0,e2,e4,e6,e1,e3,e5,e7 so that masking with 0x000f000f yields the adjacent pair (e0,e1) as a half2.
__device__ __forceinline__ void dec_dequant_word(uint32_t w, __half2 s2, __half2 z2, uint32_t* out4) {
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

__device__ __forceinline__ void dec_dequant_half(const uint4& w0, const uint4& w1, __half2 s2, __half2 z2,
                                                 uint32_t* o) {
  dec_dequant_word(w0.x, s2, z2, o + 0);
  dec_dequant_word(w0.y, s2, z2, o + 4);
  dec_dequant_word(w0.z, s2, z2, o + 8);
  dec_dequant_word(w0.w, s2, z2, o + 12);
  dec_dequant_word(w1.x, s2, z2, o + 16);
  dec_dequant_word(w1.y, s2, z2, o + 20);
  dec_dequant_word(w1.z, s2, z2, o + 24);
  dec_dequant_word(w1.w, s2, z2, o + 28);
}

// Bounded wait until a flag word in global memory holds `want`.
__device__ __forceinline__ bool dec_wait_flag(const uint32_t* flag, uint32_t want, volatile int* abort_flag, Status* st,
                                              unsigned where, unsigned detail) {
  if (ld_acquire_gpu_u32(flag) == want) return true;
  const uint64_t t0 = globaltimer_ns();
  unsigned spins = 0;
  while (ld_acquire_gpu_u32(flag) != want) {
    if ((++spins & 0x3F) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > kWaitLimitNs) {
        report(st, kWaitTimeout, where, detail);
        *abort_flag = 1;
        __threadfence_block();
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// Barrier of the 128 epilogue threads that also ANDs a predicate: after a bounded wait all of them take the same
// branch, so nobody is left alone at a later barrier.
__device__ __forceinline__ bool epi_all(bool v) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.and.pred q, 1, 128, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"(uint32_t(v))
      : "memory");
  return r != 0;
}

// First step of CTA c.  stream plan: balanced cut of the linear step space; split plan: segment (c % S) of pair c / S.
__device__ __forceinline__ int dec_range_begin(const DecArgs& a, int c, int n_cta) {
  if (a.split > 0) {
    const int pair = c / a.split, seg = c - pair * a.split;
    if (pair >= a.n_pairs) return a.total_steps;
    return pair * a.k_stages + int((long long)seg * a.k_stages / a.split);
  }
  return int((long long)c * a.total_steps / n_cta);
}

template <int NT, int EPI>
__global__ void __launch_bounds__(kDecThreads, 1)
gemm_w4_dec_kernel(const __grid_constant__ CUtensorMap tmap_x, const DecArgs a) {
  using Cfg = DecCfg<NT>;
  constexpr int SX = kDecSX, SW = kDecSW;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* x_ring = smem;                                        // [SX][2][NT*128]
  uint8_t* w_ring = smem + Cfg::kXRing;                          // [2][SW][8704]
  float* stage = reinterpret_cast<float*>(smem + Cfg::kStageOff);   // [NT][128]
  DecBars* bars = reinterpret_cast<DecBars*>(smem + Cfg::kBarsOff);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // The next kernel of the stream may start its own set-up now; this kernel in turn starts before the one ahead of it
  // has finished: set-up, the weight stream and the dequantisation (constant data) run at once, the activation
  // producer and the epilogue wait for the producer of the activations (pdl_wait below).
  pdl_launch_dependents();
  const int cta = blockIdx.x, n_cta = gridDim.x;
  const int ks = a.k_stages;
  const int g0 = dec_range_begin(a, cta, n_cta);
  const int g1 = dec_range_begin(a, cta + 1, n_cta);
  const int n_steps = g1 - g0;
  // the last pair of an odd tile count has one tile: pipeline 1 has nothing to do from `single_from` on
  const int single_from = (a.n_tiles & 1) ? (a.n_pairs - 1) * ks : a.total_steps;
  const int n_real1 = max(0, min(g1, single_from) - g0);        // steps of this CTA in which pipeline 1 has a chunk

  if (threadIdx.x == 0) {
    for (int p = 0; p < 2; ++p) {
      for (int i = 0; i < SW; ++i) {
        mbar_init(&bars->w_full[p][i], 1);
        mbar_init(&bars->w_empty[p][i], 4);
      }
      for (int i = 0; i < 2; ++i) {
        mbar_init(&bars->a_ready[p][i], 4);
        mbar_init(&bars->slot_free[p][i], 1);
        mbar_init(&bars->acc_full[p][i], 1);
        mbar_init(&bars->acc_empty[p][i], 4);
      }
    }
    for (int i = 0; i < SX; ++i) {
      mbar_init(&bars->x_full[i], 1);
      mbar_init(&bars->x_empty[i], 2);
    }
    bars->abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmap_x);
  }
  if (warp == 2) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;
  volatile int* abort_flag = &bars->abort_flag;
  // TMEM columns: accumulator (pipeline p, buffer b) at (2p + b) * 64; operand slot (pipeline p, slot s) at
  // 256 + (2p + s) * 64 (a dequantised 128 x 128 fp16 chunk = 64 columns of 32 bits)

  if (warp == 0) {
    // ------------------------------------------------------------------ weight producer (both rings)
    if (lane == 0) {
      int cnt[2] = {0, 0};
      bool ok = true;
      for (int s = 0; s < n_steps && ok; ++s) {
        const int g = g0 + s, pair = g / ks, k = g - pair * ks;
        const int ntp = g < single_from ? 2 : 1;
        for (int r = 0; r < ntp; ++r) {
          const int slot = cnt[r] % SW, use = cnt[r] / SW;
          if (use > 0 && !mbar_wait(&bars->w_empty[r][slot], (use - 1) & 1, abort_flag, a.status, 1, s)) {
            ok = false;
            break;
          }
          const uint8_t* src = a.w + (size_t(2 * pair + r) * ks + k) * kW4ChunkBytes;
          mbar_arrive_expect_tx(&bars->w_full[r][slot], kW4ChunkBytes);
          bulk_g2s(w_ring + (r * SW + slot) * kW4ChunkBytes, src, kW4ChunkBytes, &bars->w_full[r][slot]);
          ++cnt[r];
        }
      }
      if (*abort_flag) {                       // every issued copy must land before the CTA may exit
        for (int r = 0; r < 2; ++r)
          for (int it = max(0, cnt[r] - SW); it < cnt[r]; ++it) {
            const uint64_t t0 = globaltimer_ns();
            while (!mbar_try_wait(&bars->w_full[r][it % SW], (it / SW) & 1) && globaltimer_ns() - t0 < kWaitLimitNs) {
            }
          }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ activation producer
    if (lane == 0) {
      int issued = 0;
      pdl_wait();                                          // the activations come from the previous kernel
      for (int s = 0; s < n_steps; ++s) {
        const int st = s % SX, use = s / SX;
        if (use > 0 && !mbar_wait(&bars->x_empty[st], (use - 1) & 1, abort_flag, a.status, 2, s)) break;
        const int k0 = ((g0 + s) % ks) * kW4StageK;
        mbar_arrive_expect_tx(&bars->x_full[st], Cfg::kXStage);
        tma_load_2d(x_ring + st * Cfg::kXStage, &tmap_x, k0, 0, &bars->x_full[st]);
        tma_load_2d(x_ring + st * Cfg::kXStage + Cfg::kXBytes, &tmap_x, k0 + 64, 0, &bars->x_full[st]);
        issued = s + 1;
      }
      if (*abort_flag) {
        for (int it = max(0, issued - SX); it < issued; ++it) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&bars->x_full[it % SX], (it / SX) & 1) && globaltimer_ns() - t0 < kWaitLimitNs) {
          }
        }
      }
    }
  } else if (warp == 2 || warp == 3) {
    // ------------------------------------------------------------------ MMA issuer of pipeline p
    const int p = warp - 2;
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(kTileN, NT);
      const uint64_t desc0 = make_desc_sw128(smem_u32(x_ring));
      int c = 0, item = -1, prev_pair = -1;
      for (int s = 0; s < n_steps; ++s) {
        const int g = g0 + s, pair = g / ks, k = g - pair * ks;
        const bool first = pair != prev_pair;
        if (first) {
          ++item;
          prev_pair = pair;
        }
        const int st = s % SX;
        if (!mbar_wait_spin(&bars->x_full[st], (s / SX) & 1, abort_flag, a.status, 3, s)) break;
        if (p == 1 && g >= single_from) {                    // no second tile: only hand the stage back
          mbar_arrive(&bars->x_empty[st]);
          continue;
        }
        const int b = item & 1, sub = c & 1;
        if (first && item >= 2 &&
            !mbar_wait_spin(&bars->acc_empty[p][b], ((item >> 1) - 1) & 1, abort_flag, a.status, 4, item))
          break;
        if (!mbar_wait_spin(&bars->a_ready[p][sub], (c >> 1) & 1, abort_flag, a.status, 5, c)) break;
        tc_fence_after_sync();
        // the start-address field counts 16-byte units: a K step of 16 halfs is +2, the second 64-wide sub-tile is
        // +kXBytes/16
        const uint64_t bd = desc0 + uint64_t((st * Cfg::kXStage) >> 4);
        const uint32_t at = tmem + 256 + (2 * p + sub) * 64, dt = tmem + (2 * p + b) * 64;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          umma_ts(dt, at + j * 8, bd + uint64_t((j >> 2) * (Cfg::kXBytes >> 4) + (j & 3) * 2), idesc,
                  (!first) || (j != 0));
        tc_commit(&bars->slot_free[p][sub]);
        if (k == ks - 1 || s == n_steps - 1) tc_commit(&bars->acc_full[p][b]);
        ++c;
      }
    }
  } else if (warp < kDecEpiWarp0) {
    // ------------------------------------------------------------------ dequant: chunk -> fp16 -> TMEM slot
    // group = (pipeline p, slot sub): chunks sub, sub+2, ... of pipeline p.  A thread owns one weight row of the
    // chunk: 128 nibbles in, 64 half2 out, written as two 32-column TMEM stores.  Chunk c of a pipeline belongs to
    // step c of the CTA (pipeline 1 only runs out earlier when the last pair has a single tile).
    const int q = warp & 3;
    const int grp = (warp - 4) >> 2, p = grp >> 1, sub = grp & 1;
    const int row = q * 32 + lane;
    const int n_chunks = p == 0 ? n_steps : n_real1;
    const uint32_t dst = tmem + (uint32_t(q * 32) << 16) + 256 + (2 * p + sub) * 64;
    int last = -1;
    for (int c = sub; c < n_chunks; c += 2) {
      const int slot = c % SW;
      if (!mbar_wait(&bars->w_full[p][slot], (c / SW) & 1, abort_flag, a.status, 6, c)) break;
      const uint8_t* chunk = w_ring + (p * SW + slot) * kW4ChunkBytes;
      uint4 pk[4];
#pragma unroll
      for (int p4 = 0; p4 < 4; ++p4) pk[p4] = *reinterpret_cast<const uint4*>(chunk + (p4 * 128 + row) * 16);
      const __half2 sz = *reinterpret_cast<const __half2*>(chunk + 8192 + row * 4);
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->w_empty[p][slot]);     // the chunk is in registers: its slot may be refilled
      const __half2 s2 = __half2half2(__low2half(sz)), z2 = __half2half2(__high2half(sz));
      uint32_t o[32];
      // the first half is dequantised while the MMAs that still read this TMEM slot (chunk c-2) run
      dec_dequant_half(pk[0], pk[1], s2, z2, o);
      if (c >= 2) {
        if (!mbar_wait(&bars->slot_free[p][sub], ((c >> 1) - 1) & 1, abort_flag, a.status, 7, c)) break;
        // the MMAs of chunk c-2 are complete: its activation stage has one reader less
        if (q == 0 && lane == 0) mbar_arrive(&bars->x_empty[(c - 2) % SX]);
      }
      tc_fence_after_sync();
      ZSE_TMEM_ST_X32(dst, o);
      dec_dequant_half(pk[2], pk[3], s2, z2, o);
      ZSE_TMEM_ST_X32(dst + 32, o);
      tc_wait_st();
      tc_fence_before_sync();
      if (lane == 0) mbar_arrive(&bars->a_ready[p][sub]);
      last = c;
    }
    // hand back the stage of this group's last chunk as well (the activation producer may still need it when the
    // other pipeline goes on alone)
    if (last >= 0 && !*abort_flag) {
      if (mbar_wait(&bars->slot_free[p][sub], (last >> 1) & 1, abort_flag, a.status, 8, last)) {
        if (q == 0 && lane == 0) mbar_arrive(&bars->x_empty[last % SX]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (128 threads)
    const int q = warp & 3, row = q * 32 + lane, et = threadIdx.x - kDecEpiWarp0 * 32;
    const uint32_t lane_addr = uint32_t(q * 32) << 16;
    pdl_wait();                     // outputs, workspace and flags may still be in use by the previous kernel
    const uint32_t epoch1 = ld_acquire_gpu_u32(a.sync) + 1u;
    uint32_t* flags = a.sync + 8;
    const int S = a.split;
    const int seg = S > 0 ? cta % S : 0;
    int s = 0, item = 0;
    bool alive = true;
    while (s < n_steps && alive) {
      const int g = g0 + s, pair = g / ks, ka = g - pair * ks;
      const int len = min(ks - ka, n_steps - s);
      const int ntp = g < single_from ? 2 : 1;
      const int b = item & 1;
      // who adds what: `own_mod`/`own_res` select the column granules this CTA finishes (granule % own_mod == own_res;
      // own_mod 0 = none); src0..src0+n_src-1 are the CTAs whose partial sums it needs (itself excluded)
      int own_mod, own_res = 0, src0 = 0, n_src = 0;
      if (S > 0) {
        own_mod = S;
        own_res = seg;
        src0 = cta - seg;
        n_src = S;
      } else if (ka == 0) {
        own_mod = 1;
        src0 = cta + 1;
        if (len < ks)
          while (src0 + n_src < n_cta && dec_range_begin(a, src0 + n_src, n_cta) < (pair + 1) * ks) ++n_src;
      } else {
        own_mod = 0;
      }
      for (int r = 0; r < ntp && alive; ++r)
        alive = mbar_wait(&bars->acc_full[r][b], (item >> 1) & 1, abort_flag, a.status, 9, item);
      alive = epi_all(alive);
      if (!alive) break;
      tc_fence_after_sync();
      // ---- partial sums this CTA does not finish go to the workspace
      bool dumped = false;
      for (int r = 0; r < ntp; ++r) {
        float* dstw = a.ws + (size_t(cta) * 2 + r) * NT * 128 + row;
#pragma unroll 1
        for (int gr = 0; gr < Cfg::kGranules; ++gr) {
          if (own_mod != 0 && gr % own_mod == own_res) continue;
          uint32_t v[8];
          ZSE_TMEM_LD_X8(v, tmem + lane_addr + (2 * r + b) * 64 + gr * 8);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 8; ++i) dstw[(gr * 8 + i) * 128] = __uint_as_float(v[i]);
          dumped = true;
        }
      }
      if (dumped) {
        __threadfence();
        epi_bar();
        if (et == 0) st_release_gpu_u32(flags + cta, epoch1);
      }
      if (own_mod != 0) {
        // ---- wait for the other CTAs' partial sums of this pair
        for (int j = 0; j < n_src && alive; ++j) {
          const int c2 = src0 + j;
          if (c2 == cta) continue;
          if (lane == 0) alive = dec_wait_flag(flags + c2, epoch1, abort_flag, a.status, 10, c2);
          __syncwarp();
        }
        alive = epi_all(alive);
        for (int r = 0; r < ntp && alive; ++r) {
          const int tile = 2 * pair + r;
          // ---- phase 1: finished sums of the owned columns -> stage[col][row]
          float bias = 0.f;
          if ((EPI == kDecF16 || EPI == kDecQkvRope) && a.bias != nullptr && tile * kTileN + row < a.N)
            bias = __half2float(a.bias[tile * kTileN + row]);
#pragma unroll 1
          for (int gr = own_res; gr < Cfg::kGranules; gr += own_mod) {
            uint32_t raw[8];
            ZSE_TMEM_LD_X8(raw, tmem + lane_addr + (2 * r + b) * 64 + gr * 8);
            tc_wait_ld();
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(raw[i]) + bias;
            for (int j = 0; j < n_src; ++j) {                   // fixed order: the sum is reproducible
              const int c2 = src0 + j;
              if (c2 == cta) continue;
              const float* srcw = a.ws + (size_t(c2) * 2 + r) * NT * 128 + row;
              float t8[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) t8[i] = __ldcg(srcw + (gr * 8 + i) * 128);
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] += t8[i];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) stage[(gr * 8 + i) * 128 + row] = v[i];
          }
          epi_bar();
          // ---- phase 2: 16-byte stores; thread -> (column et >> 4 of the granule, 8 rows from (et & 15) * 8)
#pragma unroll 1
          for (int gr = own_res; gr < Cfg::kGranules; gr += own_mod) {
            const int col = gr * 8 + (et >> 4), t = col;
            if (t >= a.M) continue;
            if (EPI == kDecF16 || EPI == kDecF32) {
              const int r0 = (et & 15) * 8, n = tile * kTileN + r0;
              if (n >= a.N) continue;
              const float4 lo = *reinterpret_cast<const float4*>(stage + col * 128 + r0);
              const float4 hi = *reinterpret_cast<const float4*>(stage + col * 128 + r0 + 4);
              if (EPI == kDecF16) {
                uint4 pk;
                pk.x = pack_half2(clamp_f16(lo.x), clamp_f16(lo.y));
                pk.y = pack_half2(clamp_f16(lo.z), clamp_f16(lo.w));
                pk.z = pack_half2(clamp_f16(hi.x), clamp_f16(hi.y));
                pk.w = pack_half2(clamp_f16(hi.z), clamp_f16(hi.w));
                *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(a.out) + size_t(t) * a.ldo + n) = pk;
              } else {
                float* o = reinterpret_cast<float*>(a.out) + size_t(t) * a.ldo + n;
                *reinterpret_cast<float4*>(o) = lo;
                *reinterpret_cast<float4*>(o + 4) = hi;
              }
            } else if (EPI == kDecSwiGLU) {
              // tile rows 0..63 = gate, 64..127 = up of the same 64 outputs: four outputs per thread
              const int o0 = (et & 15) * 4, n = tile * 64 + o0;
              if (n >= a.N / 2) continue;
              const float4 gt = *reinterpret_cast<const float4*>(stage + col * 128 + o0);
              const float4 up = *reinterpret_cast<const float4*>(stage + col * 128 + 64 + o0);
              uint2 pk;
              pk.x = pack_half2(clamp_f16(silu_f(gt.x) * up.x), clamp_f16(silu_f(gt.y) * up.y));
              pk.y = pack_half2(clamp_f16(silu_f(gt.z) * up.z), clamp_f16(silu_f(gt.w) * up.w));
              *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(a.out) + size_t(t) * a.ldo + n) = pk;
            } else if (EPI == kDecQkvRope) {
              // tile = one head of 128 dims: q heads, then k heads, then v heads; eight dims per thread
              const DecRope& rp = a.rope;
              const int d0 = (et & 15) * 8;
              const float* sv = stage + col * 128;
              float val[8];
              if (tile < rp.nh + rp.nkv) {
                const int pos = min(max(rp.positions[t], 0), rp.max_position - 1);
                const float2* cs = rp.cos_sin + size_t(pos) * 64 + (d0 & 63);
                const float* xa = sv + (d0 & 63);           // first half of the head
                const float* xb = xa + 64;                  // second half
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const float2 c2 = cs[i];
                  val[i] = d0 < 64 ? xa[i] * c2.x - xb[i] * c2.y : xb[i] * c2.x + xa[i] * c2.y;
                }
              } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) val[i] = sv[d0 + i];
              }
              uint4 pk;
              pk.x = pack_half2(clamp_f16(val[0]), clamp_f16(val[1]));
              pk.y = pack_half2(clamp_f16(val[2]), clamp_f16(val[3]));
              pk.z = pack_half2(clamp_f16(val[4]), clamp_f16(val[5]));
              pk.w = pack_half2(clamp_f16(val[6]), clamp_f16(val[7]));
              if (tile < rp.nh) {                           // q: what attention reads
                *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(a.out) + size_t(t) * a.ldo + tile * 128 + d0) = pk;
              } else if (tile < rp.nh + 2 * rp.nkv) {
                const long long slot = rp.slots[t];
                if (slot >= 0) {
                  const bool is_v = tile >= rp.nh + rp.nkv;
                  const int kvh = tile - rp.nh - (is_v ? rp.nkv : 0);
                  const long long blk = slot / rp.block_size, off = slot % rp.block_size;
                  __half* dstp = rp.kv_layer + (((blk * 2 + (is_v ? 1 : 0)) * rp.nkv + kvh) * rp.block_size + off) * 128;
                  *reinterpret_cast<uint4*>(dstp + d0) = pk;
                }
              }
            }
          }
          epi_bar();                                   // the stage is reused by the next tile
        }
      }
      // the accumulators of this item are read: the pipelines may overwrite them (item + 2)
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0)
        for (int r = 0; r < ntp; ++r) mbar_arrive(&bars->acc_empty[r][b]);
      s += len;
      ++item;
    }
  }

  // ---------------------------------------------------------------------- exit
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem, 512);
  if (threadIdx.x == kDecEpiWarp0 * 32) {
    // the last CTA to leave moves the launch epoch on (every CTA read it after its pdl_wait, i.e. long ago)
    __threadfence();
    const uint32_t t = atomicAdd(a.sync + 1, 1u);
    if (t == uint32_t(n_cta) - 1u) {
      a.sync[1] = 0u;
      __threadfence();
      atomicAdd(a.sync, 1u);
    }
  }
}

// ---- host side --------------------------------------------------------------------------------------------------
struct DecPlan {
  int n_cta, split;
};

// tuning knobs (tests and the microbenchmark move them): smallest number of steps worth a CTA in the stream plan,
// largest number of segments per pair in the split plan
static int g_dec_min_steps = 4;
static int g_dec_max_split = 8;

static DecPlan plan_dec(int n_pairs, int k_stages, int sm_count) {
  DecPlan p{1, 0};
  const int total = n_pairs * k_stages;
  if (2 * n_pairs <= sm_count) {
    // split plan: S segments per pair, at least two steps per segment
    int S = min(min(g_dec_max_split, sm_count / n_pairs), max(1, k_stages / 2));
    S = max(1, S);
    p.split = S;
    p.n_cta = n_pairs * S;
  } else {
    p.split = 0;
    p.n_cta = max(1, min(sm_count, total / g_dec_min_steps));
  }
  return p;
}

template <int NT, int EPI>
static int launch_dec(const CUtensorMap& tx, const DecArgs& a, int n_cta, cudaStream_t st) {
  auto kern = gemm_w4_dec_kernel<NT, EPI>;
  constexpr int smem = DecCfg<NT>::kSmemBytes;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return ZSE_ERR_SHAPE;
  if (!attr_done[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return ZSE_ERR_LAUNCH;
    attr_done[dev] = true;
  }
  return launch_pdl(kern, dim3(n_cta), dim3(kDecThreads), size_t(smem), st, tx, a) == cudaSuccess ? 0
                                                                                                  : ZSE_ERR_LAUNCH;
}

template <int NT>
static int launch_dec_epi(int epi, const CUtensorMap& tx, const DecArgs& a, int n_cta, cudaStream_t st) {
  switch (epi) {
    case kDecF16: return launch_dec<NT, kDecF16>(tx, a, n_cta, st);
    case kDecSwiGLU: return launch_dec<NT, kDecSwiGLU>(tx, a, n_cta, st);
    case kDecF32: return launch_dec<NT, kDecF32>(tx, a, n_cta, st);
    case kDecQkvRope: return launch_dec<NT, kDecQkvRope>(tx, a, n_cta, st);
    default: return ZSE_ERR_SHAPE;
  }
}

static int dec_sm_count() {
  static int sm[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (sm[dev] == 0) {
    cudaDeviceGetAttribute(&sm[dev], cudaDevAttrMultiProcessorCount, dev);
    if (sm[dev] <= 0) sm[dev] = 148;
  }
  return sm[dev];
}

}  // namespace zse

using namespace zse;

// Bytes of workspace a caller has to provide (zeroed once): partial sums of up to `sm_count` CTAs plus the
// synchronisation words.  One workspace serves every call that is ordered on one stream.
extern "C" long long zse_gemm_w4_dec_workspace_bytes(int sm_count) {
  if (sm_count <= 0) sm_count = 148;
  return (long long)sm_count * 2 * 64 * 128 * 4 + (8 + sm_count) * 4 + 256;
}

extern "C" void zse_gemm_w4_dec_set_tuning(int min_steps, int max_split) {
  if (min_steps > 0) zse::g_dec_min_steps = min_steps;
  if (max_split > 0) zse::g_dec_max_split = min(max_split, 64);
}

// out2 = {CTAs, segments per pair (0 = stream plan)} for a call with these sizes
extern "C" void zse_gemm_w4_dec_plan(int N, int K, int epilogue, int sm_count, int* out2) {
  const int n_tiles = epilogue == kDecSwiGLU ? (N / 2 + 63) / 64 : (N + kTileN - 1) / kTileN;
  const DecPlan p = plan_dec((n_tiles + 1) / 2, K / kW4StageK, sm_count > 0 ? sm_count : 148);
  out2[0] = p.n_cta;
  out2[1] = p.split;
}

// 1 when zse_gemm_w4_dec takes a call with these sizes (otherwise the caller uses zse_gemm_w4)
extern "C" int zse_gemm_w4_dec_supported(int M, int N, int K, int epilogue) {
  if (M <= 0 || M > 64 || K <= 0 || K % kW4StageK != 0 || N <= 0) return 0;
  if (epilogue == kDecSwiGLU) return (N % 8) == 0 ? 1 : 0;
  if (epilogue == kDecQkvRope) return (N % 128) == 0 ? 1 : 0;
  return (epilogue == kDecF16 || epilogue == kDecF32) && (N % 8) == 0 ? 1 : 0;
}

static int run_dec(const void* w_tiled, const void* x, int x_rows_cap, const void* bias, void* out, int M, int N,
                   int K, int ldo, int epilogue, void* workspace, const DecRope* rope, void* status, void* stream) {
  if (M <= 0) return 0;
  if (!zse_gemm_w4_dec_supported(M, N, K, epilogue) || workspace == nullptr) return ZSE_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(workspace) & 15)) return ZSE_ERR_ALIGN;
  if (epilogue == kDecF32 ? (ldo % 4) : (ldo % 8)) return ZSE_ERR_ALIGN;
  const int sm_count = dec_sm_count();
  const int k_stages = K / kW4StageK;
  const int n_tiles = epilogue == kDecSwiGLU ? (N / 2 + 63) / 64 : (N + kTileN - 1) / kTileN;
  const int n_pairs = (n_tiles + 1) / 2;
  const DecPlan p = plan_dec(n_pairs, k_stages, sm_count);
  const int nt = pick_nt(M);
  CUtensorMap tx;
  if (int rc = get_tmap(x, uint64_t(max(x_rows_cap, M)), uint64_t(K), uint32_t(nt), &tx)) return rc;
  DecArgs a{};
  a.w = reinterpret_cast<const uint8_t*>(w_tiled);
  a.bias = reinterpret_cast<const __half*>(bias);
  a.out = out;
  a.M = M;
  a.N = N;
  a.ldo = ldo;
  a.k_stages = k_stages;
  a.n_tiles = n_tiles;
  a.n_pairs = n_pairs;
  a.total_steps = n_pairs * k_stages;
  a.split = p.split;
  a.ws = reinterpret_cast<float*>(workspace);
  a.sync = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(workspace) +
                                       (size_t)sm_count * 2 * 64 * 128 * 4);
  a.status = reinterpret_cast<Status*>(status);
  if (rope != nullptr) a.rope = *rope;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (nt) {
    case 16: return launch_dec_epi<16>(epilogue, tx, a, p.n_cta, st);
    case 32: return launch_dec_epi<32>(epilogue, tx, a, p.n_cta, st);
    default: return launch_dec_epi<64>(epilogue, tx, a, p.n_cta, st);
  }
}

// Decode-sized INT4 GEMM (M <= 64).  epilogue: 0 = fp16 store (+bias), 1 = SwiGLU, 2 = fp32 store (one plane).
extern "C" int zse_gemm_w4_dec(const void* w_tiled, const void* x, int x_rows_cap, const void* bias, void* out, int M,
                               int N, int K, int ldo, int epilogue, void* workspace, void* status, void* stream) {
  if (epilogue != kDecF16 && epilogue != kDecSwiGLU && epilogue != kDecF32) return ZSE_ERR_SHAPE;
  return run_dec(w_tiled, x, x_rows_cap, bias, out, M, N, K, ldo, epilogue, workspace, nullptr, status, stream);
}

// Fused QKV projection of a decode-sized pass, head_dim 128, full rotary: bias, rotate-half RoPE (cos/sin table
// [max_position][64] of float2) and the K/V rows stored straight into the paged cache
// (kv_layer [blocks][2][nkv][block_size][128], slot = block * block_size + offset, -1 = skip); `qkv_out` [M, ldo]
// receives the rotated q heads (columns 0 .. nh*128).
extern "C" int zse_gemm_w4_dec_qkv_rope(const void* w_tiled, const void* x, int x_rows_cap, const void* bias,
                                        void* qkv_out, int ldo, int M, int K, int nh, int nkv, void* kv_layer,
                                        int block_size, const void* positions_i32, const void* slots_i64,
                                        const void* cos_sin_f32x2, int max_position, void* workspace, void* status,
                                        void* stream) {
  if (nh <= 0 || nkv <= 0 || block_size <= 0 || max_position <= 0 || kv_layer == nullptr || positions_i32 == nullptr ||
      slots_i64 == nullptr || cos_sin_f32x2 == nullptr)
    return ZSE_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(kv_layer) & 15) || (reinterpret_cast<uintptr_t>(cos_sin_f32x2) & 7))
    return ZSE_ERR_ALIGN;
  DecRope rp{};
  rp.positions = reinterpret_cast<const int*>(positions_i32);
  rp.slots = reinterpret_cast<const long long*>(slots_i64);
  rp.cos_sin = reinterpret_cast<const float2*>(cos_sin_f32x2);
  rp.kv_layer = reinterpret_cast<__half*>(kv_layer);
  rp.nh = nh;
  rp.nkv = nkv;
  rp.block_size = block_size;
  rp.max_position = max_position;
  return run_dec(w_tiled, x, x_rows_cap, bias, qkv_out, M, (nh + 2 * nkv) * 128, K, ldo, kDecQkvRope, workspace, &rp,
                 status, stream);
}

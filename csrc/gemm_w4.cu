// INT4 group-128 weight linear layers on the 5th-generation tensor cores.
//
//   Y[t, n] = sum_k X[t, k] * (nibble[n, k] * scale[n, k/128] + zero[n, k/128])
//
// Computed transposed ("swap AB"): UMMA M (128) runs over weight rows, UMMA N (16..256) over tokens, so a decode step
// with a few tokens fills the TMEM lanes and the weight stream is read exactly once.
//
// Data flow of one CTA (608 threads):
//   warp 0      streams 8704-byte weight chunks (8192 B nibbles + 128 x {scale, zero}) with 1-D bulk TMA copies
//               into a deep ring (up to 12 chunks in flight: this ring is what hides HBM latency);
//   warp 18     streams the activation tile (tiled TMA, 128-byte swizzle) into a short ring (it comes from L2);
//   warps 2-17  turn chunks into fp16 in registers (lop3 nibble extraction, exact q*s+z in half2) and write them
//               with tcgen05.st straight into TMEM: four groups of four warps work on four chunks at a time, a thread
//               owning one weight row of its chunk;
//   warp 1      issues tcgen05.mma with A from TMEM and B (activations) from shared memory; accumulators in TMEM.
// The dequantised weights never touch shared memory.  A CTA owns R = 1 or 2 adjacent 128-row weight tiles and reuses
// every activation stage for all of them (the activation tile is re-read from L2 by every CTA, so R halves that
// traffic).  Split-K runs as a thread-block cluster along K: the non-leading CTAs park their accumulators in their
// shared memory, the leading CTA adds them through distributed shared memory and runs the epilogue, so split-K costs
// no global-memory traffic and works with every epilogue.
//
// Epilogues: fp16 store (+bias), SwiGLU (tile rows 0..63 = gate, 64..127 = up of the same 64 outputs), fp32 store
// (row-parallel projections; consumed by add_rmsnorm / tp_reduce_add_rmsnorm together with the residual).
//
// Replaces the scalar dequant GEMV / 32x32 tiled matmul kernels of the reference
// (zse-engine/zse_engine/orchestrator/kernels.py:1129-1192,1906-2073,2114-2203).
#include "gemm_common.cuh"

namespace zse {

constexpr int kMaxPlanes = 8;

// Two shapes of CTA.  The wide one (608 threads, all 512 TMEM columns, most of the shared memory) lives alone on its
// SM.  The narrow one (DUAL: 384 threads, 256 TMEM columns, < 113 KB) is for N <= 64 tokens.  Measured on B200: one
// thread cannot issue tcgen05.mma faster than one per ~50 cycles whatever N is, while the tensor pipe itself needs
// only 32 cycles at N = 64 and 8 at N = 16; several issuing threads (in one CTA or in two CTAs of an SM) add up
// until the pipe is full.  So the narrow CTA runs TWO independent pipelines - dequant group p + MMA warp p work on
// the chunks of parity p with their own accumulator and their own TMEM slot - and two such CTAs share an SM.
template <int NT, int R, bool DUAL>
struct W4Cfg {
  static_assert(R == 1 || R == 2, "a CTA owns one or two weight tiles");
  static_assert(!(R == 2 && NT > 128), "two accumulators of 256 columns do not fit next to the A ring");
  static_assert(!DUAL || (R == 1 && NT <= 64), "the narrow CTA holds one accumulator of at most 64 columns");
  static constexpr int kGroups = DUAL ? 2 : 4;                     // dequant groups of four warps
  static constexpr int kDqWarps = 4 * kGroups;
  static constexpr int kXWarp = 2 + kDqWarps;
  static constexpr int kThreads = 32 * (kXWarp + 1) + (DUAL ? 32 : 0);      // DUAL: second MMA warp at the end
  static constexpr int kMinBlocks = DUAL ? 2 : 1;
  static constexpr int kTmemCols = DUAL ? 256 : 512;
  static constexpr int kXBytes = NT * 128;                         // one 64-wide K sub-tile of X
  static constexpr int kXStage = 2 * kXBytes;
  // A slot of the TMEM ring holds kCPS consecutive chunks and is released by ONE tcgen05.commit (a commit costs
  // about as much tensor pipe time as two MMAs).  Where possible the activation ring is laid out so that the same
  // commit also frees the activation stages the slot used: kCPS / R stages per slot.
  static constexpr int kCPS = DUAL ? 1 : 2;                        // chunks per slot
  static constexpr bool kTiedX = !DUAL && NT <= 128;
  static constexpr int kSP = DUAL ? 2 : (NT <= 64 ? 3 : 2);        // slots in TMEM (DUAL: one per pipeline)
  static constexpr int kSX = DUAL ? 4 : (kTiedX ? kSP * kCPS / R : 2);      // activation stages
  static constexpr int kSW = DUAL ? (NT == 64 ? 5 : 6) : (NT <= 64 ? 12 : (NT == 128 ? (R == 2 ? 10 : 8) : 8));
  static constexpr int kAcc = (DUAL ? 2 : R) * NT;                 // accumulator columns (DUAL: one per pipeline)
  static_assert(kAcc + kSP * kCPS * 64 <= kTmemCols, "TMEM budget");
  static constexpr int kRingBytes = kSX * kXStage + kSW * kW4ChunkBytes;
  static constexpr int kParkBytes = R * NT * 128 * 4;              // accumulators parked for the cluster reduce
  static constexpr int kDataBytes = ((kRingBytes > kParkBytes ? kRingBytes : kParkBytes) + 15) & ~15;
  // SwiGLU gate/up exchange: after the barriers, or (DUAL) inside the idle rings behind the parked accumulators
  static constexpr int kXchBytes = 2 * kGroups * 32 * 16 * 4;
  static_assert(!DUAL || kParkBytes + kXchBytes <= kRingBytes, "exchange buffer must fit behind the park area");
  static constexpr int kSmemBytes = kDataBytes + 512 + (DUAL ? 0 : kXchBytes) + 1024;
  static_assert(kSmemBytes <= (DUAL ? 115712 : 232448), "shared memory budget");
};

struct W4Bars {
  uint64_t w_full[12], w_empty[12];
  uint64_t x_full[6], x_empty[6];
  uint64_t a_ready[6];            // [pair slot][half]
  uint64_t pair_done[3];
  uint64_t acc_ready;
  uint32_t tmem_base;
  int abort_flag;
};

struct W4Args {
  const uint8_t* w;        // tiled chunks [n_tiles][k_stages][8704]
  const __half* bias;      // [N] or null (kEpiF16)
  void* out;
  int M, N, K, ldo;
  int k_stages;            // K / 128
  int stages_per_split;    // K stages handled by one CTA of the cluster
  int cluster_k;           // CTAs per cluster along K (1: every K split writes its own fp32 plane)
  Status* status;
  long long* timing;       // debug builds (ZSE_W4_TIMING): per-role cycle counters, else unused
  PushTable push;          // kEpiPushF16: where the partial tiles go (every rank's inbox over NVLink)
  SpTable sp;              // kEpiScatterF16: where the partial tiles go (the owner of each 64-row block)
  GatherWait gather;       // the activations are a gathered buffer: wait for the row blocks of this CTA's token tile
};

__device__ __forceinline__ void multimem_st_v4(void* mc_ptr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f16x2 [%0], {%1,%2,%3,%4};" ::"l"(mc_ptr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void multimem_red_add_release(uint32_t* mc_ptr, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc_ptr), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void red_add_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t w4_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// All-gather in the prologue: the rows of token tile [t0, t0 + nt) were written into this GPU's memory by their
// owners (other GPUs, plain or multicast stores); a row block is complete when its flag holds the pass epoch.  One
// thread waits (bounded), then orders those writes before the TMA loads it is about to issue (async proxy).
__device__ __forceinline__ bool gather_wait_tile(const GatherWait& g, int t0, int nt, int M, volatile int* abort_flag,
                                                 Status* st) {
  const uint32_t want = *reinterpret_cast<const volatile uint32_t*>(g.epoch);
  bool ok = true;
  for (int t = t0; t < t0 + nt && t < M && ok; t += kSpRowBlock) {
    const uint32_t* f = g.flags + t / kSpRowBlock;
    if (w4_ld_acquire_sys(f) == want) continue;
    SpinClock clk;
    while (w4_ld_acquire_sys(f) != want) {
      if (clk.expired(0x3F) || ((clk.spins & 0x3F) == 0 && *abort_flag)) {
        report(st, kPeerTimeout, 36, unsigned(t / kSpRowBlock));
        *abort_flag = 1;
        ok = false;
        break;
      }
    }
  }
  asm volatile("fence.proxy.async;" ::: "memory");
  return ok;
}

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

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ float ld_dsmem_f32(uint32_t local_smem_addr, uint32_t cta_rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(cta_rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// Drain helper for an aborted producer: every issued copy must land before the CTA may exit.
__device__ __forceinline__ void drain(uint64_t* full, int ring, int issued) {
  for (int it = max(0, issued - ring); it < issued; ++it) {
    const uint64_t t0 = globaltimer_ns();
    while (!mbar_try_wait(&full[it % ring], (it / ring) & 1) && globaltimer_ns() - t0 < kWaitLimitNs) {
    }
  }
}

#ifdef ZSE_W4_SPIN
#define ZSE_W4_ISSUER_WAIT mbar_wait_spin
#else
#define ZSE_W4_ISSUER_WAIT mbar_wait
#endif

#ifdef ZSE_W4_TIMING
#define TICK(var) long long var = clock64()
#define ACC(slot, t0) tacc[slot] += clock64() - (t0)
#else
#define TICK(var)
#define ACC(slot, t0)
#endif

template <int NT, int R, int EPI, bool DUAL>
__global__ void __launch_bounds__((W4Cfg<NT, R, DUAL>::kThreads), (W4Cfg<NT, R, DUAL>::kMinBlocks))
gemm_w4_kernel(const __grid_constant__ CUtensorMap tmap_x, const W4Args a) {
  using Cfg = W4Cfg<NT, R, DUAL>;
  constexpr int SW = Cfg::kSW, SX = Cfg::kSX, SP = Cfg::kSP, CPS = Cfg::kCPS, G = Cfg::kGroups;
  constexpr int kDqWarps = Cfg::kDqWarps, kXWarp = Cfg::kXWarp;
  constexpr bool kTied = Cfg::kTiedX;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* x_ring = smem;                                    // [SX][2][NT*128]
  uint8_t* w_ring = smem + SX * Cfg::kXStage;                // [SW][8704]
  W4Bars* bars = reinterpret_cast<W4Bars*>(smem + Cfg::kDataBytes);
  float* xch_base = reinterpret_cast<float*>(DUAL ? smem + Cfg::kParkBytes : smem + Cfg::kDataBytes + 512);
  float* park = reinterpret_cast<float*>(smem);              // reused after the main loop: [R*NT cols][128 rows]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef ZSE_W4_TIMING
  const long long t_entry = clock64();
#endif
  // The next kernel of the stream may start its own set-up now.  This kernel in turn starts before the one ahead
  // of it has finished: barrier set-up, the TMEM allocation and the weight stream (constant data) run at once,
  // while the activation producer and the epilogue wait for the producer of the activations (pdl_wait below).
  pdl_launch_dependents();
  const int s_begin = blockIdx.z * a.stages_per_split;
  const int n_k = max(0, min(a.k_stages, s_begin + a.stages_per_split) - s_begin);
  const int n_units = n_k * R;
  const int tile0 = blockIdx.x * R;                          // first weight tile of this CTA

  if (threadIdx.x == 0) {
    for (int i = 0; i < SW; ++i) {
      mbar_init(&bars->w_full[i], 1);
      mbar_init(&bars->w_empty[i], 4);
    }
    for (int i = 0; i < SX; ++i) {
      mbar_init(&bars->x_full[i], 1);
      mbar_init(&bars->x_empty[i], 1);
    }
    for (int i = 0; i < SP; ++i) {
      for (int h = 0; h < CPS; ++h) mbar_init(&bars->a_ready[CPS * i + h], 4);
      mbar_init(&bars->pair_done[i], 1);
    }
    mbar_init(&bars->acc_ready, DUAL ? 2 : 1);
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
  const uint32_t a_base = tmem + Cfg::kAcc;
  volatile int* abort_flag = &bars->abort_flag;
  bool acc_ok = false;
#ifdef ZSE_W4_TIMING
  long long tacc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const long long t_start = clock64();
  const long long t_setup = t_start - t_entry;
#endif

  if constexpr (DUAL) {
    // ================================================================== narrow CTA: two pipelines
    // chunk u (= K stage u, R is 1) belongs to pipeline p = u & 1: dequant group p fills TMEM slot p, MMA warp p
    // accumulates into accumulator p.  Weight ring and activation ring are shared and filled in chunk order.
    constexpr int kIssuer1 = kXWarp + 1;
    if (warp == 0) {
      if (lane == 0) {
        int issued = 0, s = 0;
        uint32_t ph = 1;
        for (int u = 0; u < n_units; ++u) {
          TICK(tw);
          if (u >= SW && !mbar_wait(&bars->w_empty[s], ph, abort_flag, a.status, 1, u)) break;
          ACC(0, tw);
          const uint8_t* src = a.w + (size_t(tile0) * a.k_stages + (s_begin + u)) * kW4ChunkBytes;
          mbar_arrive_expect_tx(&bars->w_full[s], kW4ChunkBytes);
          bulk_g2s(w_ring + s * kW4ChunkBytes, src, kW4ChunkBytes, &bars->w_full[s]);
          issued = u + 1;
          if (++s == SW) { s = 0; ph ^= 1; }
        }
        if (*abort_flag) drain(bars->w_full, SW, issued);
      }
    } else if (warp == kXWarp) {
      if (lane == 0) {
        int issued = 0, s = 0;
        uint32_t ph = 1;
        pdl_wait();                                      // the activations come from the previous kernel
        for (int kk = 0; kk < n_k; ++kk) {
          if (kk >= SX && !mbar_wait(&bars->x_empty[s], ph, abort_flag, a.status, 2, kk)) break;
          mbar_arrive_expect_tx(&bars->x_full[s], Cfg::kXStage);
          const int k0 = (s_begin + kk) * kW4StageK;
          tma_load_2d(x_ring + s * Cfg::kXStage, &tmap_x, k0, blockIdx.y * NT, &bars->x_full[s]);
          tma_load_2d(x_ring + s * Cfg::kXStage + Cfg::kXBytes, &tmap_x, k0 + 64, blockIdx.y * NT, &bars->x_full[s]);
          issued = kk + 1;
          if (++s == SX) { s = 0; ph ^= 1; }
        }
        if (*abort_flag) drain(bars->x_full, SX, issued);
      }
    } else if (warp == 1 || warp == kIssuer1) {
      const int p = warp == 1 ? 0 : 1;
      if (lane == 0) {
        constexpr uint32_t idesc = make_idesc_f16(kTileN, NT);
        const uint64_t desc0 = make_desc_sw128(smem_u32(x_ring));
        const uint32_t at = a_base + p * 64, dt = tmem + p * NT;
        uint32_t aph = 0;
        for (int u = p; u < n_units; u += 2) {
          const int sx = u % SX;
          TICK(tx);
          if (!ZSE_W4_ISSUER_WAIT(&bars->x_full[sx], (u / SX) & 1, abort_flag, a.status, 3, u)) break;
          ACC(0, tx);
          TICK(ta);
          if (!ZSE_W4_ISSUER_WAIT(&bars->a_ready[p], aph, abort_flag, a.status, 4, u)) break;
          ACC(1, ta);
          TICK(ti);
          tc_fence_after_sync();
          // slot p was refilled for this chunk only after the MMAs of chunk u-2 had completed, so the activation
          // stage that chunk used is free as well
#ifndef ZSE_W4_EARLY_X
          if (u >= 2) mbar_arrive(&bars->x_empty[(u - 2) % SX]);
#endif
          const uint64_t bd = desc0 + uint64_t((sx * Cfg::kXStage) >> 4);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            umma_ts(dt, at + j * 8, bd + uint64_t((j >> 2) * (Cfg::kXBytes >> 4) + (j & 3) * 2), idesc,
                    (u >= 2) || (j != 0));
          tc_commit(&bars->pair_done[p]);
          aph ^= 1;
          ACC(2, ti);
        }
        tc_commit(&bars->acc_ready);
      }
    } else {
      const int q = warp & 3;                  // TMEM lane quarter this warp may touch
      const int p = (warp - 2) >> 2;           // pipeline = dequant group
      const int row = q * 32 + lane;
      const uint32_t dst = a_base + (uint32_t(q * 32) << 16) + p * 64;
      int sw = p % SW;
      uint32_t wph = 0, dph = 0;
      for (int u = p; u < n_units; u += 2) {
        TICK(t0);
        if (!mbar_wait(&bars->w_full[sw], wph, abort_flag, a.status, 5, u)) break;
        ACC(0, t0);
#ifdef ZSE_W4_TIMING
        if (u == p) tacc[6] = clock64() - t_start;
#endif
        TICK(t1);
        const uint8_t* chunk = w_ring + sw * kW4ChunkBytes;
        uint4 pk[4];
#pragma unroll
        for (int p4 = 0; p4 < 4; ++p4) pk[p4] = *reinterpret_cast<const uint4*>(chunk + (p4 * 128 + row) * 16);
        const __half2 sz = *reinterpret_cast<const __half2*>(chunk + 8192 + row * 4);
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->w_empty[sw]);        // the chunk is in registers: its slot may be refilled
        ACC(1, t1);
        const __half2 s2 = __half2half2(__low2half(sz)), z2 = __half2half2(__high2half(sz));
        uint32_t o[32];
#ifdef ZSE_W4_HOIST
        // the first half of the chunk is dequantised while the MMAs of this pipeline's previous chunk still run
#pragma unroll
        for (int p2 = 0; p2 < 2; ++p2) {
          const uint4 w4 = pk[p2];
          dequant_word(w4.x, s2, z2, o + p2 * 16 + 0);
          dequant_word(w4.y, s2, z2, o + p2 * 16 + 4);
          dequant_word(w4.z, s2, z2, o + p2 * 16 + 8);
          dequant_word(w4.w, s2, z2, o + p2 * 16 + 12);
        }
#endif
        TICK(t2);
        if (u >= 2) {
          if (!mbar_wait(&bars->pair_done[p], dph, abort_flag, a.status, 6, u)) break;
          dph ^= 1;
#ifdef ZSE_W4_EARLY_X
          // the MMAs of chunk u-2 are complete: its activation stage may be refilled
          if (q == 0 && lane == 0) mbar_arrive(&bars->x_empty[(u - 2) % SX]);
#endif
        }
        ACC(2, t2);
        TICK(t3);
        tc_fence_after_sync();
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
#ifdef ZSE_W4_HOIST
          if (hh == 1)
#endif
          {
#pragma unroll
            for (int p2 = 0; p2 < 2; ++p2) {
              const uint4 w4 = pk[hh * 2 + p2];
              dequant_word(w4.x, s2, z2, o + p2 * 16 + 0);
              dequant_word(w4.y, s2, z2, o + p2 * 16 + 4);
              dequant_word(w4.z, s2, z2, o + p2 * 16 + 8);
              dequant_word(w4.w, s2, z2, o + p2 * 16 + 12);
            }
          }
          ZSE_TMEM_ST_X32(dst + hh * 32, o);
        }
        ACC(3, t3);
        TICK(t4);
        tc_wait_st();
        tc_fence_before_sync();
        if (lane == 0) mbar_arrive(&bars->a_ready[p]);
        ACC(4, t4);
        sw += 2;
        if (sw >= SW) { sw -= SW; wph ^= 1; }
      }
      TICK(t5);
      acc_ok = mbar_wait(&bars->acc_ready, 0, abort_flag, a.status, 7, 0);
      tc_fence_after_sync();
      ACC(5, t5);
#ifdef ZSE_W4_TIMING
      tacc[7] = clock64() - t_start;
#endif
    }
  } else
  if (warp == 0) {
    // ------------------------------------------------------------------ weight producer
    if (lane == 0) {
      int issued = 0, s = 0, kk = 0, r = 0;
      uint32_t ph = 1;                                   // parity of the *previous* completion of w_empty[s]
      for (int u = 0; u < n_units; ++u) {
        TICK(tw);
        if (u >= SW && !mbar_wait(&bars->w_empty[s], ph, abort_flag, a.status, 1, u)) break;
        ACC(0, tw);
        const uint8_t* src = a.w + (size_t(tile0 + r) * a.k_stages + (s_begin + kk)) * kW4ChunkBytes;
        mbar_arrive_expect_tx(&bars->w_full[s], kW4ChunkBytes);
        bulk_g2s(w_ring + s * kW4ChunkBytes, src, kW4ChunkBytes, &bars->w_full[s]);
        issued = u + 1;
        if (++r == R) { r = 0; ++kk; }
        if (++s == SW) { s = 0; ph ^= 1; }
      }
      if (*abort_flag) drain(bars->w_full, SW, issued);
    }
  } else if (warp == kXWarp) {
    // ------------------------------------------------------------------ activation producer
    if (lane == 0) {
      int issued = 0, s = 0;
      uint32_t ph = 1;
      pdl_wait();                                        // the activations come from the previous kernel
      bool gathered = true;
      if (a.gather.flags != nullptr)
        gathered = gather_wait_tile(a.gather, blockIdx.y * NT, NT, a.M, abort_flag, a.status);
      for (int kk = 0; kk < n_k && gathered; ++kk) {
        if (kk >= SX) {
          // tied: the commit that ends the pair holding this stage's last chunk frees the stage as well
          uint64_t* freed = kTied ? &bars->pair_done[s / (CPS / R)] : &bars->x_empty[s];
          if (!mbar_wait(freed, ph, abort_flag, a.status, 2, kk)) break;
        }
        mbar_arrive_expect_tx(&bars->x_full[s], Cfg::kXStage);
        const int k0 = (s_begin + kk) * kW4StageK;
        tma_load_2d(x_ring + s * Cfg::kXStage, &tmap_x, k0, blockIdx.y * NT, &bars->x_full[s]);
        tma_load_2d(x_ring + s * Cfg::kXStage + Cfg::kXBytes, &tmap_x, k0 + 64, blockIdx.y * NT, &bars->x_full[s]);
        issued = kk + 1;
        if (++s == SX) { s = 0; ph ^= 1; }
      }
      if (*abort_flag) drain(bars->x_full, SX, issued);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(kTileN, NT);
      const uint64_t desc0 = make_desc_sw128(smem_u32(x_ring));
      int sx = 0, slot = 0, r = 0, kk = 0;
      uint32_t xph = 0, cyc = 0;
      for (int u = 0; u < n_units; ++u) {
        const int half = u % CPS;
        TICK(tx);
        if (r == 0 && !mbar_wait(&bars->x_full[sx], xph, abort_flag, a.status, 3, kk)) break;
        ACC(0, tx);
        TICK(ta);
        if (!mbar_wait(&bars->a_ready[CPS * slot + half], cyc, abort_flag, a.status, 4, u)) break;
        ACC(1, ta);
        TICK(ti);
        tc_fence_after_sync();
        // the start-address field counts 16-byte units: a K step of 16 halfs is +2, the second 64-wide sub-tile
        // is +kXBytes/16
        const uint64_t bd = desc0 + uint64_t((sx * Cfg::kXStage) >> 4);
        const uint32_t at = a_base + (slot * CPS + half) * 64, dt = tmem + r * NT;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          umma_ts(dt, at + j * 8, bd + uint64_t((j >> 2) * (Cfg::kXBytes >> 4) + (j & 3) * 2), idesc,
                  (kk | j) != 0);
        if (++r == R) {
          if (!kTied) tc_commit(&bars->x_empty[sx]);
          r = 0;
          ++kk;
          if (++sx == SX) { sx = 0; xph ^= 1; }
        }
        if (half == CPS - 1 || u == n_units - 1) {
          tc_commit(&bars->pair_done[slot]);
          if (++slot == SP) { slot = 0; cyc ^= 1; }
        }
        ACC(2, ti);
      }
      tc_commit(&bars->acc_ready);
    }
  } else {
    // ------------------------------------------------------------------ dequant: chunk -> fp16 -> TMEM
    // G groups of four warps; group g takes the units g, g+G, g+2G, ...  A thread owns one weight row of the
    // chunk: 128 nibbles in, 64 half2 out, written as two 32-column TMEM stores.
    const int q = warp & 3;                  // TMEM lane quarter this warp may touch
    const int grp = (warp - 2) >> 2;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = uint32_t(q * 32) << 16;
    int sw = grp % SW;
    uint32_t wph = 0;
    for (int u = grp; u < n_units; u += G) {
      // unit u -> slot (u / CPS) % SP, position u % CPS inside it; cyc = how often the slot has been used before
      const int su = u / CPS, half = u % CPS;
      const int slot = su % SP, cyc = su / SP;
      TICK(t0);
      if (!mbar_wait(&bars->w_full[sw], wph, abort_flag, a.status, 5, u)) break;
      ACC(0, t0);
      TICK(t1);
      const uint8_t* chunk = w_ring + sw * kW4ChunkBytes;
      uint4 pk[4];
#pragma unroll
      for (int p4 = 0; p4 < 4; ++p4) pk[p4] = *reinterpret_cast<const uint4*>(chunk + (p4 * 128 + row) * 16);
      const __half2 sz = *reinterpret_cast<const __half2*>(chunk + 8192 + row * 4);
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->w_empty[sw]);          // the chunk is in registers: its slot may be refilled
      ACC(1, t1);
      TICK(t2);
      if (cyc > 0 && !mbar_wait(&bars->pair_done[slot], (cyc - 1) & 1, abort_flag, a.status, 6, u)) break;
      ACC(2, t2);
      TICK(t3);
      tc_fence_after_sync();
      const __half2 s2 = __half2half2(__low2half(sz)), z2 = __half2half2(__high2half(sz));
      const uint32_t dst = a_base + lane_addr + (slot * CPS + half) * 64;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t o[32];
#pragma unroll
        for (int p2 = 0; p2 < 2; ++p2) {
          const uint4 w4 = pk[hh * 2 + p2];
          dequant_word(w4.x, s2, z2, o + p2 * 16 + 0);
          dequant_word(w4.y, s2, z2, o + p2 * 16 + 4);
          dequant_word(w4.z, s2, z2, o + p2 * 16 + 8);
          dequant_word(w4.w, s2, z2, o + p2 * 16 + 12);
        }
        ZSE_TMEM_ST_X32(dst + hh * 32, o);
      }
      ACC(3, t3);
      TICK(t4);
      tc_wait_st();
      tc_fence_before_sync();
      if (lane == 0) mbar_arrive(&bars->a_ready[CPS * slot + half]);
      ACC(4, t4);
      sw += G;
      if (sw >= SW) { sw -= SW; wph ^= 1; }
    }
    TICK(t5);
    acc_ok = mbar_wait(&bars->acc_ready, 0, abort_flag, a.status, 7, 0);
    tc_fence_after_sync();
    ACC(5, t5);
  }
#ifdef ZSE_W4_TIMING
  if (a.timing != nullptr && lane == 0 && blockIdx.x == 1 && blockIdx.z == 0) {
    // role rows: 0 = weight producer, 1 = MMA issuer, 2 = activation producer, 3.. = dequant warps (first group)
    const int role = warp == 0 ? 0 : warp == 1 ? 1 : warp == kXWarp ? 2 : 3 + (warp - 2);
    for (int i = 0; i < 8; ++i) a.timing[role * 8 + i] = tacc[i];
    if (warp == 1) a.timing[19 * 8] = clock64() - t_start;
  }
  const long long t_epi = clock64();
#endif

  // ---------------------------------------------------------------------- cluster reduce + epilogue
  // one verdict for the whole CTA, so that paired warps never disagree about taking part in the exchange barriers
  const bool dq_role = warp >= 2 && warp < 2 + kDqWarps;
  acc_ok = __syncthreads_and(dq_role ? int(acc_ok) : 1) != 0;
  pdl_wait();                                            // output buffers may still be read by the previous kernel
  const int ks = a.cluster_k;
  const bool in_cluster = ks > 1;
  const uint32_t crank = in_cluster ? cluster_ctarank() : 0u;
  const int q = warp & 3;                                       // TMEM lane quarter / row quarter
  const int cgw = (warp - 2) >> 2;                              // 0..G-1: which chunks of the CTA this warp takes
  const int row = q * 32 + lane;
  constexpr int kChunks = R * (NT / 16);                        // 16-column chunks of the CTA's accumulators

  if (in_cluster) {
    // every CTA parks its accumulators: park[(chunk*16 + i) * 128 + row]; chunk = r * (NT/16) + column group
    if (dq_role && acc_ok) {
#pragma unroll 1
      for (int ch = cgw; ch < kChunks; ch += G) {
        uint32_t v[16];
        ZSE_TMEM_LD_X16(v, tmem + (uint32_t(q * 32) << 16) + ch * 16);
        tc_wait_ld();
        if (DUAL && n_units > 1) {                               // second pipeline's accumulator
          uint32_t v1[16];
          ZSE_TMEM_LD_X16(v1, tmem + (uint32_t(q * 32) << 16) + NT + ch * 16);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + __uint_as_float(v1[i]));
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) park[(ch * 16 + i) * 128 + row] = __uint_as_float(v[i]);
      }
    }
    cluster_sync_all();
  }
  if (dq_role && acc_ok) {
    const int t0 = blockIdx.y * NT;
    const int plane_z = in_cluster ? 0 : int(blockIdx.z);
    // chunk ch belongs to the CTA with rank ch % ks; inside the CTA the four warp groups take its chunks in turn
    int mine = 0;
#pragma unroll 1
    for (int ch = int(crank); ch < kChunks; ch += ks, ++mine) {
      if ((mine % G) != cgw) continue;
      const int r = ch / (NT / 16), c0 = (ch % (NT / 16)) * 16;
      float v[16];
      if (in_cluster) {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
        const uint32_t base = smem_u32(park + (ch * 16) * 128 + row);
        for (int peer = 0; peer < ks; ++peer) {                 // fixed order: the sum is reproducible
          float tmp[16];
          uint32_t remote;
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(base), "r"(peer));
#pragma unroll
          for (int i = 0; i < 16; ++i)
            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(tmp[i]) : "r"(remote + i * 512));
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] += tmp[i];
        }
      } else {
        uint32_t raw[16];
        ZSE_TMEM_LD_X16(raw, tmem + (uint32_t(q * 32) << 16) + ch * 16);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(raw[i]);
        if (DUAL && n_units > 1) {                               // second pipeline's accumulator
          ZSE_TMEM_LD_X16(raw, tmem + (uint32_t(q * 32) << 16) + NT + ch * 16);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] += __uint_as_float(raw[i]);
        }
      }
      const int n_tile = tile0 + r;
      if (EPI == kEpiSwiGLU) {
        // rows 64..127 (q = 2, 3) hold `up`: hand them to the warp that holds the matching `gate` rows
        float* xch = xch_base + ((q & 1) + 2 * cgw) * (32 * 16);
        const int bar_id = 1 + (q & 1) + 2 * cgw;
        const int n = n_tile * 64 + (q & 1) * 32 + lane;
        if (q >= 2) {
#pragma unroll
          for (int i = 0; i < 16; ++i) xch[i * 32 + lane] = v[i];
          asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");
          asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");
        } else {
          asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");
          __half* out = reinterpret_cast<__half*>(a.out);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int t = t0 + c0 + i;
            if (t < a.M && n < a.N / 2)
              out[size_t(t) * a.ldo + n] = __float2half_rn(clamp_f16(silu_f(v[i]) * xch[i * 32 + lane]));
          }
          asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");
        }
      } else if (EPI == kEpiPushF16 || EPI == kEpiScatterF16) {
        // keep the finished sums in this CTA's park area, token-major, for the coalesced push below (the entries of
        // the chunks a CTA owns are read by nobody else)
#pragma unroll
        for (int i = 0; i < 16; ++i) park[(ch * 16 + i) * 128 + row] = v[i];
      } else {
        const int n = n_tile * kTileN + row;
        float bias = 0.f;
        if (EPI == kEpiF16 && a.bias != nullptr && n < a.N) bias = __half2float(a.bias[n]);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int t = t0 + c0 + i;
          if (t < a.M && n < a.N) {
            if (EPI == kEpiF16)
              reinterpret_cast<__half*>(a.out)[size_t(t) * a.ldo + n] = __float2half_rn(clamp_f16(v[i] + bias));
            else
              reinterpret_cast<float*>(a.out)[(size_t(plane_z) * a.M + t) * a.ldo + n] = v[i];
          }
        }
      }
    }
  }
  if (EPI == kEpiPushF16 && dq_role && acc_ok) {
    // ---- tensor-parallel exchange inside the GEMM: this rank's fp16 partial rows go to slot `rank` of every rank's
    // inbox (one multimem.st through the switch, or one store per peer), 16 bytes per thread, 256 contiguous bytes
    // per token and tile; then the CTA counts itself in on every rank.  Nothing here waits for a peer.
    constexpr int kDqThreads = kDqWarps * 32;
    asm volatile("bar.sync 15, %0;" ::"n"(kDqThreads) : "memory");
    const PushTable& pt = a.push;
    const int d = (warp - 2) * 32 + lane;
    const int t0 = blockIdx.y * NT;
    const int owned = int(crank) < kChunks ? (kChunks - int(crank) + ks - 1) / ks : 0;
    for (int item = d; item < owned * 256; item += kDqThreads) {
      const int ch = int(crank) + (item >> 8) * ks;
      const int tok = (item & 255) >> 4, seg = item & 15;
      const int r = ch / (NT / 16), c0 = (ch % (NT / 16)) * 16;
      const int t = t0 + c0 + tok;
      const int n = (tile0 + r) * kTileN + seg * 8;
      if (t < a.M && n < a.N) {
        const float4* src = reinterpret_cast<const float4*>(park + (ch * 16 + tok) * 128 + seg * 8);
        const float4 lo = src[0], hi = src[1];
        uint4 pk;
        pk.x = pack_half2(lo.x, lo.y);
        pk.y = pack_half2(lo.z, lo.w);
        pk.z = pack_half2(hi.x, hi.y);
        pk.w = pack_half2(hi.z, hi.w);
        const size_t off = ((size_t(pt.slot) * pt.tp + pt.rank) * pt.m_cap + t) * pt.H + n;
        if (pt.mc_inbox != nullptr) {
          multimem_st_v4(pt.mc_inbox + off, pk);
        } else {
#pragma unroll
          for (int k = 0; k < kPushMaxTp; ++k)
            if (k < pt.tp) *reinterpret_cast<uint4*>(pt.inbox[k] + off) = pk;
        }
      }
    }
    asm volatile("bar.sync 15, %0;" ::"n"(kDqThreads) : "memory");
    if (d == 0) {
      __threadfence_system();
      const int ctr = pt.slot * pt.tp + pt.rank;
      if (pt.mc_arrive != nullptr) {
        multimem_red_add_release(pt.mc_arrive + ctr, 1u);
      } else {
        // one system-scope fence (above) orders the CTA's stores before all of the counter updates
        for (int k = 0; k < pt.tp; ++k) red_add_relaxed_sys(pt.arrive[k] + ctr, 1u);
      }
    }
  }
  if (EPI == kEpiScatterF16 && dq_role && acc_ok) {
    // ---- reduce-scatter inside the GEMM: every 64-row block of tokens has one owner; this rank's fp16 partial rows
    // go to slot `rank` of the owner's inbox only, and the owner's counter of (source, block) gains one unit per
    // (weight tile, 16-token chunk) - the same total whatever K split each rank's shard width made it choose.
    constexpr int kDqThreads = kDqWarps * 32;
    constexpr int kBlocksPerTile = NT / kSpRowBlock;
    static_assert(EPI != kEpiScatterF16 || NT % kSpRowBlock == 0, "token tiles hold whole row blocks");
    asm volatile("bar.sync 15, %0;" ::"n"(kDqThreads) : "memory");
    const SpTable& sp = a.sp;
    const int d = (warp - 2) * 32 + lane;
    const int t0 = blockIdx.y * NT;
    const int owned = int(crank) < kChunks ? (kChunks - int(crank) + ks - 1) / ks : 0;
    for (int item = d; item < owned * 256; item += kDqThreads) {
      const int ch = int(crank) + (item >> 8) * ks;
      const int tok = (item & 255) >> 4, seg = item & 15;
      const int r = ch / (NT / 16), c0 = (ch % (NT / 16)) * 16;
      const int t = t0 + c0 + tok;
      const int n = (tile0 + r) * kTileN + seg * 8;
      if (t < a.M && n < a.N) {
        const float4* src = reinterpret_cast<const float4*>(park + (ch * 16 + tok) * 128 + seg * 8);
        const float4 lo = src[0], hi = src[1];
        uint4 pk;
        pk.x = pack_half2(clamp_f16(lo.x), clamp_f16(lo.y));
        pk.y = pack_half2(clamp_f16(lo.z), clamp_f16(lo.w));
        pk.z = pack_half2(clamp_f16(hi.x), clamp_f16(hi.y));
        pk.w = pack_half2(clamp_f16(hi.z), clamp_f16(hi.w));
        const int b = t / kSpRowBlock;
        const int owner = b % sp.tp;
        const int local = (b / sp.tp) * kSpRowBlock + (t % kSpRowBlock);
        const size_t off = ((size_t(sp.slot) * sp.tp + sp.rank) * sp.own_cap + local) * sp.H + n;
        *reinterpret_cast<uint4*>(sp.inbox[owner] + off) = pk;
      }
    }
    asm volatile("bar.sync 15, %0;" ::"n"(kDqThreads) : "memory");
    if (d < kBlocksPerTile) {
      const int b = t0 / kSpRowBlock + d;
      if (b * kSpRowBlock < a.M) {
        uint32_t units = 0;
        for (int i = 0; i < owned; ++i) {
          const int ch = int(crank) + i * ks;
          if (((ch % (NT / 16)) * 16) / kSpRowBlock == d) ++units;
        }
        if (units > 0) {
          __threadfence_system();               // the CTA's stores (ordered by the barrier above) before the count
          red_add_relaxed_sys(sp.arrive[b % sp.tp] + (size_t(sp.slot) * sp.tp + sp.rank) * sp.nblk_cap + b, units);
        }
      }
    }
  }
  if (in_cluster) cluster_sync_all();          // nobody leaves while its parked values may still be read
#ifdef ZSE_W4_TIMING
  if (a.timing != nullptr && threadIdx.x == 64 && blockIdx.x == 1 && blockIdx.z == 0) {
    a.timing[19 * 8 + 1] = clock64() - t_epi;
    a.timing[19 * 8 + 2] = n_units;
    a.timing[19 * 8 + 3] = clock64() - t_start;
    a.timing[19 * 8 + 4] = t_setup;
  }
#endif
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, Cfg::kTmemCols);
}

template <int NT, int R, int EPI, bool DUAL>
static int launch_w4(const CUtensorMap& tx, const W4Args& a, dim3 grid, cudaStream_t st) {
  auto kern = gemm_w4_kernel<NT, R, EPI, DUAL>;
  using Cfg = W4Cfg<NT, R, DUAL>;
  constexpr int smem = Cfg::kSmemBytes;
  static bool attr_done[kMaxDevices] = {};
  const int dev_slot = current_device_slot();
  if (!attr_done[dev_slot]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return ZSE_ERR_LAUNCH;
    attr_done[dev_slot] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(Cfg::kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = a.cluster_k;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, tx, a) == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

template <int NT, int R, bool DUAL = false>
static int launch_w4_epi(int epilogue, const CUtensorMap& tx, const W4Args& a, dim3 grid, cudaStream_t st) {
  if (epilogue == kEpiF16) return launch_w4<NT, R, kEpiF16, DUAL>(tx, a, grid, st);
  if (epilogue == kEpiSwiGLU) return launch_w4<NT, R, kEpiSwiGLU, DUAL>(tx, a, grid, st);
  if (epilogue == kEpiPartialF32) return launch_w4<NT, R, kEpiPartialF32, DUAL>(tx, a, grid, st);
  if (epilogue == kEpiPushF16) return launch_w4<NT, R, kEpiPushF16, DUAL>(tx, a, grid, st);
  if constexpr (NT >= 128) {         // the row-block exchange is for passes of many rows
    if (epilogue == kEpiScatterF16) return launch_w4<NT, R, kEpiScatterF16, DUAL>(tx, a, grid, st);
  }
  return ZSE_ERR_SHAPE;
}

// 0 = the planner decides, 1 = wide CTAs only, 2 = narrow (two per SM) CTAs wherever they are allowed;
// adding 4 keeps one- and two-token calls on the tensor cores instead of the CUDA-core GEMV
static int g_w4_mode = 0;

// How the launcher tiles a problem: weight tiles per CTA (R) and K splits (ks).  Measured on B200: a tcgen05.mma of
// M=128, K=16 occupies the tensor pipe for about 50 cycles whatever N <= 64 is, so a 128x128 weight chunk costs about
// 450 cycles on one SM and a CTA is tensor-issue bound, not bandwidth bound; what matters is an even spread of chunks
// over the SMs and a small fixed cost per CTA.  Row-parallel projections (fp32 epilogue) split K into planes that the
// consumer adds; the other epilogues need the whole K in one CTA (or an explicit cluster split).
// Relative cost of a chunk in a narrow CTA: when two CTAs share the SM's tensor pipe (per CTA) and when one runs alone.
constexpr double kW4DualPairCost = 0.65;
constexpr double kW4DualSoloCost = 0.95;

static void plan_w4(int M, int N, int K, int epilogue, int sm_count, int want_split, int* R_out, int* ks_out,
                    int* cluster_out, int* dual_out) {
  const int nt = pick_nt(M);
  const int n_tiles = epilogue == kEpiSwiGLU ? (N / 2 + 63) / 64 : (N + kTileN - 1) / kTileN;
  const int m_tiles = (M + nt - 1) / nt;
  const int k_stages = K / kW4StageK;
  const bool planes_ok = epilogue == kEpiPartialF32;
  double best_cost = -1.0;
  int best_r = 1, best_ks = 1, best_dual = 0;
  for (int dual = 0; dual <= 1; ++dual) {
    if (dual && (nt > 64 || (g_w4_mode & 3) == 1)) continue;
    if (!dual && (g_w4_mode & 3) == 2 && nt <= 64) continue;
    for (int R = 1; R <= (dual ? 1 : 2); ++R) {
      if (n_tiles % R != 0) continue;
      if (R == 2 && nt > 128) continue;                         // accumulators + A ring must fit 512 TMEM columns
      const long ctas = long(n_tiles / R) * m_tiles;
      // K splits: fp32 planes where the consumer adds them; otherwise a thread-block cluster along K that adds the
      // accumulators through distributed shared memory before the epilogue (worth it only when tiles alone cannot
      // fill the machine, e.g. a tensor-parallel shard of the gate/up projection)
      const int max_ks = min(kMaxPlanes, k_stages);
      for (int ks = 1; ks <= max_ks; ++ks) {
        if (!planes_ok && ks != 1 && ks != 2 && ks != 4 && ks != 8) continue;
        const long total = ctas * ks;
        const long cap = long(sm_count) * (dual ? 2 : 1);
        const long waves = (total + cap - 1) / cap;
        const long last = total - (waves - 1) * cap;            // CTAs of the last wave
        const double chunks = double((k_stages + ks - 1) / ks) * double(R);
        // time of one chunk in units of a wide CTA's chunk: activation share, and for narrow CTAs the tensor pipe
        // shared by the two CTAs of an SM (each runs slower, together they are faster)
        const double xshare = 0.1 * double(nt) / 64.0 / double(R);
        const double pair_chunk = 2.0 * kW4DualPairCost, solo_chunk = kW4DualSoloCost;
        double cost;
        if (!dual) {
          cost = double(waves) * (chunks * (1.0 + xshare) + 8.0);
        } else {
          const double full = chunks * (pair_chunk + 2.0 * xshare) + 9.0;      // an SM with two CTAs
          const double tail = last > sm_count ? full : chunks * (solo_chunk + xshare) + 8.0;
          cost = double(waves - 1) * full + tail;
        }
        cost += ks > 1 ? (planes_ok ? 1.0 : 6.0 + 0.5 * ks) : 0.0;
        if (best_cost < 0 || cost < best_cost - 1e-9 || (cost < best_cost + 1e-9 && !dual && R > best_r)) {
          best_cost = cost;
          best_r = R;
          best_ks = ks;
          best_dual = dual;
        }
      }
    }
  }
  *cluster_out = (!planes_ok && best_ks > 1) ? best_ks : 1;
  if (want_split > 0) {                                         // explicit request: planes if possible, else a cluster
    best_ks = max(1, min(want_split, min(8, k_stages)));
    if (!planes_ok) *cluster_out = best_ks;
  }
  *R_out = best_r;
  *ks_out = best_ks;
  *dual_out = best_dual;
}

}  // namespace zse

using namespace zse;

static long long* g_w4_timing = nullptr;
// Debug hook (only meaningful in builds with ZSE_W4_TIMING): device buffer of 20 x 8 counters.
extern "C" void zse_gemm_w4_set_timing(void* dev_buffer) { g_w4_timing = reinterpret_cast<long long*>(dev_buffer); }
// Tuning hook: 0 = planner decides between wide and narrow CTAs, 1 = wide only, 2 = narrow wherever allowed.
extern "C" void zse_gemm_w4_set_mode(int mode) { zse::g_w4_mode = mode; }

static int run_gemm_w4(const void* w_tiled, const void* x, int x_rows_cap, const void* bias, void* out, int M, int N,
                       int K, int ldo, int epilogue, int k_split, void* status, void* stream, const PushTable* push,
                       int* ctas_out, const SpTable* sp = nullptr, const GatherWait* gather = nullptr) {
  if (M <= 0) return 0;
  if (K % kW4StageK != 0 || N <= 0 || K <= 0) return ZSE_ERR_SHAPE;
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  if ((sp != nullptr || gather != nullptr) && M <= 64) return ZSE_ERR_SHAPE;   // wide CTAs (128 / 256 tokens) only
  if (!(g_w4_mode & 4) && push == nullptr) {
    const int gks = gemv_w4_plan(M, N, K, epilogue, sm_count, k_split);
    if (gks > 0)
      return gemv_w4_launch(w_tiled, x, bias, out, M, N, K, ldo, epilogue, gks, reinterpret_cast<cudaStream_t>(stream));
  }
  const int k_stages = K / kW4StageK;
  int R = 1, ks = 1, cluster = 1, dual = 0;
  plan_w4(M, N, K, epilogue, sm_count, k_split, &R, &ks, &cluster, &dual);
  const int spp = (k_stages + ks - 1) / ks;
  ks = (k_stages + spp - 1) / spp;                     // no empty split
  if (cluster > 1) cluster = ks;
  const int nt = pick_nt(M);
  const int n_tiles = epilogue == kEpiSwiGLU ? (N / 2 + 63) / 64 : (N + kTileN - 1) / kTileN;
  CUtensorMap tx;
  if (int rc = get_tmap(x, uint64_t(max(x_rows_cap, M)), uint64_t(K), uint32_t(nt), &tx)) return rc;
  W4Args a{reinterpret_cast<const uint8_t*>(w_tiled), reinterpret_cast<const __half*>(bias), out, M, N, K, ldo,
           k_stages, spp, cluster, reinterpret_cast<Status*>(status), g_w4_timing, PushTable{}, SpTable{},
           GatherWait{nullptr, nullptr}};
  if (push != nullptr) a.push = *push;
  if (sp != nullptr) a.sp = *sp;
  a.gather = gather != nullptr ? *gather : GatherWait{nullptr, nullptr};
  dim3 grid(n_tiles / R, (M + nt - 1) / nt, ks);
  if (ctas_out != nullptr) *ctas_out = int(grid.x * grid.y * grid.z);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int rc = ZSE_ERR_SHAPE;
  if (dual) {
    switch (nt) {
      case 16: rc = launch_w4_epi<16, 1, true>(epilogue, tx, a, grid, st); break;
      case 32: rc = launch_w4_epi<32, 1, true>(epilogue, tx, a, grid, st); break;
      default: rc = launch_w4_epi<64, 1, true>(epilogue, tx, a, grid, st); break;
    }
  } else if (R == 1) {
    ZSE_DISPATCH_NT(nt, rc = (launch_w4_epi<NT, 1>(epilogue, tx, a, grid, st)))
  } else if (R == 2) {
    switch (nt) {
      case 16: rc = launch_w4_epi<16, 2>(epilogue, tx, a, grid, st); break;
      case 32: rc = launch_w4_epi<32, 2>(epilogue, tx, a, grid, st); break;
      case 64: rc = launch_w4_epi<64, 2>(epilogue, tx, a, grid, st); break;
      default: rc = launch_w4_epi<128, 2>(epilogue, tx, a, grid, st); break;
    }
  }
  return rc;
}

extern "C" int zse_gemm_w4(const void* w_tiled, const void* x, int x_rows_cap, const void* bias, void* out, int M,
                           int N, int K, int ldo, int epilogue, int k_split, void* status, void* stream) {
  if (epilogue == kEpiPushF16) return ZSE_ERR_SHAPE;          // needs a tensor-parallel context: zse_tp_gemm_w4_push
  return run_gemm_w4(w_tiled, x, x_rows_cap, bias, out, M, N, K, ldo, epilogue, k_split, status, stream, nullptr,
                     nullptr);
}

// Row-parallel projection whose epilogue is the tensor-parallel exchange: every CTA sends its fp16 partial rows to
// every rank's inbox and counts itself in (see PushTable).  Returns the number of CTAs launched - the amount the
// consumer (zse_tp_sum_add_rmsnorm) must wait for from every rank - or a negative error.  N must equal the hidden
// size of the context and M must fit its row capacity.  rank_override >= 0 plays another rank (single-GPU tests).
extern "C" int zse_tp_gemm_w4_push(void* ctx, const void* w_tiled, const void* x, int x_rows_cap, int M, int N, int K,
                                   int slot, int use_multimem, int rank_override, void* status, void* stream) {
  PushTable pt;
  if (int rc = tp_fill_push_table(ctx, slot, use_multimem != 0, rank_override, &pt)) return rc;
  if (N != pt.H || M > pt.m_cap || N % 8) return ZSE_ERR_SHAPE;
  int ctas = 0;
  const int rc = run_gemm_w4(w_tiled, x, x_rows_cap, nullptr, nullptr, M, N, K, N, kEpiPushF16, 0, status, stream, &pt,
                             &ctas);
  return rc != 0 ? rc : ctas;
}

// Sequence-parallel prefill (see SpTable).  zse_tp_gemm_w4_scatter: row-parallel projection whose epilogue is the
// reduce-scatter (N = hidden size of the context, more than 64 rows).  zse_tp_gemm_w4_gathered: any epilogue of
// zse_gemm_w4, for a GEMM whose activations `x` are the context's gathered buffer - its prologue is the all-gather's
// receiving side.  `wait_gather` != 0 on both: also wait for the gathered rows of the own token tile.
// Replaces ncclAllReduce after o_proj / down_proj in the reference's prefill
// (zse-engine/zse_engine/orchestrator/model_runner.py:2823-2827,2872-2876).
extern "C" int zse_tp_gemm_w4_scatter(void* ctx, const void* w_tiled, const void* x, int x_rows_cap, int M, int N,
                                      int K, int slot, int rank_override, void* status, void* stream) {
  SpTable sp;
  if (int rc = tp_fill_sp_table(ctx, slot, false, rank_override, &sp)) return rc;
  if (N != sp.H || N % kTileN || M <= 64 || (M + kSpRowBlock - 1) / kSpRowBlock > sp.nblk_cap) return ZSE_ERR_SHAPE;
  return run_gemm_w4(w_tiled, x, x_rows_cap, nullptr, nullptr, M, N, K, N, kEpiScatterF16, 0, status, stream, nullptr,
                     nullptr, &sp, nullptr);
}

extern "C" int zse_tp_gemm_w4_gathered(void* ctx, const void* w_tiled, const void* x, int x_rows_cap,
                                       const void* bias, void* out, int M, int N, int K, int ldo, int epilogue,
                                       int k_split, int rank_override, void* status, void* stream) {
  if (epilogue == kEpiPushF16 || epilogue == kEpiScatterF16) return ZSE_ERR_SHAPE;
  SpTable sp;
  if (int rc = tp_fill_sp_table(ctx, 0, false, rank_override, &sp)) return rc;
  if (M <= 64 || (M + kSpRowBlock - 1) / kSpRowBlock > sp.nblk_cap) return ZSE_ERR_SHAPE;
  const GatherWait g{sp.gflag[sp.rank], sp.state};
  return run_gemm_w4(w_tiled, x, x_rows_cap, bias, out, M, N, K, ldo, epilogue, k_split, status, stream, nullptr,
                     nullptr, nullptr, &g);
}

// How many clusters of `cluster` CTAs of the 64-token kernel (narrow: two CTAs per SM, or wide) the device can hold at
// once (cudaOccupancyMaxActiveClusters); -1 on error.  The planner's wave model and the tests use it.
extern "C" int zse_gemm_w4_max_clusters(int narrow, int cluster) {
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = cluster;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.gridDim = dim3(64, 1, cluster);
  int n = -1;
  if (narrow) {
    using Cfg = W4Cfg<64, 1, true>;
    auto kern = gemm_w4_kernel<64, 1, kEpiF16, true>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (cluster > 8) cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    cfg.blockDim = dim3(Cfg::kThreads);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); return -1; }
  } else {
    using Cfg = W4Cfg<64, 1, false>;
    auto kern = gemm_w4_kernel<64, 1, kEpiF16, false>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (cluster > 8) cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    cfg.blockDim = dim3(Cfg::kThreads);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); return -1; }
  }
  return n;
}

// What the launcher would do for these arguments: out4 = {weight tiles per wide CTA, K splits, cluster size along K,
// CTA shape (0 wide, 1 narrow)}; -1 in out4[3] = CUDA-core GEMV.
extern "C" void zse_gemm_w4_plan(int M, int N, int K, int epilogue, int k_split, int sm_count, int* out4) {
  if (sm_count <= 0) sm_count = 148;
  if (!(g_w4_mode & 4)) {
    const int gks = gemv_w4_plan(M, N, K, epilogue, sm_count, k_split);
    if (gks > 0) {
      out4[0] = 1, out4[1] = gks, out4[2] = 1, out4[3] = -1;
      return;
    }
  }
  plan_w4(M, N, K, epilogue, sm_count, k_split, &out4[0], &out4[1], &out4[2], &out4[3]);
}

// Number of fp32 planes zse_gemm_w4 writes for an fp32-epilogue call with these arguments (the caller sizes the plane
// buffer and tells the consumer how many planes to add).
extern "C" int zse_gemm_w4_splits(int M, int N, int K, int k_split) {
  if (M <= 0 || K % kW4StageK != 0 || K <= 0) return 1;
  int sm_count = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  if (sm_count <= 0) sm_count = 148;
  if (!(g_w4_mode & 4)) {
    const int gks = gemv_w4_plan(M, N, K, kEpiPartialF32, sm_count, k_split);
    if (gks > 0) return gks;
  }
  int R = 1, ks = 1, cluster = 1, dual = 0;
  plan_w4(M, N, K, kEpiPartialF32, sm_count, k_split, &R, &ks, &cluster, &dual);
  const int k_stages = K / kW4StageK;
  const int spp = (k_stages + ks - 1) / ks;
  return (k_stages + spp - 1) / spp;
}

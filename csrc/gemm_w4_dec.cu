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
//  * Inside a CTA two pipelines run side by side, one per tile of the pair, and share every activation stage.  Each
//    pipeline is worked by two lanes (even and odd K stages), and a lane is a closed loop of its own: a dequant group
//    of four warps, one TMEM operand slot, one MMA-issuing warp and one accumulator.  Measured on B200, a thread that
//    issues tcgen05.mma back to back gets one through every ~85 cycles (M 128, N 64, K 16, A in TMEM) whatever else
//    it executes, while the tensor pipe needs 32: four issuing threads, one per scheduler, are what fills the pipe.
//      warps 0-3   MMA issuers of lane (pipeline p, parity s) (tcgen05.mma, A = dequantised weights in TMEM, B =
//                  activations in shared memory); the two accumulators of a tile are added in the epilogue,
//      warp 4      producer: bulk TMA of the weight chunks (one ring per pipeline), tiled TMA of the activations,
//      warps 5-20  dequant: four groups of four warps, group (p, s) fills the operand slot of lane (p, s), so
//                  dequantising chunk c+1 (other lane) overlaps the MMAs of chunk c,
//      warps 21-24 epilogue: takes the finished tile pairs one after the other; the pipelines only wait for it
//                  until it has read the accumulators out of TMEM.
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

constexpr int kDecWarps = 25;
constexpr int kDecThreads = kDecWarps * 32;
constexpr int kDecSX = 6;            // activation stages (INT4; INT8 chunks are twice as large: 5)
constexpr int kDecSW = 5;            // weight chunks per pipeline ring (INT4; INT8: 3)
constexpr int kW8ChunkBytes = 16640; // INT8 chunk: 128 rows x 128 K int8 + 128 fp16 scales
constexpr int kDecProducerWarp = 4;
constexpr int kDecDqWarp0 = 5;
constexpr int kDecEpiWarp0 = 21;
constexpr int kDecWorkerWarps = 20;      // dequant + epilogue warps: what runs the tails of the kernel
constexpr int kDecStageBytes = 64 * 128 * 4;     // finished sums of one tile: [token column][128 rows] fp32

enum DecEpilogue : int { kDecF16 = 0, kDecSwiGLU = 1, kDecF32 = 2, kDecQkvRope = 3, kDecAllReduceNorm = 4 };

struct DecBars {
  uint64_t w_full[2][kDecSW], w_empty[2][kDecSW];
  uint64_t x_full[kDecSX], x_empty[kDecSX];
  uint64_t a_ready[2][2], slot_free[2][2];
  uint64_t acc_full[2][2], acc_empty[2][2];
  uint64_t bdesc[kDecSX][8];     // activation descriptors of every (stage, K step): the MMA issuers only load them
  uint32_t tmem_base;
  int abort_flag;
};

template <int NT, bool W8 = false>
struct DecCfg {
  static constexpr int kSX = W8 ? 5 : kDecSX;
  static constexpr int kSW = W8 ? 3 : kDecSW;
  static constexpr int kChunk = W8 ? kW8ChunkBytes : kW4ChunkBytes;
  static constexpr int kXBytes = NT * 128;                  // one 64-wide K sub-tile of X
  static constexpr int kXStage = 2 * kXBytes;
  static constexpr int kXRing = ((kSX * kXStage + 1023) / 1024) * 1024;
  static constexpr int kWRing = 2 * kSW * kChunk;
  static constexpr int kStageOff = kXRing + ((kWRing + 127) / 128) * 128;
  static constexpr int kBarsOff = kStageOff + kDecStageBytes;
  static constexpr int kSmemBytes = kBarsOff + 1024 + 1024;   // barriers + alignment slack
  static constexpr int kGranules = NT / 8;                    // 8-column granules of the token dimension
  static_assert(kSmemBytes <= 232448, "shared memory budget");
  // split plan: the receive area [S][2][ceil(G/S)][8][128] fp32 lies over both rings (S * ceil(G/S) <= G + S - 1)
  static_assert((kGranules + 7) * 2 * 8 * 128 * 4 <= kStageOff, "receive area of the split plan");
};

struct DecRope {
  const int* positions;        // [M]
  const long long* slots;      // [M] cache slot = block * block_size + offset; -1 = do not store
  const float2* cos_sin;       // [max_position][64] {cos, sin} of position * inv_freq[i]
  __half* kv_layer;            // [blocks][2][nkv][block_size][128]
  int nh, nkv, block_size, max_position;
};

// Row-parallel projection whose epilogue is the tensor-parallel all-reduce, the residual add and the next RMSNorm
// (kDecAllReduceNorm).  Every CTA sends the fp16 sums it finishes to slot `rank` of EVERY rank's inbox (one
// multimem.st through the NVSwitch, or one store per peer) and adds the number of (tile, column granule) units it
// finished to the counter [slot][rank] on every rank.  Then the CTAs that own a token row wait until every source's
// counter has gained n_tiles * granules units, add the tp inbox rows in rank order (so the replicated residual stream
// stays bit-identical on all ranks), add the fp32 residual and normalise.  Counting units instead of CTAs makes the
// target the same whatever plan each rank chose for its own shard width.  The running total a counter must reach
// lives in device memory (state[slot]) and is advanced by the last CTA to leave, so a CUDA graph replays the launch
// unchanged; two inbox slots alternate between calls.
struct DecTpNorm {
  PushTable push;              // inboxes [2 slots][tp][m_cap][H] and counters [2 slots][tp] of every rank
  uint32_t* state;             // this rank's words {expected slot 0, expected slot 1, exit ticket}
  float* residual;             // fp32 [M, H], in/out
  const __half* norm_w;        // fp16 [H]
  __half* xnorm;               // fp16 [M, H] out (null: residual only)
  float eps;
  uint32_t units_total;        // what every source adds to its counter in one call
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
  long long* timing;           // debug builds (ZSE_DEC_TIMING): per-role cycle counters of one CTA, else unused
  DecRope rope;
  DecTpNorm tpn;
};

__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void dec_multimem_st_v4(void* mc_ptr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f16x2 [%0], {%1,%2,%3,%4};" ::"l"(mc_ptr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void dec_multimem_red_add_release(uint32_t* mc_ptr, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc_ptr), "r"(v) : "memory");
}
__device__ __forceinline__ void dec_red_add_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t dec_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void dec_red_add_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t dec_ld_acquire(const uint32_t* p, bool device_scope) {
  return device_scope ? ld_acquire_gpu_u32(p) : dec_ld_acquire_sys(p);
}
__device__ __forceinline__ uint4 dec_ld_relaxed_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p)
               : "memory");
  return v;
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

#ifdef ZSE_DEC_TIMING
#define DTICK(var) long long var = clock64()
#define DACC(slot, t0) tacc[slot] += clock64() - (t0)
#else
#define DTICK(var)
#define DACC(slot, t0)
#endif

// Sixteen int8 (one 16-byte part of a row: K = 16p .. 16p+15) -> eight half2 words, times the group's scale.  A byte b
// is placed under the exponent of 1024 as 0x6400 | (b ^ 0x80), i.e. 1024 + (b + 128); subtracting 1152 leaves b
// exactly, the multiplication by the scale rounds once.
__device__ __forceinline__ void dec_dequant_w8_part(const uint4& w, __half2 s2, uint32_t* out8) {
  const __half2 k1152 = __half2half2(__ushort_as_half(0x6480));      // 1152
  const uint32_t in[4] = {w.x ^ 0x80808080u, w.y ^ 0x80808080u, w.z ^ 0x80808080u, w.w ^ 0x80808080u};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t lo = __byte_perm(in[i], 0x64646464u, 0x4140);            // bytes 0, 1 -> (k, k+1)
    uint32_t hi = __byte_perm(in[i], 0x64646464u, 0x4342);            // bytes 2, 3 -> (k+2, k+3)
    __half2 a = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&lo), k1152), s2);
    __half2 b = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&hi), k1152), s2);
    out8[2 * i] = *reinterpret_cast<uint32_t*>(&a);
    out8[2 * i + 1] = *reinterpret_cast<uint32_t*>(&b);
  }
}

// Bounded wait until a flag word in global memory holds `want`.
__device__ __forceinline__ bool dec_wait_flag(const uint32_t* flag, uint32_t want, volatile int* abort_flag, Status* st,
                                              unsigned where, unsigned detail) {
  if (ld_acquire_gpu_u32(flag) == want) return true;
  SpinClock clk;
  while (ld_acquire_gpu_u32(flag) != want) {
    const bool late = clk.expired(0x3F);
    if ((clk.spins & 0x3F) == 0) {
      if (*abort_flag) return false;
      if (late) {
        report(st, kWaitTimeout, where, detail);
        *abort_flag = 1;
        __threadfence_block();
        return false;
      }
    }
  }
  return true;
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

// Eight tcgen05.mma of one 128 x 128 chunk, back to back.  The issuing thread shares its scheduler with five busy
// warps and gets an issue slot only every ten to thirty cycles, so what counts is the number of instructions it
// executes per chunk: the eight activation descriptors of a stage come out of a table in shared memory (four 16-byte
// loads), the eight TMEM operand addresses are loop-invariant registers, the predicate is set twice.
__device__ __forceinline__ void dec_mma_chunk(uint32_t dt, const uint32_t (&at)[8], const uint64_t* bdesc_stage,
                                              uint32_t idesc, uint32_t accumulate_first) {
  const ulonglong2* tab = reinterpret_cast<const ulonglong2*>(bdesc_stage);
  const ulonglong2 d01 = tab[0], d23 = tab[1], d45 = tab[2], d67 = tab[3];
  asm volatile(
      "{\n\t"
      ".reg .pred p, t;\n\t"
      "setp.ne.b32 p, %17, 0;\n\t"
      "setp.eq.b32 t, %18, %18;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %9, %18, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%2], %10, %18, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%3], %11, %18, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%4], %12, %18, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%5], %13, %18, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%6], %14, %18, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%7], %15, %18, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%8], %16, %18, t;\n\t"
      "}" ::"r"(dt),
      "r"(at[0]), "r"(at[1]), "r"(at[2]), "r"(at[3]), "r"(at[4]), "r"(at[5]), "r"(at[6]), "r"(at[7]), "l"(d01.x),
      "l"(d01.y), "l"(d23.x), "l"(d23.y), "l"(d45.x), "l"(d45.y), "l"(d67.x), "l"(d67.y), "r"(accumulate_first),
      "r"(idesc)
      : "memory");
}

// Barriers of the threads that run an epilogue together: 128 (the four epilogue warps) or 640 (with the sixteen dequant
// warps, for the last tile pair of a CTA, when those have nothing else left to do).
__device__ __forceinline__ void epi_bar(int wide) {
  if (wide)
    asm volatile("bar.sync 2, 640;" ::: "memory");
  else
    asm volatile("bar.sync 1, 128;" ::: "memory");
}
// Barrier that also ANDs a predicate: after a bounded wait all threads take the same branch, so nobody is left alone
// at a later barrier.
__device__ __forceinline__ bool epi_all(bool v, int wide) {
  uint32_t r;
  if (wide)
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.and.pred q, 2, 640, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(r)
        : "r"(uint32_t(v))
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.and.pred q, 1, 128, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(r)
        : "r"(uint32_t(v))
        : "memory");
  return r != 0;
}

// ---- epilogue ---------------------------------------------------------------------------------------------------
// Finished sums reach the stores through a `fetch`: four consecutive rows of one token column of a tile.
//   StageFetch  - the sums are in this CTA's shared memory (stream plan);
//   RecvFetch   - split plan: the S partial sums of a column granule were pushed into the shared memory of the CTA
//                 that finishes it; the fetch adds them in rank order.
struct StageFetch {
  const float* stage;                                 // [col][128]
  __device__ __forceinline__ float4 get4(int col, int row) const {
    return *reinterpret_cast<const float4*>(stage + col * 128 + row);
  }
};
struct RecvFetch {
  const float* recv;                                  // [S sources][2 tiles][go_max][8 cols][128] of this CTA
  int S, r, j, go_max;                                // tile of the pair, index of the owned granule
  __device__ __forceinline__ float4 get4(int col, int row) const {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int c = 0; c < 8; ++c) {                     // rank order: the sum is reproducible
      if (c < S) {
        const float4 t =
            *reinterpret_cast<const float4*>(recv + ((((c * 2 + r) * go_max + j) * 8 + (col & 7)) * 128 + row));
        v.x += t.x;
        v.y += t.y;
        v.z += t.z;
        v.w += t.w;
      }
    }
    return v;
  }
};

__device__ __forceinline__ void cluster_sync_all_threads() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t dec_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// One work item of the stores: token column `col` of tile `tile`, position e7 (0..127) inside the granule's 8 x 16
// grid -> 16 bytes of output (8 bytes for SwiGLU).  `add_bias`: the fetch delivers sums without the bias.
template <int NT, int EPI, typename Fetch>
__device__ __forceinline__ void dec_store_item(const DecArgs& a, const Fetch& f, int tile, int col, int e7,
                                               bool add_bias) {
  const int t = col;
  if (t >= a.M) return;
  if (EPI == kDecAllReduceNorm) {
    // this rank's partial row segment (8 columns of the hidden dimension) -> slot `rank` of every rank's inbox
    const int r0 = (e7 & 15) * 8, n = tile * kTileN + r0;
    if (n >= a.N) return;
    const float4 lo = f.get4(col, r0), hi = f.get4(col, r0 + 4);
    uint4 pk;
    pk.x = pack_half2(clamp_f16(lo.x), clamp_f16(lo.y));
    pk.y = pack_half2(clamp_f16(lo.z), clamp_f16(lo.w));
    pk.z = pack_half2(clamp_f16(hi.x), clamp_f16(hi.y));
    pk.w = pack_half2(clamp_f16(hi.z), clamp_f16(hi.w));
    const PushTable& pt = a.tpn.push;
    const size_t off = ((size_t(pt.slot) * pt.tp + pt.rank) * pt.m_cap + t) * pt.H + n;
    if (pt.mc_inbox != nullptr) {
      dec_multimem_st_v4(pt.mc_inbox + off, pk);
    } else {
#pragma unroll
      for (int k = 0; k < kPushMaxTp; ++k)
        if (k < pt.tp) *reinterpret_cast<uint4*>(pt.inbox[k] + off) = pk;
    }
    return;
  }
  if (EPI == kDecF16 || EPI == kDecF32) {
    const int r0 = (e7 & 15) * 8, n = tile * kTileN + r0;
    if (n >= a.N) return;
    float4 lo = f.get4(col, r0), hi = f.get4(col, r0 + 4);
    if (add_bias && a.bias != nullptr) {
      const uint4 bw = *reinterpret_cast<const uint4*>(a.bias + n);
      const __half2* bh = reinterpret_cast<const __half2*>(&bw);
      const float2 b0 = __half22float2(bh[0]), b1 = __half22float2(bh[1]), b2 = __half22float2(bh[2]),
                   b3 = __half22float2(bh[3]);
      lo.x += b0.x; lo.y += b0.y; lo.z += b1.x; lo.w += b1.y;
      hi.x += b2.x; hi.y += b2.y; hi.z += b3.x; hi.w += b3.y;
    }
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
    // tile rows 0..63 = gate, 64..127 = up of the same 64 outputs: four outputs per work item
    const int o0 = (e7 & 15) * 4, n = tile * 64 + o0;
    if (n >= a.N / 2) return;
    const float4 gt = f.get4(col, o0), up = f.get4(col, 64 + o0);
    uint2 pk;
    pk.x = pack_half2(clamp_f16(silu_f(gt.x) * up.x), clamp_f16(silu_f(gt.y) * up.y));
    pk.y = pack_half2(clamp_f16(silu_f(gt.z) * up.z), clamp_f16(silu_f(gt.w) * up.w));
    *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(a.out) + size_t(t) * a.ldo + n) = pk;
  } else if (EPI == kDecQkvRope) {
    // tile = one head of 128 dims: q heads, then k heads, then v heads; eight dims per work item
    const DecRope& rp = a.rope;
    const int d0 = (e7 & 15) * 8, dl = d0 & 63;
    float val[8];
    if (tile < rp.nh + rp.nkv) {
      float xa[8], xb[8];                           // dims dl.. of the first half, of the second half
      *reinterpret_cast<float4*>(xa) = f.get4(col, dl);
      *reinterpret_cast<float4*>(xa + 4) = f.get4(col, dl + 4);
      *reinterpret_cast<float4*>(xb) = f.get4(col, 64 + dl);
      *reinterpret_cast<float4*>(xb + 4) = f.get4(col, 64 + dl + 4);
      if (add_bias && a.bias != nullptr) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xa[i] += __half2float(a.bias[tile * 128 + dl + i]);
          xb[i] += __half2float(a.bias[tile * 128 + 64 + dl + i]);
        }
      }
      const int pos = min(max(rp.positions[t], 0), rp.max_position - 1);
      const float2* cs = rp.cos_sin + size_t(pos) * 64 + dl;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 c2 = cs[i];
        val[i] = d0 < 64 ? xa[i] * c2.x - xb[i] * c2.y : xb[i] * c2.x + xa[i] * c2.y;
      }
    } else {
      *reinterpret_cast<float4*>(val) = f.get4(col, d0);
      *reinterpret_cast<float4*>(val + 4) = f.get4(col, d0 + 4);
      if (add_bias && a.bias != nullptr) {
#pragma unroll
        for (int i = 0; i < 8; ++i) val[i] += __half2float(a.bias[tile * 128 + d0 + i]);
      }
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

// Eight columns of tile r's sum: the accumulators of the two lanes (even / odd K stages), whichever took part.
__device__ __forceinline__ void dec_load_acc8(uint32_t tmem, uint32_t lane_addr, int r, int gr, bool lane0, bool lane1,
                                              float (&v)[8]) {
  uint32_t x[8], y[8];
  // both are loaded whatever took part (an accumulator that was not written holds garbage that is not used): loads
  // under a condition would force the arrays into local memory
  ZSE_TMEM_LD_X8(x, tmem + lane_addr + (2 * r) * 64 + gr * 8);
  ZSE_TMEM_LD_X8(y, tmem + lane_addr + (2 * r + 1) * 64 + gr * 8);
  tc_wait_ld();
#pragma unroll
  for (int i = 0; i < 8; ++i)
    v[i] = (lane0 ? __uint_as_float(x[i]) : 0.f) + (lane1 ? __uint_as_float(y[i]) : 0.f);
}

// Stream plan: one tile pair of one CTA, from finished MMAs to memory.  Run by W warps per TMEM lane quarter (W = 1:
// the epilogue warps alone, while the pipelines work on the next pair; W = 5: all twenty worker warps, for the CTA's
// last pair); `wi` is this warp's index among them.  stage0 / stage1: where the finished sums of the two tiles are
// staged (the same buffer for W = 1: the tiles then go one after the other).
template <int NT, int EPI>
__device__ __forceinline__ bool dec_epilogue_item(const DecArgs& a, DecBars* bars, float* stage0, float* stage1,
                                                  uint32_t tmem, int cta, int n_cta, int pair, int ka, int len,
                                                  int ntp, bool lane0, bool lane1, uint32_t par0, uint32_t par1,
                                                  bool release, uint32_t epoch1, int q, int lane, int wi, int W,
                                                  bool alive_in, long long* tacc) {
  constexpr int G = NT / 8;
  const int ks = a.k_stages;
  const int wide = W > 1;
  const int row = q * 32 + lane, et = wi * 128 + row;
  const uint32_t lane_addr = uint32_t(q * 32) << 16;
  volatile int* abort_flag = &bars->abort_flag;
  uint32_t* flags = a.sync + 8;
  // the CTA that holds K stage 0 of the pair finishes it; src0 .. src0 + n_src - 1 are the CTAs whose partial sums
  // it needs
  const bool owner = ka == 0;
  int src0 = cta + 1, n_src = 0;
  if (owner && len < ks)
    while (src0 + n_src < n_cta && dec_range_begin(a, src0 + n_src, n_cta) < (pair + 1) * ks) ++n_src;
  DTICK(e0);
  // every thread of the group comes through the vote below whatever happened before, so a failed wait anywhere ends
  // the epilogue for all of them together
  bool alive = alive_in && !*abort_flag;
  for (int r = 0; r < ntp && alive; ++r) {
    if (lane0) alive = mbar_wait(&bars->acc_full[r][0], par0, abort_flag, a.status, 9, r);
    if (lane1 && alive) alive = mbar_wait(&bars->acc_full[r][1], par1, abort_flag, a.status, 9, 2 + r);
  }
  if (owner && alive && lane == 0)
    for (int j = wi; j < n_src && alive; j += W)
      alive = dec_wait_flag(flags + src0 + j, epoch1, abort_flag, a.status, 10, src0 + j);
  alive = epi_all(alive, wide);
  if (!alive) return false;
  DACC(0, e0);
  DTICK(e1);
  tc_fence_after_sync();
  if (!owner) {
    // ---- partial sums go to the workspace (units = granules of both tiles, dealt to the warps); the barrier orders
    // every thread's stores before the one release that publishes them
#pragma unroll 1
    for (int u = wi; u < ntp * G; u += W) {
      const int r = u / G, gr = u - r * G;
      float v[8];
      dec_load_acc8(tmem, lane_addr, r, gr, lane0, lane1, v);
      float* dstw = a.ws + ((size_t(cta) * 2 + r) * NT + gr * 8) * 128 + row;
#pragma unroll
      for (int i = 0; i < 8; ++i) __stcg(dstw + i * 128, v[i]);
    }
    if (release) {                                     // the accumulators are read: the lanes may go on
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0)
        for (int r = 0; r < ntp; ++r) {
          if (lane0) mbar_arrive(&bars->acc_empty[r][0]);
          if (lane1) mbar_arrive(&bars->acc_empty[r][1]);
        }
    }
    epi_bar(wide);
    if (et == 0) {
      __threadfence();
      st_release_gpu_u32(flags + cta, epoch1);
    }
    DACC(1, e1);
    return true;
  }
  const bool two_stages = stage0 != stage1;
  for (int r0 = 0; r0 < ntp; r0 += (two_stages ? 2 : 1)) {
    const int r1 = two_stages ? ntp : r0 + 1;
    DTICK(e3);
    // ---- phase 1: finished sums -> stage[col][row]
    for (int r = r0; r < r1; ++r) {
      float* stage = r == 0 ? stage0 : stage1;
      float bias = 0.f;
      const int tile = 2 * pair + r;
      if ((EPI == kDecF16 || EPI == kDecQkvRope) && a.bias != nullptr && tile * kTileN + row < a.N)
        bias = __half2float(a.bias[tile * kTileN + row]);
#pragma unroll 1
      for (int gr = wi; gr < G; gr += W) {
        // partial sums of the other CTAs (one or two as a rule): their loads are in flight together with the TMEM
        // loads; added in CTA order (the sum is reproducible)
        float t8[2][8];
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          const bool use = jj < n_src;
          const float* srcw = a.ws + ((size_t(use ? src0 + jj : cta) * 2 + r) * NT + gr * 8) * 128 + row;
#pragma unroll
          for (int i = 0; i < 8; ++i) t8[jj][i] = use ? __ldcg(srcw + i * 128) : 0.f;
        }
        float v[8];
        dec_load_acc8(tmem, lane_addr, r, gr, lane0, lane1, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = (v[i] + bias) + t8[0][i] + t8[1][i];
        for (int j = 2; j < n_src; ++j) {                       // rare: a pair cut into more than three pieces
          const float* srcw = a.ws + ((size_t(src0 + j) * 2 + r) * NT + gr * 8) * 128 + row;
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] += __ldcg(srcw + i * 128);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) stage[(gr * 8 + i) * 128 + row] = v[i];
      }
      if (release) {                                   // tile r's accumulators are read: its lanes may go on
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if (lane0) mbar_arrive(&bars->acc_empty[r][0]);
          if (lane1) mbar_arrive(&bars->acc_empty[r][1]);
        }
      }
    }
    epi_bar(wide);
    DACC(3, e3);
    DTICK(e4);
    // ---- phase 2: 16-byte stores; work item -> (tile, granule, column of the granule, 8 rows)
#pragma unroll 1
    for (int idx = et; idx < (r1 - r0) * G * 128; idx += 128 * W) {
      const int r = r0 + idx / (G * 128), rem = idx % (G * 128);
      StageFetch f{r == 0 ? stage0 : stage1};
      dec_store_item<NT, EPI>(a, f, 2 * pair + r, (rem >> 7) * 8 + ((rem & 127) >> 4), rem & 127, false);
    }
    if (r1 < ntp) epi_bar(wide);                      // the stage is reused by the second tile
    DACC(4, e4);
  }
  return true;
}

// Split plan: the S CTAs that share a tile pair form a thread-block cluster; segment `seg` finishes the column
// granules g with g mod S == seg.  Once every CTA of the cluster is through its MMAs (first cluster barrier: all
// rings are idle), each one sends its fp32 partial sums of every granule to the shared memory of the CTA that
// finishes it - plain remote stores, nothing waits for a round trip - into slot [source rank]; after the second
// cluster barrier the owner adds the S slots in rank order.  Remote loads are avoided on purpose: measured here, a
// thread's loads from another SM's shared memory complete one after the other at ~800 cycles each.
template <int NT>
__device__ __forceinline__ void dec_split_push(float* recv, uint32_t tmem, int ntp, bool lane0, bool lane1, int seg,
                                               int S, int go_max, int q, int lane, int wi) {
  constexpr int G = NT / 8;
  const int row = q * 32 + lane;
  const uint32_t lane_addr = uint32_t(q * 32) << 16;
#pragma unroll 1
  for (int u = wi; u < ntp * G; u += 5) {
    const int r = u / G, gr = u - r * G;
    const int owner = gr % S, j = gr / S;
    float v[8];
    dec_load_acc8(tmem, lane_addr, r, gr, lane0, lane1, v);
    const uint32_t local = smem_u32(recv + ((((seg * 2 + r) * go_max + j) * 8) * 128 + row));
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(owner));
#pragma unroll
    for (int i = 0; i < 8; ++i)
      asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + i * 512), "f"(v[i]) : "memory");
  }
}

template <int NT, int EPI>
__device__ __forceinline__ void dec_split_finish(const DecArgs& a, const float* recv, int pair, int ntp, int seg, int S,
                                                 int go_max, int et) {
  constexpr int G = NT / 8;
  const int Go = seg < G ? (G - seg + S - 1) / S : 0;               // granules per tile this CTA finishes
#pragma unroll 1
  for (int idx = et; idx < ntp * Go * 128; idx += 640) {
    const int r = idx / (Go * 128), rem = idx - r * (Go * 128);
    const int j = rem >> 7, gr = seg + j * S;
    RecvFetch f{recv, S, r, j, go_max};
    dec_store_item<NT, EPI>(a, f, 2 * pair + r, gr * 8 + ((rem & 127) >> 4), rem & 127, true);
  }
}

// Second half of kDecAllReduceNorm, run by the twenty worker warps (640 threads, index `et`) of every CTA after its
// own sums are on their way: count this CTA's units in on every rank, then, for the token rows this CTA owns
// (row = cta, cta + grid, ...), wait for all sources, add, residual, RMSNorm.
__device__ __forceinline__ void dec_allreduce_norm_tail(const DecArgs& a, DecBars* bars, float* red, int cta,
                                                        int n_cta, uint32_t my_units, bool pushed_ok, int et,
                                                        long long* tacc = nullptr, long long t_entry = 0) {
  const DecTpNorm& tn = a.tpn;
  const PushTable& pt = tn.push;
  volatile int* abort_flag = &bars->abort_flag;
  const int tp = pt.tp, H = pt.H, nch = H / 8;
  const int ctr_i = pt.slot * tp + pt.rank;
  const bool local_fast = pt.mc_arrive == nullptr;        // own counter at device scope, counted per warp
  // ---- count in.  This GPU's own waiters are served first and cheaply: every worker warp releases its own stores
  // at device scope (no CTA barrier, no system-scope fence on that path), so the own counter runs kDecWorkerWarps
  // times as fast as the ones the peers see.
  __syncwarp();
  if (local_fast && (et & 31) == 0 && pushed_ok && my_units > 0)
    dec_red_add_release_gpu(pt.arrive[pt.rank] + ctr_i, my_units);
  // what does not depend on anybody else is fetched while the counters fill: the residual row and the norm weights
  const bool owner = cta < a.M;
  float4 rx[2], ry[2];
  uint4 wr[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int c = et + j * 640;
    if (owner && c < nch) {
      const float4* res = reinterpret_cast<const float4*>(tn.residual + size_t(cta) * H) + 2 * c;
      rx[j] = res[0];
      ry[j] = res[1];
      wr[j] = reinterpret_cast<const uint4*>(tn.norm_w)[c];
    }
  }
  if (tp > 1 || !local_fast) {
    epi_bar(1);                                            // every store of this CTA has been issued
    if (et == 0 && pushed_ok && my_units > 0) {
      __threadfence_system();
      if (pt.mc_arrive != nullptr) {
        dec_multimem_red_add_release(pt.mc_arrive + ctr_i, my_units);
      } else {
        for (int k = 0; k < tp; ++k)
          if (k != pt.rank) dec_red_add_relaxed_sys(pt.arrive[k] + ctr_i, my_units);   // released by the fence above
      }
    }
  }
#ifdef ZSE_DEC_TIMING
#define DTAIL(i) if (tacc != nullptr && cta == 1 && et == 512) a.timing[200 + (i)] = clock64() - t_entry
#else
#define DTAIL(i)
#endif
  DTAIL(0);
  bool ok = pushed_ok;
  if (owner) {
    // ---- wait until every source has delivered its rows (bounded; a lost peer ends in a status, not a hang)
    if (et < tp) {
      const bool local = local_fast && et == pt.rank;
      const uint32_t base = tn.state[pt.slot] + tn.units_total;
      const uint32_t target = local ? base * uint32_t(kDecWorkerWarps) : base;
      const uint32_t* ctr = pt.arrive[pt.rank] + pt.slot * tp + et;
      if (int32_t(dec_ld_acquire(ctr, local) - target) < 0) {
        SpinClock clk;
        while (int32_t(dec_ld_acquire(ctr, local) - target) < 0) {
          if (clk.expired(0x3F) || ((clk.spins & 0x3F) == 0 && *abort_flag)) {
            report(a.status, kPeerTimeout, 35, et);
            ok = false;
            break;
          }
        }
      }
    }
    ok = epi_all(ok, 1);
#ifdef ZSE_DEC_TIMING
    if (tacc != nullptr) tacc[5] = clock64() - t_entry;
#endif
    int it = 0;
    for (int row = cta; row < a.M; row += n_cta, ++it) {
      const __half* box = pt.inbox[pt.rank] + (size_t(pt.slot) * tp * pt.m_cap + row) * H;
      float vals[2][8];
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int c = et + j * 640;
        if (c < nch) {
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          if (ok) {
            uint4 got[kPushMaxTp];
#pragma unroll
            for (int r = 0; r < kPushMaxTp; ++r)
              if (r < tp)         // ordered by the acquire above; L2 is where peer stores land, so bypass L1 only
                got[r] = __ldcg(reinterpret_cast<const uint4*>(box + size_t(r) * pt.m_cap * H + size_t(c) * 8));
#pragma unroll
            for (int r = 0; r < kPushMaxTp; ++r) {           // rank order: the same sum on every rank
              if (r < tp) {
                const __half2* h = reinterpret_cast<const __half2*>(&got[r]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 fv = __half22float2(h[i]);
                  acc[2 * i] += fv.x;
                  acc[2 * i + 1] += fv.y;
                }
              }
            }
          }
#ifdef ZSE_DEC_TIMING
          if (tacc != nullptr && cta == 1 && et == 512 && j == 0)
            a.timing[204] = (clock64() - t_entry) + (__float_as_uint(acc[0]) & 1u);
#endif
          float4* res = reinterpret_cast<float4*>(tn.residual + size_t(row) * H) + 2 * c;
          if (it > 0) {                                     // rows after the first: nothing was fetched ahead
            rx[j] = res[0];
            ry[j] = res[1];
          }
          float4 x = rx[j], y = ry[j];
          x.x += acc[0]; x.y += acc[1]; x.z += acc[2]; x.w += acc[3];
          y.x += acc[4]; y.y += acc[5]; y.z += acc[6]; y.w += acc[7];
#ifdef ZSE_DEC_TIMING
          if (tacc != nullptr && cta == 1 && et == 512 && j == 0)
            a.timing[205] = (clock64() - t_entry) + (__float_as_uint(x.x) & 1u);
#endif
          res[0] = x;
          res[1] = y;
          vals[j][0] = x.x; vals[j][1] = x.y; vals[j][2] = x.z; vals[j][3] = x.w;
          vals[j][4] = y.x; vals[j][5] = y.y; vals[j][6] = y.z; vals[j][7] = y.w;
#pragma unroll
          for (int i = 0; i < 8; ++i) ss += vals[j][i] * vals[j][i];
        }
      }
      DTAIL(1);
      if (tn.xnorm != nullptr) {
        float* rd = red + (it & 1) * 32;                   // two buffers: one barrier per row is enough
        ss = warp_sum(ss);
        if ((et & 31) == 0) rd[et >> 5] = ss;
        epi_bar(1);
        DTAIL(2);
        float tot = 0.f;
#pragma unroll
        for (int i = 0; i < kDecWorkerWarps; ++i) tot += rd[i];
        const float inv = rsqrtf(tot / float(H) + tn.eps);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int c = et + j * 640;
          if (c < nch) {
            const __half2* wh = reinterpret_cast<const __half2*>(&wr[j]);
            uint4 pk;
            uint32_t* po = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 w2 = __half22float2(wh[i]);
              po[i] = pack_half2(vals[j][2 * i] * inv * w2.x, vals[j][2 * i + 1] * inv * w2.y);
            }
            reinterpret_cast<uint4*>(tn.xnorm + size_t(row) * H)[c] = pk;
          }
        }
        DTAIL(3);
      }
    }
  }
#ifdef ZSE_DEC_TIMING
  if (tacc != nullptr) tacc[6] = clock64() - t_entry;
#endif
  // the last CTA of the launch moves the running total on (every CTA that reads it has done so by then)
  epi_bar(1);
  if (et == 0) {
    __threadfence();
    const uint32_t t = atomicAdd(tn.state + 2, 1u);
    if (t == uint32_t(n_cta) - 1u) {
      tn.state[pt.slot] += tn.units_total;
      tn.state[2] = 0u;
      __threadfence();
    }
  }
}

template <int NT, int EPI, bool W8>
__global__ void __launch_bounds__(kDecThreads, 1)
gemm_w4_dec_kernel(const __grid_constant__ CUtensorMap tmap_x, const DecArgs a) {
  using Cfg = DecCfg<NT, W8>;
  constexpr int SX = Cfg::kSX, SW = Cfg::kSW;
  constexpr int kChunk = Cfg::kChunk;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* x_ring = smem;                                        // [SX][2][NT*128]
  uint8_t* w_ring = smem + Cfg::kXRing;                          // [2][SW][8704]
  float* stage = reinterpret_cast<float*>(smem + Cfg::kStageOff);   // [NT][128]
  DecBars* bars = reinterpret_cast<DecBars*>(smem + Cfg::kBarsOff);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef ZSE_DEC_TIMING
  long long tacc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const long long t_entry = clock64();
#else
  long long* tacc = nullptr;
#endif
  // The next kernel of the stream may start its own set-up now; this kernel in turn starts before the one ahead of it
  // has finished: set-up, the first ring-full of weights and their dequantisation (constant data) run at once, the
  // activation loads and the epilogue wait for the producer of the activations (pdl_wait below).
  pdl_launch_dependents();
  const int cta = blockIdx.x, n_cta = gridDim.x;
  const int ks = a.k_stages;
  const int g0 = dec_range_begin(a, cta, n_cta);
  const int g1 = dec_range_begin(a, cta + 1, n_cta);
  const int n_steps = g1 - g0;
  const int pair0 = g0 / ks, k_first = g0 - pair0 * ks;
  // the last pair of an odd tile count has one tile: pipeline 1 has nothing to do from `single_from` on
  const int single_from = (a.n_tiles & 1) ? (a.n_pairs - 1) * ks : a.total_steps;
  const int n_real1 = max(0, min(g1, single_from) - g0);        // steps of this CTA in which pipeline 1 has a chunk

  if (threadIdx.x == kDecProducerWarp * 32) {
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
    // the first ring-full of weight chunks is requested before the CTA has even finished its set-up
    int pair = pair0, k = k_first;
    for (int s = 0; s < n_steps && s < SW; ++s) {
      const uint8_t* src = a.w + (size_t(2 * pair) * ks + k) * kChunk;
      mbar_arrive_expect_tx(&bars->w_full[0][s], kChunk);
      bulk_g2s(w_ring + s * kChunk, src, kChunk, &bars->w_full[0][s]);
      if (s < n_real1) {
        mbar_arrive_expect_tx(&bars->w_full[1][s], kChunk);
        bulk_g2s(w_ring + (SW + s) * kChunk, src + size_t(ks) * kChunk, kChunk,
                 &bars->w_full[1][s]);
      }
      if (++k == ks) {
        k = 0;
        ++pair;
      }
    }
    prefetch_tmap(&tmap_x);
  }
  if (warp == 0) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  if (threadIdx.x == 32) {
    // the start-address field counts 16-byte units: a K step of 16 halfs is +2, the second 64-wide K sub-tile of a
    // stage is +kXBytes/16
    const uint64_t desc0 = make_desc_sw128(smem_u32(x_ring));
    for (int st = 0; st < SX; ++st)
      for (int j = 0; j < 8; ++j)
        bars->bdesc[st][j] =
            desc0 + uint64_t(((st * Cfg::kXStage) >> 4) + (j >> 2) * (Cfg::kXBytes >> 4) + (j & 3) * 2);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;
  volatile int* abort_flag = &bars->abort_flag;
  // TMEM columns: accumulator of lane (pipeline p, parity s) at (2p + s) * 64; its operand slot at 256 + (2p + s) * 64
  // (a dequantised 128 x 128 fp16 chunk = 64 columns of 32 bits)

  bool split_ok = false;
  if (warp < 4) {
    // ------------------------------------------------------------------ MMA issuer of lane (p, sub)
    // steps sub, sub + 2, ... of the CTA; waits are polled without the suspend hint (its wake-up is on the critical
    // path); every index is carried along, nothing is divided
    const int p = warp >> 1, sub = warp & 1;
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(kTileN, NT);
      const uint32_t acc = tmem + (2 * p + sub) * 64;
      uint32_t at[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) at[j] = tmem + 256 + (2 * p + sub) * 64 + j * 8;
      const int my_steps = p == 0 ? n_steps : n_real1;
      int k = k_first + sub, item = 0, cur_item = -1, uses = 0;
      while (k >= ks) {
        k -= ks;
        ++item;
      }
      int st = sub % SX;
      uint32_t xph = 0, aph = 0;
      int s = sub;
      for (; s < my_steps; s += 2) {
        DTICK(tx);
        if (!mbar_wait_spin(&bars->x_full[st], xph, abort_flag, a.status, 3, s)) break;
        DACC(0, tx);
        const bool first = item != cur_item;             // this lane's first chunk of a tile pair
        if (first) {
          if (uses > 0 && !mbar_wait_spin(&bars->acc_empty[p][sub], (uses - 1) & 1, abort_flag, a.status, 4, item))
            break;
          cur_item = item;
        }
        DTICK(ta);
        if (!mbar_wait_spin(&bars->a_ready[p][sub], aph, abort_flag, a.status, 5, s)) break;
        DACC(1, ta);
        DTICK(ti);
        aph ^= 1;
        tc_fence_after_sync();
        dec_mma_chunk(acc, at, bars->bdesc[st], idesc, first ? 0u : 1u);
        tc_commit(&bars->slot_free[p][sub]);
        if (k + 2 >= ks || s + 2 >= n_steps) {             // this lane's last chunk of the pair
          tc_commit(&bars->acc_full[p][sub]);
          ++uses;
        }
        DACC(2, ti);
        k += 2;
        while (k >= ks) {
          k -= ks;
          ++item;
        }
        st += 2;
        if (st >= SX) {
          st -= SX;
          xph ^= 1;
        }
      }
      // no second tile in the rest of the range (pipeline 1 only): hand the stages back
      if (!*abort_flag) {
        for (; s < n_steps; s += 2) {
          if (!mbar_wait_spin(&bars->x_full[st], xph, abort_flag, a.status, 3, s)) break;
          mbar_arrive(&bars->x_empty[st]);
          st += 2;
          if (st >= SX) {
            st -= SX;
            xph ^= 1;
          }
        }
      }
#ifdef ZSE_DEC_TIMING
      tacc[3] = clock64() - t_entry;
#endif
    }
  } else if (warp == kDecProducerWarp) {
    // ------------------------------------------------------------------ producer: activations, weights
    if (lane == 0) {
      int x_issued = 0, cnt0 = min(n_steps, SW), cnt1 = min(n_real1, SW);
      int st = 0, wslot = 0, k = k_first;
      uint32_t xph = 1, wph = 0;        // xph flips to 0 when the activation ring wraps for the first time
      int pair_w = pair0, k_w = k_first + cnt0;         // position of weight step s + SW
      while (k_w >= ks) {
        k_w -= ks;
        ++pair_w;
      }
      pdl_wait();                                          // the activations come from the previous kernel
      for (int s = 0; s < n_steps; ++s) {
        if (s >= SX && !mbar_wait(&bars->x_empty[st], xph, abort_flag, a.status, 2, s)) break;
        mbar_arrive_expect_tx(&bars->x_full[st], Cfg::kXStage);
        tma_load_2d(x_ring + st * Cfg::kXStage, &tmap_x, k * kW4StageK, 0, &bars->x_full[st]);
        tma_load_2d(x_ring + st * Cfg::kXStage + Cfg::kXBytes, &tmap_x, k * kW4StageK + 64, 0, &bars->x_full[st]);
        x_issued = s + 1;
        if (++k == ks) k = 0;
        if (++st == SX) {
          st = 0;
          xph ^= 1;
        }
        // weights of step s + SW go into the slots that the chunks of step s leave
        const int sw = s + SW;
        if (sw < n_steps) {
          if (!mbar_wait(&bars->w_empty[0][wslot], wph, abort_flag, a.status, 1, sw)) break;
          const uint8_t* src = a.w + (size_t(2 * pair_w) * ks + k_w) * kChunk;
          mbar_arrive_expect_tx(&bars->w_full[0][wslot], kChunk);
          bulk_g2s(w_ring + wslot * kChunk, src, kChunk, &bars->w_full[0][wslot]);
          ++cnt0;
          if (sw < n_real1) {
            if (!mbar_wait(&bars->w_empty[1][wslot], wph, abort_flag, a.status, 1, sw)) break;
            mbar_arrive_expect_tx(&bars->w_full[1][wslot], kChunk);
            bulk_g2s(w_ring + (SW + wslot) * kChunk, src + size_t(ks) * kChunk, kChunk,
                     &bars->w_full[1][wslot]);
            ++cnt1;
          }
          if (++k_w == ks) {
            k_w = 0;
            ++pair_w;
          }
          if (++wslot == SW) {
            wslot = 0;
            wph ^= 1;
          }
        }
      }
      if (*abort_flag) {                       // every issued copy must land before the CTA may exit
        for (int r = 0; r < 2; ++r) {
          const int cnt = r == 0 ? cnt0 : cnt1;
          for (int it = max(0, cnt - SW); it < cnt; ++it) {
            const uint64_t t0 = globaltimer_ns();
            while (!mbar_try_wait(&bars->w_full[r][it % SW], (it / SW) & 1) && globaltimer_ns() - t0 < kWaitLimitNs) {
            }
          }
        }
        for (int it = max(0, x_issued - SX); it < x_issued; ++it) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&bars->x_full[it % SX], (it / SX) & 1) && globaltimer_ns() - t0 < kWaitLimitNs) {
          }
        }
      }
    }
  } else {
    const int q = warp & 3;
    if (warp < kDecEpiWarp0) {
      // ---------------------------------------------------------------- dequant: chunk -> fp16 -> TMEM slot
      // group = lane (pipeline p, parity sub): chunks sub, sub+2, ... of pipeline p.  A thread owns one weight row of
      // the chunk: 128 nibbles in, 64 half2 out, written as two 32-column TMEM stores.  Chunk c of a pipeline belongs
      // to step c of the CTA (pipeline 1 only runs out earlier when the last pair has a single tile).
      const int grp = (warp - kDecDqWarp0) >> 2, p = grp >> 1, sub = grp & 1;
      const int row = q * 32 + lane;
      const int n_chunks = p == 0 ? n_steps : n_real1;
      const uint32_t dst = tmem + (uint32_t(q * 32) << 16) + 256 + (2 * p + sub) * 64;
      int last = -1;
      int slot = sub % SW, xst = sub % SX;       // weight-ring slot of chunk c; activation stage of chunk c - 2
      uint32_t wph = 0, sph = 0;                 // parities: w_full of chunk c, slot_free of chunk c - 2
      for (int c = sub; c < n_chunks; c += 2) {
        DTICK(t0);
        if (!mbar_wait(&bars->w_full[p][slot], wph, abort_flag, a.status, 6, c)) break;
        DACC(0, t0);
#ifdef ZSE_DEC_TIMING
        if (c == sub) tacc[6] = clock64() - t_entry;
#endif
        DTICK(t1);
        const uint8_t* chunk = w_ring + (p * SW + slot) * kChunk;
        uint32_t o[32];
        if constexpr (!W8) {
          uint4 pk[4];
#pragma unroll
          for (int p4 = 0; p4 < 4; ++p4) pk[p4] = *reinterpret_cast<const uint4*>(chunk + (p4 * 128 + row) * 16);
          const __half2 sz = *reinterpret_cast<const __half2*>(chunk + 8192 + row * 4);
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->w_empty[p][slot]); // the chunk is in registers: its slot may be refilled
          const __half2 s2 = __half2half2(__low2half(sz)), z2 = __half2half2(__high2half(sz));
          // the first half is dequantised while the MMAs that still read this TMEM slot (chunk c-2) run
          dec_dequant_half(pk[0], pk[1], s2, z2, o);
          DACC(1, t1);
          DTICK(t2);
          if (c >= 2) {
            if (!mbar_wait(&bars->slot_free[p][sub], sph, abort_flag, a.status, 7, c)) break;
            sph ^= 1;
            // the MMAs of chunk c-2 are complete: its activation stage has one reader less
            if (q == 0 && lane == 0) mbar_arrive(&bars->x_empty[xst]);
            xst += 2;
            if (xst >= SX) xst -= SX;
          }
          DACC(2, t2);
          DTICK(t3);
          tc_fence_after_sync();
          ZSE_TMEM_ST_X32(dst, o);
          dec_dequant_half(pk[2], pk[3], s2, z2, o);
          ZSE_TMEM_ST_X32(dst + 32, o);
          DACC(3, t3);
        } else {
          // INT8: a row is 128 bytes in eight 16-byte parts; K 0..63 first, the rest after the first TMEM store
          uint4 pk[4];
#pragma unroll
          for (int p4 = 0; p4 < 4; ++p4) pk[p4] = *reinterpret_cast<const uint4*>(chunk + (p4 * 128 + row) * 16);
          const __half2 s2 = __half2half2(*reinterpret_cast<const __half*>(chunk + 16384 + row * 2));
#pragma unroll
          for (int p4 = 0; p4 < 4; ++p4) dec_dequant_w8_part(pk[p4], s2, o + p4 * 8);
          DACC(1, t1);
          DTICK(t2);
          if (c >= 2) {
            if (!mbar_wait(&bars->slot_free[p][sub], sph, abort_flag, a.status, 7, c)) break;
            sph ^= 1;
            if (q == 0 && lane == 0) mbar_arrive(&bars->x_empty[xst]);
            xst += 2;
            if (xst >= SX) xst -= SX;
          }
          DACC(2, t2);
          DTICK(t3);
          tc_fence_after_sync();
          ZSE_TMEM_ST_X32(dst, o);
#pragma unroll
          for (int p4 = 0; p4 < 4; ++p4) pk[p4] = *reinterpret_cast<const uint4*>(chunk + ((4 + p4) * 128 + row) * 16);
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->w_empty[p][slot]); // the chunk is in registers: its slot may be refilled
#pragma unroll
          for (int p4 = 0; p4 < 4; ++p4) dec_dequant_w8_part(pk[p4], s2, o + p4 * 8);
          ZSE_TMEM_ST_X32(dst + 32, o);
          DACC(3, t3);
        }
        DTICK(t4);
        tc_wait_st();
        tc_fence_before_sync();
        if (lane == 0) mbar_arrive(&bars->a_ready[p][sub]);
        DACC(4, t4);
        last = c;
        slot += 2;
        if (slot >= SW) {
          slot -= SW;
          wph ^= 1;
        }
      }
      // hand back the stage of this group's last chunk as well (the producer may still need it when the other
      // pipeline goes on alone)
      if (last >= 0 && !*abort_flag) {
        if (mbar_wait(&bars->slot_free[p][sub], sph, abort_flag, a.status, 8, last)) {
          if (q == 0 && lane == 0) mbar_arrive(&bars->x_empty[xst]);
        }
      }
    }
    // ------------------------------------------------------------------ epilogue
    pdl_wait();                     // outputs, workspace and flags may still be in use by the previous kernel
    const bool is_epi = warp >= kDecEpiWarp0;
    const int wi_wide = is_epi ? 4 : (warp - kDecDqWarp0) >> 2;  // index among the five warps of this lane quarter
#ifdef ZSE_DEC_TIMING
    long long tdummy[8];
    long long* tepi = is_epi ? tacc : tdummy;
#else
    long long* tepi = nullptr;
#endif
    if (a.split > 0) {
      // split plan: one tile pair, cut into S segments that form a thread-block cluster (continued below, where all
      // threads of the CTA meet at the cluster barriers)
      bool alive = !*abort_flag;
      const int ntp = g0 < single_from ? 2 : 1;
      for (int r = 0; r < ntp && alive; ++r) {
        alive = mbar_wait(&bars->acc_full[r][0], 0, abort_flag, a.status, 9, r);
        if (alive && n_steps > 1) alive = mbar_wait(&bars->acc_full[r][1], 0, abort_flag, a.status, 9, 2 + r);
      }
      split_ok = epi_all(alive, 1);
      tc_fence_after_sync();
#ifdef ZSE_DEC_TIMING
      tacc[0] = clock64() - t_entry;
#endif
    } else {
      // stream plan: the four epilogue warps take the tile pairs one after the other.  The lanes of the next pair run
      // on as soon as the accumulators are out of TMEM.  The CTA's last pair is shared by all twenty worker warps:
      // nothing is left to overlap it with, and the idle activation ring serves as the second staging buffer.
      const uint32_t epoch1 = ld_acquire_gpu_u32(a.sync) + 1u;
      int s = 0, pair = pair0, ka = k_first;
      uint32_t use0 = 0, use1 = 0;                          // tile pairs the even / odd lanes took part in so far
      bool ok = true;
      while (s < n_steps) {
        const int len = min(ks - ka, n_steps - s);
        const int ntp = g0 + s < single_from ? 2 : 1;
        const bool last_item = s + len == n_steps;
        const bool lane0 = len >= 2 || (s & 1) == 0, lane1 = len >= 2 || (s & 1) == 1;
        // all twenty warps call the last item (it begins with a vote of all of them), also after a failure
        if (last_item)
          ok = dec_epilogue_item<NT, EPI>(a, bars, stage, reinterpret_cast<float*>(x_ring), tmem, cta, n_cta, pair, ka,
                                          len, ntp, lane0, lane1, use0 & 1, use1 & 1, false, epoch1, q, lane, wi_wide, 5,
                                          ok, tepi);
        else if (is_epi && ok)
          ok = dec_epilogue_item<NT, EPI>(a, bars, stage, stage, tmem, cta, n_cta, pair, ka, len, ntp, lane0, lane1,
                                          use0 & 1, use1 & 1, true, epoch1, q, lane, 0, 1, ok, tepi);
        use0 += lane0 ? 1 : 0;
        use1 += lane1 ? 1 : 0;
        s += len;
        ka = 0;
        ++pair;
      }
    }
  }
  __syncwarp();
  if (a.split > 0) {
    // every thread of every CTA of the cluster passes both barriers, whatever happened before.  First barrier: this
    // CTA's MMAs are complete and its TMA copies have landed, i.e. its rings may be written by the peers.
    const int S = a.split, seg = int(dec_cluster_rank()), ntp = g0 < single_from ? 2 : 1;
    const int go_max = (Cfg::kGranules + S - 1) / S;
    float* recv = reinterpret_cast<float*>(x_ring);      // [S][2][go_max][8][128] fp32 over the idle rings
    const int wi = warp >= kDecEpiWarp0 ? 4 : (warp - kDecDqWarp0) >> 2;
    cluster_sync_all_threads();
#ifdef ZSE_DEC_TIMING
    if (warp >= kDecEpiWarp0) tacc[1] = clock64() - t_entry;
#endif
    if (warp >= kDecDqWarp0 && split_ok)
      dec_split_push<NT>(recv, tmem, ntp, true, n_steps > 1, seg, S, go_max, warp & 3, lane, wi);
    __syncwarp();
#ifdef ZSE_DEC_TIMING
    if (warp >= kDecEpiWarp0) tacc[2] = clock64() - t_entry;
#endif
    cluster_sync_all_threads();
#ifdef ZSE_DEC_TIMING
    if (warp >= kDecEpiWarp0) tacc[3] = clock64() - t_entry;
#endif
    if (warp >= kDecDqWarp0 && split_ok)
      dec_split_finish<NT, EPI>(a, recv, pair0, ntp, seg, S, go_max, wi * 128 + (warp & 3) * 32 + lane);
#ifdef ZSE_DEC_TIMING
    if (warp >= kDecEpiWarp0) tacc[4] = clock64() - t_entry;
#endif
    if (EPI == kDecAllReduceNorm && warp >= kDecDqWarp0) {
      constexpr int G = Cfg::kGranules;
      const uint32_t units = seg < G ? uint32_t(ntp * ((G - seg + S - 1) / S)) : 0u;
      // the staging buffer of the stream plan is idle in the split plan: scratch for the block reduction
#ifdef ZSE_DEC_TIMING
      dec_allreduce_norm_tail(a, bars, stage, cta, n_cta, units, split_ok, wi * 128 + (warp & 3) * 32 + lane,
                              warp >= kDecEpiWarp0 ? tacc : nullptr, t_entry);
#else
      dec_allreduce_norm_tail(a, bars, stage, cta, n_cta, units, split_ok, wi * 128 + (warp & 3) * 32 + lane);
#endif
    }
  }

  // ---------------------------------------------------------------------- exit
#ifdef ZSE_DEC_TIMING
  if (a.timing != nullptr && lane == 0 && cta == 1) {
    tacc[7] = clock64() - t_entry;
    for (int i = 0; i < 8; ++i) a.timing[warp * 8 + i] = tacc[i];
  }
#endif
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
  if (a.split == 0 && threadIdx.x == kDecEpiWarp0 * 32) {
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
static long long* g_dec_timing = nullptr;
static int g_dec_min_steps = 4;
static int g_dec_max_split = 8;

// Clusters of S CTAs of this kernel (one CTA per SM) that fit on the device at once.  Measured on B200 (148 SMs):
// 148, 74, 45, 33, 26, 22, 15, 15 for S = 1..8; the driver is asked once per device, the table is the fallback.
static int dec_max_clusters(int S);

static DecPlan plan_dec(int n_pairs, int k_stages, int sm_count) {
  DecPlan p{1, 0};
  const int total = n_pairs * k_stages;
  if (2 * n_pairs <= sm_count) {
    // split plan: the largest S whose clusters are all resident at once (one wave), at least two steps per segment
    int best = 1;
    for (int S = 2; S <= min(g_dec_max_split, 8); ++S)
      if (S <= max(1, k_stages / 2) && n_pairs <= dec_max_clusters(S) && n_pairs * S <= sm_count) best = S;
    p.split = best;
    p.n_cta = n_pairs * best;
  } else {
    p.split = 0;
    p.n_cta = max(1, min(sm_count, total / g_dec_min_steps));
  }
  return p;
}

template <int NT, int EPI, bool W8>
static int launch_dec(const CUtensorMap& tx, const DecArgs& a, int n_cta, cudaStream_t st) {
  auto kern = gemm_w4_dec_kernel<NT, EPI, W8>;
  constexpr int smem = DecCfg<NT, W8>::kSmemBytes;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return ZSE_ERR_SHAPE;
  if (!attr_done[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return ZSE_ERR_LAUNCH;
    attr_done[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_cta);
  cfg.blockDim = dim3(kDecThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = a.split > 0 ? a.split : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, tx, a) == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

static int dec_max_clusters(int S) {
  static const int kTable[9] = {0, 148, 74, 45, 33, 26, 22, 15, 15};
  static int cached[64][9] = {};
  if (S < 1 || S > 8) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return kTable[S];
  }
  if (cached[dev][S] == 0) {
    auto kern = gemm_w4_dec_kernel<64, kDecF16, false>;
    constexpr int smem = DecCfg<64, false>::kSmemBytes;
    int n = 0;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.gridDim = dim3(S * 8);
    cfg.blockDim = dim3(kDecThreads);
    cfg.dynamicSmemBytes = smem;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = kTable[S];
    }
    cached[dev][S] = n;
  }
  return cached[dev][S];
}

template <int NT, bool W8>
static int launch_dec_epi(int epi, const CUtensorMap& tx, const DecArgs& a, int n_cta, cudaStream_t st) {
  switch (epi) {
    case kDecF16: return launch_dec<NT, kDecF16, W8>(tx, a, n_cta, st);
    case kDecSwiGLU: return launch_dec<NT, kDecSwiGLU, W8>(tx, a, n_cta, st);
    case kDecF32: return launch_dec<NT, kDecF32, W8>(tx, a, n_cta, st);
    case kDecQkvRope: return launch_dec<NT, kDecQkvRope, W8>(tx, a, n_cta, st);
    case kDecAllReduceNorm: return launch_dec<NT, kDecAllReduceNorm, W8>(tx, a, n_cta, st);
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

// Debug hook (only meaningful in builds with ZSE_DEC_TIMING): device buffer of 24 x 8 cycle counters.
extern "C" void zse_gemm_w4_dec_set_timing(void* dev_buffer) { zse::g_dec_timing = reinterpret_cast<long long*>(dev_buffer); }

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
  if (epilogue == kDecAllReduceNorm) return (N % 8) == 0 && N <= 10240 ? 1 : 0;
  return (epilogue == kDecF16 || epilogue == kDecF32) && (N % 8) == 0 ? 1 : 0;
}

static int run_dec(bool w8, const void* w_tiled, const void* x, int x_rows_cap, const void* bias, void* out, int M,
                   int N, int K, int ldo, int epilogue, void* workspace, const DecRope* rope, void* status,
                   void* stream, const DecTpNorm* tpn = nullptr) {
  if (M <= 0) return 0;
  if (!zse_gemm_w4_dec_supported(M, N, K, epilogue) || workspace == nullptr) return ZSE_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(workspace) & 15) ||
      (reinterpret_cast<uintptr_t>(bias) & 15))
    return ZSE_ERR_ALIGN;
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
  a.timing = g_dec_timing;
  if (rope != nullptr) a.rope = *rope;
  if (epilogue == kDecAllReduceNorm) {
    if (tpn == nullptr || p.split <= 0) return ZSE_ERR_SHAPE;      // the exchange is part of the split plan only
    a.tpn = *tpn;
    a.tpn.units_total = uint32_t(n_tiles) * uint32_t(nt / 8);
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (nt) {
    case 16:
      return w8 ? launch_dec_epi<16, true>(epilogue, tx, a, p.n_cta, st)
                : launch_dec_epi<16, false>(epilogue, tx, a, p.n_cta, st);
    case 32:
      return w8 ? launch_dec_epi<32, true>(epilogue, tx, a, p.n_cta, st)
                : launch_dec_epi<32, false>(epilogue, tx, a, p.n_cta, st);
    default:
      return w8 ? launch_dec_epi<64, true>(epilogue, tx, a, p.n_cta, st)
                : launch_dec_epi<64, false>(epilogue, tx, a, p.n_cta, st);
  }
}

// Decode-sized INT4 GEMM (M <= 64).  epilogue: 0 = fp16 store (+bias), 1 = SwiGLU, 2 = fp32 store (one plane).
extern "C" int zse_gemm_w4_dec(const void* w_tiled, const void* x, int x_rows_cap, const void* bias, void* out, int M,
                               int N, int K, int ldo, int epilogue, void* workspace, void* status, void* stream) {
  if (epilogue != kDecF16 && epilogue != kDecSwiGLU && epilogue != kDecF32) return ZSE_ERR_SHAPE;
  return run_dec(false, w_tiled, x, x_rows_cap, bias, out, M, N, K, ldo, epilogue, workspace, nullptr, status, stream);
}

// The same for INT8 weights (symmetric groups of 128, tiled by zse_repack_w8): the weights stay 8 bits wide in memory
// and are expanded in registers on their way to the tensor cores
// (reference: tiled_dequant_matmul_int8, zse-engine/zse_engine/orchestrator/kernels.py:1195-1249).
extern "C" int zse_gemm_w8_dec(const void* w_tiled, const void* x, int x_rows_cap, const void* bias, void* out, int M,
                               int N, int K, int ldo, int epilogue, void* workspace, void* status, void* stream) {
  if (epilogue != kDecF16 && epilogue != kDecSwiGLU && epilogue != kDecF32) return ZSE_ERR_SHAPE;
  return run_dec(true, w_tiled, x, x_rows_cap, bias, out, M, N, K, ldo, epilogue, workspace, nullptr, status, stream);
}

// Fused QKV projection of a decode-sized pass, head_dim 128, full rotary: bias, rotate-half RoPE (cos/sin table
// [max_position][64] of float2) and the K/V rows stored straight into the paged cache
// (kv_layer [blocks][2][nkv][block_size][128], slot = block * block_size + offset, -1 = skip); `qkv_out` [M, ldo]
// receives the rotated q heads (columns 0 .. nh*128).
static int run_qkv_rope(bool int8_weights, const void* w_tiled, const void* x, int x_rows_cap, const void* bias,
                        void* qkv_out, int ldo, int M, int K, int nh, int nkv, void* kv_layer, int block_size,
                        const void* positions_i32, const void* slots_i64, const void* cos_sin_f32x2, int max_position,
                        void* workspace, void* status, void* stream) {
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
  return run_dec(int8_weights, w_tiled, x, x_rows_cap, bias, qkv_out, M, (nh + 2 * nkv) * 128, K, ldo, kDecQkvRope,
                 workspace, &rp, status, stream);
}

// Row-parallel projection + tensor-parallel all-reduce + residual add + RMSNorm in ONE kernel (see DecTpNorm):
//   residual[M, H] += sum over ranks of x W^T;   xnorm = RMSNorm(residual) * norm_w
// `ctx` is a tensor-parallel context with the push buffers set (zse_tp_ctx_set_push); N must be its hidden size and M
// at most its row capacity.  tp = 1 works as well (no peers: the kernel then only fuses projection, residual and
// norm).  `slot` alternates between consecutive calls.  rank_override >= 0 plays another rank (single-GPU tests).
// Replaces ncclAllReduce + residual_add + rmsnorm of the reference
// (zse-engine/zse_engine/orchestrator/model_runner.py:2622-2635,2694-2705).
extern "C" int zse_tp_gemm_dec_allreduce_norm(void* ctx, const void* w_tiled, int int8_weights, const void* x,
                                              int x_rows_cap, int M, int N, int K, int slot, int use_multimem,
                                              int rank_override, void* residual, const void* norm_w, void* xnorm,
                                              float eps, void* workspace, void* status, void* stream) {
  DecTpNorm tn{};
  if (int rc = tp_fill_push_table(ctx, slot, use_multimem != 0, rank_override, &tn.push)) return rc;
  tn.state = tp_push_state(ctx, rank_override);
  if (tn.state == nullptr || residual == nullptr || norm_w == nullptr) return ZSE_ERR_SHAPE;
  if (N != tn.push.H || M > tn.push.m_cap) return ZSE_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(residual) & 15) || (reinterpret_cast<uintptr_t>(norm_w) & 15) ||
      (reinterpret_cast<uintptr_t>(xnorm) & 15))
    return ZSE_ERR_ALIGN;
  tn.residual = reinterpret_cast<float*>(residual);
  tn.norm_w = reinterpret_cast<const __half*>(norm_w);
  tn.xnorm = reinterpret_cast<__half*>(xnorm);
  tn.eps = eps;
  // `out` is not written by this epilogue; the residual pointer stands in for the alignment check
  return run_dec(int8_weights != 0, w_tiled, x, x_rows_cap, nullptr, residual, M, N, K, N, kDecAllReduceNorm, workspace,
                 nullptr, status, stream, &tn);
}

extern "C" int zse_gemm_w4_dec_qkv_rope(const void* w_tiled, const void* x, int x_rows_cap, const void* bias,
                                        void* qkv_out, int ldo, int M, int K, int nh, int nkv, void* kv_layer,
                                        int block_size, const void* positions_i32, const void* slots_i64,
                                        const void* cos_sin_f32x2, int max_position, void* workspace, void* status,
                                        void* stream) {
  return run_qkv_rope(false, w_tiled, x, x_rows_cap, bias, qkv_out, ldo, M, K, nh, nkv, kv_layer, block_size,
                      positions_i32, slots_i64, cos_sin_f32x2, max_position, workspace, status, stream);
}

extern "C" int zse_gemm_w8_dec_qkv_rope(const void* w_tiled, const void* x, int x_rows_cap, const void* bias,
                                        void* qkv_out, int ldo, int M, int K, int nh, int nkv, void* kv_layer,
                                        int block_size, const void* positions_i32, const void* slots_i64,
                                        const void* cos_sin_f32x2, int max_position, void* workspace, void* status,
                                        void* stream) {
  return run_qkv_rope(true, w_tiled, x, x_rows_cap, bias, qkv_out, ldo, M, K, nh, nkv, kv_layer, block_size,
                      positions_i32, slots_i64, cos_sin_f32x2, max_position, workspace, status, stream);
}

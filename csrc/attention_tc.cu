// Chunked-prefill attention on the tcgen05 tensor cores (head_dim 128, fp16, causal over a paged KV cache, GQA).
//
// One CTA owns 128 query rows of one head of one sequence and walks the keys in tiles of 128 tokens:
//   S = Q K^T     tcgen05.mma, both operands in shared memory (K-major, 128-byte swizzle, brought by TMA - the K tile
//                 of a head is made of boxes of 16, 32 or 64 tokens, whatever divides the block size, fetched through
//                 the sequence's block table by a loader warp, one lane per box), S in TMEM
//   softmax       128 threads, thread i owns TMEM lane i = query row i, no cross-thread reduction at all.  Usually one
//                 pass with tcgen05.ld: probabilities against the maximum in use while the new maximum is tracked;
//                 two passes (row maximum, then exp2 and the fp16 probabilities) when some row of the warp outgrew
//                 its reference, and where masking applies (the diagonal tile, tiles with dropped blocks)
//   O += P V      tcgen05.mma with P as the A operand FROM TMEM (written by tcgen05.st over the scores it replaces) and
//                 V from shared memory as an MN-major operand - the cache stores V as [token][head_dim], which is
//                 exactly that layout, so nothing is transposed; O accumulates in TMEM across the tiles
// The running maximum is only moved when a row's maximum grew by more than 2^8 (probabilities then stay below 256,
// well inside fp16), so the rescaling pass over O (tcgen05.ld, multiply, tcgen05.st) is rare after the first tiles.
// TMEM per CTA: 128 columns S / P + 128 columns O; shared memory: Q, one K and one V tile (96 KB); two CTAs share an
// SM, so one CTA's softmax overlaps the other's MMAs.  K is released as soon as S is complete and V as soon as the
// P V product is, so the next tile's loads run under the current tile's softmax.  One tcgen05.commit per event: the
// barrier that tells the softmax warps that S is complete also tells the loader that the K slot is free, and the one
// that frees the V slot tells the epilogue that O is complete.
// Every wait is bounded and reports through the status word; on a failure the CTA frees its TMEM and leaves.  The waits
// of the MMA issuer and the loader poll without the suspend hint: a suspended thread wakes up microseconds after its
// barrier flips, and a tile passes several such hand-overs.
//
// Replaces the reference's flash_attention_prefill kernel (zse-engine/zse_engine/orchestrator/kernels.py:859-957) for
// the shapes it covers; attention.cu::attn_prefill_kernel (mma.sync) keeps the rest (other head sizes, soft-capped
// scores, sliding windows).
#include "api.h"
#include "common.cuh"
#include "gemm_common.cuh"

namespace zse {

constexpr int kTcRows = 128;          // query rows per CTA (UMMA M)
constexpr int kTcKv = 128;            // keys per tile (UMMA N of S, K of P V)
constexpr int kTcHd = 128;
constexpr int kTcThreads = 192;       // warps 0-3 softmax, warp 4 loader, warp 5 MMA issuer
constexpr int kTcTileBytes = kTcKv * kTcHd * 2;                      // 32 KB: [2 halves of 64 columns][128 rows][128 B]
constexpr int kTcSmemBytes = 3 * kTcTileBytes + 1024 + 256;           // Q, K, V + alignment + barriers

struct TcBars {
  uint64_t q_full, k_full, v_full, v_empty, s_full, p_full;
  uint32_t tmem_base;
  int abort_flag;
};

struct TcArgs {
  const int* bt;            // block tables [num_seqs][max_blocks]
  const int* cu_q;          // [num_seqs + 1]
  const int* q_pos0;        // [num_seqs]
  __half* out;
  int ldo, max_blocks, nh, nkv, block_size;
  float scale_log2;
  int box_rows;             // cache rows per K/V load: 16, 32 or 64, the largest that divides the block size
  int packed;               // > 0: chunks of at most 16 rows; the CTA owns ONE kv head and packs the `packed` query
                            // heads that share it as 16-row slots of its 128 rows (keys and values read once per group)
  Status* status;
  long long* timing;        // instrumented builds (ZSE_ATTN_TIMING): clock64() stamps of CTA (0, 0, 0), else unused
};

// Instrumented builds: stamp `slot` of key tile `t` (16 slots per tile, the first 24 tiles of the heaviest CTA).
#ifdef ZSE_ATTN_TIMING
#define ATIME(t, slot)                                                                                   \
  do {                                                                                                   \
    if (a.timing != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (t) < 24)       \
      a.timing[(t) * 16 + (slot)] = clock64();                                                           \
  } while (0)
#else
#define ATIME(t, slot)
#endif

// MN-major operand in shared memory, 128-byte swizzle: rows of the K dimension are 128 bytes (64 MN elements) long,
// groups of eight K rows lie `k8_bytes` apart, the next 64 MN elements `mn64_bytes` apart.
__device__ __forceinline__ uint64_t make_desc_sw128_mn(uint32_t smem_addr, uint32_t mn64_bytes, uint32_t k8_bytes) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr >> 4) & 0x3FFF);
  d |= uint64_t((mn64_bytes >> 4) & 0x3FFF) << 16;     // leading dimension byte offset
  d |= uint64_t((k8_bytes >> 4) & 0x3FFF) << 32;       // stride dimension byte offset
  d |= uint64_t(1) << 46;
  d |= uint64_t(2) << 61;                              // SWIZZLE_128B
  return d;
}


// 64 consecutive 32-bit columns of the thread's TMEM lane in one instruction (the loads of a tile are few and wide:
// a tcgen05.ld + wait::ld round trip costs several hundred cycles whatever its width).
// 2^x on the special-function unit, one instruction (exp2f() adds range handling around it that softmax does not need)
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

#define ZSE_TMEM_LD_X64(r, taddr)                                                                                  \
  asm volatile(                                                                                                    \
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "                                                                    \
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31," \
      "%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61," \
      "%62,%63}, [%64];"                                                                                           \
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),    \
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),       \
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),      \
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]),      \
        "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]),      \
        "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]),      \
        "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]),      \
        "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])                     \
      : "r"(taddr)                                                                                                 \
      : "memory")

__global__ void __launch_bounds__(kTcThreads, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv,
                       const __grid_constant__ CUtensorMap tmap_q16, const TcArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* k_s = smem + kTcTileBytes;
  uint8_t* v_s = smem + 2 * kTcTileBytes;
  TcBars* bars = reinterpret_cast<TcBars*>(smem + 3 * kTcTileBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the last query tile of a chunk sees the most keys: hand the heavy tiles out first, so that the light ones fill
  // the tail of the grid (causal work per tile grows linearly with its index)
  const int qt = int(gridDim.x) - 1 - int(blockIdx.x), head = blockIdx.y, seq = blockIdx.z;
  pdl_launch_dependents();
  const int q_begin = a.cu_q[seq], q_len = a.cu_q[seq + 1] - q_begin;
  if (qt * kTcRows >= q_len) return;                     // before any barrier or TMEM use: the whole CTA leaves
  const int pos0 = a.q_pos0[seq];
  const int G = a.packed;                                // query heads per kv head in packed mode (else 0)
  const int kvh = G > 0 ? head : head / (a.nh / a.nkv);  // packed: blockIdx.y walks the kv heads
  const int last_row = min(q_len, qt * kTcRows + kTcRows) - 1;
  const int kv_len = pos0 + last_row + 1;                // keys visible to the last query row of this CTA
  const int n_tiles = (kv_len + kTcKv - 1) / kTcKv;
  const int* my_bt = a.bt + size_t(seq) * a.max_blocks;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    mbar_init(&bars->k_full, 1);
    mbar_init(&bars->v_full, 1);
    mbar_init(&bars->v_empty, 1);
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->p_full, 128);
    bars->abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(G > 0 ? &tmap_q16 : &tmap_q);
    prefetch_tmap(&tmap_kv);
  }
  // V must never hold a NaN bit pattern where a probability is zero (0 * NaN): clear it once; afterwards it only ever
  // holds cache contents
  for (int i = threadIdx.x; i < kTcTileBytes / 16; i += kTcThreads) reinterpret_cast<uint4*>(v_s)[i] = make_uint4(0, 0, 0, 0);
  fence_proxy_async_smem();
  if (warp == 5) {
    tmem_alloc(&bars->tmem_base, 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;
  const uint32_t tm_s = tmem, tm_p = tmem, tm_o = tmem + 128;
  volatile int* abort_flag = &bars->abort_flag;

  if (warp == 4) {
    // ------------------------------------------------------------------ producer (the whole warp)
    // One thread issuing the 32 loads of a key tile (16 cache rows x 64 columns each) takes ~2.7 k cycles, and looking
    // eight block-table entries up one after the other another ~3.5 k: more than the rest of the tile's chain.  So the
    // warp shares the work: lane 2 g + half looks up group g of the NEXT tile while the current one is in flight, and
    // issues one K and one V load; 16 loads leave in one warp-wide instruction.
    pdl_wait();                                        // q and the cache rows of this chunk come from the previous kernels
    if (lane == 0) {
      if (G > 0) {
        // slot s = rows 16 s .. 16 s + 15 = the chunk's (at most 16) rows of query head kvh * G + s
        mbar_arrive_expect_tx(&bars->q_full, uint32_t(G) * 4096u);
        for (int sl = 0; sl < G; ++sl) {
          const int x = (kvh * G + sl) * kTcHd;
          tma_load_2d(q_s + sl * 2048, &tmap_q16, x, q_begin, &bars->q_full);
          tma_load_2d(q_s + kTcTileBytes / 2 + sl * 2048, &tmap_q16, x + 64, q_begin, &bars->q_full);
        }
      } else {
        mbar_arrive_expect_tx(&bars->q_full, kTcTileBytes);
        const int y = q_begin + qt * kTcRows;
        tma_load_2d(q_s, &tmap_q, head * kTcHd, y, &bars->q_full);
        tma_load_2d(q_s + kTcTileBytes / 2, &tmap_q, head * kTcHd + 64, y, &bars->q_full);
      }
    }
    // a load covers `box_rows` consecutive tokens of one block (64 columns of them): 128 / box_rows groups per tile,
    // two loads per group
    const int br = a.box_rows, n_groups = kTcKv / br;
    const int g = lane >> 1, half = lane & 1;          // lanes past 2 * n_groups issue nothing
    const int v_off = a.nkv * a.block_size;            // rows between the K half and the V half of a block
    const uint32_t box_bytes = uint32_t(br) * 128u;
    // block of group g of tile t (a hole or past the end: -1).  Only the load is issued here; its result is first
    // touched one tile later, so the latency of the table lookup never sits in the chain.
    auto group_block = [&](int t) {
      const int tok = t * kTcKv + g * br;
      return (g < n_groups && t < n_tiles && tok < kv_len) ? my_bt[tok / a.block_size] : -1;
    };
    int pb_next = group_block(0);
    uint32_t ph = 1;                                   // "empty" barriers: the first wait passes
    for (int t = 0; t < n_tiles; ++t) {
      if (lane == 0) ATIME(t, 14);
      const int pb = pb_next;
      const int tok = t * kTcKv + g * br;
      const int row0 = pb >= 0 ? ((pb * 2) * a.nkv + kvh) * a.block_size + tok % a.block_size : -1;
      const bool issue = row0 >= 0;
      const uint32_t n_loads = __popc(__ballot_sync(0xffffffffu, issue));
      pb_next = group_block(t + 1);                    // in flight while this tile's loads are issued
      bool ok = true;
      if (lane == 0) ATIME(t, 15);
      // the K slot is free once Q K^T of the previous tile is complete: the event `s_full` already announces (a second
      // tcgen05.commit for the loader alone was seen ~1 k cycles later than the first)
      if (lane == 0 && t > 0) ok = mbar_wait_spin(&bars->s_full, ph, abort_flag, a.status, 41, t);
      if (!__shfl_sync(0xffffffffu, ok, 0)) break;
      if (lane == 0) {
        ATIME(t, 10);
        mbar_arrive_expect_tx(&bars->k_full, n_loads * box_bytes);
      }
      __syncwarp();
      if (issue) tma_load_2d(k_s + half * (kTcTileBytes / 2) + g * box_bytes, &tmap_kv, half * 64, row0, &bars->k_full);
      __syncwarp();
      if (lane == 0) {
        ATIME(t, 11);
        ok = mbar_wait_spin(&bars->v_empty, ph, abort_flag, a.status, 42, t);
      }
      if (!__shfl_sync(0xffffffffu, ok, 0)) break;
      if (lane == 0) {
        ATIME(t, 12);
        mbar_arrive_expect_tx(&bars->v_full, n_loads * box_bytes);
      }
      __syncwarp();
      if (issue)
        tma_load_2d(v_s + half * (kTcTileBytes / 2) + g * box_bytes, &tmap_kv, half * 64, row0 + v_off, &bars->v_full);
      __syncwarp();
      if (lane == 0) ATIME(t, 13);
      ph ^= 1;
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_f16(kTcRows, kTcKv);
      constexpr uint32_t idesc_pv = make_idesc_f16(kTcRows, kTcHd) | (1u << 16);       // B is MN-major
      const uint64_t q_desc = make_desc_sw128(smem_u32(q_s));
      const uint64_t k_desc = make_desc_sw128(smem_u32(k_s));
      // V [keys][head_dim] as the MN-major B operand: 64 head_dim elements per 128-byte row, eight keys per 1024 bytes,
      // the second half of head_dim 16 KB further on
      const uint32_t mn64 = uint32_t(kTcTileBytes / 2), k8 = 1024u;
      bool ok = mbar_wait_spin(&bars->q_full, 0, abort_flag, a.status, 43, 0);
      uint32_t ph = 0;
      for (int t = 0; t < n_tiles && ok; ++t) {
        if (!mbar_wait_spin(&bars->k_full, ph, abort_flag, a.status, 44, t)) break;
        ATIME(t, 0);
        // the probabilities of the previous tile live in the columns this product overwrites: let P V finish reading
        // them first (v_empty of tile t-1 is committed behind that product)
        if (t > 0 && !mbar_wait_spin(&bars->v_empty, ph ^ 1, abort_flag, a.status, 49, t)) break;
        ATIME(t, 1);
        tc_fence_after_sync();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint64_t adv = uint64_t((j >> 2) * (kTcTileBytes / 2 >> 4) + (j & 3) * 2);
          umma_ss(tm_s, q_desc + adv, k_desc + adv, idesc_qk, j != 0);
        }
        tc_commit(&bars->s_full);                     // S complete (and every earlier MMA, i.e. the previous P V)
        ATIME(t, 2);
        if (!mbar_wait_spin(&bars->v_full, ph, abort_flag, a.status, 45, t)) break;
        ATIME(t, 3);
        if (!mbar_wait_spin(&bars->p_full, ph, abort_flag, a.status, 46, t)) break;
        ATIME(t, 4);
        tc_fence_after_sync();
#pragma unroll
        for (int j = 0; j < 8; ++j) {                 // 16 keys per step: two groups of eight cache rows
          const uint64_t v_desc = make_desc_sw128_mn(smem_u32(v_s) + j * 2048, mn64, k8);
          umma_ts(tm_o, tm_p + j * 8, v_desc, idesc_pv, (t != 0) || (j != 0));
        }
        tc_commit(&bars->v_empty);
        ATIME(t, 5);
        ph ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue: thread = query row
    const int r = warp * 32 + lane;                   // row inside the CTA = TMEM lane
    const int slot = r >> 4;                          // packed mode: which query head of the group
    const int row = G > 0 ? (r & 15) : qt * kTcRows + r;      // row inside the sequence's chunk
    const int out_head = G > 0 ? kvh * G + slot : head;
    const bool row_live = row < q_len && (G == 0 || slot < G);
    const int limit = pos0 + row;                     // last key this row may see
    const uint32_t lane_addr = uint32_t(warp * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    uint32_t ph = 0;
    bool ok = true;
    for (int t = 0; t < n_tiles; ++t) {
      const int k0 = t * kTcKv;
      // which 16-key groups of the tile exist: a block table entry < 0 is a hole (a block the cache has dropped); its
      // keys were not loaded and must not be seen.  Looked up while S is still being computed.
      const int g_tok = k0 + (lane & 7) * 16;         // lanes 0..7 look one group up each
      const uint32_t groups =
          __ballot_sync(0xffffffffu, g_tok < kv_len && my_bt[g_tok / a.block_size] >= 0) & 0xFFu;
      // one verdict per warp: the tcgen05.ld / st below are warp-wide
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->s_full, ph, abort_flag, a.status, 47, t))) { ok = false; break; }
      if (threadIdx.x == 0) ATIME(t, 6);
      tc_fence_after_sync();
      // Most tiles lie entirely below the diagonal and have no holes: every row of the warp sees every key, and the
      // per-element masking (a third of the instructions of this loop) is skipped.
      const bool full = __all_sync(0xffffffffu, groups == 0xFFu && k0 + kTcKv - 1 <= limit);
      // One pass instead of two when the running maximum is likely to hold: probabilities are computed against the
      // maximum in use while the new maximum is tracked; they are kept in registers, and stored only if no row of the
      // warp outgrew its reference by more than 2^8 (else the scores, still intact in TMEM, go through the two passes).
      if (full && __all_sync(0xffffffffu, m_used > -INFINITY)) {
        uint32_t pk[64];
        float s0 = 0.f, s1 = 0.f, x0 = -INFINITY, x1 = -INFINITY;
#pragma unroll
        for (int h = 0; h < 4; ++h) {                  // 32 columns at a time: 64 + 32 live registers
          uint32_t v[32];
          ZSE_TMEM_LD_X16(v, tm_s + lane_addr + h * 32);
          ZSE_TMEM_LD_X16((v + 16), tm_s + lane_addr + h * 32 + 16);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float e0 = fmaf(__uint_as_float(v[2 * i]), a.scale_log2, -m_used);
            const float e1 = fmaf(__uint_as_float(v[2 * i + 1]), a.scale_log2, -m_used);
            x0 = fmaxf(x0, e0);
            x1 = fmaxf(x1, e1);
            const float p0 = ex2_fast(e0), p1 = ex2_fast(e1);
            s0 += p0;
            s1 += p1;
            pk[h * 16 + i] = pack_half2(p0, p1);
          }
        }
        if (!__any_sync(0xffffffffu, fmaxf(x0, x1) > 8.f)) {
          ZSE_TMEM_ST_X32(tm_p + lane_addr, pk);
          ZSE_TMEM_ST_X32(tm_p + lane_addr + 32, (pk + 32));
          l += s0 + s1;
          if (threadIdx.x == 0) ATIME(t, 7);
          tc_wait_st();
          tc_fence_before_sync();
          mbar_arrive(&bars->p_full);
          if (threadIdx.x == 0) ATIME(t, 8);
          ph ^= 1;
          continue;
        }
      }
      // pass 1: row maximum of the visible scores (two loads of 64 columns)
      float mx = -INFINITY;
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        uint32_t v[64];
        ZSE_TMEM_LD_X64(v, tm_s + lane_addr + h * 64);
        tc_wait_ld();
        if (full) {
          float m0 = mx, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;      // four chains instead of one
#pragma unroll
          for (int i = 0; i < 64; i += 4) {
            m0 = fmaxf(m0, __uint_as_float(v[i]));
            m1 = fmaxf(m1, __uint_as_float(v[i + 1]));
            m2 = fmaxf(m2, __uint_as_float(v[i + 2]));
            m3 = fmaxf(m3, __uint_as_float(v[i + 3]));
          }
          mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
        } else {
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const bool seen = ((groups >> (h * 4 + (i >> 4))) & 1u) && (k0 + h * 64 + i <= limit);
            mx = seen ? fmaxf(mx, __uint_as_float(v[i])) : mx;
          }
        }
      }
      mx *= a.scale_log2;                              // scale > 0: the maximum commutes with it
      // move the reference maximum only when some row of the warp needs it (tcgen05.ld/st are warp-wide)
      const bool grow = mx > m_used + 8.f;
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = fmaxf(m_used, mx);
        const float alpha = (m_used == -INFINITY) ? 0.f : ex2_fast(m_used - m_new);
        if (t > 0) {
          // s_full of this tile means every earlier MMA has completed, the previous P V included: O is stable
#pragma unroll 1
          for (int h = 0; h < 2; ++h) {
            uint32_t o[64];
            ZSE_TMEM_LD_X64(o, tm_o + lane_addr + h * 64);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 64; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            ZSE_TMEM_ST_X32(tm_o + lane_addr + h * 64, o);
            ZSE_TMEM_ST_X32(tm_o + lane_addr + h * 64 + 32, (o + 32));
          }
          tc_wait_st();
        }
        l *= alpha;
        m_used = m_new;
      }
      // pass 2: probabilities (fp16) over the scores they replace, and the row sum
      const float m_ref = (m_used == -INFINITY) ? 0.f : m_used;
      float psum = 0.f;
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        uint32_t v[64];
        ZSE_TMEM_LD_X64(v, tm_s + lane_addr + h * 64);
        tc_wait_ld();
        uint32_t pk[32];
        if (full) {
          float s0 = 0.f, s1 = 0.f;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float p0 = ex2_fast(fmaf(__uint_as_float(v[2 * i]), a.scale_log2, -m_ref));
            const float p1 = ex2_fast(fmaf(__uint_as_float(v[2 * i + 1]), a.scale_log2, -m_ref));
            s0 += p0;
            s1 += p1;
            pk[i] = pack_half2(p0, p1);
          }
          psum += s0 + s1;
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            // a hole: no key of its 16-key group is visible
            const int lim_g = ((groups >> (h * 4 + (i >> 3))) & 1u) ? limit : -1;
            const int k = k0 + h * 64 + 2 * i;
            const float p0 = k <= lim_g ? ex2_fast(__uint_as_float(v[2 * i]) * a.scale_log2 - m_ref) : 0.f;
            const float p1 = k + 1 <= lim_g ? ex2_fast(__uint_as_float(v[2 * i + 1]) * a.scale_log2 - m_ref) : 0.f;
            psum += p0 + p1;
            pk[i] = pack_half2(p0, p1);
          }
        }
        // P columns h*32 .. h*32+31 lie under score columns that this pass has already read
        ZSE_TMEM_ST_X32(tm_p + lane_addr + h * 32, pk);
      }
      l += psum;
      if (threadIdx.x == 0) ATIME(t, 9);
      tc_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&bars->p_full);
      if (threadIdx.x == 0) ATIME(t, 8);
      ph ^= 1;
    }
    // ---- epilogue: O / l -> fp16 rows
    // O is complete when P V of the last tile is: the event `v_empty` announces for that tile
    if (ok)
      ok = __all_sync(0xffffffffu,
                      mbar_wait_spin(&bars->v_empty, uint32_t(n_tiles - 1) & 1u, abort_flag, a.status, 48, 0));
    tc_fence_after_sync();
    if (ok) {
      // every lane takes part in the warp-wide tcgen05.ld (rows past the chunk included); only the stores are per row
      const bool live = row_live;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __half* dst = a.out + size_t(q_begin + (live ? row : 0)) * a.ldo + size_t(live ? out_head : 0) * kTcHd;
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        uint32_t o[64];
        ZSE_TMEM_LD_X64(o, tm_o + lane_addr + h * 64);
        tc_wait_ld();
        if (live) {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            uint4 w;
            w.x = pack_half2(__uint_as_float(o[8 * c]) * inv, __uint_as_float(o[8 * c + 1]) * inv);
            w.y = pack_half2(__uint_as_float(o[8 * c + 2]) * inv, __uint_as_float(o[8 * c + 3]) * inv);
            w.z = pack_half2(__uint_as_float(o[8 * c + 4]) * inv, __uint_as_float(o[8 * c + 5]) * inv);
            w.w = pack_half2(__uint_as_float(o[8 * c + 6]) * inv, __uint_as_float(o[8 * c + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + h * 64 + c * 8) = w;
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem, 256);
}

}  // namespace zse

using namespace zse;

// Debug hook (only meaningful in builds with ZSE_ATTN_TIMING): device buffer of 24 x 16 cycle stamps.
static long long* g_attn_tc_timing = nullptr;
extern "C" void zse_attn_prefill_tc_set_timing(void* dev_buffer) {
  g_attn_tc_timing = reinterpret_cast<long long*>(dev_buffer);
}

// out[q_begin + r, head * 128 ...] = softmax(q K^T * scale, causal) V for every sequence's chunk of query rows.
//   q [total_rows, ldq] fp16 (head h at columns h * 128), kv_layer [num_blocks][2][nkv][block_size][128] fp16,
//   block_tables [num_seqs][max_blocks], cu_q [num_seqs + 1], q_pos0 [num_seqs] (position of each chunk's first row).
// head_dim 128 only; block_size a multiple of 16.  Returns ZSE_ERR_SHAPE for anything else (the caller then uses
// zse_attn_prefill).
extern "C" int zse_attn_prefill_tc(const void* q, int ldq, int total_rows, const void* kv_layer, int num_blocks,
                                   const void* block_tables, int max_blocks, const void* cu_q, const void* q_pos0,
                                   void* out, int ldo, int num_seqs, int max_q_len, int nh, int nkv, int hd,
                                   int block_size, float scale, int variant, void* status, void* stream) {
  if (num_seqs <= 0 || max_q_len <= 0) return 0;
  if (hd != kTcHd || nh % nkv || block_size % 16 || ldq % 8 || ldo % 8 || total_rows <= 0 || num_blocks <= 0)
    return ZSE_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(kv_layer) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return ZSE_ERR_ALIGN;
  CUtensorMap tq, tkv, tq16;
  if (int rc = get_tmap(q, uint64_t(total_rows), uint64_t(ldq), uint32_t(kTcRows), &tq)) return rc;
  if (int rc = get_tmap(q, uint64_t(total_rows), uint64_t(ldq), 16u, &tq16)) return rc;
  // chunks of at most 16 rows (speculative verification, short tails): one CTA per kv head serves the whole group of
  // query heads, so keys and values are read once per group instead of once per query head
  const int group = nh / nkv;
  const int packed = (max_q_len <= 16 && group <= 8 && variant != 2) ? group : 0;
  const int box_rows = block_size % 64 == 0 ? 64 : block_size % 32 == 0 ? 32 : 16;
  if (int rc = get_tmap(kv_layer, uint64_t(num_blocks) * 2 * nkv * block_size, uint64_t(kTcHd), uint32_t(box_rows), &tkv))
    return rc;
  static bool attr[kMaxDevices] = {};
  const int dev_slot = current_device_slot();
  if (!attr[dev_slot]) {
    if (cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes) !=
        cudaSuccess)
      return ZSE_ERR_LAUNCH;
    attr[dev_slot] = true;
  }
  TcArgs a{reinterpret_cast<const int*>(block_tables), reinterpret_cast<const int*>(cu_q),
           reinterpret_cast<const int*>(q_pos0), reinterpret_cast<__half*>(out), ldo, max_blocks, nh, nkv, block_size,
           scale * 1.4426950408889634f, box_rows, packed, reinterpret_cast<Status*>(status), g_attn_tc_timing};
  dim3 grid((max_q_len + kTcRows - 1) / kTcRows, packed > 0 ? nkv : nh, num_seqs);
  return launch_pdl(attn_prefill_tc_kernel, grid, dim3(kTcThreads), size_t(kTcSmemBytes),
                    reinterpret_cast<cudaStream_t>(stream), tq, tkv, tq16, a) == cudaSuccess
             ? 0
             : ZSE_ERR_LAUNCH;
}

// Definitions shared by the tensor-core GEMM kernels (gemm.cu: fp16 weights, gemm_w4.cu: INT4 weights).
#pragma once
#include <cuda.h>

#include "api.h"
#include "common.cuh"

namespace zse {

constexpr int kTileN = 128;          // weight rows per CTA (UMMA M)
constexpr int kW4StageK = 128;       // K per pipeline stage of the INT4 kernel (= quantisation group)
constexpr int kW4ChunkBytes = 8704;  // 8192 nibble bytes + 512 bytes of {scale, zero}
constexpr int kGemmThreads = 320;    // fp16 kernel: warp 0 producer, warp 1 MMA issuer, warps 2..9 epilogue

enum Epilogue : int { kEpiF16 = 0, kEpiSwiGLU = 1, kEpiPartialF32 = 2, kEpiPushF16 = 3, kEpiScatterF16 = 4 };

struct GemmArgs {
  const uint8_t* w;        // W4: tiled chunks [n_tiles][k_stages][8704]; F16: unused (tensor map)
  const __half* bias;      // [N] or null (kEpiF16 only)
  void* out;               // fp16 [M, ldo] / fp32 planes [M, ldo] (fp16 kernel: one plane per K split)
  int M, N, K;
  int ldo;                 // output row stride in elements
  int k_stages;            // total K stages
  int stages_per_split;
  Status* status;
};



// fp16 [rows, cols] row-major tensor map: box = 64 columns x box_rows rows, 128-byte swizzle, zero fill out of
// bounds; cached per (pointer, shape, box).  Defined in gemm.cu.
int get_tmap(const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows, CUtensorMap* out);

// Where a row-parallel GEMM sends its partial output tiles when the tensor-parallel exchange is part of the GEMM
// (gemm_w4.cu, kEpiPushF16): rank r's tile goes, as fp16, into slot r of EVERY rank's inbox - one multimem.st through
// the NVSwitch, or one store per peer - and each CTA then adds 1 to the counter `arrive[k][slot][r]` on every rank k.
// The consumer (comm.cu, tp_sum_add_rmsnorm) waits for the counters and adds the tp rows from its own inbox.
constexpr int kPushMaxTp = 8;
struct PushTable {
  __half* inbox[kPushMaxTp];       // inbox[k]: rank k's inbox [2 slots][tp sources][m_cap][H], as mapped here
  uint32_t* arrive[kPushMaxTp];    // arrive[k]: rank k's counters [2 slots][tp sources]
  __half* mc_inbox;                // multicast view of the inbox (null: plain peer stores)
  uint32_t* mc_arrive;             // multicast view of the counters
  int tp, rank, m_cap, H, slot;
};
// Fills `out` from a tensor-parallel context (comm.cu).  rank_override >= 0 plays another rank (single-GPU tests).
int tp_fill_push_table(const void* ctx, int slot, bool multimem, int rank_override, PushTable* out);
// This rank's running totals of the push exchange {expected slot 0, expected slot 1, exit ticket} (comm.cu), or null.
uint32_t* tp_push_state(const void* ctx, int rank_override);

// Sequence-parallel exchange for passes of many rows (prefill).  Token rows are owned in blocks of kSpRowBlock:
// block b = t / 64 belongs to rank b % tp and sits at local row (b / tp) * 64 + t % 64 of the owner's buffers.
//   scatter  - the row-parallel GEMM (gemm_w4.cu, kEpiScatterF16) stores each fp16 partial tile into slot `rank` of the
//              OWNER's inbox only and adds the (tile, 16-token chunk) units it finished to the owner's counter of
//              that (source, row block): (tp-1)/tp of a row per rank crosses NVLink instead of tp-1.
//   reduce   - the owner (comm.cu, tp_sp_sum_norm_gather_kernel) waits for 4 * H/128 units per source and block, adds
//              the tp rows in rank order and its fp32 residual row (the residual stream is sharded by rows during such
//              a pass), normalises, and
//   gather   - stores the fp16 row into `xg` on EVERY rank; the CTA that completes a block publishes the pass epoch
//              in gflag[b] on every rank.  The column-parallel GEMM that consumes `xg` (gemm_w4.cu, activation
//              producer) waits for the flags of the row blocks of its own token tile before its TMA loads: the gather
//              is part of that GEMM's prologue, tile by tile.
// The epoch lives in device memory (state[0], advanced by the last CTA of every reduce launch), so CUDA graphs
// replay the launches unchanged.
constexpr int kSpRowBlock = 64;
struct SpTable {
  __half* inbox[kPushMaxTp];       // inbox[k]: rank k's inbox [2 slots][tp sources][own_cap][H], as mapped here
  uint32_t* arrive[kPushMaxTp];    // arrive[k]: rank k's unit counters [2 slots][tp sources][nblk_cap]
  __half* xg[kPushMaxTp];          // xg[k]: rank k's gathered activations [m_cap][H]
  uint32_t* gflag[kPushMaxTp];     // gflag[k]: rank k's row-block flags [nblk_cap]
  __half* mc_xg;                   // multicast view of xg (null: one store per rank)
  uint32_t* state;                 // this rank's device words {epoch, exit ticket, pad, pad, tickets[nblk_cap]}
  int tp, rank, H, own_cap, nblk_cap, slot;
};
// What the activation producer of a GEMM waits for when its input is a gathered buffer (null flags: nothing).
struct GatherWait {
  const uint32_t* flags;           // this rank's gflag
  const uint32_t* epoch;           // this rank's state[0]
};
int tp_fill_sp_table(const void* ctx, int slot, bool multimem, int rank_override, SpTable* out);

// CUDA-core path for one or two tokens (gemv_w4.cu).  gemv_w4_plan returns the number of K splits (fp32 planes) the
// GEMV would use, or 0 when the tensor-core kernel should run instead.
int gemv_w4_plan(int M, int N, int K, int epilogue, int sm_count, int want_split);
int gemv_w4_launch(const void* w_tiled, const void* x, const void* bias, void* out, int M, int N, int K, int ldo,
                   int epilogue, int ks, cudaStream_t st);

inline int pick_nt(int M) {
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128) return 128;
  return 256;
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

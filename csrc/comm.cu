// Tensor-parallel reductions done inside the consuming kernel, over NVLink peer memory.
//
// tp_reduce_add_rmsnorm - what follows every row-parallel projection (o_proj, down_proj):
//     residual += sum over ranks of (sum of this rank's split-K planes);  out = RMSNorm(residual) * w
//   One CTA per token row.  Phase A sums the local fp32 planes, rounds to fp16 and stores the row into this rank's
//   symmetric buffer, then raises a per-row flag in every peer's flag array with st.release.sys.  Phase B waits
//   (bounded) until the flags of all ranks for this row are up, takes them down again, then either pulls the row from every peer
//   with plain 16-byte loads over NVLink and adds them in rank order, or - when a multicast mapping exists - lets
//   the NVSwitch add them with multimem.ld_reduce.  Residual add and RMSNorm run on the row while it is in
//   registers.  No NCCL call, no separate all-reduce kernel, no grid-wide barrier: row r of one rank only depends on
//   row r of the others.  The reference does ncclAllReduce + residual_add + rmsnorm as three steps on the NULL
//   stream (zse-engine/zse_engine/orchestrator/model_runner.py:2622-2635,2694-2705).
// tp_argmax             - greedy token selection over a vocabulary-sharded lm_head: local arg-max, 8-byte exchange
//                         through the same flag protocol, global arg-max (ties -> lowest token id).
//
// Buffers alternate between two slots so that a fast rank starting call c+2 cannot overwrite what a slow rank still
// reads for call c (a rank can only enter call c+2 after every rank finished its part of call c+1); for the same
// reason a flag taken down in call c is not raised again before call c+2.  Flags carry no epoch, so a launch can be
// replayed from a CUDA graph unchanged.
// Waits give up after kWaitLimitNs and report through the status word; the kernel then finishes normally.
//
// Emulation: with grid.y == tp the launch plays every rank itself (blockIdx.y = rank) on buffers of one GPU; it is
// started cooperatively so that all CTAs are resident.  That is how the protocol is tested on a single GPU.
#include <cooperative_groups.h>

#include <stdlib.h>

#include "api.h"
#include "common.cuh"
#include "gemm_common.cuh"

namespace zse {

constexpr int kMaxTp = 8;
constexpr int kRedThreads = 256;
constexpr int kRedMaxChunks = 4;          // 8-element chunks per thread -> H <= 8192

struct TpTable {
  __half* data[kMaxTp];        // data[r]: rank r's row buffer [2][m_cap][H] as mapped into this process
  uint32_t* flags[kMaxTp];     // flags[r]: rank r's flag words [2][tp][m_cap]
  const __half* mc_data;       // multicast view of the row buffer (null: peer loads)
  int tp;
  int m_cap;
};

struct TpRankArgs {            // per emulated rank (index 0 in a real launch)
  float* residual;
  const float* partials;
  __half* out;
  int rank;
};

struct TpReduceArgs {
  TpRankArgs r[kMaxTp];
  const __half* weight;
  int n_planes, M, H, row0;
  float eps;
  int slot;
  Status* status;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// To be used right after __threadfence_system(): fence + strong store is a release pattern, and it costs ONE
// system-scope fence where fence + st.release would cost two (measured on B200: several microseconds each).
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ uint4 multimem_ld_reduce_f16x8(const void* mc_ptr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_ptr)
               : "memory");
  return v;
}

// Bounded wait until *flag is raised, then takes it down.  Returns false on timeout.
__device__ __forceinline__ bool wait_flag(uint32_t* flag, Status* st, unsigned where, unsigned detail) {
  if (ld_acquire_sys(flag) == 0u) {
    SpinClock clk;
    while (ld_acquire_sys(flag) == 0u) {
      if (clk.expired(0x3F)) {
        report(st, kPeerTimeout, where, detail);
        return false;
      }
    }
  }
  *reinterpret_cast<volatile uint32_t*>(flag) = 0u;
  return true;
}

__device__ __forceinline__ void acc_h8(float* a, const uint4& v) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    a[2 * i] += f.x;
    a[2 * i + 1] += f.y;
  }
}

// Phase A of both reductions: sum of this rank's fp32 split-K planes of one row, rounded to fp16, into the rank's
// symmetric row buffer.
__device__ __forceinline__ void reduce_phase_a(const TpTable& tb, const TpReduceArgs& a, const TpRankArgs& me, int rank,
                                               int row, size_t row_off) {
  const int H = a.H, nch = H / 8;
  const size_t plane = size_t(a.M) * H;
#pragma unroll
  for (int j = 0; j < kRedMaxChunks; ++j) {
    const int c = threadIdx.x + j * kRedThreads;
    if (c < nch) {
      float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      // the first eight planes are loaded together (predicated, unrolled) so that the loads overlap
      float4 px[8], py[8];
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        const float4* src = reinterpret_cast<const float4*>(me.partials + p * plane + size_t(row) * H) + 2 * c;
        px[p] = p < a.n_planes ? __ldcs(src) : make_float4(0, 0, 0, 0);
        py[p] = p < a.n_planes ? __ldcs(src + 1) : make_float4(0, 0, 0, 0);
      }
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        v[0] += px[p].x; v[1] += px[p].y; v[2] += px[p].z; v[3] += px[p].w;
        v[4] += py[p].x; v[5] += py[p].y; v[6] += py[p].z; v[7] += py[p].w;
      }
      for (int p = 8; p < a.n_planes; ++p) {
        const float4* src = reinterpret_cast<const float4*>(me.partials + p * plane + size_t(row) * H) + 2 * c;
        const float4 x = src[0], y = src[1];
        v[0] += x.x; v[1] += x.y; v[2] += x.z; v[3] += x.w;
        v[4] += y.x; v[5] += y.y; v[6] += y.z; v[7] += y.w;
      }
      uint4 pk;
      pk.x = pack_half2(v[0], v[1]);
      pk.y = pack_half2(v[2], v[3]);
      pk.z = pack_half2(v[4], v[5]);
      pk.w = pack_half2(v[6], v[7]);
      reinterpret_cast<uint4*>(tb.data[rank] + row_off)[c] = pk;
    }
  }
}

template <bool kMultimem>
__global__ void __launch_bounds__(kRedThreads)
tp_reduce_add_rmsnorm_kernel(const TpTable tb, const TpReduceArgs a) {
  __shared__ float red[32];
  __shared__ int ok_flag;
  // the next kernel (a GEMM) may set itself up and stream weights while this one waits for its peers
  pdl_launch_dependents();
  pdl_wait();
  const int er = blockIdx.y;                      // emulated rank slot (0 in a real launch)
  const TpRankArgs me = a.r[er];
  const int rank = me.rank;
  const int row = a.row0 + blockIdx.x;
  const int H = a.H, nch = H / 8;
  const size_t slot_off = size_t(a.slot) * tb.m_cap * H;
  const size_t row_off = slot_off + size_t(row) * H;
  if (threadIdx.x == 0) ok_flag = 1;

  // ---- phase A: local planes -> fp16 row in this rank's symmetric buffer ------------------------------------
  reduce_phase_a(tb, a, me, rank, row, row_off);
  __syncthreads();
  if (threadIdx.x < tb.tp) {
    __threadfence_system();
    st_relaxed_sys(tb.flags[threadIdx.x] + (size_t(a.slot) * tb.tp + rank) * tb.m_cap + row, 1u);
  }
  // ---- phase B: wait for every rank's row, reduce, residual add, RMSNorm -------------------------------------
  if (threadIdx.x < tb.tp) {
    if (!wait_flag(tb.flags[rank] + (size_t(a.slot) * tb.tp + threadIdx.x) * tb.m_cap + row, a.status, 31,
                   threadIdx.x))
      ok_flag = 0;
  }
  __syncthreads();
  const bool ok = ok_flag != 0;                   // on timeout the row keeps its old residual; the host sees the status
  float vals[kRedMaxChunks][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kRedMaxChunks; ++j) {
    const int c = threadIdx.x + j * kRedThreads;
    if (c < nch) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (ok) {
        if (kMultimem) {
          acc_h8(acc, multimem_ld_reduce_f16x8(tb.mc_data + row_off + size_t(c) * 8));
        } else {
          uint4 got[kMaxTp];
#pragma unroll
          for (int r = 0; r < kMaxTp; ++r)
            if (r < tb.tp) got[r] = ld_relaxed_sys_v4(tb.data[r] + row_off + size_t(c) * 8);
#pragma unroll
          for (int r = 0; r < kMaxTp; ++r)
            if (r < tb.tp) acc_h8(acc, got[r]);
        }
      }
      float4* res = reinterpret_cast<float4*>(me.residual + size_t(row) * H) + 2 * c;
      float4 x = res[0], y = res[1];
      x.x += acc[0]; x.y += acc[1]; x.z += acc[2]; x.w += acc[3];
      y.x += acc[4]; y.y += acc[5]; y.z += acc[6]; y.w += acc[7];
      res[0] = x;
      res[1] = y;
      vals[j][0] = x.x; vals[j][1] = x.y; vals[j][2] = x.z; vals[j][3] = x.w;
      vals[j][4] = y.x; vals[j][5] = y.y; vals[j][6] = y.z; vals[j][7] = y.w;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += vals[j][i] * vals[j][i];
    }
  }
  if (me.out == nullptr) return;
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = (threadIdx.x & 31) < (kRedThreads >> 5) ? red[threadIdx.x & 31] : 0.f;
  tot = warp_sum(tot);
  const float inv = rsqrtf(tot / float(H) + a.eps);
#pragma unroll
  for (int j = 0; j < kRedMaxChunks; ++j) {
    const int c = threadIdx.x + j * kRedThreads;
    if (c < nch) {
      const uint4 wr = reinterpret_cast<const uint4*>(a.weight)[c];
      const __half2* wh = reinterpret_cast<const __half2*>(&wr);
      uint4 pk;
      uint32_t* po = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 w = __half22float2(wh[i]);
        po[i] = pack_half2(vals[j][2 * i] * inv * w.x, vals[j][2 * i + 1] * inv * w.y);
      }
      reinterpret_cast<uint4*>(me.out + size_t(row) * H)[c] = pk;
    }
  }
}

// ---- two-shot variant for many rows (prefill): reduce-scatter + all-gather inside one kernel -------------------
// Row r belongs to rank r % tp.  Every rank still sums its own planes of every row (phase A) and raises the row's flag,
// but only at the owner.  The owner waits for all ranks, adds their rows (peer loads in rank order, or one
// multimem.ld_reduce), adds its residual row and normalises: the fp32 residual stream is therefore sharded by rows -
// nobody else needs it, because the same owner reduces that row in every layer of the pass.  The normalised fp16 row
// goes to the owner's own output AND back into its symmetric row (whose phase-A content is spent), and a second flag is
// raised at every peer; the other ranks wait for that flag and pull the finished row.  Per row and rank 1 row crosses
// NVLink inwards in the scatter phase (owner: tp-1 rows) and 1 in the gather phase, instead of tp-1 rows for every
// rank in the one-shot kernel: 2 (tp-1)/tp of a row per rank instead of tp-1.
template <bool kMultimem>
__global__ void __launch_bounds__(kRedThreads)
tp_reduce_scatter_add_rmsnorm_kernel(const TpTable tb, const TpReduceArgs a) {
  __shared__ float red[32];
  __shared__ int ok_flag;
  pdl_launch_dependents();
  pdl_wait();
  const int er = blockIdx.y;
  const TpRankArgs me = a.r[er];
  const int rank = me.rank, tp = tb.tp;
  const int row = a.row0 + blockIdx.x;
  const int owner = row % tp;
  const int H = a.H, nch = H / 8;
  const size_t row_off = (size_t(a.slot) * tb.m_cap + size_t(row)) * H;
  if (threadIdx.x == 0) ok_flag = 1;

  reduce_phase_a(tb, a, me, rank, row, row_off);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    st_relaxed_sys(tb.flags[owner] + (size_t(a.slot) * tp + rank) * tb.m_cap + row, 1u);
  }
  if (rank != owner) {
    // ---- gather side: wait for the owner's finished row, copy it
    if (threadIdx.x == 0 &&
        !wait_flag(tb.flags[rank] + (size_t(a.slot) * tp + owner) * tb.m_cap + row, a.status, 33, owner))
      ok_flag = 0;
    __syncthreads();
    if (ok_flag != 0) {
#pragma unroll
      for (int j = 0; j < kRedMaxChunks; ++j) {
        const int c = threadIdx.x + j * kRedThreads;
        if (c < nch)
          reinterpret_cast<uint4*>(me.out + size_t(row) * H)[c] =
              ld_relaxed_sys_v4(tb.data[owner] + row_off + size_t(c) * 8);
      }
    }
    return;
  }
  // ---- owner: wait for every rank's row, reduce, residual add, RMSNorm, publish
  if (threadIdx.x < tp) {
    if (!wait_flag(tb.flags[rank] + (size_t(a.slot) * tp + threadIdx.x) * tb.m_cap + row, a.status, 32, threadIdx.x))
      ok_flag = 0;
  }
  __syncthreads();
  const bool ok = ok_flag != 0;
  float vals[kRedMaxChunks][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kRedMaxChunks; ++j) {
    const int c = threadIdx.x + j * kRedThreads;
    if (c < nch) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (ok) {
        if (kMultimem) {
          acc_h8(acc, multimem_ld_reduce_f16x8(tb.mc_data + row_off + size_t(c) * 8));
        } else {
          uint4 got[kMaxTp];
#pragma unroll
          for (int r = 0; r < kMaxTp; ++r)
            if (r < tp) got[r] = ld_relaxed_sys_v4(tb.data[r] + row_off + size_t(c) * 8);
#pragma unroll
          for (int r = 0; r < kMaxTp; ++r)
            if (r < tp) acc_h8(acc, got[r]);
        }
      }
      float4* res = reinterpret_cast<float4*>(me.residual + size_t(row) * H) + 2 * c;
      float4 x = res[0], y = res[1];
      x.x += acc[0]; x.y += acc[1]; x.z += acc[2]; x.w += acc[3];
      y.x += acc[4]; y.y += acc[5]; y.z += acc[6]; y.w += acc[7];
      res[0] = x;
      res[1] = y;
      vals[j][0] = x.x; vals[j][1] = x.y; vals[j][2] = x.z; vals[j][3] = x.w;
      vals[j][4] = y.x; vals[j][5] = y.y; vals[j][6] = y.z; vals[j][7] = y.w;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += vals[j][i] * vals[j][i];
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();                                  // also: every thread has finished reading the symmetric rows
  float tot = (threadIdx.x & 31) < (kRedThreads >> 5) ? red[threadIdx.x & 31] : 0.f;
  tot = warp_sum(tot);
  const float inv = rsqrtf(tot / float(H) + a.eps);
#pragma unroll
  for (int j = 0; j < kRedMaxChunks; ++j) {
    const int c = threadIdx.x + j * kRedThreads;
    if (c < nch) {
      const uint4 wr = reinterpret_cast<const uint4*>(a.weight)[c];
      const __half2* wh = reinterpret_cast<const __half2*>(&wr);
      uint4 pk;
      uint32_t* po = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 w = __half22float2(wh[i]);
        po[i] = pack_half2(vals[j][2 * i] * inv * w.x, vals[j][2 * i + 1] * inv * w.y);
      }
      reinterpret_cast<uint4*>(me.out + size_t(row) * H)[c] = pk;
      reinterpret_cast<uint4*>(tb.data[rank] + row_off)[c] = pk;       // what the other ranks pull
    }
  }
  __syncthreads();
  if (threadIdx.x < tp && threadIdx.x != rank) {
    __threadfence_system();
    st_relaxed_sys(tb.flags[threadIdx.x] + (size_t(a.slot) * tp + owner) * tb.m_cap + row, 1u);
  }
}

// ---- consumer of the push exchange: the GEMM (gemm_w4.cu, kEpiPushF16) of every rank has written its fp16 partial
// rows into slot `src` of this rank's inbox and counted its CTAs into arrive[slot][src].  This kernel waits until
// every source has delivered `expected_add` more CTAs than before, adds the tp rows in rank order (the same order on
// every rank, so the replicated residual stays bit-identical), adds the residual and normalises.  Nothing is read
// from a peer here: the NVLink transfers happened while the GEMMs were still running.
// The running total the counters must reach lives in device memory (state[slot]) and is advanced by the last CTA of
// the launch, so a CUDA graph can replay the launch unchanged.
struct TpSumArgs {
  TpRankArgs r[kMaxTp];            // per emulated rank: residual, (unused), out, rank
  const __half* inbox[kMaxTp];     // inbox[r]: rank r's own inbox [2][tp][m_cap][H]
  const uint32_t* arrive[kMaxTp];  // arrive[r]: rank r's own counters [2][tp]
  uint32_t* state[kMaxTp];         // state[r]: {expected slot 0, expected slot 1, ticket}
  const __half* weight;
  int tp, m_cap, M, H, slot;
  uint32_t expected_add;
  float eps;
  Status* status;
};

__global__ void __launch_bounds__(kRedThreads)
tp_sum_add_rmsnorm_kernel(const TpSumArgs a) {
  __shared__ float red[32];
  __shared__ int ok_flag;
  pdl_launch_dependents();
  pdl_wait();
  const int er = blockIdx.y;
  const TpRankArgs me = a.r[er];
  const int rank = me.rank, tp = a.tp, row = blockIdx.x;
  const int H = a.H, nch = H / 8;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (threadIdx.x < tp) {
    const uint32_t target = a.state[rank][a.slot] + a.expected_add;
    const uint32_t* ctr = a.arrive[rank] + a.slot * tp + threadIdx.x;
    if (int32_t(ld_acquire_sys(ctr) - target) < 0) {
      SpinClock clk;
      while (int32_t(ld_acquire_sys(ctr) - target) < 0) {
        if (clk.expired(0x3F)) {
          report(a.status, kPeerTimeout, 34, threadIdx.x);
          ok_flag = 0;
          break;
        }
      }
    }
  }
  __syncthreads();
  const bool ok = ok_flag != 0;
  const __half* box = a.inbox[rank] + size_t(a.slot) * tp * a.m_cap * H + size_t(row) * H;
  float vals[kRedMaxChunks][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kRedMaxChunks; ++j) {
    const int c = threadIdx.x + j * kRedThreads;
    if (c < nch) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (ok) {
        uint4 got[kMaxTp];
#pragma unroll
        for (int r = 0; r < kMaxTp; ++r)
          if (r < tp) got[r] = ld_relaxed_sys_v4(box + size_t(r) * a.m_cap * H + size_t(c) * 8);
#pragma unroll
        for (int r = 0; r < kMaxTp; ++r)
          if (r < tp) acc_h8(acc, got[r]);
      }
      float4* res = reinterpret_cast<float4*>(me.residual + size_t(row) * H) + 2 * c;
      float4 x = res[0], y = res[1];
      x.x += acc[0]; x.y += acc[1]; x.z += acc[2]; x.w += acc[3];
      y.x += acc[4]; y.y += acc[5]; y.z += acc[6]; y.w += acc[7];
      res[0] = x;
      res[1] = y;
      vals[j][0] = x.x; vals[j][1] = x.y; vals[j][2] = x.z; vals[j][3] = x.w;
      vals[j][4] = y.x; vals[j][5] = y.y; vals[j][6] = y.z; vals[j][7] = y.w;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += vals[j][i] * vals[j][i];
    }
  }
  if (me.out != nullptr) {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = (threadIdx.x & 31) < (kRedThreads >> 5) ? red[threadIdx.x & 31] : 0.f;
    tot = warp_sum(tot);
    const float inv = rsqrtf(tot / float(H) + a.eps);
#pragma unroll
    for (int j = 0; j < kRedMaxChunks; ++j) {
      const int c = threadIdx.x + j * kRedThreads;
      if (c < nch) {
        const uint4 wr = reinterpret_cast<const uint4*>(a.weight)[c];
        const __half2* wh = reinterpret_cast<const __half2*>(&wr);
        uint4 pk;
        uint32_t* po = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 w = __half22float2(wh[i]);
          po[i] = pack_half2(vals[j][2 * i] * inv * w.x, vals[j][2 * i + 1] * inv * w.y);
        }
        reinterpret_cast<uint4*>(me.out + size_t(row) * H)[c] = pk;
      }
    }
  }
  // the last CTA of this rank's launch moves the running total on (every CTA has read it by then)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t t = atomicAdd(a.state[rank] + 2, 1u);
    if (t == gridDim.x - 1) {
      a.state[rank][a.slot] += a.expected_add;
      a.state[rank][2] = 0u;
      __threadfence();
    }
  }
}

// ---- greedy selection over a vocabulary-sharded lm_head --------------------------------------------------
struct TpArgmaxArgs {
  const __half* logits[kMaxTp];   // per emulated rank: [M, ld] local logits
  int* out[kMaxTp];
  int rank[kMaxTp];
  unsigned long long* xchg[kMaxTp];   // xchg[r]: rank r's exchange words [2][tp][m_cap] as mapped here
  uint32_t* flags[kMaxTp];
  int ld, V_local, vocab_stride;      // global token id = rank * vocab_stride + local index
  int tp, m_cap;
  int slot;
  Status* status;
};

__device__ __forceinline__ uint32_t f16_key(__half h) {
  const uint32_t b = __half_as_ushort(h);
  return (b & 0x8000u) ? (~b & 0xFFFFu) : (b | 0x8000u);
}

__global__ void __launch_bounds__(1024) tp_argmax_kernel(const TpArgmaxArgs a) {
  __shared__ unsigned long long red[32];
  __shared__ int ok_flag;
  const int er = blockIdx.y, rank = a.rank[er], row = blockIdx.x;
  const __half* lrow = a.logits[er] + size_t(row) * a.ld;
  if (threadIdx.x == 0) ok_flag = 1;
  unsigned long long best = 0ull;
  for (int i = threadIdx.x; i < a.V_local; i += blockDim.x) {
    const unsigned gid = unsigned(rank) * unsigned(a.vocab_stride) + unsigned(i);
    const unsigned long long cand = ((unsigned long long)f16_key(lrow[i]) << 32) | (0xFFFFFFFFu - gid);
    best = cand > best ? cand : best;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x < 32) {
    unsigned long long t = red[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, t, o);
      t = other > t ? other : t;
    }
    best = t;
  }
  const size_t base = size_t(a.slot) * a.tp * a.m_cap;
  if (threadIdx.x < a.tp) {
    // push my candidate into peer threadIdx.x's exchange area, then raise the flag there
    const size_t idx = base + size_t(rank) * a.m_cap + row;
    a.xchg[threadIdx.x][idx] = __shfl_sync((1u << a.tp) - 1u, best, 0);
    __threadfence_system();
    st_relaxed_sys(a.flags[threadIdx.x] + idx, 1u);
    if (!wait_flag(a.flags[rank] + base + size_t(threadIdx.x) * a.m_cap + row, a.status, 41, threadIdx.x))
      ok_flag = 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long g = 0ull;
    if (ok_flag) {
      for (int r = 0; r < a.tp; ++r) {
        const unsigned long long c = *reinterpret_cast<volatile unsigned long long*>(
            a.xchg[rank] + base + size_t(r) * a.m_cap + row);
        g = c > g ? c : g;
      }
    } else {
      g = best;
    }
    a.out[er][row] = int(0xFFFFFFFFu - unsigned(g & 0xFFFFFFFFull));
  }
}


// ---- all-gather of vocabulary-sharded logits (sampling with temperature under tensor parallelism) ---------------
// One CTA per logits row: it stores this rank's shard [W] of the row into columns rank * W .. of EVERY rank's gathered
// buffer (16-byte peer stores), raises the row's flag for this source on every rank, then waits (bounded) until all tp
// sources have raised theirs here and takes the flags down - when the launch is over, this rank holds the full rows.
// Two slots alternate between calls, as in the other exchanges.  Replaces ncclAllGather + concatenation of the
// reference-style path (NcclComm.gather_logits); shards must be equally wide with W a multiple of 8.
struct TpGatherArgs {
  const __half* src[kMaxTp];       // per emulated rank: local logits [M, ld]
  int rank[kMaxTp];
  __half* buf[kMaxTp];             // buf[k]: rank k's gathered rows [2][rows_cap][tp * W] as mapped here
  uint32_t* flags[kMaxTp];         // flags[k]: rank k's flags [2][tp][rows_cap]
  int ld, W, tp, rows_cap, slot;
  Status* status;
};

__global__ void __launch_bounds__(512) tp_gather_rows_kernel(const TpGatherArgs a) {
  __shared__ int ok_flag;
  const int er = blockIdx.y, rank = a.rank[er], row = blockIdx.x;
  if (threadIdx.x == 0) ok_flag = 1;
  const uint4* src = reinterpret_cast<const uint4*>(a.src[er] + size_t(row) * a.ld);
  const size_t row_off = (size_t(a.slot) * a.rows_cap + row) * (size_t(a.tp) * a.W) + size_t(rank) * a.W;
  for (int c = threadIdx.x; c < a.W / 8; c += blockDim.x) {
    const uint4 v = src[c];
#pragma unroll
    for (int k = 0; k < kMaxTp; ++k)
      if (k < a.tp) reinterpret_cast<uint4*>(a.buf[k] + row_off)[c] = v;
  }
  __syncthreads();
  const size_t base = size_t(a.slot) * a.tp * a.rows_cap;
  if (threadIdx.x < a.tp) {
    __threadfence_system();
    st_relaxed_sys(a.flags[threadIdx.x] + base + size_t(rank) * a.rows_cap + row, 1u);
    if (!wait_flag(a.flags[rank] + base + size_t(threadIdx.x) * a.rows_cap + row, a.status, 39, threadIdx.x))
      ok_flag = 0;
  }
  __syncthreads();
}

// ---- sequence-parallel exchange for passes of many rows: the reduce + all-gather half (see SpTable) -------------
// One CTA per token row; rows this rank does not own leave at once.  The owner waits (bounded) until every source's
// counter for the row's 64-row block holds `units`, adds the tp fp16 rows of its inbox in rank order, adds its fp32
// residual row, normalises and stores the fp16 row into the gathered buffer of EVERY rank.  The CTA that finishes a
// block last takes the block's counters down and publishes the pass epoch in the block's flag on every rank - the
// GEMM that consumes the gathered rows (gemm_w4.cu, gather_wait_tile) and tp_sp_wait_kernel wait for exactly that.
// The last CTA of the launch stores the epoch into state[0]; consumers launched after this kernel read it there.
struct TpSpArgs {
  SpTable sp;                      // sp.rank / sp.state are per emulated rank below
  float* residual[kMaxTp];
  uint32_t* state[kMaxTp];
  int rank[kMaxTp];
  const __half* weight;
  int M;
  float eps;
  uint32_t units;
  Status* status;
};

__device__ __forceinline__ void multimem_st_f16x8(void* mc_ptr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f16x2 [%0], {%1,%2,%3,%4};" ::"l"(mc_ptr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

__global__ void __launch_bounds__(kRedThreads)
tp_sp_sum_norm_gather_kernel(const TpSpArgs a) {
  __shared__ float red[32];
  __shared__ int ok_flag;
  const SpTable& sp = a.sp;
  const int er = blockIdx.y;
  const int rank = a.rank[er], tp = sp.tp, H = sp.H, nch = H / 8;
  uint32_t* st = a.state[er];
  const int row = blockIdx.x;
  const int b = row / kSpRowBlock;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(st) + 1u;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (b % tp == rank) {
    const int local = (b / tp) * kSpRowBlock + (row % kSpRowBlock);
    if (threadIdx.x < tp) {
      const uint32_t* ctr = sp.arrive[rank] + (size_t(sp.slot) * tp + threadIdx.x) * sp.nblk_cap + b;
      if (int32_t(ld_acquire_sys(ctr) - a.units) < 0) {
        SpinClock clk;
        while (int32_t(ld_acquire_sys(ctr) - a.units) < 0) {
          if (clk.expired(0x3F)) {
            report(a.status, kPeerTimeout, 37, threadIdx.x);
            ok_flag = 0;
            break;
          }
        }
      }
    }
    __syncthreads();
    const bool ok = ok_flag != 0;
    const __half* box = sp.inbox[rank] + (size_t(sp.slot) * tp * sp.own_cap + local) * H;
    float vals[kRedMaxChunks][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < kRedMaxChunks; ++j) {
      const int c = threadIdx.x + j * kRedThreads;
      if (c < nch) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (ok) {
          uint4 got[kMaxTp];
#pragma unroll
          for (int r = 0; r < kMaxTp; ++r)
            if (r < tp) got[r] = ld_relaxed_sys_v4(box + size_t(r) * sp.own_cap * H + size_t(c) * 8);
#pragma unroll
          for (int r = 0; r < kMaxTp; ++r)
            if (r < tp) acc_h8(acc, got[r]);
        }
        float4* res = reinterpret_cast<float4*>(a.residual[er] + size_t(row) * H) + 2 * c;
        float4 x = res[0], y = res[1];
        x.x += acc[0]; x.y += acc[1]; x.z += acc[2]; x.w += acc[3];
        y.x += acc[4]; y.y += acc[5]; y.z += acc[6]; y.w += acc[7];
        res[0] = x;
        res[1] = y;
        vals[j][0] = x.x; vals[j][1] = x.y; vals[j][2] = x.z; vals[j][3] = x.w;
        vals[j][4] = y.x; vals[j][5] = y.y; vals[j][6] = y.z; vals[j][7] = y.w;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += vals[j][i] * vals[j][i];
      }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = (threadIdx.x & 31) < (kRedThreads >> 5) ? red[threadIdx.x & 31] : 0.f;
    tot = warp_sum(tot);
    const float inv = rsqrtf(tot / float(H) + a.eps);
#pragma unroll
    for (int j = 0; j < kRedMaxChunks; ++j) {
      const int c = threadIdx.x + j * kRedThreads;
      if (c < nch) {
        const uint4 wr = reinterpret_cast<const uint4*>(a.weight)[c];
        const __half2* wh = reinterpret_cast<const __half2*>(&wr);
        uint4 pk;
        uint32_t* po = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 w = __half22float2(wh[i]);
          po[i] = pack_half2(vals[j][2 * i] * inv * w.x, vals[j][2 * i + 1] * inv * w.y);
        }
        const size_t off = size_t(row) * H + size_t(c) * 8;
        if (sp.mc_xg != nullptr) {
          multimem_st_f16x8(sp.mc_xg + off, pk);
        } else {
#pragma unroll
          for (int k = 0; k < kMaxTp; ++k)
            if (k < tp) *reinterpret_cast<uint4*>(sp.xg[k] + off) = pk;
        }
      }
    }
    __syncthreads();                                 // every store of the row has been issued
    if (threadIdx.x == 0) {
      __threadfence_system();
      const int rows_in_block = min(kSpRowBlock, a.M - b * kSpRowBlock);
      const uint32_t tk = atomicAdd(st + 4 + b, 1u);
      if (tk == uint32_t(rows_in_block) - 1u) {
        // every row of the block has been stored (their fences precede their tickets): take the counters down for
        // the call after next, then tell every rank that the block is complete
        st[4 + b] = 0u;
        for (int r = 0; r < tp; ++r)
          *reinterpret_cast<volatile uint32_t*>(sp.arrive[rank] + (size_t(sp.slot) * tp + r) * sp.nblk_cap + b) = 0u;
        __threadfence_system();
        for (int k = 0; k < tp; ++k) st_relaxed_sys(sp.gflag[k] + b, epoch);
      }
    }
  }
  // the last CTA of the launch moves the epoch on (every CTA has read it by then)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t t = atomicAdd(st + 1, 1u);
    if (t == gridDim.x - 1u) {
      st[1] = 0u;
      *reinterpret_cast<volatile uint32_t*>(st) = epoch;
      __threadfence();
    }
  }
}

// Waits (bounded) until every row block of a pass of M rows has been gathered on this rank: for readers of the
// gathered buffer that are not GEMMs of this library (row selection before the lm_head, adapters).
__global__ void __launch_bounds__(kRedThreads)
tp_sp_wait_kernel(const uint32_t* flags, const uint32_t* epoch_word, int n_blocks, Status* status) {
  const uint32_t want = *reinterpret_cast<const volatile uint32_t*>(epoch_word);
  for (int b = threadIdx.x; b < n_blocks; b += kRedThreads) {
    if (ld_acquire_sys(flags + b) == want) continue;
    SpinClock clk;
    while (ld_acquire_sys(flags + b) != want) {
      if (clk.expired(0x3F)) {
        report(status, kPeerTimeout, 38, b);
        break;
      }
    }
  }
}

}  // namespace zse

using namespace zse;

// Host-side description of one tensor-parallel group member (filled by the Python side after the rendezvous).
struct zse_tp_ctx {
  TpTable table;
  unsigned long long* xchg[kMaxTp];
  uint32_t* xflags[kMaxTp];
  int rank;
  int H;
  // push exchange (GEMM epilogue -> inboxes): set by zse_tp_ctx_set_push
  __half* inbox[kMaxTp] = {};
  uint32_t* arrive[kMaxTp] = {};
  uint32_t* state[kMaxTp] = {};      // state[r]: rank r's local words {expected slot 0, expected slot 1, ticket, -}
  __half* mc_inbox = nullptr;
  uint32_t* mc_arrive = nullptr;
  int push_m_cap = 0;                // rows per source in the inbox
  // sequence-parallel exchange (set by zse_tp_ctx_set_sp)
  __half* sp_inbox[kMaxTp] = {};
  uint32_t* sp_arrive[kMaxTp] = {};
  __half* sp_xg[kMaxTp] = {};
  uint32_t* sp_gflag[kMaxTp] = {};
  uint32_t* sp_state[kMaxTp] = {};   // sp_state[r]: rank r's local words {epoch, exit ticket, -, -, tickets[nblk_cap]}
  __half* mc_xg = nullptr;
  int sp_own_cap = 0, sp_nblk_cap = 0;
  // logits all-gather (set by zse_tp_ctx_set_gather)
  __half* g_buf[kMaxTp] = {};
  uint32_t* g_flags[kMaxTp] = {};
  int g_rows_cap = 0, g_width = 0;
};

extern "C" void* zse_tp_ctx_create(int tp, int rank, int m_cap, int H, const uint64_t* data_ptrs,
                                   const uint64_t* flag_ptrs, uint64_t mc_data, const uint64_t* xchg_ptrs,
                                   const uint64_t* xflag_ptrs) {
  if (tp < 1 || tp > kMaxTp) return nullptr;
  zse_tp_ctx* c = new zse_tp_ctx();
  c->table.tp = tp;
  c->table.m_cap = m_cap;
  c->table.mc_data = reinterpret_cast<const __half*>(mc_data);
  for (int r = 0; r < tp; ++r) {
    c->table.data[r] = reinterpret_cast<__half*>(data_ptrs[r]);
    c->table.flags[r] = reinterpret_cast<uint32_t*>(flag_ptrs[r]);
    c->xchg[r] = reinterpret_cast<unsigned long long*>(xchg_ptrs[r]);
    c->xflags[r] = reinterpret_cast<uint32_t*>(xflag_ptrs[r]);
  }
  c->rank = rank;
  c->H = H;
  return c;
}

extern "C" void zse_tp_ctx_destroy(void* ctx) { delete reinterpret_cast<zse_tp_ctx*>(ctx); }

extern "C" int zse_tp_ctx_set_push(void* ctx, int push_m_cap, const uint64_t* inbox_ptrs, uint64_t mc_inbox,
                                   const uint64_t* arrive_ptrs, uint64_t mc_arrive, const uint64_t* state_ptrs) {
  zse_tp_ctx* c = reinterpret_cast<zse_tp_ctx*>(ctx);
  if (c == nullptr || push_m_cap <= 0) return ZSE_ERR_SHAPE;
  c->push_m_cap = push_m_cap;
  for (int r = 0; r < c->table.tp; ++r) {
    c->inbox[r] = reinterpret_cast<__half*>(inbox_ptrs[r]);
    c->arrive[r] = reinterpret_cast<uint32_t*>(arrive_ptrs[r]);
    c->state[r] = reinterpret_cast<uint32_t*>(state_ptrs[r]);
  }
  c->mc_inbox = reinterpret_cast<__half*>(mc_inbox);
  c->mc_arrive = reinterpret_cast<uint32_t*>(mc_arrive);
  return 0;
}

namespace zse {
int tp_fill_push_table(const void* ctx, int slot, bool multimem, int rank_override, PushTable* out) {
  const zse_tp_ctx* c = reinterpret_cast<const zse_tp_ctx*>(ctx);
  if (c == nullptr || c->inbox[0] == nullptr) return ZSE_ERR_SHAPE;
  if (multimem && (c->mc_inbox == nullptr || c->mc_arrive == nullptr)) return ZSE_ERR_SHAPE;
  for (int r = 0; r < kPushMaxTp; ++r) {
    out->inbox[r] = r < c->table.tp ? c->inbox[r] : nullptr;
    out->arrive[r] = r < c->table.tp ? c->arrive[r] : nullptr;
  }
  out->mc_inbox = multimem ? c->mc_inbox : nullptr;
  out->mc_arrive = multimem ? c->mc_arrive : nullptr;
  out->tp = c->table.tp;
  out->rank = rank_override >= 0 ? rank_override : c->rank;
  out->m_cap = c->push_m_cap;
  out->H = c->H;
  out->slot = slot & 1;
  return 0;
}
uint32_t* tp_push_state(const void* ctx, int rank_override) {
  const zse_tp_ctx* c = reinterpret_cast<const zse_tp_ctx*>(ctx);
  if (c == nullptr) return nullptr;
  const int r = rank_override >= 0 ? rank_override : c->rank;
  return (r >= 0 && r < c->table.tp) ? c->state[r] : nullptr;
}
}  // namespace zse

// Buffers of the sequence-parallel exchange (see SpTable): per rank r the mapped addresses of its inbox
// [2][tp][own_cap][H] fp16, counters [2][tp][nblk_cap] u32, gathered activations [nblk_cap * 64][H] fp16 and flags
// [nblk_cap] u32; `state_ptrs[r]`: rank r's local words (4 + nblk_cap u32, zero-initialised; other ranks' entries may
// be 0 outside single-GPU tests).  own_cap must hold ceil(nblk_cap / tp) blocks of 64 rows.
extern "C" int zse_tp_ctx_set_sp(void* ctx, int own_cap, int nblk_cap, const uint64_t* inbox_ptrs,
                                 const uint64_t* arrive_ptrs, const uint64_t* xg_ptrs, uint64_t mc_xg,
                                 const uint64_t* gflag_ptrs, const uint64_t* state_ptrs) {
  zse_tp_ctx* c = reinterpret_cast<zse_tp_ctx*>(ctx);
  if (c == nullptr || nblk_cap <= 0) return ZSE_ERR_SHAPE;
  const int tp = c->table.tp;
  if (own_cap < ((nblk_cap + tp - 1) / tp) * kSpRowBlock) return ZSE_ERR_SHAPE;
  c->sp_own_cap = own_cap;
  c->sp_nblk_cap = nblk_cap;
  for (int r = 0; r < tp; ++r) {
    c->sp_inbox[r] = reinterpret_cast<__half*>(inbox_ptrs[r]);
    c->sp_arrive[r] = reinterpret_cast<uint32_t*>(arrive_ptrs[r]);
    c->sp_xg[r] = reinterpret_cast<__half*>(xg_ptrs[r]);
    c->sp_gflag[r] = reinterpret_cast<uint32_t*>(gflag_ptrs[r]);
    c->sp_state[r] = reinterpret_cast<uint32_t*>(state_ptrs[r]);
  }
  c->mc_xg = reinterpret_cast<__half*>(mc_xg);
  return 0;
}

namespace zse {
int tp_fill_sp_table(const void* ctx, int slot, bool multimem, int rank_override, SpTable* out) {
  const zse_tp_ctx* c = reinterpret_cast<const zse_tp_ctx*>(ctx);
  if (c == nullptr || c->sp_inbox[0] == nullptr) return ZSE_ERR_SHAPE;
  if (multimem && c->mc_xg == nullptr) return ZSE_ERR_SHAPE;
  const int rank = rank_override >= 0 ? rank_override : c->rank;
  if (rank < 0 || rank >= c->table.tp || c->sp_state[rank] == nullptr) return ZSE_ERR_SHAPE;
  for (int r = 0; r < kPushMaxTp; ++r) {
    const bool in = r < c->table.tp;
    out->inbox[r] = in ? c->sp_inbox[r] : nullptr;
    out->arrive[r] = in ? c->sp_arrive[r] : nullptr;
    out->xg[r] = in ? c->sp_xg[r] : nullptr;
    out->gflag[r] = in ? c->sp_gflag[r] : nullptr;
  }
  out->mc_xg = multimem ? c->mc_xg : nullptr;
  out->state = c->sp_state[rank];
  out->tp = c->table.tp;
  out->rank = rank;
  out->H = c->H;
  out->own_cap = c->sp_own_cap;
  out->nblk_cap = c->sp_nblk_cap;
  out->slot = slot & 1;
  return 0;
}
}  // namespace zse

static int fill_sp_args(const zse_tp_ctx* c, TpSpArgs& a, const void* weight, int M, float eps, int slot,
                        bool multimem, void* status) {
  if (c == nullptr || M <= 0 || c->H % kTileN || c->H > 8 * kRedThreads * kRedMaxChunks) return ZSE_ERR_SHAPE;
  if (int rc = tp_fill_sp_table(c, slot, multimem, -1, &a.sp)) return rc;
  if ((M + kSpRowBlock - 1) / kSpRowBlock > c->sp_nblk_cap) return ZSE_ERR_SHAPE;
  a.weight = reinterpret_cast<const __half*>(weight);
  a.M = M;
  a.eps = eps;
  a.units = uint32_t(kSpRowBlock / 16) * uint32_t(c->H / kTileN);   // (16-token chunks per block) x (weight tiles)
  a.status = reinterpret_cast<Status*>(status);
  return 0;
}

// residual[own rows] += sum over ranks of the scattered partial rows; gathered buffer of every rank = RMSNorm of
// those rows (see tp_sp_sum_norm_gather_kernel).  Follows zse_tp_gemm_w4_scatter of the same slot on every rank.
extern "C" int zse_tp_sp_sum_norm_gather(void* ctx, void* residual, const void* weight, int M, float eps, int slot,
                                         int use_multimem, void* status, void* stream) {
  zse_tp_ctx* c = reinterpret_cast<zse_tp_ctx*>(ctx);
  TpSpArgs a{};
  if (int rc = fill_sp_args(c, a, weight, M, eps, slot, use_multimem != 0, status)) return rc;
  a.residual[0] = reinterpret_cast<float*>(residual);
  a.state[0] = c->sp_state[c->rank];
  a.rank[0] = c->rank;
  tp_sp_sum_norm_gather_kernel<<<dim3(M, 1), kRedThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

// All ranks of a single-GPU test in one launch (blockIdx.y = rank).  The scatter GEMMs of every emulated rank have
// finished before it starts, and no CTA of it waits for another CTA.
extern "C" int zse_tp_sp_sum_norm_gather_emulated(void* ctx, const uint64_t* residuals, const void* weight, int M,
                                                  float eps, int slot, void* status, void* stream) {
  zse_tp_ctx* c = reinterpret_cast<zse_tp_ctx*>(ctx);
  TpSpArgs a{};
  if (int rc = fill_sp_args(c, a, weight, M, eps, slot, false, status)) return rc;
  for (int r = 0; r < c->table.tp; ++r) {
    if (c->sp_state[r] == nullptr) return ZSE_ERR_SHAPE;
    a.residual[r] = reinterpret_cast<float*>(residuals[r]);
    a.state[r] = c->sp_state[r];
    a.rank[r] = r;
  }
  tp_sp_sum_norm_gather_kernel<<<dim3(M, c->table.tp), kRedThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

// Bounded wait until all row blocks of a pass of M rows have arrived in this rank's gathered buffer.
extern "C" int zse_tp_sp_wait(void* ctx, int M, int rank_override, void* status, void* stream) {
  zse_tp_ctx* c = reinterpret_cast<zse_tp_ctx*>(ctx);
  SpTable sp;
  if (int rc = tp_fill_sp_table(c, 0, false, rank_override, &sp)) return rc;
  const int nb = (M + kSpRowBlock - 1) / kSpRowBlock;
  if (M <= 0 || nb > sp.nblk_cap) return ZSE_ERR_SHAPE;
  tp_sp_wait_kernel<<<1, kRedThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(sp.gflag[sp.rank], sp.state, nb,
                                                                                 reinterpret_cast<Status*>(status));
  return cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

// Buffers of the logits all-gather: per rank r its gathered rows [2][rows_cap][tp * width] fp16 and flags
// [2][tp][rows_cap] u32 (zero at start), both in symmetric memory.
extern "C" int zse_tp_ctx_set_gather(void* ctx, int rows_cap, int width, const uint64_t* buf_ptrs,
                                     const uint64_t* flag_ptrs) {
  zse_tp_ctx* c = reinterpret_cast<zse_tp_ctx*>(ctx);
  if (c == nullptr || rows_cap <= 0 || width <= 0 || width % 8) return ZSE_ERR_SHAPE;
  c->g_rows_cap = rows_cap;
  c->g_width = width;
  for (int r = 0; r < c->table.tp; ++r) {
    c->g_buf[r] = reinterpret_cast<__half*>(buf_ptrs[r]);
    c->g_flags[r] = reinterpret_cast<uint32_t*>(flag_ptrs[r]);
  }
  return 0;
}

static int fill_gather_args(const zse_tp_ctx* c, TpGatherArgs& a, int ld, int M, int slot, void* status) {
  if (c == nullptr || c->g_buf[0] == nullptr || M <= 0 || M > c->g_rows_cap || ld % 8 || ld < c->g_width)
    return ZSE_ERR_SHAPE;
  for (int r = 0; r < c->table.tp; ++r) {
    a.buf[r] = c->g_buf[r];
    a.flags[r] = c->g_flags[r];
  }
  a.ld = ld;
  a.W = c->g_width;
  a.tp = c->table.tp;
  a.rows_cap = c->g_rows_cap;
  a.slot = slot & 1;
  a.status = reinterpret_cast<Status*>(status);
  return 0;
}

// After the launch, rows [0, M) of slot `slot` of this rank's gathered buffer hold the logits of all ranks
// (columns r * width .. (r + 1) * width from rank r).
extern "C" int zse_tp_gather_rows(void* ctx, const void* logits, int ld, int M, int slot, void* status, void* stream) {
  zse_tp_ctx* c = reinterpret_cast<zse_tp_ctx*>(ctx);
  TpGatherArgs a{};
  if (int rc = fill_gather_args(c, a, ld, M, slot, status)) return rc;
  if (reinterpret_cast<uintptr_t>(logits) & 15) return ZSE_ERR_ALIGN;
  a.src[0] = reinterpret_cast<const __half*>(logits);
  a.rank[0] = c->rank;
  tp_gather_rows_kernel<<<dim3(M, 1), 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

// All ranks of a single-GPU test in one cooperative launch (blockIdx.y = rank): every CTA is resident, so the waits
// between the emulated ranks are waits inside one kernel.
extern "C" int zse_tp_gather_rows_emulated(void* ctx, const uint64_t* logits, int ld, int M, int slot, void* status,
                                           void* stream) {
  zse_tp_ctx* c = reinterpret_cast<zse_tp_ctx*>(ctx);
  TpGatherArgs a{};
  if (int rc = fill_gather_args(c, a, ld, M, slot, status)) return rc;
  for (int r = 0; r < c->table.tp; ++r) {
    a.src[r] = reinterpret_cast<const __half*>(logits[r]);
    a.rank[r] = r;
  }
  void* params[] = {&a};
  return cudaLaunchCooperativeKernel((const void*)tp_gather_rows_kernel, dim3(M, c->table.tp), dim3(512), params, 0,
                                     reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess
             ? 0
             : ZSE_ERR_LAUNCH;
}

// Programmatic dependent launch for the reduce kernels: off unless ZSE_TP_PDL=1.  Measured on 2 GPUs: a reduce kernel
// that starts early spins on its peers' flags while the GEMM before it still runs and slows the whole step
// (7.5 ms vs 6.4 ms per decode step), so these kernels keep the ordinary stream order.
static bool tp_pdl_allowed() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("ZSE_TP_PDL");
    v = (e != nullptr && e[0] == '1') ? 1 : 0;
  }
  return v != 0;
}

static int launch_reduce(const zse_tp_ctx* c, TpReduceArgs& a, int rows, int emulate, bool multimem,
                         cudaStream_t st) {
  dim3 grid(rows, emulate > 0 ? emulate : 1);
  if (emulate > 0) {
    void* params[] = {const_cast<TpTable*>(&c->table), &a};
    const void* fn = multimem ? (const void*)tp_reduce_add_rmsnorm_kernel<true>
                              : (const void*)tp_reduce_add_rmsnorm_kernel<false>;
    return cudaLaunchCooperativeKernel(fn, grid, dim3(kRedThreads), params, 0, st) == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
  }
  const bool pdl = tp_pdl_allowed();
  const cudaError_t e = multimem ? launch_pdl_if(pdl, tp_reduce_add_rmsnorm_kernel<true>, grid, dim3(kRedThreads), 0,
                                                 st, c->table, a)
                                 : launch_pdl_if(pdl, tp_reduce_add_rmsnorm_kernel<false>, grid, dim3(kRedThreads), 0,
                                                 st, c->table, a);
  return e == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

static int launch_reduce_scatter(const zse_tp_ctx* c, TpReduceArgs& a, int rows, int emulate, bool multimem,
                                 cudaStream_t st) {
  dim3 grid(rows, emulate > 0 ? emulate : 1);
  if (emulate > 0) {
    void* params[] = {const_cast<TpTable*>(&c->table), &a};
    return cudaLaunchCooperativeKernel((const void*)tp_reduce_scatter_add_rmsnorm_kernel<false>, grid,
                                       dim3(kRedThreads), params, 0, st) == cudaSuccess
               ? 0
               : ZSE_ERR_LAUNCH;
  }
  const bool pdl = tp_pdl_allowed();
  const cudaError_t e = multimem ? launch_pdl_if(pdl, tp_reduce_scatter_add_rmsnorm_kernel<true>, grid,
                                                 dim3(kRedThreads), 0, st, c->table, a)
                                 : launch_pdl_if(pdl, tp_reduce_scatter_add_rmsnorm_kernel<false>, grid,
                                                 dim3(kRedThreads), 0, st, c->table, a);
  return e == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

// Real launch: residual/partials/out are this rank's.  Rows are processed in launches of at most 512 so that every
// CTA of a launch is resident on every rank (a CTA waits for its peers' CTAs of the same row).
extern "C" int zse_tp_reduce_add_rmsnorm(void* ctx, void* residual, const void* partials, int n_planes,
                                         const void* weight, void* out, int M, float eps, int slot,
                                         int use_multimem, void* status, void* stream) {
  zse_tp_ctx* c = reinterpret_cast<zse_tp_ctx*>(ctx);
  if (M <= 0) return 0;
  if (c == nullptr || c->H % 8 || c->H > 8 * kRedThreads * kRedMaxChunks || M > c->table.m_cap) return ZSE_ERR_SHAPE;
  if (use_multimem && c->table.mc_data == nullptr) return ZSE_ERR_SHAPE;
  TpReduceArgs a{};
  a.r[0] = TpRankArgs{reinterpret_cast<float*>(residual), reinterpret_cast<const float*>(partials),
                      reinterpret_cast<__half*>(out), c->rank};
  a.weight = reinterpret_cast<const __half*>(weight);
  a.n_planes = n_planes;
  a.M = M;
  a.H = c->H;
  a.eps = eps;
  a.slot = slot & 1;
  a.status = reinterpret_cast<Status*>(status);
  for (int row0 = 0; row0 < M; row0 += 512) {
    a.row0 = row0;
    if (int rc = launch_reduce(c, a, min(512, M - row0), 0, use_multimem != 0, reinterpret_cast<cudaStream_t>(stream)))
      return rc;
  }
  return 0;
}

// Two-shot variant (see the kernel): after it the fp32 residual is current only in the rows this rank owns
// (row % tp == rank); `out` is complete on every rank.
extern "C" int zse_tp_reduce_scatter_add_rmsnorm(void* ctx, void* residual, const void* partials, int n_planes,
                                                 const void* weight, void* out, int M, float eps, int slot,
                                                 int use_multimem, void* status, void* stream) {
  zse_tp_ctx* c = reinterpret_cast<zse_tp_ctx*>(ctx);
  if (M <= 0) return 0;
  if (c == nullptr || out == nullptr || c->H % 8 || c->H > 8 * kRedThreads * kRedMaxChunks || M > c->table.m_cap)
    return ZSE_ERR_SHAPE;
  if (use_multimem && c->table.mc_data == nullptr) return ZSE_ERR_SHAPE;
  TpReduceArgs a{};
  a.r[0] = TpRankArgs{reinterpret_cast<float*>(residual), reinterpret_cast<const float*>(partials),
                      reinterpret_cast<__half*>(out), c->rank};
  a.weight = reinterpret_cast<const __half*>(weight);
  a.n_planes = n_planes;
  a.M = M;
  a.H = c->H;
  a.eps = eps;
  a.slot = slot & 1;
  a.status = reinterpret_cast<Status*>(status);
  for (int row0 = 0; row0 < M; row0 += 512) {
    a.row0 = row0;
    if (int rc = launch_reduce_scatter(c, a, min(512, M - row0), 0, use_multimem != 0,
                                       reinterpret_cast<cudaStream_t>(stream)))
      return rc;
  }
  return 0;
}

extern "C" int zse_tp_reduce_scatter_add_rmsnorm_emulated(void* ctx, const uint64_t* residuals,
                                                          const uint64_t* partials, int n_planes, const void* weight,
                                                          const uint64_t* outs, int M, float eps, int slot,
                                                          void* status, void* stream) {
  zse_tp_ctx* c = reinterpret_cast<zse_tp_ctx*>(ctx);
  if (c == nullptr || M <= 0 || M > c->table.m_cap || M * c->table.tp > 256) return ZSE_ERR_SHAPE;
  TpReduceArgs a{};
  for (int r = 0; r < c->table.tp; ++r)
    a.r[r] = TpRankArgs{reinterpret_cast<float*>(residuals[r]), reinterpret_cast<const float*>(partials[r]),
                        reinterpret_cast<__half*>(outs[r]), r};
  a.weight = reinterpret_cast<const __half*>(weight);
  a.n_planes = n_planes;
  a.M = M;
  a.H = c->H;
  a.eps = eps;
  a.slot = slot & 1;
  a.row0 = 0;
  a.status = reinterpret_cast<Status*>(status);
  return launch_reduce_scatter(c, a, M, c->table.tp, false, reinterpret_cast<cudaStream_t>(stream));
}

// Single-GPU emulation of all ranks in one cooperative launch (tests): arrays hold one pointer per rank.
extern "C" int zse_tp_reduce_add_rmsnorm_emulated(void* ctx, const uint64_t* residuals, const uint64_t* partials,
                                                  int n_planes, const void* weight, const uint64_t* outs, int M,
                                                  float eps, int slot, void* status, void* stream) {
  zse_tp_ctx* c = reinterpret_cast<zse_tp_ctx*>(ctx);
  if (c == nullptr || M <= 0 || M > c->table.m_cap || M * c->table.tp > 256) return ZSE_ERR_SHAPE;
  TpReduceArgs a{};
  for (int r = 0; r < c->table.tp; ++r)
    a.r[r] = TpRankArgs{reinterpret_cast<float*>(residuals[r]), reinterpret_cast<const float*>(partials[r]),
                        reinterpret_cast<__half*>(outs[r]), r};
  a.weight = reinterpret_cast<const __half*>(weight);
  a.n_planes = n_planes;
  a.M = M;
  a.H = c->H;
  a.eps = eps;
  a.slot = slot & 1;
  a.row0 = 0;
  a.status = reinterpret_cast<Status*>(status);
  return launch_reduce(c, a, M, c->table.tp, false, reinterpret_cast<cudaStream_t>(stream));
}

static int fill_sum_args(const zse_tp_ctx* c, TpSumArgs& a, const void* weight, int M, float eps, int slot,
                         int expected_add, void* status) {
  if (c == nullptr || c->inbox[0] == nullptr || M <= 0 || M > c->push_m_cap || c->H % 8 ||
      c->H > 8 * kRedThreads * kRedMaxChunks || expected_add <= 0)
    return ZSE_ERR_SHAPE;
  for (int r = 0; r < c->table.tp; ++r) {
    a.inbox[r] = c->inbox[r];
    a.arrive[r] = c->arrive[r];
    a.state[r] = c->state[r];
  }
  a.weight = reinterpret_cast<const __half*>(weight);
  a.tp = c->table.tp;
  a.m_cap = c->push_m_cap;
  a.M = M;
  a.H = c->H;
  a.slot = slot & 1;
  a.expected_add = uint32_t(expected_add);
  a.eps = eps;
  a.status = reinterpret_cast<Status*>(status);
  return 0;
}

// Consumer of the push exchange (see tp_sum_add_rmsnorm_kernel).  `expected_add`: what zse_tp_gemm_w4_push returned
// for the GEMM of this call (its CTA count, the same on every rank).
extern "C" int zse_tp_sum_add_rmsnorm(void* ctx, void* residual, const void* weight, void* out, int M, float eps,
                                      int slot, int expected_add, void* status, void* stream) {
  zse_tp_ctx* c = reinterpret_cast<zse_tp_ctx*>(ctx);
  TpSumArgs a{};
  if (int rc = fill_sum_args(c, a, weight, M, eps, slot, expected_add, status)) return rc;
  if (c->state[c->rank] == nullptr) return ZSE_ERR_SHAPE;
  a.r[0] = TpRankArgs{reinterpret_cast<float*>(residual), nullptr, reinterpret_cast<__half*>(out), c->rank};
  return launch_pdl_if(tp_pdl_allowed(), tp_sum_add_rmsnorm_kernel, dim3(M, 1), dim3(kRedThreads), 0,
                       reinterpret_cast<cudaStream_t>(stream), a) == cudaSuccess
             ? 0
             : ZSE_ERR_LAUNCH;
}

// All ranks of a single-GPU test in one launch (blockIdx.y = rank).  The producers have finished before it starts,
// so nothing here waits for a kernel that is not running.
extern "C" int zse_tp_sum_add_rmsnorm_emulated(void* ctx, const uint64_t* residuals, const void* weight,
                                               const uint64_t* outs, int M, float eps, int slot, int expected_add,
                                               void* status, void* stream) {
  zse_tp_ctx* c = reinterpret_cast<zse_tp_ctx*>(ctx);
  TpSumArgs a{};
  if (int rc = fill_sum_args(c, a, weight, M, eps, slot, expected_add, status)) return rc;
  for (int r = 0; r < c->table.tp; ++r) {
    if (c->state[r] == nullptr) return ZSE_ERR_SHAPE;
    a.r[r] = TpRankArgs{reinterpret_cast<float*>(residuals[r]), nullptr, reinterpret_cast<__half*>(outs[r]), r};
  }
  tp_sum_add_rmsnorm_kernel<<<dim3(M, c->table.tp), kRedThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

extern "C" int zse_tp_argmax(void* ctx, const void* logits, int ld, void* out, int M, int V_local, int vocab_stride,
                             int slot, void* status, void* stream) {
  zse_tp_ctx* c = reinterpret_cast<zse_tp_ctx*>(ctx);
  if (M <= 0) return 0;
  if (c == nullptr || M > c->table.m_cap) return ZSE_ERR_SHAPE;
  TpArgmaxArgs a{};
  a.logits[0] = reinterpret_cast<const __half*>(logits);
  a.out[0] = reinterpret_cast<int*>(out);
  a.rank[0] = c->rank;
  for (int r = 0; r < c->table.tp; ++r) {
    a.xchg[r] = c->xchg[r];
    a.flags[r] = c->xflags[r];
  }
  a.ld = ld;
  a.V_local = V_local;
  a.vocab_stride = vocab_stride;
  a.tp = c->table.tp;
  a.m_cap = c->table.m_cap;
  a.slot = slot & 1;
  a.status = reinterpret_cast<Status*>(status);
  tp_argmax_kernel<<<dim3(M, 1), 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : ZSE_ERR_LAUNCH;
}

extern "C" int zse_tp_argmax_emulated(void* ctx, const uint64_t* logits, int ld, const uint64_t* outs, int M,
                                      int V_local, int vocab_stride, int slot, void* status,
                                      void* stream) {
  zse_tp_ctx* c = reinterpret_cast<zse_tp_ctx*>(ctx);
  if (c == nullptr || M <= 0 || M > c->table.m_cap || M * c->table.tp > 128) return ZSE_ERR_SHAPE;
  TpArgmaxArgs a{};
  for (int r = 0; r < c->table.tp; ++r) {
    a.logits[r] = reinterpret_cast<const __half*>(logits[r]);
    a.out[r] = reinterpret_cast<int*>(outs[r]);
    a.rank[r] = r;
    a.xchg[r] = c->xchg[r];
    a.flags[r] = c->xflags[r];
  }
  a.ld = ld;
  a.V_local = V_local;
  a.vocab_stride = vocab_stride;
  a.tp = c->table.tp;
  a.m_cap = c->table.m_cap;
  a.slot = slot & 1;
  a.status = reinterpret_cast<Status*>(status);
  void* params[] = {&a};
  return cudaLaunchCooperativeKernel((const void*)tp_argmax_kernel, dim3(M, c->table.tp), dim3(1024), params, 0,
                                     reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess
             ? 0
             : ZSE_ERR_LAUNCH;
}

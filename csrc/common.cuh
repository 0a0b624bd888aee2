// Shared device helpers for the sm_100a kernels: mbarrier, TMA (bulk and tiled, never multicast),
// tcgen05 (TMEM allocation, MMA, commit, ld/st, fences), bounded waits and the status word.
//
// Every wait in this library is bounded: when a limit runs out the waiter records
// {code, block, detail} in a status word that the host reads after the launch, raises a CTA-wide
// abort flag and the kernel unwinds normally (TMEM is released, in-flight copies are drained).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace zse {

// ---- status word -----------------------------------------------------------------------------
// One per library instance (device memory, zeroed at init); kernels only ever write to it on
// failure, so the normal path costs nothing.
struct Status {
  unsigned int code;      // 0 = ok
  unsigned int block;     // linear block id of the first reporter
  unsigned int where;     // site id inside the kernel
  unsigned int detail;    // e.g. stage index / expected value
};
enum StatusCode : unsigned int {
  kOk = 0,
  kWaitTimeout = 1,       // an mbarrier / flag wait ran out
  kBadArgument = 2,       // device-side argument check failed (index out of range, ...)
  kPeerTimeout = 3,       // a wait on another GPU's flag ran out
};

__device__ __forceinline__ void report(Status* st, unsigned code, unsigned where, unsigned detail) {
  if (st != nullptr && atomicCAS(&st->code, 0u, code) == 0u) {
    st->block = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    st->where = where;
    st->detail = detail;
    __threadfence_system();
  }
}

// ---- programmatic dependent launch ----------------------------------------------------------------------------
// A kernel launched with launch_pdl() may start while the kernel before it on the stream is still running.
// pdl_wait() returns once that kernel has finished and its writes are visible: everything a kernel reads from or
// writes to memory that an earlier kernel of the stream touches has to come after it.  Work that only needs
// constant data (weights, tensor maps, barrier set-up, TMEM allocation) may come before.  Both calls do nothing in a
// kernel that was launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

constexpr uint64_t kWaitLimitNs = 2000000000ull;   // 2 s: far beyond any legitimate wait

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier --------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Same test, but the thread may stay suspended for up to `hint_ns` before it reports "not yet": a waiting warp then
// costs the scheduler almost nothing (the hardware wakes it when the phase completes).
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}

// Deadline of a bounded spin.  The global timer is slow to read (of the order of a microsecond), so a wait consults it
// only every `mask + 1` polls and starts its clock at the first such reading: a wait that ends soon never reads it.
struct SpinClock {
  uint64_t t0 = 0;
  unsigned spins = 0;
  __device__ __forceinline__ bool expired(unsigned mask) {
    if ((++spins & mask) != 0) return false;
    const uint64_t now = globaltimer_ns();
    if (t0 == 0) t0 = now;
    return now - t0 > kWaitLimitNs;
  }
};

// Bounded wait.  Returns false when it gave up (timeout, or another thread of the CTA aborted).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, Status* st,
                                          unsigned where, unsigned detail) {
  if (mbar_try_wait(bar, parity)) return true;
  // the global timer is slow to read (of the order of a microsecond): it is first read after 16 unsuccessful polls, never
  // on the path of a wait that ends soon
  uint64_t t0 = 0;
  unsigned spins = 0;
  while (!mbar_try_wait_hint(bar, parity, 20000u)) {
    if ((++spins & 0xF) == 0) {
      if (*abort_flag) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > kWaitLimitNs) {
        report(st, kWaitTimeout, where, detail);
        *abort_flag = 1;
        __threadfence_block();
        return false;
      }
    }
  }
  return true;
}

// Same contract, for the one thread whose wake-up latency is on the critical path (an MMA issuer): it polls without
// the suspend hint, so it sees the phase flip within a few cycles instead of after a scheduler wake-up.
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity, volatile int* abort_flag, Status* st,
                                               unsigned where, unsigned detail) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;                                    // first read after 256 polls (see mbar_wait)
  unsigned spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0xFF) == 0) {
      if (*abort_flag) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > kWaitLimitNs) {
        report(st, kWaitTimeout, where, detail);
        *abort_flag = 1;
        __threadfence_block();
        return false;
      }
    }
  }
  return true;
}

// ---- TMA -------------------------------------------------------------------------------------
// 1-D bulk copy global -> shared (16-byte aligned addresses, size a multiple of 16).
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// 2-D tiled load; x is the innermost (contiguous) coordinate in elements and must be a multiple of
// 16 bytes / element size.
__device__ __forceinline__ void tma_load_2d(void* dst_smem, const void* tmap, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(dst_smem)),
      "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- tcgen05 / TMEM --------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {   // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {    // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {   // one thread
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem], kind::f16 (fp16 or bf16 inputs, fp32 accumulate); one thread.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; A is K-major, lane = row, one 32-bit column per two K values.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Instruction descriptor for kind::f16: fp32 accumulator, A and B K-major, fp16 (fmt 0) or bf16 (fmt 1).
__host__ __device__ constexpr uint32_t make_idesc_f16(int m, int n, int ab_fmt = 0) {
  return (1u << 4) | (uint32_t(ab_fmt) << 7) | (uint32_t(ab_fmt) << 10) | (uint32_t(n >> 3) << 17) |
         (uint32_t(m >> 4) << 24);
}
// Shared-memory matrix descriptor, K-major operand in the 128-byte-swizzle layout that a tiled TMA
// load with CU_TENSOR_MAP_SWIZZLE_128B produces: rows of 128 bytes, 8-row groups 1024 bytes apart.
// The tile base must be 1024-byte aligned; a K step of 16 halfs advances the start address by 32 bytes.
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr >> 4) & 0x3FFF);          // start address
  d |= uint64_t(1) << 16;                            // leading byte offset (unused with swizzle)
  d |= uint64_t(1024 >> 4) << 32;                    // stride byte offset: 8 rows * 128 B
  d |= uint64_t(1) << 46;                            // descriptor version (sm_100)
  d |= uint64_t(2) << 61;                            // SWIZZLE_128B
  return d;
}

// 32 lanes x 32-bit x N columns, lane i of the warp <-> TMEM lane (base + i).
#define ZSE_TMEM_LD_X16(r, taddr)                                                                              \
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, " \
               "[%16];"                                                                                        \
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), \
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),       \
                 "=r"(r[15])                                                                                   \
               : "r"(taddr)                                                                                    \
               : "memory")

#define ZSE_TMEM_ST_X16(taddr, r)                                                                              \
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" \
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),      \
               "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),    \
               "r"(r[15])                                                                                      \
               : "memory")

#define ZSE_TMEM_ST_X32(taddr, r)                                                                              \
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "                                                  \
               "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"                                       \
               "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"                              \
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),      \
               "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),    \
               "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), \
               "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), \
               "r"(r[31])                                                                                      \
               : "memory")

// ---- small math ------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + __expf(-g)); }
__device__ __forceinline__ float clamp_f16(float v) { return fminf(fmaxf(v, -65504.0f), 65504.0f); }

// ---- host side: function attributes are per device ------------------------------------------------------------
// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) applies to the current device only, so "already done" is kept per
// device (a process that drives several GPUs raises it on each of them).
constexpr int kMaxDevices = 64;
inline int current_device_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
  return dev;
}

// ---- host side: launch with the programmatic-serialization attribute (see pdl_wait) ---------------------------
int pdl_enabled();   // runtime.cu; 1 unless switched off by zse_set_pdl(0) or ZSE_PDL=0

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_if(bool allow, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (allow && pdl_enabled()) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

}  // namespace zse

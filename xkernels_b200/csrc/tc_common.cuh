// sm_100a building blocks used by the tcgen05 kernels: mbarriers with BOUNDED
// waits, TMA tile loads (never multicast), tensor-memory management, UMMA
// descriptors and the tcgen05 load/store/MMA instructions as inline PTX.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace xkb {
namespace tc {

// Error codes a kernel writes to its status word when a bounded wait runs out.
constexpr int kErrWaitTimeout = 1;

// Time budget of one wait.  A healthy pipeline completes every wait within microseconds; a wait
// that lasts this long means a lost arrival, and the kernel gives up instead of hanging the GPU.
constexpr uint64_t kWaitBudgetNs = 1000000000ull;   // one second

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
// One probe of the barrier phase.  try_wait may park the thread for a hardware-defined time while
// the phase is incomplete (it is woken when the phase completes), so waiting roles burn fewer of
// the issue slots the dequantiser warps need than with test_wait.  (An explicit suspend-time hint
// measured 1 % slower than none.)
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
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

// Shared abort word + global status word of one CTA.
struct Guard {
  volatile int* abort_flag;  // shared memory
  int* status;               // global memory (may be shared by all CTAs)
  __device__ __forceinline__ bool aborted() const { return *abort_flag != 0; }
  __device__ __forceinline__ void raise(int code) {
    *abort_flag = code;
    atomicCAS(status, 0, code);
  }
};

// Bounded wait: returns false (after recording the failure) if the barrier has not completed the
// phase within `budget_ns` of wall-clock time (read from %globaltimer every 64 probes) or another
// role aborted.  `sleep_ns` > 0 backs off between probes: roles that run ahead of the pipeline
// (the TMA producers) and roles that wait on the slower side (the MMA issuers) would otherwise
// spend issue slots on probes that the dequantiser warps need.
// The polling loop lives out of line: the callers' fast path (phase already complete) is then one
// probe and one predicated call, without the loop's divergence bookkeeping in every inlined copy.
static __device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, Guard g, int where, uint32_t sleep_ns,
                                            uint64_t budget_ns) {
  uint64_t t0 = 0;
  for (uint32_t i = 1;; ++i) {
    if (sleep_ns) __nanosleep(sleep_ns);
    if (mbar_try(bar, parity)) return true;
    if ((i & 63u) == 0u) {
      if (g.aborted()) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > budget_ns) break;
    }
  }
  g.raise(kErrWaitTimeout + (where << 8));
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, Guard& g, int where,
                                          uint32_t sleep_ns = 0, uint64_t budget_ns = kWaitBudgetNs) {
  if (mbar_try(bar, parity)) return true;   // the common case: already complete
  return mbar_wait_slow(bar, parity, g, where, sleep_ns, budget_ns);
}

// Variants for warp-uniform code: every lane of the warp executes the call with the same operands
// and `leader` (non-zero in exactly one lane) selects the lane whose instruction takes effect.
__device__ __forceinline__ void mbar_arrive_if(uint64_t* bar, uint32_t leader) {
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %1, 0;\n\t@q mbarrier.arrive.shared::cta.b64 _, [%0];\n\t}"
               ::"r"(smem_u32(bar)), "r"(leader) : "memory");
}

// ---- shared-memory loads by 32-bit shared address (keeps the loads in the shared state space) ----
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

// ---- TMA (plain tile loads; no multicast anywhere) ---------------------------
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x,
                                            int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- tensor memory -------------------------------------------------------------
// Whole-warp calls.  The allocation result lands in shared memory.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tc_commit_if(uint64_t* bar, uint32_t leader) {
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
      ::"r"(smem_u32(bar)), "r"(leader) : "memory");
}

// 32 lanes x 8 columns store (registers r[0..7] of each thread).
__device__ __forceinline__ void tmem_st_32x8(uint32_t taddr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3,
                                             uint32_t r4, uint32_t r5, uint32_t r6, uint32_t r7) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"r"(taddr), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(r4), "r"(r5), "r"(r6), "r"(r7)
               : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x 16 columns load (fp32 accumulators): thread i reads lane
// (lane_base + i), columns [col, col+16).
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- UMMA descriptors ----------------------------------------------------------
// Instruction descriptor, kind::f16: bf16 x bf16 -> fp32, both operands K-major,
// M = 128, N = n.  Field layout: c_format [4,6), a_format [7,10), b_format
// [10,13), a_major 15, b_major 16, n>>3 [17,23), m>>4 [24,29).
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes
// (64 bf16) in the 128-byte swizzle: 8-row groups 1024 bytes apart.
// start>>4 [0,14), LBO>>4 [16,30) (unused with swizzle: 1), SBO>>4 [32,46) = 64,
// version [46,48) = 1, layout [61,64) = 2 (SWIZZLE_128B).  The tile base must be
// 1024-byte aligned; advancing K by 16 elements adds 32 bytes to the start.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// D[tmem] (+)= A[tmem] * B[smem]^T ; one thread issues.
__device__ __forceinline__ void umma_ts_bf16(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The same, executed by a whole warp with identical operands; only the lane with `leader` != 0 issues.
__device__ __forceinline__ void umma_ts_bf16_if(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate, uint32_t leader) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader)
      : "memory");
}

}  // namespace tc
}  // namespace xkb

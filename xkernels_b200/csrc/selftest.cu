// Self-test of the abort path of the tcgen05 kernels, without faulting or hanging anything:
// a one-CTA kernel with the same building blocks (tensor-memory allocation, an mbarrier, the
// bounded wait, the shared abort word, the status word) in which one role waits on a barrier
// that nobody ever arrives on.  The wait runs out after a few microseconds, the role records the
// status code, the second role leaves its own wait through the abort word, tensor memory is
// released and the kernel returns.  The host then reads the status like after any fused call.
#include "common.cuh"
#include "tc_common.cuh"

namespace xkb {
namespace {

using namespace tc;

constexpr int kSelftestWaitSite = 99;      // the "where" code the timed-out wait reports
constexpr uint64_t kSelftestBudgetNs = 20000;   // 20 us instead of the one second of the real kernels

__global__ void __launch_bounds__(96, 1) bounded_wait_selftest_kernel(int* status) {
  __shared__ __align__(8) uint64_t never_arrives, also_never;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_word;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(&never_arrives, 1);
    mbar_init(&also_never, 1);
    abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 512);   // everything, as the grouped-GEMM kernels do
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  Guard guard{&abort_word, status};
  if (warp == 1 && lane == 0) {
    // the role whose wait runs out: records kErrWaitTimeout + (site << 8) and raises the abort word
    mbar_wait(&never_arrives, 0, guard, kSelftestWaitSite, 32, kSelftestBudgetNs);
  } else if (warp == 2 && lane == 0) {
    // a role with the full one-second budget: it must leave early, through the abort word
    mbar_wait(&also_never, 0, guard, kSelftestWaitSite + 1, 32);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace
}  // namespace xkb

extern "C" int xkb_selftest_bounded_wait(void* workspace, int64_t workspace_bytes, void* stream_) {
  using namespace xkb;
  XKB_REQUIRE(workspace != nullptr && workspace_bytes >= 256, "xkb_selftest_bounded_wait: workspace of at least 256 bytes needed");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  XKB_CHECK_CUDA(cudaMemsetAsync(workspace, 0, sizeof(int), stream));
  bounded_wait_selftest_kernel<<<1, 96, 0, stream>>>(static_cast<int*>(workspace));
  XKB_CHECK_LAUNCH("bounded_wait_selftest_kernel");
  return XKB_OK;
}

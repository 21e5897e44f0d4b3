// Shared host/device helpers for the xkb200 library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "../../include/xkb200.h"

namespace xkb {

// ---- error plumbing -------------------------------------------------------
char* last_error_buf();  // thread-local, 512 bytes
int fail(int code, const char* fmt, ...);
extern std::atomic<int64_t> g_launches;
inline void count_launch(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

#define XKB_CHECK_CUDA(expr)                                                        \
  do {                                                                              \
    cudaError_t _e = (expr);                                                        \
    if (_e != cudaSuccess)                                                          \
      return ::xkb::fail(XKB_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,              \
                         cudaGetErrorString(_e), __FILE__, __LINE__);               \
  } while (0)

#define XKB_CHECK_LAUNCH(name)                                                      \
  do {                                                                              \
    cudaError_t _e = cudaGetLastError();                                            \
    if (_e != cudaSuccess)                                                          \
      return ::xkb::fail(XKB_ERR_CUDA, "launch of %s failed: %s", name,             \
                         cudaGetErrorString(_e));                                   \
    ::xkb::count_launch();                                                          \
  } while (0)

#define XKB_REQUIRE(cond, ...)                                                      \
  do {                                                                              \
    if (!(cond)) return ::xkb::fail(XKB_ERR_ARG, __VA_ARGS__);                      \
  } while (0)

inline int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Bump allocator over the caller's workspace (256-byte aligned slices).
struct Carver {
  char* base;
  int64_t off = 0;
  explicit Carver(void* p) : base(static_cast<char*>(p)) {}
  template <typename T>
  T* take(int64_t n) {
    T* p = reinterpret_cast<T*>(base + off);
    off += align_up(n * (int64_t)sizeof(T), 256);
    return p;
  }
};

// ---- layout of the routing produced by the align stage ---------------------
// sorted_ids[p]  slot id (token*top_k + j) at sorted position p, or `numel`
//                for a padding position.
// expert_ids[b]  expert of block b (block = `block_size` consecutive positions).
// expert_off[e]  first position of expert e's padded run; [E] = num_post_pad.
struct Routing {
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* num_post;
  const int32_t* expert_off;
  int64_t numel;     // M * top_k
  int64_t max_pad;   // length of sorted_ids
  int64_t max_blocks;
  int block;
  // two arrays of `counters_each` ints, zeroed with the status word at the start of a fused call:
  // [0] rows the gather kernel has delivered per token block, [1] finished read-outs of the first
  // GEMM of a two-GEMM layer per token block (nullptr: the kernels do not overlap that way)
  int32_t* block_counters;
  int64_t counters_each;
};

// Internal launchers shared between translation units --------------------------
int launch_align(const int32_t* topk_ids, int64_t numel, int num_experts, int block_size,
                 const int32_t* expert_map, int num_map, int32_t* sorted_ids,
                 int32_t* expert_ids, int32_t* num_post, int32_t* expert_off,
                 void* workspace, int64_t workspace_bytes, cudaStream_t stream);
int64_t align_workspace_bytes(int64_t numel, int num_experts);

// out[m,n] = sum_j scratch[m*top_k+j, n] over the slots whose (mapped) expert id lies in [0, E)
// (the slots the align stage kept), ascending j, fp32.
int launch_combine(const float* scratch, const int32_t* topk_ids, const int32_t* expert_map,
                   int num_map, int E, void* out, int out_dtype, int64_t M, int top_k, int64_t N,
                   cudaStream_t stream);

// Records one event pair of the optional GEMM timer (xkb_gemm_timer_enable) around
// the launches made while it is alive; does nothing when the timer is not armed.
struct GemmTimerScope {
  cudaStream_t stream;
  int slot;
  explicit GemmTimerScope(cudaStream_t s);
  ~GemmTimerScope();
};

// ---- programmatic dependent launch ------------------------------------------------
// The kernels of one fused call form a chain on the caller's stream (align -> gather -> grouped
// GEMM -> combine).  A link launched with launch_chained() may START while its predecessor is still
// running, once every CTA of the predecessor has executed chain_trigger() (or exited); it must call
// chain_wait() before it touches anything the predecessor writes - that returns when the predecessor
// (and, transitively, everything before it) has completed and its writes are visible.  What this
// buys is the launch latency and the prologue of each link (for the GEMM: barrier set-up, tensor
// memory allocation, descriptor prefetch), a few microseconds per link in a 200 microsecond call.
// A kernel launched the ordinary way sees both calls as no-ops.
#ifdef __CUDACC__
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                           Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#endif

// ---- device helpers --------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) {
  return __uint_as_float(bits16 << 16);
}
__device__ __forceinline__ float round_to_bf16(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}
// e2m1 magnitude table {0,.5,1,1.5,2,3,4,6}; bit 3 of the code is the sign.
__device__ __forceinline__ float e2m1_to_float(uint32_t code) {
  const uint32_t mag = code & 7u;
  // 2*value is the integer {0,1,2,3,4,6,8,12}
  const float v2 = (mag < 2u) ? (float)mag : (float)((2u + (mag & 1u)) << ((mag >> 1) - 1u));
  const float v = 0.5f * v2;
  return (code & 8u) ? -v : v;
}
// e8m0 scale: 2^(s-127); 0xFF decodes to 0 (the reference treats the NaN code as 0).
__device__ __forceinline__ float e8m0_to_float(uint32_t s) {
  if (s == 0xFFu) return 0.f;
  if (s == 0u) return __uint_as_float(0x00400000u);  // 2^-127 (subnormal)
  return __uint_as_float(s << 23);
}
#endif

}  // namespace xkb

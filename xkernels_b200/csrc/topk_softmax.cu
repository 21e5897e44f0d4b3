// MoE router: softmax over the experts, top-k, optional renormalisation (sm_100a).
//
// Contract (src/xkernels/ops/moe/topk_softmax.py:33-95 in the reference): logits are upcast to
// fp32, softmax runs over ALL experts, then the k largest probabilities are taken in DESCENDING
// probability with ties broken by ASCENDING expert id (a stable descending argsort), then the
// selected weights are optionally divided by their sum.  Equal logits give equal probabilities
// here as there, so the tie rule decides the same way.
//
// One warp per token row: lane l holds experts l, l + 32, ...; row maximum and sum by shuffles;
// k rounds of "best of my lane, then best of the warp" on the key (probability, -id).

#include <cuda_fp16.h>

#include "common.cuh"

namespace xkb {
namespace {

constexpr int kMaxPerLane = 32;               // experts per lane -> at most 1024 experts
constexpr int kWarpsPerBlock = 8;

template <typename T> __device__ __forceinline__ float load_logit(const T* p);
template <> __device__ __forceinline__ float load_logit<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float load_logit<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
template <> __device__ __forceinline__ float load_logit<__half>(const __half* p) { return __half2float(*p); }

// (probability, id) ordering of the contract: larger probability first, then smaller id
__device__ __forceinline__ bool better(float pa, int ia, float pb, int ib) {
  return pa > pb || (pa == pb && ia < ib);
}

template <typename T, int PER_LANE>
__global__ void __launch_bounds__(32 * kWarpsPerBlock)
topk_softmax_kernel(const T* __restrict__ gating, float* __restrict__ topk_w, int32_t* __restrict__ topk_ids,
                    int64_t M, int E, int topk, int renormalize) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= M) return;
  const T* x = gating + row * E;

  float p[PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int t = 0; t < PER_LANE; ++t) {
    const int e = lane + 32 * t;
    p[t] = e < E ? load_logit<T>(x + e) : -INFINITY;
    mx = fmaxf(mx, p[t]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int t = 0; t < PER_LANE; ++t) {
    const int e = lane + 32 * t;
    p[t] = e < E ? expf(p[t] - mx) : 0.f;
    sum += p[t];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
  for (int t = 0; t < PER_LANE; ++t) {
    const int e = lane + 32 * t;
    p[t] = e < E ? p[t] / sum : -1.f;   // -1 marks "not a candidate" (probabilities are >= 0)
  }

  float wsum = 0.f;
  float my_w = 0.f;     // lane j keeps the j-th selected weight (j < 32), further ones go out directly
  for (int j = 0; j < topk; ++j) {
    float bp = -1.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int t = 0; t < PER_LANE; ++t) {
      const int e = lane + 32 * t;
      if (better(p[t], e, bp, bi)) { bp = p[t]; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float op = __shfl_xor_sync(0xffffffffu, bp, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(op, oi, bp, bi)) { bp = op; bi = oi; }
    }
    // every lane now holds the same winner; its owner retires it
    if ((bi & 31) == lane) {
#pragma unroll
      for (int t = 0; t < PER_LANE; ++t)
        if (t == (bi >> 5)) p[t] = -1.f;
    }
    wsum += bp;
    if (lane == 0) topk_ids[row * topk + j] = bi;
    if (renormalize) {
      if (j < 32) { if (lane == j) my_w = bp; }
      else if (lane == 0) topk_w[row * topk + j] = bp;   // divided below
    } else if (lane == 0) {
      topk_w[row * topk + j] = bp;
    }
  }
  if (renormalize) {
    if (lane < topk) topk_w[row * topk + lane] = my_w / wsum;
    if (lane == 0)
      for (int j = 32; j < topk; ++j) topk_w[row * topk + j] = topk_w[row * topk + j] / wsum;
  }
}

template <typename T>
int launch_for_type(const void* gating, float* w, int32_t* ids, int64_t M, int E, int topk, int renorm,
                    cudaStream_t s) {
  const unsigned blocks = (unsigned)ceil_div(M, (int64_t)kWarpsPerBlock);
  const T* g = static_cast<const T*>(gating);
  const int per_lane = (E + 31) / 32;
#define XKB_TS_CASE(PL)                                                                                  \
  if (per_lane <= PL) {                                                                                  \
    topk_softmax_kernel<T, PL><<<blocks, 32 * kWarpsPerBlock, 0, s>>>(g, w, ids, M, E, topk, renorm);  \
    XKB_CHECK_LAUNCH("topk_softmax_kernel");                                                             \
    return XKB_OK;                                                                                       \
  }
  XKB_TS_CASE(1)
  XKB_TS_CASE(2)
  XKB_TS_CASE(4)
  XKB_TS_CASE(8)
  XKB_TS_CASE(16)
  XKB_TS_CASE(32)
#undef XKB_TS_CASE
  return fail(XKB_ERR_ARG, "topk_softmax: E=%d exceeds %d experts", E, 32 * kMaxPerLane);
}

}  // namespace
}  // namespace xkb

extern "C" int xkb_topk_softmax(const void* gating_output, int dtype, float* topk_weights, int32_t* topk_ids,
                                int64_t M, int E, int topk, int renormalize, void* stream) {
  using namespace xkb;
  XKB_REQUIRE(M >= 0 && E >= 1, "topk_softmax: bad shape M=%lld E=%d", (long long)M, E);
  XKB_REQUIRE(topk >= 1 && topk <= E, "topk_softmax: topk must satisfy 1 <= topk <= E (got topk=%d, E=%d)", topk, E);
  XKB_REQUIRE(E <= 32 * kMaxPerLane, "topk_softmax: E=%d exceeds %d experts", E, 32 * kMaxPerLane);
  if (M == 0) return XKB_OK;
  XKB_REQUIRE(gating_output != nullptr && topk_weights != nullptr && topk_ids != nullptr,
              "topk_softmax: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case XKB_BF16: return launch_for_type<__nv_bfloat16>(gating_output, topk_weights, topk_ids, M, E, topk, renormalize, s);
    case XKB_F32: return launch_for_type<float>(gating_output, topk_weights, topk_ids, M, E, topk, renormalize, s);
    case XKB_F16: return launch_for_type<__half>(gating_output, topk_weights, topk_ids, M, E, topk, renormalize, s);
    default: return fail(XKB_ERR_ARG, "topk_softmax: unsupported logits dtype code %d", dtype);
  }
}

// moe_sum_reduce and the fused ops' top-k combine for sm_100a.
//
//   out[m, h] = rsf * sum_k (w[m,k] or 1) * y[m,k,h]        fp32, ascending k
//
// HBM-bound: every thread owns 8 consecutive h of one token row and streams the
// top_k partial rows with 128-bit loads (bf16: one load, fp32: two), so a warp
// reads 512 B / 1 KiB contiguous per k.  No atomics, fixed summation order: the
// result is bit-reproducible run to run.  Reference semantics:
// src/xkernels/ops/moe/sum_reduce.py:20-39.
#include "common.cuh"

namespace xkb {
namespace {

template <typename T> struct Vec8;
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);   // plain loads: the rows may come from a kernel this one overlaps
    const uint32_t u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(u[i] << 16);
      v[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint32_t u[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      u[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(u[0], u[1], u[2], u[3]);
  }
};
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
};

__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ void from_f(float& d, float x) { d = x; }
__device__ __forceinline__ void from_f(__nv_bfloat16& d, float x) { d = __float2bfloat16_rn(x); }

// Validity of slot (m,k): the same predicate as the align stage (align.cu:map_expert), which
// drops a slot whose (mapped) expert id falls outside [0, E) and therefore never has its fp32
// row written.  The reference skips those slots too (src/xkernels/ops/moe/reference.py:59-63,
// mxfp4_reference.py:82-83).  ids == nullptr means every slot contributes (moe_sum_reduce).
__device__ __forceinline__ bool slot_valid(const int32_t* ids, const int32_t* emap, int num_map,
                                           int E, int64_t slot) {
  if (ids == nullptr) return true;
  int g = ids[slot];
  if (emap != nullptr) {
    if (g < 0 || g >= num_map) return false;
    g = emap[g];
  }
  return g >= 0 && g < E;
}

template <typename TY, typename TW, typename TO>
__global__ void __launch_bounds__(256)
sum_reduce_vec8_kernel(const TY* y, const TW* __restrict__ w, TO* __restrict__ out,
                       int64_t M, int top_k, int64_t H, float rsf, const int32_t* __restrict__ ids,
                       const int32_t* __restrict__ emap, int num_map, int E) {
  // As the combine of a fused call the slot rows come from the GEMM kernel before this one, which is
  // still running when this kernel starts: `y` is therefore not `const __restrict__` (no invariant /
  // non-coherent loads, which may deliver what was there before the wait).
  chain_wait();
  const int64_t hv = H >> 3;  // 8-wide columns per row
  const int64_t total = M * hv;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = idx / hv;
    const int64_t h = (idx - m * hv) << 3;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const TY* row = y + (m * top_k) * H + h;
#pragma unroll 4
    for (int k = 0; k < top_k; ++k) {
      if (!slot_valid(ids, emap, num_map, E, m * top_k + k)) continue;
      float v[8];
      Vec8<TY>::load(row + (int64_t)k * H, v);
      if (w != nullptr) {
        const float wk = to_f(w[m * top_k + k]);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += v[i] * wk;
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += v[i];
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] *= rsf;
    Vec8<TO>::store(out + m * H + h, acc);
  }
}

// Any H / any alignment.
template <typename TY, typename TW, typename TO>
__global__ void __launch_bounds__(256)
sum_reduce_scalar_kernel(const TY* __restrict__ y, const TW* __restrict__ w, TO* __restrict__ out,
                         int64_t M, int top_k, int64_t H, float rsf,
                         const int32_t* __restrict__ ids, const int32_t* __restrict__ emap,
                         int num_map, int E) {
  const int64_t total = M * H;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = idx / H, h = idx - m * H;
    float acc = 0.f;
    for (int k = 0; k < top_k; ++k) {
      if (!slot_valid(ids, emap, num_map, E, m * top_k + k)) continue;
      const float v = to_f(y[(m * top_k + k) * H + h]);
      acc += (w != nullptr) ? v * to_f(w[m * top_k + k]) : v;
    }
    from_f(out[idx], acc * rsf);
  }
}

template <typename TY, typename TW, typename TO>
int launch_typed(const void* y, const void* w, void* out, int64_t M, int top_k, int64_t H, float rsf,
                 const int32_t* ids, const int32_t* emap, int num_map, int E, cudaStream_t stream) {
  if (M == 0 || H == 0) return XKB_OK;
  const bool vec_ok = (H % 8 == 0) && (reinterpret_cast<uintptr_t>(y) % 16 == 0) &&
                      (reinterpret_cast<uintptr_t>(out) % 16 == 0);
  const int64_t work = vec_ok ? M * (H / 8) : M * H;
  // 148 SMs x 8 resident 256-thread CTAs; grid-stride covers the rest
  int64_t blocks = ceil_div(work, 256);
  const int64_t cap = 148 * 8 * 4;
  if (blocks > cap) blocks = cap;
  if (vec_ok) {
    XKB_CHECK_CUDA(launch_chained(sum_reduce_vec8_kernel<TY, TW, TO>, dim3((unsigned)blocks), dim3(256), 0, stream,
                                  static_cast<const TY*>(y), static_cast<const TW*>(w), static_cast<TO*>(out), M, top_k,
                                  H, rsf, ids, emap, num_map, E));
    XKB_CHECK_LAUNCH("sum_reduce_vec8_kernel");
  } else {
    sum_reduce_scalar_kernel<TY, TW, TO><<<(unsigned)blocks, 256, 0, stream>>>(
        static_cast<const TY*>(y), static_cast<const TW*>(w), static_cast<TO*>(out), M, top_k, H, rsf,
        ids, emap, num_map, E);
    XKB_CHECK_LAUNCH("sum_reduce_scalar_kernel");
  }
  return XKB_OK;
}

template <typename TY, typename TW>
int dispatch_out(int out_dtype, const void* y, const void* w, void* out, int64_t M, int top_k,
                 int64_t H, float rsf, const int32_t* ids, const int32_t* emap, int num_map,
                 int E, cudaStream_t s) {
  if (out_dtype == XKB_BF16)
    return launch_typed<TY, TW, __nv_bfloat16>(y, w, out, M, top_k, H, rsf, ids, emap, num_map, E, s);
  return launch_typed<TY, TW, float>(y, w, out, M, top_k, H, rsf, ids, emap, num_map, E, s);
}

// out[m, :] = sum_k w[m,k] * rows[row_index[m,k], :]   (fp32 rows, ascending k, fp32 sum).
// row_index < 0 skips the term.  One thread = 4 consecutive columns.
template <typename TO>
__global__ void __launch_bounds__(256)
gather_reduce_kernel(const float* __restrict__ rows, const int32_t* __restrict__ row_index,
                     const float* __restrict__ w, TO* __restrict__ out, int64_t M, int top_k, int64_t H) {
  const int64_t hv = H >> 2;
  const int64_t total = M * hv;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = idx / hv;
    const int64_t h = (idx - m * hv) << 2;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < top_k; ++k) {
      const int32_t r = row_index[m * top_k + k];
      if (r < 0) continue;
      const float4 v = __ldg(reinterpret_cast<const float4*>(rows + (int64_t)r * H + h));
      const float wk = (w != nullptr) ? w[m * top_k + k] : 1.f;
      acc.x += wk * v.x; acc.y += wk * v.y; acc.z += wk * v.z; acc.w += wk * v.w;
    }
    TO* o = out + m * H + h;
    from_f(o[0], acc.x); from_f(o[1], acc.y); from_f(o[2], acc.z); from_f(o[3], acc.w);
  }
}

}  // namespace

int launch_combine(const float* scratch, const int32_t* topk_ids, const int32_t* expert_map,
                   int num_map, int E, void* out, int out_dtype, int64_t M, int top_k, int64_t N,
                   cudaStream_t stream) {
  return dispatch_out<float, float>(out_dtype, scratch, nullptr, out, M, top_k, N, 1.0f, topk_ids,
                                    expert_map, num_map, E, stream);
}

}  // namespace xkb

extern "C" int xkb_moe_sum_reduce(const void* y, int y_dtype, const void* w, int w_dtype, void* out,
                                  int out_dtype, int64_t M, int top_k, int64_t H,
                                  float routed_scaling_factor, void* stream) {
  using namespace xkb;
  XKB_REQUIRE(M >= 0 && H >= 0 && top_k >= 0, "moe_sum_reduce: negative dimension");
  XKB_REQUIRE((y_dtype == XKB_BF16 || y_dtype == XKB_F32) &&
                  (out_dtype == XKB_BF16 || out_dtype == XKB_F32) &&
                  (w == nullptr || w_dtype == XKB_BF16 || w_dtype == XKB_F32),
              "moe_sum_reduce: dtype codes must be XKB_BF16 or XKB_F32");
  XKB_REQUIRE(M * H == 0 || (y != nullptr && out != nullptr) || top_k == 0,
              "moe_sum_reduce: null y/out pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const float rsf = routed_scaling_factor;
  if (y_dtype == XKB_BF16) {
    if (w != nullptr && w_dtype == XKB_BF16)
      return dispatch_out<__nv_bfloat16, __nv_bfloat16>(out_dtype, y, w, out, M, top_k, H, rsf, nullptr, nullptr, 0, 0, s);
    return dispatch_out<__nv_bfloat16, float>(out_dtype, y, w, out, M, top_k, H, rsf, nullptr, nullptr, 0, 0, s);
  }
  if (w != nullptr && w_dtype == XKB_BF16)
    return dispatch_out<float, __nv_bfloat16>(out_dtype, y, w, out, M, top_k, H, rsf, nullptr, nullptr, 0, 0, s);
  return dispatch_out<float, float>(out_dtype, y, w, out, M, top_k, H, rsf, nullptr, nullptr, 0, 0, s);
}

extern "C" int xkb_moe_gather_sum_reduce(const float* rows, const int32_t* row_index, const float* w,
                                         void* out, int out_dtype, int64_t M, int top_k, int64_t H,
                                         void* stream) {
  using namespace xkb;
  XKB_REQUIRE(M >= 0 && H >= 0 && top_k >= 0, "moe_gather_sum_reduce: negative dimension");
  XKB_REQUIRE(H % 4 == 0, "moe_gather_sum_reduce: H must be a multiple of 4 (got %lld)", (long long)H);
  XKB_REQUIRE(out_dtype == XKB_BF16 || out_dtype == XKB_F32, "moe_gather_sum_reduce: bad out_dtype");
  if (M == 0 || H == 0) return XKB_OK;
  XKB_REQUIRE(rows && row_index && out, "moe_gather_sum_reduce: null pointer");
  XKB_REQUIRE(reinterpret_cast<uintptr_t>(rows) % 16 == 0, "moe_gather_sum_reduce: rows must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int64_t blocks = ceil_div(M * (H / 4), 256);
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (out_dtype == XKB_BF16)
    gather_reduce_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, s>>>(
        rows, row_index, w, static_cast<__nv_bfloat16*>(out), M, top_k, H);
  else
    gather_reduce_kernel<float><<<(unsigned)blocks, 256, 0, s>>>(rows, row_index, w,
                                                                 static_cast<float*>(out), M, top_k, H);
  XKB_CHECK_LAUNCH("gather_reduce_kernel");
  return XKB_OK;
}

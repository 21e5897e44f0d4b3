// Generic SIMT grouped expert GEMMs (INT4 W4A16 and MXFP4) for sm_100a.
//
// These kernels take ANY shape the ops accept (N, K only need the packing
// granularity; fp32 or bf16 activations; M >= 1) and are the path for the odd
// and tiny shapes and for fp32 activations.  The tcgen05 kernels cover the
// large bf16 shapes.  One CTA = one 16-position block of the sorted routing
// (one expert) x 128 weight rows; a thread owns one weight row, streams its
// packed 4-bit words from global memory, dequantises in registers exactly as
// the reference does and accumulates 16 fp32 dot products against an fp32
// activation tile staged in shared memory.
//
// Arithmetic contracts (reference file:line):
//  * INT4: W = ((nib - 8) * scale) in fp32, rounded to bf16 iff A is bf16
//    (src/xkernels/ops/moe/w4a16.py:44-50, ops/moe/reference.py:54); fp32
//    accumulate; x topk_w in fp32 (reference.py:66-69).
//  * MXFP4: W = bf16(e2m1 * 2^(s-127)), 0xFF -> 0 (ops/gather/mxfp4.py:58-68);
//    gate_up rounded to bf16 (+ bf16 bias), clamp, silu(gate)*up rounded to
//    bf16, down rounded to bf16 (+ bf16 bias), x topk_w in fp32
//    (ops/moe/mxfp4_reference.py:90-110).
#include "moe_kernels.h"

namespace xkb {

constexpr int kSimtBM = kSimtBlock;    // positions per block (must equal the align block)
constexpr int kSimtBN = 128;   // weight rows per CTA (= threads)
constexpr int kSimtKC = 256;   // K elements staged per outer step

namespace {

__device__ __forceinline__ float load_a(const float* p) { return __ldg(p); }
__device__ __forceinline__ float load_a(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// Stage As[i][k] = A_row(i)[k0 + k] for the 16 positions of the block (0 beyond
// K or for padding positions).  rows[i] = source row index or -1.
template <typename TA, bool kRoundBf16>
__device__ __forceinline__ void stage_a(float (*As)[kSimtKC], const TA* __restrict__ A, int64_t lda,
                                        const int64_t* rows, int64_t k0, int64_t K) {
  for (int idx = threadIdx.x; idx < kSimtBM * kSimtKC; idx += kSimtBN) {
    const int i = idx / kSimtKC, k = idx - i * kSimtKC;
    float v = 0.f;
    if (rows[i] >= 0 && k0 + k < K) {
      v = load_a(A + rows[i] * lda + k0 + k);
      if (kRoundBf16) v = round_to_bf16(v);
    }
    As[i][k] = v;
  }
}

}  // namespace

// ---------------------------------------------------------------------------
// INT4 W4A16
// ---------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(kSimtBN)
int4_simt_kernel(const TA* __restrict__ A, const int32_t* __restrict__ packed,
                 const __nv_bfloat16* __restrict__ scale, const int32_t* __restrict__ sorted_ids,
                 const int32_t* __restrict__ expert_ids, const int32_t* __restrict__ num_post,
                 const float* __restrict__ topk_w, float* __restrict__ scratch, int64_t numel,
                 int64_t N, int64_t K, int top_k, int group, int mul_w, int round_out) {
  __shared__ float As[kSimtBM][kSimtKC];
  __shared__ int64_t rows[kSimtBM];
  __shared__ int32_t slots[kSimtBM];
  const int64_t pos0 = (int64_t)blockIdx.y * kSimtBM;
  if (pos0 >= num_post[0]) return;
  const int e = expert_ids[blockIdx.y];
  if (threadIdx.x < kSimtBM) {
    const int32_t s = sorted_ids[pos0 + threadIdx.x];
    slots[threadIdx.x] = s;
    rows[threadIdx.x] = (s >= 0 && s < numel) ? (int64_t)(s / top_k) : -1;
  }
  __syncthreads();
  const int64_t n = (int64_t)blockIdx.x * kSimtBN + threadIdx.x;
  const bool row_ok = n < N;
  const int64_t kp = K / 8, kg = K / group;
  const int32_t* wrow = packed + ((int64_t)e * N + (row_ok ? n : 0)) * kp;
  const __nv_bfloat16* srow = scale + ((int64_t)e * N + (row_ok ? n : 0)) * kg;
  float acc[kSimtBM];
#pragma unroll
  for (int i = 0; i < kSimtBM; ++i) acc[i] = 0.f;
  constexpr bool kBf16 = sizeof(TA) == 2;

  for (int64_t k0 = 0; k0 < K; k0 += kSimtKC) {
    __syncthreads();
    stage_a<TA, false>(As, A, K, rows, k0, K);
    __syncthreads();
    if (!row_ok) continue;
    const int words = (int)(((K - k0) < kSimtKC ? (K - k0) : kSimtKC) / 8);
    for (int wi = 0; wi < words; ++wi) {
      const uint32_t word = (uint32_t)__ldg(wrow + k0 / 8 + wi);
      const float sc = __bfloat162float(srow[(k0 + (int64_t)wi * 8) / group]);
      float w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float q = (float)((int)((word >> (4 * j)) & 0xFu) - 8);
        const float v = q * sc;
        w[j] = kBf16 ? round_to_bf16(v) : v;
      }
#pragma unroll
      for (int i = 0; i < kSimtBM; ++i) {
        const float* a = &As[i][wi * 8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i] = fmaf(a[j], w[j], acc[i]);
      }
    }
  }
  if (!row_ok) return;
#pragma unroll
  for (int i = 0; i < kSimtBM; ++i) {
    const int32_t s = slots[i];
    if (s < 0 || s >= numel) continue;
    float v = acc[i];
    if (mul_w) v = topk_w[s] * v;
    if (round_out && kBf16) v = round_to_bf16(v);
    scratch[(int64_t)s * N + n] = v;
  }
}

// ---------------------------------------------------------------------------
// MXFP4 stage 0: act[p, j] = bf16( silu(clamp(gate)) * clamp(up) )
// ---------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(kSimtBN)
mxfp4_stage0_simt_kernel(const TA* __restrict__ A, const uint8_t* __restrict__ w13,
                         const uint8_t* __restrict__ w13_scale, const __nv_bfloat16* __restrict__ b13,
                         const int32_t* __restrict__ sorted_ids, const int32_t* __restrict__ expert_ids,
                         const int32_t* __restrict__ num_post, __nv_bfloat16* __restrict__ act,
                         int64_t numel, int64_t hidden, int64_t ispp, int top_k, float limit) {
  __shared__ float As[kSimtBM][kSimtKC];
  __shared__ int64_t rows[kSimtBM];
  const int64_t pos0 = (int64_t)blockIdx.y * kSimtBM;
  if (pos0 >= num_post[0]) return;
  const int e = expert_ids[blockIdx.y];
  if (threadIdx.x < kSimtBM) {
    const int32_t s = sorted_ids[pos0 + threadIdx.x];
    rows[threadIdx.x] = (s >= 0 && s < numel) ? (int64_t)(s / top_k) : -1;
  }
  __syncthreads();
  const int64_t j = (int64_t)blockIdx.x * kSimtBN + threadIdx.x;
  const bool row_ok = j < ispp;
  const int64_t kb = hidden / 2, kg = hidden / 32;
  const int64_t jr = row_ok ? j : 0;
  const uint8_t* g_w = w13 + ((int64_t)e * 2 * ispp + jr) * kb;
  const uint8_t* u_w = w13 + ((int64_t)e * 2 * ispp + ispp + jr) * kb;
  const uint8_t* g_s = w13_scale + ((int64_t)e * 2 * ispp + jr) * kg;
  const uint8_t* u_s = w13_scale + ((int64_t)e * 2 * ispp + ispp + jr) * kg;
  float ag[kSimtBM], au[kSimtBM];
#pragma unroll
  for (int i = 0; i < kSimtBM; ++i) ag[i] = au[i] = 0.f;

  for (int64_t k0 = 0; k0 < hidden; k0 += kSimtKC) {
    __syncthreads();
    stage_a<TA, true>(As, A, hidden, rows, k0, hidden);
    __syncthreads();
    if (!row_ok) continue;
    const int groups = (int)(((hidden - k0) < kSimtKC ? (hidden - k0) : kSimtKC) / 32);
    for (int gi = 0; gi < groups; ++gi) {
      const int64_t kk = k0 + (int64_t)gi * 32;
      const float sg = e8m0_to_float(g_s[kk / 32]);
      const float su = e8m0_to_float(u_s[kk / 32]);
#pragma unroll
      for (int q = 0; q < 4; ++q) {  // 4 x 4 bytes = 32 codes
        const uint32_t wg = __ldg(reinterpret_cast<const uint32_t*>(g_w + kk / 2) + q);
        const uint32_t wu = __ldg(reinterpret_cast<const uint32_t*>(u_w + kk / 2) + q);
        float vg[8], vu[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          vg[t] = round_to_bf16(e2m1_to_float((wg >> (4 * t)) & 0xFu) * sg);
          vu[t] = round_to_bf16(e2m1_to_float((wu >> (4 * t)) & 0xFu) * su);
        }
#pragma unroll
        for (int i = 0; i < kSimtBM; ++i) {
          const float* a = &As[i][gi * 32 + q * 8];
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            ag[i] = fmaf(a[t], vg[t], ag[i]);
            au[i] = fmaf(a[t], vu[t], au[i]);
          }
        }
      }
    }
  }
  if (!row_ok) return;
  float bg = 0.f, bu = 0.f;
  if (b13 != nullptr) {
    bg = __bfloat162float(b13[(int64_t)e * 2 * ispp + j]);
    bu = __bfloat162float(b13[(int64_t)e * 2 * ispp + ispp + j]);
  }
#pragma unroll
  for (int i = 0; i < kSimtBM; ++i) {
    float g = round_to_bf16(ag[i]);
    float u = round_to_bf16(au[i]);
    if (b13 != nullptr) {
      g = round_to_bf16(g + bg);
      u = round_to_bf16(u + bu);
    }
    if (limit > 0.f) {
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
    }
    const float silu = g / (1.f + expf(-g));
    act[(pos0 + i) * ispp + j] = __float2bfloat16_rn(silu * u);
  }
}

// ---------------------------------------------------------------------------
// MXFP4 stage 1: scratch[slot, h] = float(bf16(act @ w2^T (+b2))) * w
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kSimtBN)
mxfp4_stage1_simt_kernel(const __nv_bfloat16* __restrict__ act, const uint8_t* __restrict__ w2,
                         const uint8_t* __restrict__ w2_scale, const __nv_bfloat16* __restrict__ b2,
                         const int32_t* __restrict__ sorted_ids, const int32_t* __restrict__ expert_ids,
                         const int32_t* __restrict__ num_post, const float* __restrict__ topk_w,
                         float* __restrict__ scratch, int64_t numel, int64_t hidden, int64_t ispp,
                         int mul_w) {
  __shared__ float As[kSimtBM][kSimtKC];
  __shared__ int64_t rows[kSimtBM];
  __shared__ int32_t slots[kSimtBM];
  const int64_t pos0 = (int64_t)blockIdx.y * kSimtBM;
  if (pos0 >= num_post[0]) return;
  const int e = expert_ids[blockIdx.y];
  if (threadIdx.x < kSimtBM) {
    const int32_t s = sorted_ids[pos0 + threadIdx.x];
    slots[threadIdx.x] = s;
    rows[threadIdx.x] = (s >= 0 && s < numel) ? pos0 + threadIdx.x : -1;
  }
  __syncthreads();
  const int64_t h = (int64_t)blockIdx.x * kSimtBN + threadIdx.x;
  const bool row_ok = h < hidden;
  const int64_t kb = ispp / 2, kg = ispp / 32;
  const uint8_t* wr = w2 + ((int64_t)e * hidden + (row_ok ? h : 0)) * kb;
  const uint8_t* sr = w2_scale + ((int64_t)e * hidden + (row_ok ? h : 0)) * kg;
  float acc[kSimtBM];
#pragma unroll
  for (int i = 0; i < kSimtBM; ++i) acc[i] = 0.f;

  for (int64_t k0 = 0; k0 < ispp; k0 += kSimtKC) {
    __syncthreads();
    stage_a<__nv_bfloat16, false>(As, act, ispp, rows, k0, ispp);
    __syncthreads();
    if (!row_ok) continue;
    const int groups = (int)(((ispp - k0) < kSimtKC ? (ispp - k0) : kSimtKC) / 32);
    for (int gi = 0; gi < groups; ++gi) {
      const int64_t kk = k0 + (int64_t)gi * 32;
      const float sc = e8m0_to_float(sr[kk / 32]);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t word = __ldg(reinterpret_cast<const uint32_t*>(wr + kk / 2) + q);
        float v[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) v[t] = round_to_bf16(e2m1_to_float((word >> (4 * t)) & 0xFu) * sc);
#pragma unroll
        for (int i = 0; i < kSimtBM; ++i) {
          const float* a = &As[i][gi * 32 + q * 8];
#pragma unroll
          for (int t = 0; t < 8; ++t) acc[i] = fmaf(a[t], v[t], acc[i]);
        }
      }
    }
  }
  if (!row_ok) return;
  const float bias = (b2 != nullptr) ? __bfloat162float(b2[(int64_t)e * hidden + h]) : 0.f;
#pragma unroll
  for (int i = 0; i < kSimtBM; ++i) {
    const int32_t s = slots[i];
    if (s < 0 || s >= numel) continue;
    float d = round_to_bf16(acc[i]);
    if (b2 != nullptr) d = round_to_bf16(d + bias);
    if (mul_w) d = d * topk_w[s];
    scratch[(int64_t)s * hidden + h] = d;
  }
}

// ---------------------------------------------------------------------------
// host launchers (used by fused.cu)
// ---------------------------------------------------------------------------
int launch_int4_simt(const void* A, int a_dtype, const int32_t* packed, const void* scale,
                     const Routing& r, const float* topk_w, float* scratch, int64_t N, int64_t K,
                     int top_k, int group, int mul_w, cudaStream_t stream, int round_out) {
  if (r.max_blocks == 0 || N == 0) return XKB_OK;
  XKB_REQUIRE(r.block == kSimtBM, "int4 SIMT kernel needs align block %d", kSimtBM);
  XKB_REQUIRE(r.max_blocks <= 65535 * 32, "too many routing blocks for one launch");
  dim3 grid((unsigned)ceil_div(N, kSimtBN), (unsigned)r.max_blocks);
  XKB_REQUIRE(grid.y <= 65535u, "routing has %u blocks; the SIMT path supports at most 65535", grid.y);
  GemmTimerScope timed(stream);
  if (a_dtype == XKB_BF16)
    int4_simt_kernel<__nv_bfloat16><<<grid, kSimtBN, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(A), packed, static_cast<const __nv_bfloat16*>(scale),
        r.sorted_ids, r.expert_ids, r.num_post, topk_w, scratch, r.numel, N, K, top_k, group, mul_w, round_out);
  else
    int4_simt_kernel<float><<<grid, kSimtBN, 0, stream>>>(
        static_cast<const float*>(A), packed, static_cast<const __nv_bfloat16*>(scale), r.sorted_ids,
        r.expert_ids, r.num_post, topk_w, scratch, r.numel, N, K, top_k, group, mul_w, round_out);
  XKB_CHECK_LAUNCH("int4_simt_kernel");
  return XKB_OK;
}

// ---------------------------------------------------------------------------
// INT4 two-GEMM expert layer on the generic kernels: gate_up slot rows (fp32) -> SwiGLU per slot ->
// down GEMM over the slots' activation rows (every slot is its own "token": top_k = 1 below) with
// the weighted rows rounded to the activation dtype.
// ---------------------------------------------------------------------------
namespace {
template <typename TA>
__global__ void __launch_bounds__(256)
swiglu_rows_kernel(const float* __restrict__ rows1, TA* __restrict__ act, int64_t numel, int64_t inter, float limit,
                   const int32_t* __restrict__ ids, const int32_t* __restrict__ emap, int num_map, int E) {
  const int64_t total = numel * inter;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t s = i / inter, j = i - s * inter;
    // slots the align stage dropped have no gate_up row: same predicate as the combine
    int g = ids[s];
    if (emap != nullptr) g = (g < 0 || g >= num_map) ? -1 : emap[g];
    if (g < 0 || g >= E) continue;
    float gate = rows1[s * 2 * inter + j], up = rows1[s * 2 * inter + inter + j];
    if (sizeof(TA) == 2) { gate = round_to_bf16(gate); up = round_to_bf16(up); }   // the first GEMM's output dtype
    if (limit > 0.f) { gate = fminf(gate, limit); up = fminf(fmaxf(up, -limit), limit); }
    const float v = gate / (1.f + expf(-gate)) * up;
    if (sizeof(TA) == 2) act[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<float*>(act)[i] = v;
  }
}
}  // namespace

int launch_int4_ffn_simt(const void* A, int a_dtype, const int32_t* w13, const void* s13, const int32_t* w2,
                         const void* s2, const Routing& r, const int32_t* topk_ids, const int32_t* expert_map,
                         int num_map, int E, const float* topk_w, float* rows1, void* act, float* scratch,
                         int64_t hidden, int64_t inter, int top_k, int group, float limit, cudaStream_t stream) {
  int rc = launch_int4_simt(A, a_dtype, w13, s13, r, nullptr, rows1, 2 * inter, hidden, top_k, group, 0, stream);
  if (rc != XKB_OK) return rc;
  if (r.numel > 0 && inter > 0) {
    int64_t blocks = ceil_div(r.numel * inter, 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (a_dtype == XKB_BF16)
      swiglu_rows_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>(
          rows1, static_cast<__nv_bfloat16*>(act), r.numel, inter, limit, topk_ids, expert_map, num_map, E);
    else
      swiglu_rows_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>(rows1, static_cast<float*>(act), r.numel, inter,
                                                                      limit, topk_ids, expert_map, num_map, E);
    XKB_CHECK_LAUNCH("swiglu_rows_kernel");
  }
  // slot s reads activation row s: the same routing with one slot per "token"
  return launch_int4_simt(act, a_dtype, w2, s2, r, topk_w, scratch, hidden, inter, 1, group, 1, stream, 1);
}

int launch_mxfp4_simt(const void* A, int a_dtype, const uint8_t* w13, const uint8_t* w13_scale,
                      const uint8_t* w2, const uint8_t* w2_scale, const void* b13, const void* b2,
                      const Routing& r, const float* topk_w, __nv_bfloat16* act, float* scratch,
                      int64_t hidden, int64_t ispp, int top_k, float limit, int mul_w,
                      cudaStream_t stream) {
  if (r.max_blocks == 0) return XKB_OK;
  XKB_REQUIRE(r.block == kSimtBM, "mxfp4 SIMT kernels need align block %d", kSimtBM);
  XKB_REQUIRE(r.max_blocks <= 65535, "routing has %lld blocks; the SIMT path supports at most 65535",
              (long long)r.max_blocks);
  dim3 g0((unsigned)ceil_div(ispp, kSimtBN), (unsigned)r.max_blocks);
  GemmTimerScope timed(stream);
  if (a_dtype == XKB_BF16)
    mxfp4_stage0_simt_kernel<__nv_bfloat16><<<g0, kSimtBN, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(A), w13, w13_scale, static_cast<const __nv_bfloat16*>(b13),
        r.sorted_ids, r.expert_ids, r.num_post, act, r.numel, hidden, ispp, top_k, limit);
  else
    mxfp4_stage0_simt_kernel<float><<<g0, kSimtBN, 0, stream>>>(
        static_cast<const float*>(A), w13, w13_scale, static_cast<const __nv_bfloat16*>(b13),
        r.sorted_ids, r.expert_ids, r.num_post, act, r.numel, hidden, ispp, top_k, limit);
  XKB_CHECK_LAUNCH("mxfp4_stage0_simt_kernel");
  dim3 g1((unsigned)ceil_div(hidden, kSimtBN), (unsigned)r.max_blocks);
  mxfp4_stage1_simt_kernel<<<g1, kSimtBN, 0, stream>>>(
      act, w2, w2_scale, static_cast<const __nv_bfloat16*>(b2), r.sorted_ids, r.expert_ids, r.num_post,
      topk_w, scratch, r.numel, hidden, ispp, mul_w);
  XKB_CHECK_LAUNCH("mxfp4_stage1_simt_kernel");
  return XKB_OK;
}

}  // namespace xkb

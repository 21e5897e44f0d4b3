// Launchers of the grouped expert GEMM kernels (SIMT and tcgen05 paths).
#pragma once
#include "common.cuh"

namespace xkb {

constexpr int kSimtBlock = 16;  // align block the SIMT kernels consume

// ---- generic SIMT path (moe_simt.cu) ---------------------------------------
int launch_int4_simt(const void* A, int a_dtype, const int32_t* packed, const void* scale,
                     const Routing& r, const float* topk_w, float* scratch, int64_t N, int64_t K,
                     int top_k, int group, int mul_w, cudaStream_t stream, int round_out = 0);
int launch_mxfp4_simt(const void* A, int a_dtype, const uint8_t* w13, const uint8_t* w13_scale,
                      const uint8_t* w2, const uint8_t* w2_scale, const void* b13, const void* b2,
                      const Routing& r, const float* topk_w, __nv_bfloat16* act, float* scratch,
                      int64_t hidden, int64_t ispp, int top_k, float limit, int mul_w,
                      cudaStream_t stream);

// ---- tcgen05 path (moe_tc.cu) ----------------------------------------------
bool int4_tc_supported(int a_dtype, int64_t M, int64_t N, int64_t K, int E, int top_k, int group);
int int4_tc_block(int64_t numel, int E);
int64_t int4_tc_workspace_bytes(int64_t numel, int64_t N, int64_t K, int E);
int launch_int4_tc(const void* A, const int32_t* packed, const void* scale, const Routing& r,
                   const float* topk_w, float* scratch, int64_t N, int64_t K, int E, int top_k,
                   int mul_w, void* tc_ws, int* status, cudaStream_t stream);

// INT4 two-GEMM expert layer (gate_up + SwiGLU, then down with bf16-rounded weighted slot rows)
bool int4_ffn_tc_supported(int a_dtype, int64_t M, int64_t hidden, int64_t inter, int E, int top_k, int group);
int launch_int4_ffn_tc(const void* A, const int32_t* w13, const void* s13, const int32_t* w2, const void* s2,
                       const Routing& r, const float* topk_w, __nv_bfloat16* act, float* scratch, int64_t hidden,
                       int64_t inter, int E, int top_k, float limit, void* tc_ws, int* status, cudaStream_t stream);
int launch_int4_ffn_simt(const void* A, int a_dtype, const int32_t* w13, const void* s13, const int32_t* w2,
                         const void* s2, const Routing& r, const int32_t* topk_ids, const int32_t* expert_map,
                         int num_map, int E, const float* topk_w, float* rows1, void* act, float* scratch,
                         int64_t hidden, int64_t inter, int top_k, int group, float limit, cudaStream_t stream);

bool mxfp4_tc_supported(int a_dtype, int64_t M, int64_t hidden, int64_t ispp, int E, int top_k);
int mxfp4_tc_block(int64_t numel, int E);
int64_t mxfp4_tc_workspace_bytes(int64_t numel, int64_t hidden, int64_t ispp, int E);
int launch_mxfp4_tc(const void* A, const uint8_t* w13, const uint8_t* w13_scale, const uint8_t* w2,
                    const uint8_t* w2_scale, const void* b13, const void* b2, const Routing& r,
                    const float* topk_w, __nv_bfloat16* act, float* scratch, int64_t hidden,
                    int64_t ispp, int E, int top_k, float limit, int mul_w, void* tc_ws, int* status,
                    cudaStream_t stream);

}  // namespace xkb

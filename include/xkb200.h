/*
 * xkb200 — C ABI of the B200 (sm_100a) fused-MoE hot path.
 *
 * Every pointer is a raw DEVICE pointer unless the parameter name ends in
 * `_host`.  `stream` is a `cudaStream_t` passed as `void*` (NULL = the legacy
 * default stream).  Every entry point returns 0 on success and a negative
 * `XKB_ERR_*` code on failure; `xkb_last_error()` then holds a readable
 * message for the calling thread.  Nothing here allocates device memory: the
 * caller owns inputs, outputs and the workspace whose size the matching
 * `*_workspace_bytes` query reports.
 *
 * The citations name the reference interface each entry point stands in for
 * (paths inside the ResearchComputer/xkernels tree).
 */
#ifndef XKB200_H_
#define XKB200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define XKB_OK 0
#define XKB_ERR_ARG (-1)       /* bad argument / unsupported shape            */
#define XKB_ERR_CUDA (-2)      /* a CUDA runtime or driver call failed        */
#define XKB_ERR_WORKSPACE (-3) /* workspace missing or too small              */
#define XKB_ERR_DEVICE (-4)    /* a kernel reported a bounded-wait time-out   */

/* dtype codes used by the `*_dtype` parameters */
#define XKB_BF16 0
#define XKB_F32 1
#define XKB_F16 2 /* accepted for router logits only */

/* kernel-path selectors for the `path` parameters */
#define XKB_PATH_AUTO 0  /* tensor-core kernel when the shape allows, else SIMT */
#define XKB_PATH_SIMT 1  /* force the generic SIMT kernels                      */
#define XKB_PATH_TC 2    /* force the tcgen05 kernels (error if shape unfit)    */

/* Library / build identification. */
const char* xkb_version(void);
/* Message of the last failure on the calling thread ("" if none). */
const char* xkb_last_error(void);
/* Number of kernel launches issued by this library since load (all threads). */
int64_t xkb_launch_count(void);

/* ------------------------------------------------------------------------
 * moe_align_block_size
 * Replaces: src/xkernels/ops/moe/w4a16.py:53-101 (moe_align_block_size_ref),
 *           src/xkernels/ops/moe/triton/align_kernel.py:156-248 (Triton launcher)
 *           and, with `expert_map`, w4a16.py:104-155 / align_kernel.py:251-312.
 *
 * topk_ids      [numel] int32 expert id per token-slot (flattened [M, top_k]).
 * expert_map    NULL, or [num_map] int32 global->local map (-1 = not local);
 *               slots whose expert is not local are dropped.  `num_experts`
 *               is then the LOCAL expert count.
 * sorted_ids    [numel + (num_experts+1)*(block_size-1)] int32, every entry
 *               written (unused entries = numel).
 * expert_ids    [ceil(len(sorted_ids)/block_size)] int32, every entry written
 *               (entries past the used blocks = 0).
 * num_post_pad  [1] int32.
 * expert_offsets NULL or [num_experts+1] int32: start of each expert's padded
 *               run in sorted_ids (entry num_experts = num_post_pad).
 * workspace     xkb_moe_align_workspace_bytes(numel, num_experts) bytes.
 * ---------------------------------------------------------------------- */
int64_t xkb_moe_align_workspace_bytes(int64_t numel, int num_experts);
int xkb_moe_align_block_size(const int32_t* topk_ids, int64_t numel,
                             int num_experts, int block_size,
                             const int32_t* expert_map, int num_map,
                             int32_t* sorted_ids, int32_t* expert_ids,
                             int32_t* num_post_pad, int32_t* expert_offsets,
                             void* workspace, int64_t workspace_bytes,
                             void* stream);

/* ------------------------------------------------------------------------
 * xkb_moe_align_block_size_static: the same operation and outputs as
 * xkb_moe_align_block_size, for callers that cannot provide scratch memory.
 * It has no counterpart in the reference.
 *
 * Who needs it: code that is not allowed to create device memory at the point
 * of the call - a plug-in living inside another runtime's memory pool, a
 * serving loop that has frozen its allocator, a plain C caller without one.
 * The scratch of the multi-launch path (the chunk x expert count matrix) is a
 * fixed array compiled into the library, 259 KiB on every GPU that loads
 * the library, kept until the process ends.  The call makes no cudaMalloc /
 * cudaFree and uses no allocating library routine; inputs and outputs are
 * still the caller's.
 *
 * Limits: numel <= 262144 token-slots and num_experts <= 256; larger
 * arguments are refused with XKB_ERR_ARG and a message that names the limit.
 * The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress, for the device that is current at the call, which
 * must be the device `stream` belongs to) and remembers it; make that first
 * call before starting any stream capture.  All calls on a device
 * share the one array, which keeps whatever the previous call left in it (no
 * part of it needs clearing: every entry that is read is first rewritten by
 * the same call).  Two calls that overlap on the GPU - different streams, or
 * different host threads - race on it and must be serialised by the caller.
 * ---------------------------------------------------------------------- */
int xkb_moe_align_block_size_static(const int32_t* topk_ids, int64_t numel,
                                    int num_experts, int block_size,
                                    const int32_t* expert_map, int num_map,
                                    int32_t* sorted_ids, int32_t* expert_ids,
                                    int32_t* num_post_pad,
                                    int32_t* expert_offsets, void* stream);

/* ------------------------------------------------------------------------
 * topk_softmax: the router step immediately before the path.
 * Replaces: src/xkernels/ops/moe/topk_softmax.py:33-95 (topk_softmax_ref) and
 * triton/topk_softmax_kernel.py:38- (spec registry/ops/topk_softmax.spec.json).
 *
 * gating_output [M, E] logits (dtype XKB_BF16 / XKB_F32 / XKB_F16, row major),
 * topk_weights [M, topk] fp32, topk_ids [M, topk] int32.  Softmax in fp32 over
 * all E experts, then the topk largest probabilities in descending order, ties
 * broken by ascending expert id, then (renormalize != 0) divided by their sum.
 * E <= 1024; 1 <= topk <= E (XKB_ERR_ARG otherwise, as the reference raises
 * ValueError).  One launch, no workspace.
 * ---------------------------------------------------------------------- */
int xkb_topk_softmax(const void* gating_output, int dtype, float* topk_weights,
                     int32_t* topk_ids, int64_t M, int E, int topk,
                     int renormalize, void* stream);

/* ------------------------------------------------------------------------
 * moe_sum_reduce: out[m,:] = rsf * sum_k (w[m,k] or 1) * y[m,k,:]
 * Replaces: src/xkernels/ops/moe/sum_reduce.py:20-39 (reference),
 *           src/xkernels/ops/moe/triton/sum_reduce_kernel.py:66-100,
 *           src/xkernels/ops/moe/cute/entry.py:19-40.
 * y [M, top_k, H] (y_dtype), w NULL or [M, top_k] (w_dtype), out [M, H]
 * (out_dtype).  The sum runs in fp32 in ascending k, so it is deterministic.
 * ---------------------------------------------------------------------- */
int xkb_moe_sum_reduce(const void* y, int y_dtype, const void* w, int w_dtype,
                       void* out, int out_dtype, int64_t M, int top_k,
                       int64_t H, float routed_scaling_factor, void* stream);

/* ------------------------------------------------------------------------
 * fused_moe_int4_w4a16: out[m] = sum_j w[m,j] * (A[m] @ dequant(W[e_mj])^T)
 * Replaces: src/xkernels/ops/moe/reference.py:22-70 (moe_w4a16_ref) and
 *           src/xkernels/ops/moe/triton/moe_int4_kernel.py:438-577 (Triton
 *           entry: align + grouped GEMM + top-k combine).
 * A [M,K] (a_dtype), packed [E,N,K/8] int32 (low nibble = lowest k, zero
 * point 8), scale [E,N,K/group] bf16, topk_ids [M,top_k] int32, topk_w
 * [M,top_k] fp32, expert_map NULL or [num_map] int32, out [M,N] (a_dtype).
 * ---------------------------------------------------------------------- */
int64_t xkb_fused_moe_int4_w4a16_workspace_bytes(int64_t M, int64_t N,
                                                 int64_t K, int E, int top_k,
                                                 int a_dtype);
int xkb_fused_moe_int4_w4a16(const void* A, int a_dtype, const int32_t* packed,
                             const void* scale, const int32_t* topk_ids,
                             const float* topk_w, const int32_t* expert_map,
                             int num_map, void* out, int64_t M, int64_t N,
                             int64_t K, int E, int top_k, int group_size,
                             int mul_routed_weight, int path, void* workspace,
                             int64_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------
 * fused_moe_int4_ffn: one expert layer made of two INT4 W4A16 GEMMs,
 *   out[m] = sum_j bf16( w[m,j] * (act_mj @ dequant(W2[e_mj])^T) ),
 *   act_mj = bf16( silu(gate) * up ),  [gate | up] = bf16( A[m] @ dequant(W13[e_mj])^T )
 * in one call: align -> gate_up GEMM with fused SwiGLU -> down GEMM -> combine.
 * The reference has no such op; it stands for what a caller of the reference
 * composes from fused_moe_int4_w4a16 (ops/moe/interface.py:19-32) twice, with
 * top_k = 1 over the slots, and moe_sum_reduce (ops/moe/sum_reduce.py:20-39),
 * and it rounds where that composition rounds.  The two shapes are those of
 * meta/benchmarks/bench_moe_int4_w4a16.py:3-12 (gate_up N = 2*inter, K = hidden;
 * down N = hidden, K = inter).  w13_packed [E, 2*inter, hidden/8] int32 with the
 * gate rows first, w13_scale [E, 2*inter, hidden/group] bf16, w2_packed
 * [E, hidden, inter/8], w2_scale [E, hidden, inter/group]; swiglu_limit <= 0:
 * no clamp, else gate <= limit and |up| <= limit as in fused_moe_mxfp4.
 * ---------------------------------------------------------------------- */
int64_t xkb_fused_moe_int4_ffn_workspace_bytes(int64_t M, int64_t hidden,
                                               int64_t inter, int E, int top_k,
                                               int a_dtype);
int xkb_fused_moe_int4_ffn(const void* A, int a_dtype, const int32_t* w13_packed,
                           const void* w13_scale, const int32_t* w2_packed,
                           const void* w2_scale, const int32_t* topk_ids,
                           const float* topk_w, const int32_t* expert_map,
                           int num_map, void* out, int64_t M, int64_t hidden,
                           int64_t inter, int E, int top_k, int group_size,
                           float swiglu_limit, int path, void* workspace,
                           int64_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------
 * Expert-parallel building blocks (all-to-all mode).  The reference has no
 * all-to-all; its expert-parallel contract is "per-rank partials sum to the
 * dense result" (tests/test_moe_int4_ep.py:152-177).  These two calls are the
 * local halves around the NCCL exchanges:
 *
 * xkb_moe_int4_w4a16_rows: as xkb_fused_moe_int4_w4a16 but WITHOUT the top-k
 *   combine: rows_out [M*top_k, N] fp32, row = token*top_k + j (the grouped
 *   GEMM stage of triton/moe_int4_kernel.py:550-577 before its `.sum(1)`).
 *   Same workspace size as the fused call.
 * xkb_moe_gather_sum_reduce: out[m,:] = sum_k w[m,k] * rows[row_index[m,k],:]
 *   in fp32, ascending k (row_index < 0 skips); the combine of
 *   ops/moe/reference.py:59-69 over rows that came back in exchange order.
 * ---------------------------------------------------------------------- */
int xkb_moe_int4_w4a16_rows(const void* A, int a_dtype, const int32_t* packed,
                            const void* scale, const int32_t* topk_ids,
                            const float* topk_w, float* rows_out, int64_t M,
                            int64_t N, int64_t K, int E, int top_k,
                            int group_size, int mul_routed_weight, int path,
                            void* workspace, int64_t workspace_bytes,
                            void* stream);
 /* xkb_moe_int4_w4a16_partial: the expert side of the all-to-all mode in one
 *   call.  A [M,K] are the received rows, routing [M, 2*top_k] int32 what
 *   travelled with them (top_k local expert ids, -1 = slot served on another
 *   rank, then the top_k routing weights' fp32 bit patterns; the layout
 *   xkb_ep_plan writes).  out [M,N] fp32 = per received row the weighted sum
 *   over its local experts in ascending slot order, i.e. the rank's partial
 *   of ops/moe/reference.py:59-69 before the final cast. */
int64_t xkb_moe_int4_w4a16_partial_workspace_bytes(int64_t M, int64_t N,
                                                   int64_t K, int E, int top_k,
                                                   int a_dtype);
int xkb_moe_int4_w4a16_partial(const void* A, int a_dtype,
                               const int32_t* packed, const void* scale,
                               const int32_t* routing, float* out, int64_t M,
                               int64_t N, int64_t K, int E, int top_k,
                               int group_size, int path, void* workspace,
                               int64_t workspace_bytes, void* stream);
int xkb_moe_gather_sum_reduce(const float* rows, const int32_t* row_index,
                              const float* w, void* out, int out_dtype,
                              int64_t M, int top_k, int64_t H, void* stream);

/* xkb_set_sm_margin: the grouped-GEMM kernels are persistent, one CTA per SM.
 * A margin of n keeps n SMs free (process-wide, until changed), so that
 * kernels launched on other streams -- NCCL's exchanges in the chunked
 * expert-parallel pipeline -- can run beside them instead of behind them.
 * No reference counterpart.  0 <= n <= 128; default 0. */
int xkb_set_sm_margin(int sms);

/* xkb_ep_plan: the dispatch plan of the all-to-all mode, computed on the device
 * without a host read (three launches).  No reference counterpart (the
 * reference replicates tokens, ops/moe/interface.py:37-57); the host-side
 * statement of the same plan is xkernels_b200/ep.py:plan_dispatch.
 * A token goes once to every rank that owns one of its top-k experts.  Pairs
 * (token, rank) are listed grouped by (token chunk, rank), ascending token
 * inside a group.  Outputs (all int32, sized for the worst case of one pair per
 * slot): pair_token [M*top_k], pair_dest [M*top_k], routing [M*top_k, 2*top_k]
 * (top_k local expert ids, -1 where the slot goes elsewhere, then the top_k
 * routing weights' fp32 bit patterns), pair_of [M, world] (position of pair
 * (token, rank), -1 if none), counts [chunks*world] pairs per group, info[2] =
 * {number of pairs, number of expert ids outside [0, experts_per_rank*world)}.
 * round_robin = 0: rank r owns experts [r*experts_per_rank, ...); 1: expert g
 * lives on rank g % world as local expert g / world; 2: as 1, but every second
 * group of `world` experts is dealt in reverse rank order.  expert_table, if not
 * NULL, overrides all three: [experts_per_rank*world, 2] int32 on the device,
 * (destination rank, expert index on that rank) per global expert as THIS rank
 * sees it - a rank that holds a replica of a popular expert names itself there,
 * so those slots never leave the GPU.  top_k <= 32. */
int64_t xkb_ep_plan_workspace_bytes(int64_t M, int top_k, int world, int chunks);
int xkb_ep_plan(const int32_t* topk_ids, const float* topk_w, int64_t M, int top_k,
                int experts_per_rank, int world, int round_robin,
                const int32_t* expert_table, int chunks,
                int32_t* pair_token, int32_t* pair_dest, int32_t* routing,
                int32_t* pair_of, int32_t* counts, int32_t* info, void* workspace,
                int64_t workspace_bytes, void* stream);

/* xkb_gather_rows: dst[p,:] = src[index[p],:] for p < *count_dev (count_dev NULL:
 * for all max_rows positions); rows of row_bytes bytes, a multiple of 16.  Fills
 * the dispatch send buffer of the all-to-all mode from the plan's pair_token
 * list while the host still waits for the pair counts: the row count is read on
 * the device (the plan's info[0]).  No reference counterpart. */
int xkb_gather_rows(const void* src, int64_t src_rows, int64_t row_bytes,
                    const int32_t* index, const int32_t* count_dev,
                    int64_t max_rows, void* dst, void* stream);

/* ------------------------------------------------------------------------
 * fused_moe_mxfp4: gate_up GEMM -> clamped SwiGLU -> down GEMM -> combine
 * Replaces: src/xkernels/ops/moe/mxfp4_reference.py:28-112 (moe_mxfp4_ref)
 *           and src/xkernels/ops/moe/triton/moe_mxfp4_kernel.py:487-568.
 * A [M,hidden] (a_dtype), w13 [E,2*ispp,hidden/2] u8, w13_scale
 * [E,2*ispp,hidden/32] u8 (e8m0), w2 [E,hidden,ispp/2] u8, w2_scale
 * [E,hidden,ispp/32] u8, b13 NULL or [E,2*ispp] bf16, b2 NULL or [E,hidden]
 * bf16, out [M,hidden] (a_dtype).  swiglu_limit <= 0 disables the clamp.
 * ---------------------------------------------------------------------- */
int64_t xkb_fused_moe_mxfp4_workspace_bytes(int64_t M, int64_t hidden,
                                            int64_t ispp, int E, int top_k);
int xkb_fused_moe_mxfp4(const void* A, int a_dtype, const uint8_t* w13,
                        const uint8_t* w13_scale, const uint8_t* w2,
                        const uint8_t* w2_scale, const int32_t* topk_ids,
                        const float* topk_w, const void* b13, const void* b2,
                        const int32_t* expert_map, int num_map, void* out,
                        int64_t M, int64_t hidden, int64_t ispp, int E,
                        int top_k, float swiglu_limit, int mul_routed_weight,
                        int path, void* workspace, int64_t workspace_bytes,
                        void* stream);

/* ------------------------------------------------------------------------
 * Device status of the last fused call that used `workspace`: synchronises
 * `stream`, reads the status word in the workspace header and returns
 * XKB_ERR_DEVICE if the word is not zero.  Low byte of the word: 1 = a
 * tcgen05 kernel gave up one of its bounded waits (the wait site in the upper
 * bits), 2 = an MXFP4 scale byte outside the range the 128-token instance of
 * the tcgen05 path converts, 3 = a kernel read a routing value (token-block
 * count, expert id) outside what the routing buffers can hold and skipped the
 * work instead of using it as an index.
 * The reference reports kernel failures as Python exceptions raised by the
 * launch (src/xkernels/_dispatch.py:204-240); this is the explicit query.
 * ---------------------------------------------------------------------- */
int xkb_workspace_status(const void* workspace, void* stream);

/* ------------------------------------------------------------------------
 * xkb_selftest_bounded_wait: exercises the abort path of the tcgen05 kernels
 * on purpose and harmlessly.  One small kernel allocates tensor memory and
 * waits, with a 20 microsecond budget, on an mbarrier that nothing arrives on;
 * the wait runs out, the kernel writes its status word into the workspace
 * header, releases tensor memory and returns.  xkb_workspace_status on the
 * same workspace then returns XKB_ERR_DEVICE, and the next fused call works.
 * Nothing traps, faults or spins without a limit.  No reference counterpart
 * (the reference's kernels have no device-side waits to bound).
 * ---------------------------------------------------------------------- */
int xkb_selftest_bounded_wait(void* workspace, int64_t workspace_bytes,
                              void* stream);

/* ------------------------------------------------------------------------
 * Measurement support: time the expert-GEMM kernel(s) of each fused call with
 * CUDA events recorded on the caller's stream around their launch.
 * `xkb_gemm_timer_enable(n)` arms n event pairs (0 disarms); each fused call
 * then uses the next pair; `xkb_gemm_timer_read` waits for the recorded
 * pairs, writes their durations in milliseconds to the HOST array and re-arms.
 * The reference times whole ops from Python
 * (src/xkernels/utils/benchmarking.py:68-141); per-kernel timing is new here.
 * Not thread-safe: arm, run and read from one thread.
 * ---------------------------------------------------------------------- */
int xkb_gemm_timer_enable(int max_calls);
int xkb_gemm_timer_read(float* ms_host, int capacity, int* count_host);

#ifdef __cplusplus
}
#endif
#endif /* XKB200_H_ */

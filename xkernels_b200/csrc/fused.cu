// Host side of the fused ops: workspace carving, kernel-path choice and the
// launch sequence  align -> grouped GEMM(s) -> fixed-order fp32 combine.
// Everything is enqueued on the caller's stream; no host synchronisation and no
// allocation happens here.
#include "common.cuh"
#include "moe_kernels.h"

#include <vector>

namespace xkb {

std::atomic<int64_t> g_launches{0};

char* last_error_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}

// ---- optional per-call timing of the grouped-GEMM kernel(s) -----------------
// A ring of event pairs; when enabled, every fused call records one pair around
// its expert GEMM launch(es) on the caller's stream.
struct GemmTimer {
  std::vector<cudaEvent_t> start, stop;
  int used = 0;
  bool enabled = false;
};
static GemmTimer g_timer;

// Scopes nest: only the outermost one records (two GEMMs that overlap are timed as one span, and no
// event lands between them, which would serialise them).
static thread_local int g_timer_depth = 0;
GemmTimerScope::GemmTimerScope(cudaStream_t s) : stream(s), slot(-1) {
  if (g_timer_depth++ == 0 && g_timer.enabled && g_timer.used < (int)g_timer.start.size()) {
    slot = g_timer.used++;
    cudaEventRecord(g_timer.start[slot], stream);
  }
}
GemmTimerScope::~GemmTimerScope() {
  --g_timer_depth;
  if (slot >= 0) cudaEventRecord(g_timer.stop[slot], stream);
}

namespace {

struct RoutingBuffers {
  int* status;
  int32_t* counters;        // directly behind the status header: one memset clears both
  int64_t counters_each;
  int32_t* sorted_ids;
  int32_t* expert_ids;
  int32_t* num_post;
  int32_t* expert_off;
  void* align_ws;
  int64_t align_ws_bytes;
};

// Routing buffers are sized for the worst case over the block sizes any path
// may pick: the longest sorted_ids (largest block) and the most blocks
// (smallest block).
constexpr int kMaxBlock = 256;
constexpr int kMinBlock = 16;

int64_t routing_max_pad(int64_t numel, int E, int block) {
  return numel + (int64_t)(E + 1) * (block - 1);
}

RoutingBuffers carve_routing(Carver& c, int64_t numel, int E) {
  RoutingBuffers r;
  r.status = c.take<int>(64);  // workspace header: word 0 = device status of the last call
  r.counters_each = numel / kMinBlock + E + 2;     // >= token blocks at the smallest token tile
  r.counters = c.take<int32_t>(2 * r.counters_each);
  r.sorted_ids = c.take<int32_t>(routing_max_pad(numel, E, kMaxBlock));
  r.expert_ids = c.take<int32_t>(ceil_div(routing_max_pad(numel, E, kMinBlock), kMinBlock) + 1);
  r.num_post = c.take<int32_t>(1);
  r.expert_off = c.take<int32_t>(E + 1);
  r.align_ws_bytes = align_workspace_bytes(numel, E);
  r.align_ws = c.take<char>(r.align_ws_bytes);
  return r;
}

// status header and the block counters behind it, as one span
size_t header_bytes(const RoutingBuffers& r) {
  return (size_t)(reinterpret_cast<const char*>(r.counters + 2 * r.counters_each) - reinterpret_cast<const char*>(r.status));
}

int64_t routing_bytes(int64_t numel, int E) {
  Carver c(nullptr);
  carve_routing(c, numel, E);
  return c.off;
}

Routing make_routing(const RoutingBuffers& b, int64_t numel, int E, int block) {
  Routing r;
  r.sorted_ids = b.sorted_ids;
  r.expert_ids = b.expert_ids;
  r.num_post = b.num_post;
  r.expert_off = b.expert_off;
  r.numel = numel;
  r.block = block;
  r.max_pad = routing_max_pad(numel, E, block);
  r.max_blocks = ceil_div(r.max_pad, block);
  r.block_counters = b.counters;
  r.counters_each = b.counters_each;
  return r;
}

}  // namespace
}  // namespace xkb

using namespace xkb;

extern "C" const char* xkb_version(void) { return "xkb200 0.1 (sm_100a)"; }
extern "C" const char* xkb_last_error(void) { return last_error_buf(); }
extern "C" int64_t xkb_launch_count(void) { return g_launches.load(); }

// ---------------------------------------------------------------------------
// INT4 W4A16
// ---------------------------------------------------------------------------
extern "C" int64_t xkb_fused_moe_int4_w4a16_workspace_bytes(int64_t M, int64_t N, int64_t K, int E,
                                                            int top_k, int a_dtype) {
  (void)a_dtype;
  if (M < 0 || N < 0 || K < 0 || E < 0 || top_k < 0) return -1;
  const int64_t numel = M * top_k;
  int64_t total = routing_bytes(numel, E);
  total += align_up(numel * N * 4, 256);           // fp32 slot-indexed rows
  total += int4_tc_workspace_bytes(numel, N, K, E);  // gathered activations etc.
  return total + 256;
}

// rows_out == nullptr: combine into `out` ([M,N], a_dtype).  rows_out != nullptr: leave the fp32
// per-slot rows ([M*top_k, N], row = token*top_k + j) there and skip the combine.
static int int4_impl(const void* A, int a_dtype, const int32_t* packed, const void* scale,
                     const int32_t* topk_ids, const float* topk_w, const int32_t* expert_map,
                     int num_map, void* out, float* rows_out, int64_t M, int64_t N, int64_t K, int E,
                     int top_k, int group_size, int mul_routed_weight, int path, void* workspace,
                     int64_t workspace_bytes, cudaStream_t stream, int out_dtype = -1) {
  if (out_dtype < 0) out_dtype = a_dtype;
  XKB_REQUIRE(a_dtype == XKB_BF16 || a_dtype == XKB_F32, "fused_moe_int4_w4a16: bad a_dtype %d", a_dtype);
  XKB_REQUIRE(M >= 0 && N >= 0 && K >= 0 && E >= 0 && top_k >= 0, "fused_moe_int4_w4a16: negative dim");
  XKB_REQUIRE(group_size > 0 && group_size % 8 == 0 && K % group_size == 0 && K % 8 == 0,
              "fused_moe_int4_w4a16: need K %% 8 == 0, group_size %% 8 == 0, K %% group_size == 0 "
              "(K=%lld group_size=%d)", (long long)K, group_size);
  XKB_REQUIRE(path == XKB_PATH_AUTO || path == XKB_PATH_SIMT || path == XKB_PATH_TC,
              "fused_moe_int4_w4a16: bad path %d", path);
  if (M == 0 || N == 0) return XKB_OK;
  XKB_REQUIRE(A && packed && scale && topk_ids && (out || rows_out),
              "fused_moe_int4_w4a16: null pointer argument");
  XKB_REQUIRE(topk_w || !mul_routed_weight, "fused_moe_int4_w4a16: topk_w is null");
  const int64_t need = xkb_fused_moe_int4_w4a16_workspace_bytes(M, N, K, E, top_k, a_dtype);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(XKB_ERR_WORKSPACE, "fused_moe_int4_w4a16: workspace of %lld bytes needed, %lld given",
                (long long)need, (long long)workspace_bytes);
  XKB_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 256 == 0, "workspace must be 256-byte aligned");

  const int64_t numel = M * top_k;
  Carver carve(workspace);
  RoutingBuffers rb = carve_routing(carve, numel, E);
  float* scratch = carve.take<float>(numel * N);
  if (rows_out != nullptr) scratch = rows_out;
  void* tc_ws = carve.take<char>(int4_tc_workspace_bytes(numel, N, K, E));

  const bool tc_fit = int4_tc_supported(a_dtype, M, N, K, E, top_k, group_size);
  if (path == XKB_PATH_TC && !tc_fit)
    return fail(XKB_ERR_ARG,
                "fused_moe_int4_w4a16: shape not supported by the tcgen05 path (needs bf16 A, "
                "N %% 128 == 0, K %% 256 == 0, group_size 32)");
  const bool use_tc = (path == XKB_PATH_TC) || (path == XKB_PATH_AUTO && tc_fit);
  const int block = use_tc ? int4_tc_block(numel, E) : kSimtBlock;

  Routing r = make_routing(rb, numel, E, block);
  XKB_CHECK_CUDA(cudaMemsetAsync(rb.status, 0, header_bytes(rb), stream));   // status word + block counters
  int rc = launch_align(topk_ids, numel, E, block, expert_map, num_map, rb.sorted_ids, rb.expert_ids,
                        rb.num_post, rb.expert_off, rb.align_ws, rb.align_ws_bytes, stream);
  if (rc != XKB_OK) return rc;
  if (use_tc)
    rc = launch_int4_tc(A, packed, scale, r, topk_w, scratch, N, K, E, top_k, mul_routed_weight,
                        tc_ws, rb.status, stream);
  else
    rc = launch_int4_simt(A, a_dtype, packed, scale, r, topk_w, scratch, N, K, top_k, group_size,
                          mul_routed_weight, stream);
  if (rc != XKB_OK) return rc;
  if (rows_out != nullptr) return XKB_OK;
  return launch_combine(scratch, topk_ids, expert_map, num_map, E, out, out_dtype, M, top_k, N, stream);
}

extern "C" int xkb_fused_moe_int4_w4a16(const void* A, int a_dtype, const int32_t* packed,
                                        const void* scale, const int32_t* topk_ids,
                                        const float* topk_w, const int32_t* expert_map, int num_map,
                                        void* out, int64_t M, int64_t N, int64_t K, int E, int top_k,
                                        int group_size, int mul_routed_weight, int path,
                                        void* workspace, int64_t workspace_bytes, void* stream) {
  XKB_REQUIRE(out != nullptr || M == 0 || N == 0, "fused_moe_int4_w4a16: null out");
  return int4_impl(A, a_dtype, packed, scale, topk_ids, topk_w, expert_map, num_map, out, nullptr, M, N,
                   K, E, top_k, group_size, mul_routed_weight, path, workspace, workspace_bytes,
                   static_cast<cudaStream_t>(stream));
}

extern "C" int xkb_moe_int4_w4a16_rows(const void* A, int a_dtype, const int32_t* packed,
                                       const void* scale, const int32_t* topk_ids, const float* topk_w,
                                       float* rows_out, int64_t M, int64_t N, int64_t K, int E,
                                       int top_k, int group_size, int mul_routed_weight, int path,
                                       void* workspace, int64_t workspace_bytes, void* stream) {
  XKB_REQUIRE(rows_out != nullptr || M == 0 || N == 0, "moe_int4_w4a16_rows: null rows_out");
  return int4_impl(A, a_dtype, packed, scale, topk_ids, topk_w, nullptr, 0, nullptr, rows_out, M, N, K,
                   E, top_k, group_size, mul_routed_weight, path, workspace, workspace_bytes,
                   static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------
// Expert side of the all-to-all mode in one call: received rows whose routing travels with them as
// [M, 2*top_k] int32 (top_k local expert ids, -1 = slot served elsewhere, then the top_k routing
// weights' bit patterns) -> one fp32 partial row per received row (the weighted sum over its local
// experts, ascending slot order).  The routing is split into the two contiguous arrays the align
// stage and the combine read by a small kernel, so that the host makes ONE call per chunk.
// ---------------------------------------------------------------------------
namespace xkb {
namespace {
__global__ void __launch_bounds__(256)
split_routing_kernel(const int32_t* __restrict__ routing, int64_t numel, int top_k, int32_t* __restrict__ ids,
                     float* __restrict__ w) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= numel) return;
  const int64_t m = i / top_k;
  const int j = (int)(i - m * top_k);
  ids[i] = routing[m * 2 * top_k + j];
  w[i] = __int_as_float(routing[m * 2 * top_k + top_k + j]);
}
}  // namespace
}  // namespace xkb

extern "C" int64_t xkb_moe_int4_w4a16_partial_workspace_bytes(int64_t M, int64_t N, int64_t K, int E, int top_k,
                                                              int a_dtype) {
  const int64_t base = xkb_fused_moe_int4_w4a16_workspace_bytes(M, N, K, E, top_k, a_dtype);
  if (base < 0) return base;
  return base + 2 * align_up(M * top_k * 4, 256);
}

extern "C" int xkb_moe_int4_w4a16_partial(const void* A, int a_dtype, const int32_t* packed, const void* scale,
                                          const int32_t* routing, float* out, int64_t M, int64_t N, int64_t K,
                                          int E, int top_k, int group_size, int path, void* workspace,
                                          int64_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  XKB_REQUIRE(M >= 0 && N >= 0 && K >= 0 && E >= 0 && top_k >= 1, "moe_int4_w4a16_partial: bad dimension");
  if (M == 0 || N == 0) return XKB_OK;
  XKB_REQUIRE(routing != nullptr && out != nullptr, "moe_int4_w4a16_partial: null routing/out");
  const int64_t need = xkb_moe_int4_w4a16_partial_workspace_bytes(M, N, K, E, top_k, a_dtype);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(XKB_ERR_WORKSPACE, "moe_int4_w4a16_partial: workspace of %lld bytes needed, %lld given",
                (long long)need, (long long)workspace_bytes);
  XKB_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 256 == 0, "workspace must be 256-byte aligned");
  // the two routing arrays sit behind the fused op's own workspace
  const int64_t base = xkb_fused_moe_int4_w4a16_workspace_bytes(M, N, K, E, top_k, a_dtype);
  const int64_t numel = M * top_k;
  int32_t* ids = reinterpret_cast<int32_t*>(static_cast<char*>(workspace) + align_up(base, 256));
  float* w = reinterpret_cast<float*>(reinterpret_cast<char*>(ids) + align_up(numel * 4, 256));
  split_routing_kernel<<<(unsigned)ceil_div(numel, 256), 256, 0, stream>>>(routing, numel, top_k, ids, w);
  XKB_CHECK_LAUNCH("split_routing_kernel");
  return int4_impl(A, a_dtype, packed, scale, ids, w, nullptr, 0, out, nullptr, M, N, K, E, top_k, group_size, 1,
                   path, workspace, base, stream, XKB_F32);
}

// ---------------------------------------------------------------------------
// INT4 two-GEMM expert layer
// ---------------------------------------------------------------------------
extern "C" int64_t xkb_fused_moe_int4_ffn_workspace_bytes(int64_t M, int64_t hidden, int64_t inter, int E, int top_k,
                                                          int a_dtype) {
  (void)a_dtype;
  if (M < 0 || hidden < 0 || inter < 0 || E < 0 || top_k < 0) return -1;
  const int64_t numel = M * top_k;
  int64_t total = routing_bytes(numel, E);
  total += align_up(numel * hidden * 4, 256);                                   // fp32 slot rows of the down GEMM
  total += align_up(numel * 2 * inter * 4, 256);                                // fp32 gate_up slot rows (generic path)
  total += align_up(routing_max_pad(numel, E, kMaxBlock) * inter * 4, 256);     // activations (bf16 by position, or by slot)
  total += int4_tc_workspace_bytes(numel, hidden, hidden, E);                   // gathered input activations
  return total + 256;
}

extern "C" int xkb_fused_moe_int4_ffn(const void* A, int a_dtype, const int32_t* w13_packed, const void* w13_scale,
                                      const int32_t* w2_packed, const void* w2_scale, const int32_t* topk_ids,
                                      const float* topk_w, const int32_t* expert_map, int num_map, void* out,
                                      int64_t M, int64_t hidden, int64_t inter, int E, int top_k, int group_size,
                                      float swiglu_limit, int path, void* workspace, int64_t workspace_bytes,
                                      void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  XKB_REQUIRE(a_dtype == XKB_BF16 || a_dtype == XKB_F32, "fused_moe_int4_ffn: bad a_dtype %d", a_dtype);
  XKB_REQUIRE(M >= 0 && hidden >= 0 && inter >= 0 && E >= 0 && top_k >= 0, "fused_moe_int4_ffn: negative dim");
  XKB_REQUIRE(group_size > 0 && group_size % 8 == 0 && hidden % group_size == 0 && inter % group_size == 0,
              "fused_moe_int4_ffn: hidden and inter must be multiples of group_size, group_size of 8 "
              "(hidden=%lld inter=%lld group_size=%d)", (long long)hidden, (long long)inter, group_size);
  XKB_REQUIRE(path == XKB_PATH_AUTO || path == XKB_PATH_SIMT || path == XKB_PATH_TC, "fused_moe_int4_ffn: bad path %d", path);
  if (M == 0 || hidden == 0) return XKB_OK;
  XKB_REQUIRE(A && w13_packed && w13_scale && w2_packed && w2_scale && topk_ids && topk_w && out,
              "fused_moe_int4_ffn: null pointer argument");
  const int64_t need = xkb_fused_moe_int4_ffn_workspace_bytes(M, hidden, inter, E, top_k, a_dtype);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(XKB_ERR_WORKSPACE, "fused_moe_int4_ffn: workspace of %lld bytes needed, %lld given", (long long)need,
                (long long)workspace_bytes);
  XKB_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 256 == 0, "workspace must be 256-byte aligned");

  const int64_t numel = M * top_k;
  Carver carve(workspace);
  RoutingBuffers rb = carve_routing(carve, numel, E);
  float* scratch = carve.take<float>(numel * hidden);
  float* rows1 = carve.take<float>(numel * 2 * inter);
  void* act = carve.take<float>(routing_max_pad(numel, E, kMaxBlock) * inter);
  void* tc_ws = carve.take<char>(int4_tc_workspace_bytes(numel, hidden, hidden, E));

  const bool tc_fit = int4_ffn_tc_supported(a_dtype, M, hidden, inter, E, top_k, group_size);
  if (path == XKB_PATH_TC && !tc_fit)
    return fail(XKB_ERR_ARG, "fused_moe_int4_ffn: shape not supported by the tcgen05 path (needs bf16 A, "
                             "hidden %% 256 == 0, inter %% 256 == 0, group_size 32)");
  const bool use_tc = (path == XKB_PATH_TC) || (path == XKB_PATH_AUTO && tc_fit);
  const int block = use_tc ? int4_tc_block(numel, E) : kSimtBlock;
  Routing r = make_routing(rb, numel, E, block);
  XKB_CHECK_CUDA(cudaMemsetAsync(rb.status, 0, header_bytes(rb), stream));   // status word + block counters
  int rc = launch_align(topk_ids, numel, E, block, expert_map, num_map, rb.sorted_ids, rb.expert_ids, rb.num_post,
                        rb.expert_off, rb.align_ws, rb.align_ws_bytes, stream);
  if (rc != XKB_OK) return rc;
  if (use_tc)
    rc = launch_int4_ffn_tc(A, w13_packed, w13_scale, w2_packed, w2_scale, r, topk_w, static_cast<__nv_bfloat16*>(act),
                            scratch, hidden, inter, E, top_k, swiglu_limit, tc_ws, rb.status, stream);
  else
    rc = launch_int4_ffn_simt(A, a_dtype, w13_packed, w13_scale, w2_packed, w2_scale, r, topk_ids, expert_map, num_map,
                              E, topk_w, rows1, act, scratch, hidden, inter, top_k, group_size, swiglu_limit, stream);
  if (rc != XKB_OK) return rc;
  return launch_combine(scratch, topk_ids, expert_map, num_map, E, out, a_dtype, M, top_k, hidden, stream);
}

// ---------------------------------------------------------------------------
// MXFP4
// ---------------------------------------------------------------------------
extern "C" int64_t xkb_fused_moe_mxfp4_workspace_bytes(int64_t M, int64_t hidden, int64_t ispp, int E,
                                                       int top_k) {
  if (M < 0 || hidden < 0 || ispp < 0 || E < 0 || top_k < 0) return -1;
  const int64_t numel = M * top_k;
  int64_t total = routing_bytes(numel, E);
  total += align_up(numel * hidden * 4, 256);                                 // fp32 partial rows
  total += align_up(routing_max_pad(numel, E, kMaxBlock) * ispp * 2, 256);    // bf16 activations
  total += mxfp4_tc_workspace_bytes(numel, hidden, ispp, E);
  return total + 256;
}

extern "C" int xkb_fused_moe_mxfp4(const void* A, int a_dtype, const uint8_t* w13,
                                   const uint8_t* w13_scale, const uint8_t* w2,
                                   const uint8_t* w2_scale, const int32_t* topk_ids,
                                   const float* topk_w, const void* b13, const void* b2,
                                   const int32_t* expert_map, int num_map, void* out, int64_t M,
                                   int64_t hidden, int64_t ispp, int E, int top_k, float swiglu_limit,
                                   int mul_routed_weight, int path, void* workspace,
                                   int64_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  XKB_REQUIRE(a_dtype == XKB_BF16 || a_dtype == XKB_F32, "fused_moe_mxfp4: bad a_dtype %d", a_dtype);
  XKB_REQUIRE(M >= 0 && hidden >= 0 && ispp >= 0 && E >= 0 && top_k >= 0, "fused_moe_mxfp4: negative dim");
  XKB_REQUIRE(hidden % 32 == 0 && ispp % 32 == 0,
              "fused_moe_mxfp4: hidden and ispp must be multiples of the MX block 32 (got %lld, %lld)",
              (long long)hidden, (long long)ispp);
  XKB_REQUIRE(path == XKB_PATH_AUTO || path == XKB_PATH_SIMT || path == XKB_PATH_TC,
              "fused_moe_mxfp4: bad path %d", path);
  if (M == 0 || hidden == 0) return XKB_OK;
  XKB_REQUIRE(A && w13 && w13_scale && w2 && w2_scale && topk_ids && out,
              "fused_moe_mxfp4: null pointer argument");
  XKB_REQUIRE(topk_w || !mul_routed_weight, "fused_moe_mxfp4: topk_w is null");
  const int64_t need = xkb_fused_moe_mxfp4_workspace_bytes(M, hidden, ispp, E, top_k);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(XKB_ERR_WORKSPACE, "fused_moe_mxfp4: workspace of %lld bytes needed, %lld given",
                (long long)need, (long long)workspace_bytes);
  XKB_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 256 == 0, "workspace must be 256-byte aligned");

  const int64_t numel = M * top_k;
  Carver carve(workspace);
  RoutingBuffers rb = carve_routing(carve, numel, E);
  float* scratch = carve.take<float>(numel * hidden);
  __nv_bfloat16* act = carve.take<__nv_bfloat16>(routing_max_pad(numel, E, kMaxBlock) * ispp);
  void* tc_ws = carve.take<char>(mxfp4_tc_workspace_bytes(numel, hidden, ispp, E));

  const bool tc_fit = mxfp4_tc_supported(a_dtype, M, hidden, ispp, E, top_k);
  if (path == XKB_PATH_TC && !tc_fit)
    return fail(XKB_ERR_ARG,
                "fused_moe_mxfp4: shape not supported by the tcgen05 path (needs bf16 A, "
                "hidden %% 512 == 0, ispp %% 512 == 0)");
  const bool use_tc = (path == XKB_PATH_TC) || (path == XKB_PATH_AUTO && tc_fit);
  const int block = use_tc ? mxfp4_tc_block(numel, E) : kSimtBlock;

  Routing r = make_routing(rb, numel, E, block);
  XKB_CHECK_CUDA(cudaMemsetAsync(rb.status, 0, header_bytes(rb), stream));   // status word + block counters
  int rc = launch_align(topk_ids, numel, E, block, expert_map, num_map, rb.sorted_ids, rb.expert_ids,
                        rb.num_post, rb.expert_off, rb.align_ws, rb.align_ws_bytes, stream);
  if (rc != XKB_OK) return rc;
  if (use_tc)
    rc = launch_mxfp4_tc(A, w13, w13_scale, w2, w2_scale, b13, b2, r, topk_w, act, scratch, hidden,
                         ispp, E, top_k, swiglu_limit, mul_routed_weight, tc_ws, rb.status, stream);
  else
    rc = launch_mxfp4_simt(A, a_dtype, w13, w13_scale, w2, w2_scale, b13, b2, r, topk_w, act, scratch,
                           hidden, ispp, top_k, swiglu_limit, mul_routed_weight, stream);
  if (rc != XKB_OK) return rc;
  return launch_combine(scratch, topk_ids, expert_map, num_map, E, out, a_dtype, M, top_k, hidden, stream);
}

// ---------------------------------------------------------------------------
extern "C" int xkb_workspace_status(const void* workspace, void* stream_) {
  XKB_REQUIRE(workspace != nullptr, "xkb_workspace_status: null workspace");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int host = 0;
  XKB_CHECK_CUDA(cudaMemcpyAsync(&host, workspace, sizeof(int), cudaMemcpyDeviceToHost, stream));
  XKB_CHECK_CUDA(cudaStreamSynchronize(stream));
  if (host == 2)
    return fail(XKB_ERR_DEVICE, "an MXFP4 scale byte in 191..254 (weights of 2^64 and more) is outside the range "
                                "the tcgen05 dequantiser converts: status 0x2");
  if ((host & 0xFF) == 3)
    return fail(XKB_ERR_DEVICE, "a kernel read a routing value outside what the routing buffers hold and skipped the "
                                "work: status 0x%x (site %d)", host, host >> 8);
  if (host != 0)
    return fail(XKB_ERR_DEVICE, "a kernel gave up a bounded wait: status 0x%x (wait site %d)", host, host >> 8);
  return XKB_OK;
}

// ---------------------------------------------------------------------------
extern "C" int xkb_gemm_timer_enable(int max_calls) {
  XKB_REQUIRE(max_calls >= 0 && max_calls <= (1 << 16), "xkb_gemm_timer_enable: max_calls out of range");
  for (auto e : g_timer.start) cudaEventDestroy(e);
  for (auto e : g_timer.stop) cudaEventDestroy(e);
  g_timer.start.clear();
  g_timer.stop.clear();
  g_timer.used = 0;
  g_timer.enabled = max_calls > 0;
  for (int i = 0; i < max_calls; ++i) {
    cudaEvent_t a, b;
    XKB_CHECK_CUDA(cudaEventCreate(&a));
    XKB_CHECK_CUDA(cudaEventCreate(&b));
    g_timer.start.push_back(a);
    g_timer.stop.push_back(b);
  }
  return XKB_OK;
}

extern "C" int xkb_gemm_timer_read(float* ms_host, int capacity, int* count_host) {
  XKB_REQUIRE(ms_host != nullptr && count_host != nullptr, "xkb_gemm_timer_read: null output");
  const int n = g_timer.used < capacity ? g_timer.used : capacity;
  for (int i = 0; i < n; ++i) {
    XKB_CHECK_CUDA(cudaEventSynchronize(g_timer.stop[i]));
    XKB_CHECK_CUDA(cudaEventElapsedTime(&ms_host[i], g_timer.start[i], g_timer.stop[i]));
  }
  *count_host = n;
  g_timer.used = 0;
  return XKB_OK;
}

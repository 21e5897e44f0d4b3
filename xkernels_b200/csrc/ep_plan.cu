// Dispatch plan of the all-to-all expert-parallel mode, on the device and without a host read.
//
// A token goes once to every rank that owns at least one of its top-k experts (an expert whose table
// entry has a negative rank is served without dispatch - the caller computes it where the token is -
// and opens no pair).  The plan lists those
// (token, rank) pairs grouped by (token chunk, rank), ascending token inside a group, and for every
// pair the routing that travels with it.  Three launches: a key per slot (the rank of a slot that
// opens a pair, "none" otherwise), the counting sort of the align stage with one position per
// block, and the per-pair rows.  The reference has no all-to-all (its expert parallelism replicates
// the tokens, src/xkernels/ops/moe/interface.py:37-57); the host-side statement of the same plan
// is xkernels_b200/ep.py:plan_dispatch, against which this is tested for equality.

#include "common.cuh"

namespace xkb {
namespace {

constexpr int kMaxTopK = 32;

__device__ __forceinline__ void owner_local(int id, int experts_per_rank, int world, int round_robin,
                                            const int32_t* __restrict__ table, int& owner, int& local) {
  if (table != nullptr) { owner = table[2 * id]; local = table[2 * id + 1]; }   // explicit placement (replicas)
  else if (round_robin == 1) { owner = id % world; local = id / world; }
  else if (round_robin == 2) {   // snake: every second group of `world` experts in reverse rank order
    local = id / world;
    const int pos = id % world;
    owner = (local & 1) ? world - 1 - pos : pos;
  } else { owner = id / experts_per_rank; local = id - owner * experts_per_rank; }
}

// thread = token: key[slot] = chunk * world + rank for the first slot of the token that goes to that
// rank, -1 (dropped by the sort) for the others; dest/local per slot for the later stages
__global__ void __launch_bounds__(256)
ep_key_kernel(const int32_t* __restrict__ topk_ids, int64_t M, int top_k, int experts_per_rank, int world,
              int round_robin, const int32_t* __restrict__ table, int64_t tokens_per_chunk, int32_t* __restrict__ key, int32_t* __restrict__ dest,
              int32_t* __restrict__ local, int32_t* __restrict__ info) {
  const int64_t m = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= M) return;
  const int E = experts_per_rank * world;
  const int chunk = (int)(m / tokens_per_chunk);
  int d[kMaxTopK];
  int bad = 0;
  for (int j = 0; j < top_k; ++j) {
    int id = topk_ids[m * top_k + j];
    if (id < 0 || id >= E) { ++bad; id = id < 0 ? 0 : E - 1; }     // clamped; the host raises on info[1]
    int o, l;
    owner_local(id, experts_per_rank, world, round_robin, table, o, l);
    d[j] = o;
    bool first = true;
    for (int i = 0; i < j; ++i) first = first && (d[i] != o);
    key[m * top_k + j] = (first && o >= 0) ? chunk * world + o : -1;   // o < 0 (table only): not dispatched
    dest[m * top_k + j] = o;
    local[m * top_k + j] = l;
  }
  if (bad) atomicAdd(&info[1], bad);
}

// thread = sorted position p < P: the pair's token and rank, its routing row (top_k local expert
// ids, -1 where the slot goes elsewhere, then the top_k routing weights' bit patterns, 0 there),
// and its position in the token's row of pair_of
__global__ void __launch_bounds__(256)
ep_pairs_kernel(const int32_t* __restrict__ sorted_slots, const int32_t* __restrict__ num_pairs,
                const int32_t* __restrict__ group_off, int n_groups, const int32_t* __restrict__ dest,
                const int32_t* __restrict__ local, const float* __restrict__ topk_w, int top_k, int world,
                int32_t* __restrict__ pair_token, int32_t* __restrict__ pair_dest, int32_t* __restrict__ routing,
                int32_t* __restrict__ pair_of, int32_t* __restrict__ counts, int32_t* __restrict__ info) {
  const int P = num_pairs[0];
  const int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (p == 0) info[0] = P;
  if (p < n_groups) counts[p] = group_off[p + 1] - group_off[p];
  if (p >= P) return;
  const int slot = sorted_slots[p];
  const int token = slot / top_k;
  const int rank = dest[slot];
  pair_token[p] = token;
  pair_dest[p] = rank;
  int32_t* row = routing + p * 2 * (int64_t)top_k;
  for (int j = 0; j < top_k; ++j) {
    const int64_t s = (int64_t)token * top_k + j;
    const bool mine = dest[s] == rank;
    row[j] = mine ? local[s] : -1;
    row[top_k + j] = mine ? __float_as_int(topk_w[s]) : 0;
  }
  pair_of[(int64_t)token * world + rank] = (int32_t)p;
}

}  // namespace
}  // namespace xkb

extern "C" int64_t xkb_ep_plan_workspace_bytes(int64_t M, int top_k, int world, int chunks) {
  using namespace xkb;
  const int64_t numel = M * top_k;
  const int groups = world * chunks;
  return 4 * align_up(numel * 4 + 4, 256)            // key, dest, local, sorted slots
         + align_up(numel * 4 + 4, 256)              // group of each position (one position per block)
         + 2 * align_up((int64_t)(groups + 2) * 4, 256)   // number of pairs, group offsets
         + align_workspace_bytes(numel, groups) + 256;
}

extern "C" int xkb_ep_plan(const int32_t* topk_ids, const float* topk_w, int64_t M, int top_k,
                           int experts_per_rank, int world, int round_robin, const int32_t* expert_table,
                           int chunks, int32_t* pair_token,
                           int32_t* pair_dest, int32_t* routing, int32_t* pair_of, int32_t* counts,
                           int32_t* info, void* workspace, int64_t workspace_bytes, void* stream) {
  using namespace xkb;
  XKB_REQUIRE(M >= 0 && top_k >= 1 && top_k <= kMaxTopK, "ep_plan: top_k=%d outside [1,%d]", top_k, kMaxTopK);
  XKB_REQUIRE(experts_per_rank >= 1 && world >= 1 && chunks >= 1, "ep_plan: bad sharding");
  const int groups = world * chunks;
  XKB_REQUIRE(groups <= 1024, "ep_plan: world * chunks = %d exceeds 1024 groups", groups);
  XKB_REQUIRE(counts && info, "ep_plan: null output pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t numel = M * top_k;
  XKB_CHECK_CUDA(cudaMemsetAsync(info, 0, 2 * sizeof(int32_t), s));
  XKB_CHECK_CUDA(cudaMemsetAsync(counts, 0, groups * sizeof(int32_t), s));
  if (M == 0) return XKB_OK;    // no token: no pair, the per-pair outputs are empty
  XKB_REQUIRE(pair_token && pair_dest && routing && pair_of, "ep_plan: null output pointer");
  XKB_REQUIRE(workspace != nullptr && workspace_bytes >= xkb_ep_plan_workspace_bytes(M, top_k, world, chunks),
              "ep_plan: workspace too small (%lld bytes)", (long long)workspace_bytes);
  XKB_REQUIRE(topk_ids && topk_w, "ep_plan: null input pointer");
  XKB_CHECK_CUDA(cudaMemsetAsync(pair_of, 0xFF, (size_t)M * world * sizeof(int32_t), s));   // -1: no such pair
  Carver carve(workspace);
  int32_t* key = carve.take<int32_t>(numel + 1);
  int32_t* dest = carve.take<int32_t>(numel + 1);
  int32_t* local = carve.take<int32_t>(numel + 1);
  int32_t* sorted = carve.take<int32_t>(numel + 1);
  int32_t* group_of = carve.take<int32_t>(numel + 1);
  int32_t* num_pairs = carve.take<int32_t>(groups + 2);
  int32_t* group_off = carve.take<int32_t>(groups + 2);
  void* align_ws = carve.take<char>(align_workspace_bytes(numel, groups));
  const int64_t tokens_per_chunk = (M + chunks - 1) / chunks;
  ep_key_kernel<<<(unsigned)ceil_div(M, 256), 256, 0, s>>>(topk_ids, M, top_k, experts_per_rank, world, round_robin,
                                                           expert_table, tokens_per_chunk, key, dest, local, info);
  XKB_CHECK_LAUNCH("ep_key_kernel");
  // stable counting sort of the slots by key, one position per block: no padding, dropped keys (-1) leave
  int rc = launch_align(key, numel, groups, 1, nullptr, 0, sorted, group_of, num_pairs, group_off, align_ws,
                        align_workspace_bytes(numel, groups), s);
  if (rc != XKB_OK) return rc;
  ep_pairs_kernel<<<(unsigned)ceil_div(numel > groups ? numel : groups, 256), 256, 0, s>>>(
      sorted, num_pairs, group_off, groups, dest, local, topk_w, top_k, world, pair_token, pair_dest, routing,
      pair_of, counts, info);
  XKB_CHECK_LAUNCH("ep_pairs_kernel");
  return XKB_OK;
}

// ---------------------------------------------------------------------------
// Row gather with the row count on the device: dst[p, :] = src[index[p], :] for p < *count.
// Used to fill the dispatch send buffer while the host still waits for the pair counts (the
// count lives in the plan's info word), so that the copy is off the host's critical path.
// ---------------------------------------------------------------------------
namespace xkb {
namespace {
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ src, int64_t row_vecs, const int32_t* __restrict__ index,
                   const int32_t* __restrict__ count, int64_t max_rows, int64_t src_rows, uint4* __restrict__ dst) {
  int64_t n = count != nullptr ? (int64_t)count[0] : max_rows;
  if (n > max_rows) n = max_rows;
  for (int64_t p = blockIdx.x; p < n; p += gridDim.x) {
    const int64_t r = index[p];
    if (r < 0 || r >= src_rows) continue;
    const uint4* s = src + r * row_vecs;
    uint4* d = dst + p * row_vecs;
    for (int64_t i = threadIdx.x; i < row_vecs; i += blockDim.x) d[i] = __ldg(s + i);
  }
}
}  // namespace
}  // namespace xkb

extern "C" int xkb_gather_rows(const void* src, int64_t src_rows, int64_t row_bytes, const int32_t* index,
                               const int32_t* count_dev, int64_t max_rows, void* dst, void* stream) {
  using namespace xkb;
  XKB_REQUIRE(src_rows >= 0 && max_rows >= 0 && row_bytes > 0 && row_bytes % 16 == 0,
              "gather_rows: rows must be a positive multiple of 16 bytes long (got %lld)", (long long)row_bytes);
  if (max_rows == 0 || src_rows == 0) return XKB_OK;
  XKB_REQUIRE(src && index && dst, "gather_rows: null pointer");
  XKB_REQUIRE(reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0,
              "gather_rows: src and dst must be 16-byte aligned");
  int64_t blocks = max_rows < 148 * 16 ? max_rows : 148 * 16;
  gather_rows_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), row_bytes / 16, index, count_dev, max_rows, src_rows, static_cast<uint4*>(dst));
  XKB_CHECK_LAUNCH("gather_rows_kernel");
  return XKB_OK;
}

// moe_align_block_size for sm_100a: sort/pad routed token-slots into per-expert
// blocks, bit-exact with the reference (src/xkernels/ops/moe/w4a16.py:53-101):
// stable order inside an expert, every run padded to a multiple of block_size,
// unused entries of sorted_ids = numel, unused entries of expert_ids = 0.
//
// Stability without sorting: a slot's rank inside its expert is
//   (# same-expert slots in earlier 1024-slot chunks)      -> chunk x expert matrix
// + (# same-expert slots in earlier warps of its chunk)    -> warp x expert matrix (smem)
// + (# same-expert lanes below it in its warp)             -> __match_any_sync ballot
// Counters only ever count, so atomics never decide an output position.
//
// numel <= kSmallMax runs as ONE single-CTA kernel; larger inputs use three
// launches (count -> offsets -> scatter) over 1024-slot chunks.
#include "common.cuh"

namespace xkb {
namespace {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;
constexpr int kChunk = kThreads;       // slots per chunk (one per thread)
constexpr int64_t kSmallMax = 8192;    // single-CTA path up to this many slots
constexpr int kMaxExperts = 1024;

__device__ __forceinline__ int map_expert(int id, int E, const int32_t* expert_map, int num_map) {
  if (expert_map != nullptr) {
    if (id < 0 || id >= num_map) return E;
    id = expert_map[id];
  }
  return (id < 0 || id >= E) ? E : id;  // E = ghost expert (dropped)
}

// Exclusive scan of padded per-expert counts; one CTA, any E <= kMaxExperts.
// hist[e] (e < E) -> off[e], off[E] = total.  scratch: kWarps ints.
__device__ void padded_offsets(const int* hist, int* off, int* warp_tot, int E, int block) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // E <= 1024 = kThreads: one expert per thread.
  int padded = 0;
  if (tid < E) padded = (hist[tid] + block - 1) / block * block;
  int incl = padded;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int v = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += v;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int t = warp_tot[lane];
    int ti = t;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int v = __shfl_up_sync(0xffffffffu, ti, d);
      if (lane >= d) ti += v;
    }
    warp_tot[lane] = ti - t;  // exclusive
  }
  __syncthreads();
  const int excl = incl - padded + warp_tot[warp];
  if (tid < E) off[tid] = excl;
  if (tid == E - 1) off[E] = excl + padded;
  if (E == 0 && tid == 0) off[0] = 0;
  __syncthreads();
}

// expert_ids[b] for every block b < max_blocks: the expert whose padded run
// holds position b*block, 0 past the used blocks.
__device__ void write_expert_ids(const int* off, int E, int block, int32_t* expert_ids,
                                 int64_t max_blocks, int tid0, int stride) {
  const int total = off[E];
  for (int64_t b = tid0; b < max_blocks; b += stride) {
    const int64_t pos = b * block;
    int e = 0;
    if (pos < total) {
      // largest e with off[e] <= pos and off[e+1] > pos (runs of zero length skipped)
      int lo = 0, hi = E;  // invariant: off[lo] <= pos < off[hi]
      while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (off[mid] <= pos) lo = mid; else hi = mid;
      }
      e = lo;
    }
    expert_ids[b] = e;
  }
}

// One 1024-slot round of the stable scatter.  `base[e]` = position of the first
// slot of expert e that belongs to this round.  wcnt: [kWarps][E+1] uint16.
// tot[e] receives the number of slots of expert e in this round.
__device__ void scatter_round(int my_e, bool active, int64_t slot, const int* base, int E,
                              uint16_t* wcnt, int* tot, int32_t* sorted_ids) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int EP = E + 1;
  for (int i = tid; i < kWarps * EP; i += kThreads) wcnt[i] = 0;
  __syncthreads();
  // inactive lanes vote with a key no expert uses so they never match
  const int key = active ? my_e : (EP + lane);
  const unsigned peers = __match_any_sync(0xffffffffu, key);
  const int rank = __popc(peers & ((1u << lane) - 1u));
  if (active && rank == 0) wcnt[warp * EP + my_e] = (uint16_t)__popc(peers);
  __syncthreads();
  // exclusive scan over warps, one expert per scanning warp per step
  for (int e = warp; e < EP; e += kWarps) {
    int v = wcnt[lane * EP + e];
    int incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int u = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += u;
    }
    wcnt[lane * EP + e] = (uint16_t)(incl - v);
    if (lane == 31) tot[e] = incl;
  }
  __syncthreads();
  if (active && my_e < E) {
    const int pos = base[my_e] + (int)wcnt[warp * EP + my_e] + rank;
    sorted_ids[pos] = (int32_t)slot;
  }
}

// ---------------------------------------------------------------------------
// Single-CTA path
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
align_small_kernel(const int32_t* __restrict__ topk_ids, int64_t numel, int E, int block,
                   const int32_t* __restrict__ expert_map, int num_map,
                   int32_t* __restrict__ sorted_ids, int64_t max_pad,
                   int32_t* __restrict__ expert_ids, int64_t max_blocks,
                   int32_t* __restrict__ num_post, int32_t* __restrict__ expert_off_out) {
  chain_trigger();   // a kernel chained behind this one may be launched; it waits for completion itself
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int EP = E + 1;
  int* hist = reinterpret_cast<int*>(smem_raw);   // [EP]
  int* off = hist + EP;                            // [EP]   off[E] = total
  int* run = off + EP;                             // [EP]   running base per expert
  int* tot = run + EP;                             // [EP]
  int* warp_tot = tot + EP;                        // [kWarps]
  uint16_t* wcnt = reinterpret_cast<uint16_t*>(warp_tot + kWarps);  // [kWarps][EP]
  const int tid = threadIdx.x;

  for (int i = tid; i < EP; i += kThreads) hist[i] = 0;
  __syncthreads();
  for (int64_t s = tid; s < numel; s += kThreads)
    atomicAdd(&hist[map_expert(topk_ids[s], E, expert_map, num_map)], 1);
  __syncthreads();
  padded_offsets(hist, off, warp_tot, E, block);
  for (int i = tid; i < EP; i += kThreads) run[i] = (i < E) ? off[i] : 0;
  if (tid == 0) num_post[0] = off[E];
  if (expert_off_out != nullptr)
    for (int i = tid; i < EP; i += kThreads) expert_off_out[i] = off[i];
  for (int64_t i = tid; i < max_pad; i += kThreads) sorted_ids[i] = (int32_t)numel;
  write_expert_ids(off, E, block, expert_ids, max_blocks, tid, kThreads);
  __syncthreads();
  const int64_t rounds = (numel + kChunk - 1) / kChunk;
  for (int64_t r = 0; r < rounds; ++r) {
    const int64_t slot = r * kChunk + tid;
    const bool active = slot < numel;
    const int e = active ? map_expert(topk_ids[slot], E, expert_map, num_map) : E;
    scatter_round(e, active, slot, run, E, wcnt, tot, sorted_ids);
    __syncthreads();
    for (int i = tid; i < E; i += kThreads) run[i] += tot[i];
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------
// Multi-CTA path: count -> offsets -> scatter over 1024-slot chunks
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
align_count_kernel(const int32_t* __restrict__ topk_ids, int64_t numel, int E,
                   const int32_t* __restrict__ expert_map, int num_map,
                   int32_t* __restrict__ chunk_cnt /*[C][E+1]*/,
                   int32_t* __restrict__ sorted_ids, int64_t max_pad) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int* hist = reinterpret_cast<int*>(smem_raw);
  const int EP = E + 1, tid = threadIdx.x;
  for (int i = tid; i < EP; i += kThreads) hist[i] = 0;
  __syncthreads();
  const int64_t slot = (int64_t)blockIdx.x * kChunk + tid;
  if (slot < numel) atomicAdd(&hist[map_expert(topk_ids[slot], E, expert_map, num_map)], 1);
  // pre-fill this CTA's slice of sorted_ids with the padding id
  const int64_t per = (max_pad + gridDim.x - 1) / gridDim.x;
  const int64_t lo = (int64_t)blockIdx.x * per;
  const int64_t hi = (lo + per < max_pad) ? lo + per : max_pad;
  for (int64_t i = lo + tid; i < hi; i += kThreads) sorted_ids[i] = (int32_t)numel;
  __syncthreads();
  for (int i = tid; i < EP; i += kThreads) chunk_cnt[(int64_t)blockIdx.x * EP + i] = hist[i];
}

__global__ void __launch_bounds__(kThreads)
align_offsets_kernel(int32_t* __restrict__ chunk_cnt /*in: counts, out: exclusive bases*/,
                     int C, int E, int block, int32_t* __restrict__ expert_ids,
                     int64_t max_blocks, int32_t* __restrict__ num_post,
                     int32_t* __restrict__ expert_off_g /*[E+1], always written*/) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int EP = E + 1;
  int* hist = reinterpret_cast<int*>(smem_raw);  // [EP]
  int* off = hist + EP;                           // [EP]
  int* warp_tot = off + EP;                       // [kWarps]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // per expert: exclusive scan of its counts over the chunks (warp per expert)
  for (int e = warp; e < EP; e += kWarps) {
    int carry = 0;
    for (int c0 = 0; c0 < C; c0 += 32) {
      const int c = c0 + lane;
      int v = (c < C) ? chunk_cnt[(int64_t)c * EP + e] : 0;
      int incl = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        int u = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += u;
      }
      if (c < C) chunk_cnt[(int64_t)c * EP + e] = carry + incl - v;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) hist[e] = carry;
  }
  __syncthreads();
  padded_offsets(hist, off, warp_tot, E, block);
  if (tid == 0) num_post[0] = off[E];
  for (int i = tid; i < EP; i += kThreads) expert_off_g[i] = off[i];
  write_expert_ids(off, E, block, expert_ids, max_blocks, tid, kThreads);
}

__global__ void __launch_bounds__(kThreads)
align_scatter_kernel(const int32_t* __restrict__ topk_ids, int64_t numel, int E,
                     const int32_t* __restrict__ expert_map, int num_map,
                     const int32_t* __restrict__ chunk_base /*[C][E+1]*/,
                     const int32_t* __restrict__ expert_off_g, int32_t* __restrict__ sorted_ids) {
  chain_trigger();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int EP = E + 1;
  int* base = reinterpret_cast<int*>(smem_raw);   // [EP]
  int* tot = base + EP;                            // [EP]
  uint16_t* wcnt = reinterpret_cast<uint16_t*>(tot + EP);
  const int tid = threadIdx.x;
  for (int i = tid; i < EP; i += kThreads)
    base[i] = (i < E) ? expert_off_g[i] + chunk_base[(int64_t)blockIdx.x * EP + i] : 0;
  const int64_t slot = (int64_t)blockIdx.x * kChunk + tid;
  const bool active = slot < numel;
  const int e = active ? map_expert(topk_ids[slot], E, expert_map, num_map) : E;
  __syncthreads();
  scatter_round(e, active, slot, base, E, wcnt, tot, sorted_ids);
}

size_t small_smem(int E) {
  const size_t EP = E + 1;
  return 4 * EP * sizeof(int) + kWarps * sizeof(int) + kWarps * EP * sizeof(uint16_t) + 16;
}
size_t scatter_smem(int E) {
  const size_t EP = E + 1;
  return 2 * EP * sizeof(int) + kWarps * EP * sizeof(uint16_t) + 16;
}

template <typename K>
cudaError_t allow_smem(K kernel, size_t bytes) {
  if (bytes <= 48 * 1024) return cudaSuccess;
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

}  // namespace

int64_t align_workspace_bytes(int64_t numel, int num_experts) {
  const int64_t C = ceil_div(numel > 0 ? numel : 1, kChunk);
  // chunk x expert matrix + a private expert_off copy
  return align_up(C * (num_experts + 1) * 4, 256) + align_up((int64_t)(num_experts + 1) * 4, 256);
}

int launch_align(const int32_t* topk_ids, int64_t numel, int E, int block,
                 const int32_t* expert_map, int num_map, int32_t* sorted_ids,
                 int32_t* expert_ids, int32_t* num_post, int32_t* expert_off,
                 void* workspace, int64_t workspace_bytes, cudaStream_t stream) {
  XKB_REQUIRE(numel >= 0 && numel < (1ll << 30), "moe_align: numel=%lld out of range", (long long)numel);
  XKB_REQUIRE(block > 0, "moe_align: block_size must be > 0 (got %d)", block);
  XKB_REQUIRE(E >= 0 && E <= kMaxExperts, "moe_align: num_experts=%d outside [0,%d]", E, kMaxExperts);
  XKB_REQUIRE(sorted_ids && expert_ids && num_post, "moe_align: null output pointer");
  XKB_REQUIRE(numel == 0 || topk_ids, "moe_align: null topk_ids");
  const int64_t max_pad = numel + (int64_t)(E + 1) * (block - 1);
  const int64_t max_blocks = ceil_div(max_pad, block);
  if (numel <= kSmallMax) {
    const size_t smem = small_smem(E);
    XKB_CHECK_CUDA(allow_smem(align_small_kernel, smem));
    align_small_kernel<<<1, kThreads, smem, stream>>>(topk_ids, numel, E, block, expert_map, num_map,
                                                      sorted_ids, max_pad, expert_ids, max_blocks,
                                                      num_post, expert_off);
    XKB_CHECK_LAUNCH("align_small_kernel");
    return XKB_OK;
  }
  const int64_t need = align_workspace_bytes(numel, E);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(XKB_ERR_WORKSPACE, "moe_align: workspace of %lld bytes needed, %lld given",
                (long long)need, (long long)workspace_bytes);
  const int C = (int)ceil_div(numel, kChunk);
  Carver carve(workspace);
  int32_t* chunk_cnt = carve.take<int32_t>((int64_t)C * (E + 1));
  int32_t* off_priv = carve.take<int32_t>(E + 1);
  int32_t* off_g = expert_off ? expert_off : off_priv;
  const size_t smem1 = (size_t)(E + 1) * sizeof(int) + 16;
  const size_t smem2 = (size_t)(2 * (E + 1) + kWarps) * sizeof(int) + 16;
  const size_t smem3 = scatter_smem(E);
  XKB_CHECK_CUDA(allow_smem(align_scatter_kernel, smem3));
  align_count_kernel<<<C, kThreads, smem1, stream>>>(topk_ids, numel, E, expert_map, num_map,
                                                     chunk_cnt, sorted_ids, max_pad);
  XKB_CHECK_LAUNCH("align_count_kernel");
  align_offsets_kernel<<<1, kThreads, smem2, stream>>>(chunk_cnt, C, E, block, expert_ids, max_blocks,
                                                       num_post, off_g);
  XKB_CHECK_LAUNCH("align_offsets_kernel");
  align_scatter_kernel<<<C, kThreads, smem3, stream>>>(topk_ids, numel, E, expert_map, num_map,
                                                       chunk_cnt, off_g, sorted_ids);
  XKB_CHECK_LAUNCH("align_scatter_kernel");
  return XKB_OK;
}

}  // namespace xkb

extern "C" int64_t xkb_moe_align_workspace_bytes(int64_t numel, int num_experts) {
  return xkb::align_workspace_bytes(numel, num_experts);
}

extern "C" int xkb_moe_align_block_size(const int32_t* topk_ids, int64_t numel, int num_experts,
                                        int block_size, const int32_t* expert_map, int num_map,
                                        int32_t* sorted_ids, int32_t* expert_ids,
                                        int32_t* num_post_pad, int32_t* expert_offsets,
                                        void* workspace, int64_t workspace_bytes, void* stream) {
  return xkb::launch_align(topk_ids, numel, num_experts, block_size, expert_map, num_map, sorted_ids,
                           expert_ids, num_post_pad, expert_offsets, workspace, workspace_bytes,
                           static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------
// Allocation-free variant.
//
// Some hosts of this library may not create device memory at all: a plug-in that runs inside
// another runtime's memory pool, code that executes while that runtime forbids allocation (for
// example between the points where its allocator may be entered), or a C caller that simply has
// no allocator for scratch buffers.  For them the chunk x expert count matrix of the multi-launch
// align path lives in a fixed array inside the library image instead of a caller workspace.
// The price is a size limit and the loss of re-entrancy (see the header comment).
// ---------------------------------------------------------------------------
namespace xkb {
namespace {

constexpr int64_t kStaticMaxSlots = 262144;   // numel limit: 256 chunks of 1024 slots
constexpr int kStaticMaxExperts = 256;        // num_experts limit
constexpr int64_t kStaticChunks = kStaticMaxSlots / kChunk;
constexpr int64_t kStaticInts = kStaticChunks * (kStaticMaxExperts + 1) + (kStaticMaxExperts + 1) + 256;

// 265 220 bytes (259 KiB) per GPU that loads the library, held until the process exits.
static __device__ __align__(256) int32_t g_align_static_scratch[kStaticInts];

constexpr int kMaxDevices = 64;
std::atomic<void*> g_static_ptr[kMaxDevices];   // device address of the array, per device (zero-initialised)

// The array's name is only a host-side handle; the device address has to be asked for, once per
// device, with that device current.  The address is looked up for the device that is CURRENT at
// the call, so the stream passed in must belong to the current device (as for any launch).
// Threads that race on a device's first call all store the same value.
int static_scratch_address(void** out) {
  int dev = -1;
  XKB_CHECK_CUDA(cudaGetDevice(&dev));
  XKB_REQUIRE(dev >= 0 && dev < kMaxDevices, "moe_align (static): device index %d not supported", dev);
  void* p = g_static_ptr[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    XKB_CHECK_CUDA(cudaGetSymbolAddress(&p, g_align_static_scratch));
    XKB_REQUIRE(p != nullptr, "moe_align (static): cudaGetSymbolAddress returned a null address");
    g_static_ptr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return XKB_OK;
}

}  // namespace
}  // namespace xkb

extern "C" int xkb_moe_align_block_size_static(const int32_t* topk_ids, int64_t numel, int num_experts,
                                               int block_size, const int32_t* expert_map, int num_map,
                                               int32_t* sorted_ids, int32_t* expert_ids,
                                               int32_t* num_post_pad, int32_t* expert_offsets,
                                               void* stream) {
  using namespace xkb;
  XKB_REQUIRE(numel >= 0 && numel <= kStaticMaxSlots,
              "moe_align (static): numel=%lld exceeds the built-in scratch limit of %lld token-slots; "
              "use xkb_moe_align_block_size with a caller workspace",
              (long long)numel, (long long)kStaticMaxSlots);
  XKB_REQUIRE(num_experts >= 0 && num_experts <= kStaticMaxExperts,
              "moe_align (static): num_experts=%d exceeds the built-in scratch limit of %d; "
              "use xkb_moe_align_block_size with a caller workspace",
              num_experts, kStaticMaxExperts);
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != XKB_OK) return rc;
  // Nothing in the scratch has to start at zero: the count kernel writes every entry of the
  // chunk x expert matrix that the later kernels read, and the offsets slice is fully rewritten.
  return launch_align(topk_ids, numel, num_experts, block_size, expert_map, num_map, sorted_ids,
                      expert_ids, num_post_pad, expert_offsets, scratch,
                      kStaticInts * (int64_t)sizeof(int32_t), static_cast<cudaStream_t>(stream));
}

// tcgen05 grouped expert GEMM for INT4 W4A16 (sm_100a).
//
// Swap-AB formulation: the 4-bit weights are the UMMA "A" operand (M = 128
// weight rows per CTA tile) and the routed tokens the "B" operand (N = BT
// tokens of one expert block), so a decode batch with a handful of tokens per
// expert still fills the 128-row datapath and the kernel's cost is the weight
// stream.  Per CTA, twelve warps:
//
//   warp 0   TMA producer, weights: packed int32 tile [128 rows x 128 B] (128B
//            swizzle, so that one row per thread reads conflict-free) + bf16
//            scale tile [128 x 8] per 256-wide K stage.
//   warp 1   TMA producer, tokens: [BT x 64] bf16 tiles (128B swizzle = the UMMA
//            K-major canonical layout) from the gathered activation buffer.
//            It also allocates and releases tensor memory.
//   warps 2-3 MMA issuers: tcgen05.mma kind::f16, A from tensor memory, B from
//            shared memory, fp32 accumulators in tensor memory (two issuers with
//            one accumulator each for token tiles <= 64, one issuer above).
//   warps 4-11 dequantisers: thread = weight row; nibbles -> exact bf16 integers
//            by the 0x4300|nib trick, minus 136, times the group scale in one
//            bf16 multiply (= the reference's single rounding,
//            src/xkernels/ops/moe/w4a16.py:44-50), written to tensor memory with
//            tcgen05.st as the next 64-wide A slice.  They also run the epilogue:
//            tcgen05.ld, x topk_w in fp32, store to the fp32 slot-indexed rows.
//
// The dequantiser emits each packed word's nibbles in the order 0,4,1,5,2,6,3,7
// (two nibbles per mask, no cross-lane moves); the activation gather kernel
// writes A with the same permutation inside every group of eight K elements, so
// the dot products are unchanged.
//
// Every mbarrier wait is bounded (tc_common.cuh); on a time-out the CTA records
// a status code, all roles leave their loops, and tensor memory is released.
#include "moe_kernels.h"
#include "tc_common.cuh"

namespace xkb {
namespace {

using namespace tc;

constexpr int kTileRows = 128;   // weight rows per tile (UMMA M)
constexpr int kStageK = 256;     // K per weight pipeline stage
constexpr int kSubK = 64;        // K per token stage / tensor-memory A slot
constexpr int kSubs = kStageK / kSubK;
constexpr int kAColsPerSlot = kSubK / 2;               // 32 columns of bf16 pairs per A slot
constexpr int kWStages = 4;
constexpr int kCtrlWarps = 6;      // weight producer, token producer, up to four MMA issuers
constexpr int kPackedStageBytes = kTileRows * (kStageK / 2);  // 16 KiB
constexpr int kScaleStageBytes = kTileRows * (kStageK / 32) * 2;  // 2 KiB

template <int BT> struct TcCfg {
  // Token (B operand) ring: a stage holds kBSub sub-tiles of [BT x 64]; small token tiles
  // are loaded several at a time so that one barrier round trip covers up to 256 K.  With two
  // MMA issuers kBSub must be a multiple of 2 (each issuer waits/releases once per stage).
  static constexpr int kBSub = (BT <= 32) ? 4 : (BT == 64) ? 2 : 1;
  static constexpr int kBStages = (BT <= 32) ? 3 : 4;
  static constexpr int kBSubBytes = BT * kSubK * 2;
  static constexpr int kBStageBytes = kBSub * kBSubBytes;
  // MMA issuers: narrow token tiles make the MMAs short (about 45 cycles each whatever N <= 64),
  // so the issuing thread's own instruction stream becomes the limit; two issuer warps then
  // take alternate K slices, each into its own accumulator (summed in the epilogue).
  static constexpr int kIssuers = (BT <= 64) ? 2 : 1;
  // Dequantiser warpgroups (4 warps each).  Two CTAs share an SM for narrow tiles (2 x 2
  // warpgroups); wider tiles run one CTA per SM with four.  Warpgroup w owns the K slices
  // sub = w, w + kWGs, ... of every 256-wide stage.
  static constexpr int kWGs = (BT <= 32) ? 2 : 4;
  static constexpr int kDequantWarps = 4 * kWGs;
  static constexpr int kThreads = 32 * (kCtrlWarps + kDequantWarps);
  static constexpr int kAcc = kIssuers;
  static constexpr int kDCols = kAcc * BT;
  static constexpr int kTmemCols = (BT <= 32) ? 256 : 512;
  static constexpr int kASlots = (BT <= 32) ? 4 : 8;     // multiple of kIssuers and of kWGs
  static constexpr int kACol0 = kDCols;                  // A ring starts after the accumulators
  static_assert(kDCols + kASlots * kAColsPerSlot <= kTmemCols, "tensor memory overcommitted");
  static constexpr size_t kSmemBytes = 1024 /*alignment slack*/ + (size_t)kWStages * kPackedStageBytes +
                                       (size_t)kBStages * kBStageBytes + (size_t)kWStages * kScaleStageBytes +
                                       1024 /*barriers*/;
};

#ifdef XKB_TC_TRACE
// Debug builds only: CTA 0 logs (clock, tag) pairs per role into a global buffer.
constexpr int kTraceCap = 4096;
}  // namespace
__device__ long long g_trace[8][kTraceCap];
__device__ int g_trace_n[8];
namespace {
#define TRACE(role, tag)                                                         \
  do {                                                                           \
    if (blockIdx.x == 0 && trace_i < kTraceCap) {                                \
      g_trace[role][trace_i++] = (clock64() << 8) | (tag);                       \
      g_trace_n[role] = trace_i;                                                 \
    }                                                                            \
  } while (0)
#else
#define TRACE(role, tag) do {} while (0)
#endif

struct TcParams {
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* num_post;
  const float* topk_w;
  float* scratch;
  int* status;
  int64_t numel;
  int N, K;
  int mul_w;
};

// (x & 0x000F000F) | 0x43004300  ->  two bf16 values 128 + nibble
__device__ __forceinline__ uint32_t nib_pair(uint32_t x) {
  uint32_t r;
  asm("lop3.b32 %0, %1, 0x000F000F, 0x43004300, 0xEA;" : "=r"(r) : "r"(x));  // (a & b) | c
  return r;
}
__device__ __forceinline__ uint32_t dequant_pair(uint32_t biased, uint32_t scale2) {
  const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&biased);
  const uint32_t k136 = 0x43084308u;  // 136.0 = 128 + zero point 8, twice
  const __nv_bfloat162 q = __hsub2(v, *reinterpret_cast<const __nv_bfloat162*>(&k136));
  const __nv_bfloat162 w = __hmul2(q, *reinterpret_cast<const __nv_bfloat162*>(&scale2));
  return *reinterpret_cast<const uint32_t*>(&w);
}

template <int BT>
__global__ void __launch_bounds__(TcCfg<BT>::kThreads, (BT <= 32) ? 2 : 1)
int4_tc_kernel(const __grid_constant__ CUtensorMap tm_packed, const __grid_constant__ CUtensorMap tm_scale,
               const __grid_constant__ CUtensorMap tm_tokens, const TcParams p) {
  using Cfg = TcCfg<BT>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                         ~uintptr_t(1023));
  unsigned char* s_packed = smem;                                         // kWStages x 16 KiB
  unsigned char* s_tokens = s_packed + kWStages * kPackedStageBytes;      // kBStages x BT*128
  unsigned char* s_scale = s_tokens + Cfg::kBStages * Cfg::kBStageBytes;  // kWStages x 2 KiB
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_scale + kWStages * kScaleStageBytes);
  uint64_t* w_full = bars;                       // [kWStages]
  uint64_t* w_empty = w_full + kWStages;         // [kWStages]
  uint64_t* b_full = w_empty + kWStages;         // [kBStages]
  uint64_t* b_empty = b_full + Cfg::kBStages;    // [kBStages]
  uint64_t* a_full = b_empty + Cfg::kBStages;    // [kASlots]
  uint64_t* a_empty = a_full + Cfg::kASlots;     // [kASlots]
  uint64_t* d_full = a_empty + Cfg::kASlots;     // [1]
  uint64_t* d_empty = d_full + 1;                // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_empty + 1);
  int* abort_word = reinterpret_cast<int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  Guard guard{abort_word, p.status};
#ifdef XKB_TC_TRACE
  int trace_i = 0;
#endif

  if (threadIdx.x == 0) {
    for (int i = 0; i < kWStages; ++i) { mbar_init(&w_full[i], 1); mbar_init(&w_empty[i], Cfg::kDequantWarps); }
    for (int i = 0; i < Cfg::kBStages; ++i) { mbar_init(&b_full[i], 1); mbar_init(&b_empty[i], Cfg::kIssuers); }
    for (int i = 0; i < Cfg::kASlots; ++i) { mbar_init(&a_full[i], 4); mbar_init(&a_empty[i], 1); }
    mbar_init(d_full, Cfg::kIssuers);
    mbar_init(d_empty, Cfg::kDequantWarps);
    *abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, Cfg::kTmemCols);
  if (warp == 0 && lane == 0) { prefetch_tensormap(&tm_packed); prefetch_tensormap(&tm_scale); }
  if (warp == 1 && lane == 0) prefetch_tensormap(&tm_tokens);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int n_tiles = p.N / kTileRows;
  const int n_blocks = p.num_post[0] / BT;
  const int64_t total_tiles = (int64_t)n_blocks * n_tiles;
  const int k_stages = p.K / kStageK;

  if (warp == 0) {
    // ---------------- weight producer ----------------
    if (lane == 0) {
      uint32_t st = 0, ph = 0;
      for (int64_t t = blockIdx.x; t < total_tiles && !guard.aborted(); t += gridDim.x) {
        const int nt = (int)(t % n_tiles), b = (int)(t / n_tiles);
        const int row0 = p.expert_ids[b] * p.N + nt * kTileRows;
        for (int ks = 0; ks < k_stages; ++ks) {
          TRACE(0, 1);
          if (!mbar_wait(&w_empty[st], ph ^ 1, guard, 1, 400)) break;
          TRACE(0, 2);
          mbar_expect_tx(&w_full[st], kPackedStageBytes + kScaleStageBytes);
          tma_load_2d(s_packed + st * kPackedStageBytes, &tm_packed, &w_full[st], ks * (kStageK / 2), row0);
          tma_load_2d(s_scale + st * kScaleStageBytes, &tm_scale, &w_full[st], ks * (kStageK / 32), row0);
          if (++st == kWStages) { st = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- token producer ----------------
    if (lane == 0) {
      uint32_t st = 0, ph = 0;
      for (int64_t t = blockIdx.x; t < total_tiles && !guard.aborted(); t += gridDim.x) {
        const int b = (int)(t / n_tiles);
        const int pos0 = b * BT;
        for (int s = 0; s < k_stages * kSubs; s += Cfg::kBSub) {
          TRACE(1, 1);
          if (!mbar_wait(&b_empty[st], ph ^ 1, guard, 2, 400)) break;
          TRACE(1, 2);
          mbar_expect_tx(&b_full[st], Cfg::kBStageBytes);
#pragma unroll
          for (int j = 0; j < Cfg::kBSub; ++j)
            tma_load_2d(s_tokens + st * Cfg::kBStageBytes + j * Cfg::kBSubBytes, &tm_tokens, &b_full[st],
                        (s + j) * kSubK, pos0);
          if (++st == Cfg::kBStages) { st = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp < kCtrlWarps) {
    // ---------------- MMA issuer(s) ----------------
    // Issuer i takes the K slices g with g % kIssuers == i and accumulates into accumulator i.
    const int me = warp - 2;
    if (lane == 0 && me < Cfg::kIssuers) {
      constexpr uint32_t idesc = umma_idesc_bf16(kTileRows, BT);
      constexpr int kStep = Cfg::kIssuers;
      uint32_t bst = 0, bph = 0, aq = me, aph = 0, eph = 0;
      const uint32_t d_tmem = tmem_base + me * BT;
      for (int64_t t = blockIdx.x; t < total_tiles && !guard.aborted(); t += gridDim.x) {
        // the previous tile's accumulators must have been read out by every epilogue thread
        bool ok = mbar_wait(d_empty, eph ^ 1, guard, 8, 100);
        eph ^= 1;
        if (ok) tc_fence_after();
        for (int s = me; s < k_stages * kSubs && ok; s += kStep) {
          const int bsub = s % Cfg::kBSub;
          TRACE(2, 1);
          ok = mbar_wait(&a_full[aq], aph, guard, 3, 100);
          TRACE(2, 2);
          // first slice of this issuer inside a token stage: the stage must have landed
          if (ok && bsub < kStep) ok = mbar_wait(&b_full[bst], bph, guard, 4);
          if (!ok) break;
          tc_fence_after();
          TRACE(2, 3);
          const uint32_t a_tmem = tmem_base + Cfg::kACol0 + aq * kAColsPerSlot;
          const uint64_t b_desc =
              umma_desc_k_sw128(smem_u32(s_tokens + bst * Cfg::kBStageBytes + bsub * Cfg::kBSubBytes));
#pragma unroll
          for (int kk = 0; kk < kSubK / 16; ++kk)  // the first MMA of a tile overwrites the accumulator
            umma_ts_bf16(d_tmem, a_tmem + kk * 8, b_desc + (uint64_t)(kk * 2), idesc, (s != me || kk != 0) ? 1u : 0u);
          TRACE(2, 4);
          tc_commit(&a_empty[aq]);
          TRACE(2, 5);
          aq += kStep;
          if (aq >= (uint32_t)Cfg::kASlots) { aq -= Cfg::kASlots; aph ^= 1; }
          // last slice of this issuer inside the token stage: release it
          if (bsub + kStep >= Cfg::kBSub) {
            tc_commit(&b_empty[bst]);
            if (++bst == Cfg::kBStages) { bst = 0; bph ^= 1; }
          }
        }
        if (!ok) break;
        tc_commit(d_full);
      }
    }
  } else {
    // ---------------- dequantisers + epilogue ----------------
    // K slices of 64 are numbered g = 0,1,2,... across stages and tiles; slice g goes to
    // tensor-memory slot g % kASlots and is produced by warpgroup g % kWGs.
    // A slice is stored eight columns at a time as its words are dequantised and published
    // as soon as the stores have completed.
    const int wg = (warp - kCtrlWarps) >> 2;
    const int quarter = warp & 3;              // tensor-memory lane quarter this warp may access
    const int row = quarter * 32 + lane;       // weight row inside the tile
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    uint32_t wst = 0, wph = 0, dph = 0;
    uint32_t aq = wg, aph = 0;                 // next slot of this warpgroup and its phase
    for (int64_t t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      const int nt = (int)(t % n_tiles), b = (int)(t / n_tiles);
      bool ok = true;
      for (int ks = 0; ks < k_stages && ok; ++ks) {
        if (lane == 0 && quarter == 0) TRACE(3 + wg, 1);
        if (!mbar_wait(&w_full[wst], wph, guard, 5)) { ok = false; break; }
        if (lane == 0 && quarter == 0) TRACE(3 + wg, 2);
        const unsigned char* pk = s_packed + wst * kPackedStageBytes + row * 128;
        const uint4 sc = *reinterpret_cast<const uint4*>(s_scale + wst * kScaleStageBytes + row * 16);
        const uint32_t sc_w[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
        for (int i = 0; i < kSubs / Cfg::kWGs; ++i) {
          const int sub = wg + Cfg::kWGs * i;
          if (lane == 0 && quarter == 0) TRACE(3 + wg, 3);
          if (!mbar_wait(&a_empty[aq], aph ^ 1, guard, 6)) { ok = false; break; }
          tc_fence_after();
          if (lane == 0 && quarter == 0) TRACE(3 + wg, 4);
          const uint32_t dst = tmem_base + lane_base + Cfg::kACol0 + aq * kAColsPerSlot;
          uint32_t sw = sc_w[0];  // the two group scales of slice `sub` (static indices only)
#pragma unroll
          for (int q = 1; q < kSubs; ++q)
            if (q == sub) sw = sc_w[q];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int chunk = sub * 2 + h;  // 16-byte chunk = 32 weights = one scale group
            const uint4 w4 = *reinterpret_cast<const uint4*>(pk + ((chunk ^ (row & 7)) << 4));
            const uint32_t s2 = h ? __byte_perm(sw, sw, 0x3232) : __byte_perm(sw, sw, 0x1010);
            const uint32_t words[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int wp = 0; wp < 2; ++wp) {  // two words = 16 weights = 8 columns
              const uint32_t x0 = words[2 * wp], x1 = words[2 * wp + 1];
              tmem_st_32x8(dst + h * 16 + wp * 8,
                           dequant_pair(nib_pair(x0), s2), dequant_pair(nib_pair(x0 >> 4), s2),
                           dequant_pair(nib_pair(x0 >> 8), s2), dequant_pair(nib_pair(x0 >> 12), s2),
                           dequant_pair(nib_pair(x1), s2), dequant_pair(nib_pair(x1 >> 4), s2),
                           dequant_pair(nib_pair(x1 >> 8), s2), dequant_pair(nib_pair(x1 >> 12), s2));
            }
          }
          if (i == kSubs / Cfg::kWGs - 1) {  // last read of this stage is done: one arrival per warp
            __syncwarp();
            if (lane == 0) mbar_arrive(&w_empty[wst]);
          }
          if (lane == 0 && quarter == 0) TRACE(3 + wg, 5);
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&a_full[aq]);
          if (lane == 0 && quarter == 0) TRACE(3 + wg, 6);
          aq += Cfg::kWGs;
          if (aq >= (uint32_t)Cfg::kASlots) { aq -= Cfg::kASlots; aph ^= 1; }
        }
        if (++wst == kWStages) { wst = 0; wph ^= 1; }
      }
      if (!ok) break;
      // epilogue (the warpgroups take the 16-column groups round robin):
      // sum of the kAcc accumulators -> x topk_w -> fp32 slot rows
      if (!mbar_wait(d_full, dph, guard, 7)) break;
      dph ^= 1;
      tc_fence_after();
      const int64_t n_glob = (int64_t)nt * kTileRows + row;
      const int32_t* slots = p.sorted_ids + (int64_t)b * BT;
#pragma unroll 1
      for (int c0 = wg * 16; c0 < BT; c0 += 16 * Cfg::kWGs) {
        uint32_t acc[16];
        tmem_ld_32x16(tmem_base + lane_base + c0, acc);
        tmem_wait_ld();
#pragma unroll
        for (int a = 1; a < Cfg::kAcc; ++a) {
          uint32_t more[16];
          tmem_ld_32x16(tmem_base + lane_base + a * BT + c0, more);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[j] = __float_as_uint(__uint_as_float(acc[j]) + __uint_as_float(more[j]));
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int32_t slot = __ldg(slots + c0 + j);  // same address for the whole warp
          if (slot >= 0 && slot < p.numel) {
            float v = __uint_as_float(acc[j]);
            if (p.mul_w) v = p.topk_w[slot] * v;
            p.scratch[(int64_t)slot * p.N + n_glob] = v;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(d_empty);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ---------------------------------------------------------------------------
// Activation gather: Ag[p, :] = A[sorted_ids[p] / top_k, :] with the nibble-order
// permutation (0,4,1,5,2,6,3,7) applied inside every group of 8 K elements.
// Padding positions are left untouched: their accumulator columns are never read.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gather_permute_kernel(const __nv_bfloat16* __restrict__ A, const int32_t* __restrict__ sorted_ids,
                      const int32_t* __restrict__ num_post, __nv_bfloat16* __restrict__ Ag, int64_t numel,
                      int K, int top_k) {
  const int total = num_post[0];
  for (int64_t pos = blockIdx.x; pos < total; pos += gridDim.x) {
    const int32_t slot = sorted_ids[pos];
    if (slot < 0 || slot >= numel) continue;
    const uint4* src = reinterpret_cast<const uint4*>(A + (int64_t)(slot / top_k) * K);
    uint4* dst = reinterpret_cast<uint4*>(Ag + pos * K);
    for (int i = threadIdx.x; i < K / 8; i += blockDim.x) {
      const uint4 v = __ldg(src + i);  // elements e0..e7 as (e1:e0, e3:e2, e5:e4, e7:e6)
      uint4 o;
      o.x = __byte_perm(v.x, v.z, 0x5410);  // (e4 : e0)
      o.y = __byte_perm(v.x, v.z, 0x7632);  // (e5 : e1)
      o.z = __byte_perm(v.y, v.w, 0x5410);  // (e6 : e2)
      o.w = __byte_perm(v.y, v.w, 0x7632);  // (e7 : e3)
      dst[i] = o;
    }
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// 2-D row-major tensor [rows, cols] of `elem_bytes` elements, box [box_rows, box_cols].
int make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t rows,
                uint64_t cols, uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swz, const char* what) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return fail(XKB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  XKB_REQUIRE(reinterpret_cast<uintptr_t>(base) % 16 == 0, "%s: base pointer must be 16-byte aligned", what);
  XKB_REQUIRE((cols * elem_bytes) % 16 == 0, "%s: row pitch %llu B is not a multiple of 16", what,
              (unsigned long long)(cols * elem_bytes));
  XKB_REQUIRE(box_rows <= 256 && box_cols <= 256 && (box_cols * elem_bytes) % 16 == 0, "%s: bad box", what);
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * (uint64_t)elem_bytes};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(XKB_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r);
  return XKB_OK;
}

template <int BT>
int launch_bt(const CUtensorMap& tmp, const CUtensorMap& tms, const CUtensorMap& tmt, const TcParams& prm,
              int64_t max_tiles, cudaStream_t stream) {
  using Cfg = TcCfg<BT>;
  XKB_CHECK_CUDA(cudaFuncSetAttribute(int4_tc_kernel<BT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)Cfg::kSmemBytes));
  int dev = 0, sms = 148;
  XKB_CHECK_CUDA(cudaGetDevice(&dev));
  XKB_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  // resident CTAs per SM: bounded by shared memory and by 512 tensor-memory columns
  int per_sm = (int)((227 * 1024) / Cfg::kSmemBytes);
  const int by_tmem = 512 / Cfg::kTmemCols;
  if (per_sm > by_tmem) per_sm = by_tmem;
  if (per_sm < 1) per_sm = 1;
  int64_t grid = (int64_t)sms * per_sm;
  if (grid > max_tiles) grid = max_tiles;
  if (grid < 1) grid = 1;
  {
    GemmTimerScope timed(stream);
    int4_tc_kernel<BT><<<(unsigned)grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(tmp, tms, tmt, prm);
  }
  XKB_CHECK_LAUNCH("int4_tc_kernel");
  return XKB_OK;
}

}  // namespace

bool int4_tc_supported(int a_dtype, int64_t M, int64_t N, int64_t K, int E, int top_k, int group) {
  return a_dtype == XKB_BF16 && group == 32 && N > 0 && N % kTileRows == 0 && K > 0 && K % kStageK == 0 &&
         M > 0 && E > 0 && top_k > 0 && (int64_t)E * N < (1ll << 31) && K < (1 << 30);
}

int int4_tc_block(int64_t numel, int E) {
  const double avg = (double)numel / (E > 0 ? E : 1);
  if (avg <= 12) return 16;
  if (avg <= 24) return 32;
  if (avg <= 48) return 64;
  if (avg <= 96) return 128;
  return 256;
}

int64_t int4_tc_workspace_bytes(int64_t numel, int64_t N, int64_t K, int E) {
  (void)N;
  // gathered activations for the largest token tile
  return align_up((numel + (int64_t)(E + 1) * 255) * K * 2, 256);
}

int launch_int4_tc(const void* A, const int32_t* packed, const void* scale, const Routing& r,
                   const float* topk_w, float* scratch, int64_t N, int64_t K, int E, int top_k, int mul_w,
                   void* tc_ws, int* status, cudaStream_t stream) {
  Carver carve(tc_ws);
  __nv_bfloat16* Ag = carve.take<__nv_bfloat16>(r.max_pad * K);

  int64_t gblocks = r.max_pad < 148 * 16 ? r.max_pad : 148 * 16;
  if (gblocks < 1) gblocks = 1;
  gather_permute_kernel<<<(unsigned)gblocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(A),
                                                               r.sorted_ids, r.num_post, Ag, r.numel, (int)K,
                                                               top_k);
  XKB_CHECK_LAUNCH("gather_permute_kernel");

  CUtensorMap tm_packed, tm_scale, tm_tokens;
  int rc = make_map_2d(&tm_packed, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, packed, (uint64_t)E * N, (uint64_t)K / 2,
                       kTileRows, kStageK / 2, CU_TENSOR_MAP_SWIZZLE_128B, "packed weights");
  if (rc != XKB_OK) return rc;
  rc = make_map_2d(&tm_scale, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, scale, (uint64_t)E * N, (uint64_t)K / 32,
                   kTileRows, kStageK / 32, CU_TENSOR_MAP_SWIZZLE_NONE, "group scales");
  if (rc != XKB_OK) return rc;
  rc = make_map_2d(&tm_tokens, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Ag, (uint64_t)r.max_pad, (uint64_t)K,
                   (uint32_t)r.block, kSubK, CU_TENSOR_MAP_SWIZZLE_128B, "gathered activations");
  if (rc != XKB_OK) return rc;

  TcParams prm;
  prm.sorted_ids = r.sorted_ids;
  prm.expert_ids = r.expert_ids;
  prm.num_post = r.num_post;
  prm.topk_w = topk_w;
  prm.scratch = scratch;
  prm.status = status;
  prm.numel = r.numel;
  prm.N = (int)N;
  prm.K = (int)K;
  prm.mul_w = mul_w;
  const int64_t max_tiles = r.max_blocks * (N / kTileRows);
  switch (r.block) {
    case 16: return launch_bt<16>(tm_packed, tm_scale, tm_tokens, prm, max_tiles, stream);
    case 32: return launch_bt<32>(tm_packed, tm_scale, tm_tokens, prm, max_tiles, stream);
    case 64: return launch_bt<64>(tm_packed, tm_scale, tm_tokens, prm, max_tiles, stream);
    case 128: return launch_bt<128>(tm_packed, tm_scale, tm_tokens, prm, max_tiles, stream);
    case 256: return launch_bt<256>(tm_packed, tm_scale, tm_tokens, prm, max_tiles, stream);
    default: return fail(XKB_ERR_ARG, "int4 tcgen05 path: unsupported token tile %d", r.block);
  }
}

// ---- MXFP4 tcgen05 path: not built yet, the SIMT kernels serve every shape ----
bool mxfp4_tc_supported(int, int64_t, int64_t, int64_t, int, int) { return false; }
int mxfp4_tc_block(int64_t, int) { return kSimtBlock; }
int64_t mxfp4_tc_workspace_bytes(int64_t, int64_t, int64_t, int) { return 256; }
int launch_mxfp4_tc(const void*, const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, const void*,
                    const void*, const Routing&, const float*, __nv_bfloat16*, float*, int64_t, int64_t, int, int,
                    float, int, void*, int*, cudaStream_t) {
  return fail(XKB_ERR_ARG, "the MXFP4 tcgen05 path is not available");
}

}  // namespace xkb

#ifdef XKB_TC_TRACE
extern "C" int xkb_debug_trace(long long* host, int* counts_host) {
  int zero[8] = {0};
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(counts_host, xkb::g_trace_n, sizeof(int) * 8);
  cudaMemcpyFromSymbol(host, xkb::g_trace, sizeof(long long) * 8 * xkb::kTraceCap);
  cudaMemcpyToSymbol(xkb::g_trace_n, zero, sizeof(zero));
  return 0;
}
#endif

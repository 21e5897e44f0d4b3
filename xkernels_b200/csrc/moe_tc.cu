// tcgen05 grouped expert GEMM for INT4 W4A16 and MXFP4 weights (sm_100a).
//
// Swap-AB formulation: the 4-bit weights are the UMMA "A" operand (M = 128
// weight rows per CTA tile) and the routed tokens the "B" operand (N = BT
// tokens of one expert block), so a decode batch with a handful of tokens per
// expert still fills the 128-row datapath and the kernel's cost is the weight
// stream.  One persistent CTA per SM (it owns all 512 tensor-memory columns),
// twenty or twenty-one warps, everything handed over in whole 256-K stages:
//
//   warp 0   TMA producer, weights: packed tile [128 rows x 128 B] (128B swizzle, so that one
//            row per thread reads conflict-free) + scale tile per stage: bf16 [128 x 8] for INT4,
//            e8m0 bytes [128 x 16] for MXFP4 (sixteen bytes are the smallest TMA row, so a tile
//            carries the scales of two stages and each stage uses its half).
//   then     two or three MMA issuer warps (lane 0 each; warp 1 also allocates and frees tensor
//            memory): tcgen05.mma kind::f16, A from tensor memory, B from shared
//            memory, fp32 accumulators in tensor memory.  They take whole stages in
//            turn, each into its own accumulator.
//   then     TMA producer, tokens: four [BT x 64] bf16 sub-tiles per stage (128B swizzle =
//            the UMMA K-major canonical layout) from the gathered activation buffer.  (In a
//            warp of its own: two polling threads in one warp slow each other down.)
//   then     sixteen dequantiser warps: thread = weight row; nibbles -> exact bf16 integers
//            by the 0x4300|nib trick, minus 136, times the group scale in one
//            bf16 multiply (= the reference's single rounding,
//            src/xkernels/ops/moe/w4a16.py:44-50), written to tensor memory with
//            tcgen05.st as (their share of) the stage's 128-column A slot.  They
//            also run the epilogue, one stage into the next tile: tcgen05.ld, sum
//            of the issuers' partial accumulators, x topk_w in fp32, store to the
//            fp32 slot-indexed rows (or the fused SwiGLU of the MXFP4 gate_up mode).
//
// The dequantiser emits each packed word's nibbles in the order 0,4,1,5,2,6,3,7
// (two nibbles per mask, no cross-lane moves); the activation gather kernel
// writes A with the same permutation inside every group of eight K elements, so
// the dot products are unchanged.
//
// mbarrier parity waits only tell "the phase with this parity is over", so a
// waiter must never fall two phases behind a barrier.  Every role here either
// visits every use of a barrier in order or skips uses in a pattern for which the
// previous use is implied by something it has already seen; the configuration
// comments say which.
//
// Every mbarrier wait is bounded (tc_common.cuh); on a time-out the CTA records
// a status code, all roles leave their loops, and tensor memory is released.

#include <atomic>
#include <mutex>
#include "moe_kernels.h"
#include "tc_common.cuh"

namespace xkb {
std::atomic<int> g_sm_margin{0};
namespace {

using namespace tc;

constexpr int kTileRows = 128;   // weight rows per tile (UMMA M)
constexpr int kStageK = 256;     // K per pipeline stage (weights, tokens and the tensor-memory A slot alike)
constexpr int kSubK = 64;        // K per 128-byte swizzled token sub-tile / per dequantiser warpgroup
constexpr int kSubs = kStageK / kSubK;  // 4
constexpr int kSlotCols = kStageK / 2;                 // 128 columns of bf16 pairs per A slot
constexpr int kSubCols = kSubK / 2;                    // 32 of them per warpgroup
constexpr int kMaxIssuers = 4;
constexpr int kMxIssuers = 2;          // MMA issuer warps of the two-matrix modes at token tiles <= 32 (2 or 4)
constexpr int kInt4TwoMatIssuers = 4;   // measured on the two-GEMM layer at decode: 290 us with four, 307 with two
constexpr int kWStagesNarrow = 6;      // weight ring depth for token tiles of 16
constexpr int kBStages16 = 9;          // token ring depth for token tiles of 16
constexpr uint32_t kProdSleepNs = 400; // back-off of the TMA producers, which run a whole ring ahead
constexpr uint32_t kIssSleepNs = 32;   // back-off of the MMA issuers (on the critical path: short)
constexpr int kNarrowWGs = 4;          // dequantiser warpgroups for token tiles <= 64
// Hand-off units per 256-K stage (1 = the whole stage, or one unit per warpgroup that shares the
// stage): every unit has its own tensor-memory slot and its own full/empty barriers, so its MMAs
// start as soon as its warpgroup has published it and its slot is free again as soon as they end.
constexpr int kUnitsNarrow = 2;        // token tiles <= 64: two warpgroups share a stage
constexpr int kUnitsWide = 4;          // token tiles of 128: four warpgroups share a stage
// A tile's accumulators are read out by the dequantiser warps after they have converted this many
// further stages of their own: the last MMAs of the tile (about one conversion time of issue and
// commit latency behind the conversion) have then long completed and the read-out never waits.
constexpr int kEpiDelay = 2;
// The dequantiser warps hand a weight stage back to the TMA producer as soon as they have read it
// from shared memory into registers, before they convert it (one arrival per warp of the group):
// the turn-round of a ring slot (TMA latency + wait for the readers + their wake-up) then does not
// contain the conversion time.
// MMA issuer warps run their loop with all 32 lanes (waits included) and only the tcgen05.mma /
// commit / arrive instructions themselves are predicated on lane 0: the loop is then warp-uniform
// and descriptors and tensor-memory addresses are computed in uniform registers, instead of being
// moved there one by one for every MMA as in a loop that only lane 0 executes.
constexpr bool kUniformIssuer = false;
constexpr int kTmemCols = 512;     // one CTA per SM owns all of tensor memory
constexpr int kPackedStageBytes = kTileRows * (kStageK / 2);  // 16 KiB
constexpr int kScaleStageBytes = kTileRows * (kStageK / 32) * 2;  // 2 KiB

// MATS = weight matrices that alternate 256-K stages inside one tile (MXFP4 gate/up, INT4 row-tile pairs)
//
// Why the hand-off unit matters: a tensor-memory slot is busy from the first converted column until
// the commit of the MMAs that read it comes back, i.e. for (fill time + MMA issue time + barrier
// round trips), and only 384-416 columns are left for slots beside the accumulators.  With whole
// 256-K stages as units that is three slots, and the slot cycle, not any pipe, bounds the kernel.
// Units of half a stage (one warpgroup's share) halve the MMA part of the cycle and let the other
// half be converted meanwhile.
constexpr int gcd_c(int a, int b) { return b == 0 ? a : gcd_c(b, a % b); }
constexpr int lcm_c(int a, int b) { return a / gcd_c(a, b) * b; }

template <int BT, int MATS = 1, bool INT4 = true> struct TcCfg {
  // Dequantiser groups that take alternate stages.  Narrow tiles: two groups of eight warps, so
  // that one group's waits and store drains overlap the other's arithmetic.  Wide tiles are bound by
  // the tensor pipe and have only two A slots; there all sixteen warps fill one slot together,
  // which halves the fill latency in the slot's round trip.
  // dequantiser warpgroups (the four warps of one cover the four tensor-memory lane quarters)
  static constexpr int kWGs = (BT <= 64) ? kNarrowWGs : 4;
  static constexpr int kDequantWarps = 4 * kWGs;
  // Read-out of a tile's accumulators: one task per 16 token columns.  A tile with fewer tasks than
  // warpgroups (token tiles of 16 and 32) is read out by kEpiWGs warpgroups only, and the duty
  // rotates from tile to tile, so that no warpgroup carries the read-out of every tile on top of
  // its share of the conversion.
  static constexpr int kColGroups = BT / 16;
  static constexpr int kEpiWGs = kColGroups < kWGs ? kColGroups : kWGs;
  // Control warps: weight producer, the issuers, token producer.  Narrow INT4 tiles run three
  // issuers (five control warps; 21 warps get 80 registers each, enough for the INT4 dequantiser);
  // the others two issuers (four control warps, 96 registers, which the E2M1 dequantiser needs).
  static constexpr int kCtrlWarps = (BT > 32) ? 4 : (MATS == 1) ? (INT4 ? 5 : 4)
                                                : 2 + (INT4 ? kInt4TwoMatIssuers : kMxIssuers);
  static constexpr int kThreads = 32 * (kCtrlWarps + kDequantWarps);
  static constexpr int kGroups = (BT <= 64) ? kWGs / 2 : 1;
  static constexpr int kGroupWarps = kDequantWarps / kGroups;
  static constexpr int kPartsPerStage = kWGs / kGroups;      // warpgroups that share one stage
  static constexpr int kChunks = 8 / kPartsPerStage;         // 16-byte chunks (32 weights, one scale group) per thread and stage
  static constexpr int kUnits = (BT <= 64) ? kUnitsNarrow : kUnitsWide;   // hand-off units per stage
  static_assert(kUnits == 1 || kUnits == kPartsPerStage, "a unit is a whole stage or one warpgroup's share of it");
  static constexpr int kUnitCols = kSlotCols / kUnits;       // tensor-memory columns of one unit
  static constexpr int kUnitSubs = kSubs / kUnits;           // 64-K token sub-tiles one unit spans
  static_assert(kSubs % kUnits == 0, "a unit must span whole 64-K sub-tiles");
  // Token ring.  A token stage is released by the commit of the MMAs that read it and re-filled by
  // TMA from L2 about a microsecond later; narrow tiles are small, so their ring is made deep
  // enough that the issuers never wait for tokens.
  static constexpr int kBStages = (BT <= 16) ? kBStages16 : (BT <= 32) ? 6 : (BT <= 64) ? (kGroups == 3 ? 3 : 4) : 2;
  static constexpr int kBSubBytes = BT * kSubK * 2;
  static constexpr int kBStageBytes = kSubs * kBSubBytes;   // [4][BT x 64] bf16
  static constexpr int kWStages = (BT <= 16) ? kWStagesNarrow : (BT <= 32 || kGroups == 3) ? 6 : 4;
  static_assert(kWStages % kGroups == 0, "a weight stage must always be converted by the same group");
  // MMA issuers.  One thread sustains one tcgen05.mma per ~45 cycles (65-100 beside busy
  // dequantiser warps) whatever the shape, and that is an issue limit of the thread, not of the
  // tensor pipe: measured aggregate rates for N = 16 are 45 / 27 / 13 cycles per MMA with 1 / 2 / 4
  // issuing warps, while N = 128 is pipe-bound at 64 cycles.  Besides the MMAs a visit to a stage
  // costs the issuing thread several hundred cycles of waits, fences and commits, so the issuers
  // take whole stages in turn: stage g (numbered across the tiles of the CTA) belongs to issuer
  // g % kIssuers, which puts it into its own accumulator (per matrix); the epilogue adds them.
  // (Measured at decode: two issuers + token producer in its own warp 222 us, three issuers with
  // both producers in one warp 238 us, three issuers + five control warps 210 us.)
  static constexpr int kIssuers = kCtrlWarps - 2;
  static_assert(kIssuers <= kMaxIssuers, "not enough issuer warps");
  // One accumulator per issuer.  A tile has a multiple of MATS stages and kIssuers is a multiple of
  // MATS, so the matrix of stage g is g % MATS = (g % kIssuers) % MATS: issuer j only ever sees matrix
  // j % MATS, and accumulator a belongs to matrix a % MATS.  (kIssuers == MATS: one per matrix.)
  static constexpr bool kLocked = (kIssuers == MATS);
  static constexpr int kAccs = kIssuers;
  // Two or three accumulator sets when tensor memory has room beside three stages of A slots: the
  // MMAs of the next tiles start while an earlier tile's accumulators still wait to be read out.
  // (Three sets let the read-out trail two tiles behind, which short tiles need: see kEpiDelay.)
  static constexpr int kDBuf = (3 * kAccs * BT + 3 * kSlotCols <= kTmemCols) ? 3
                               : (2 * kAccs * BT + 3 * kSlotCols <= kTmemCols) ? 2 : 1;
  static constexpr int kDCols = kDBuf * kAccs * BT;         // accumulator a of set d at (d * kAccs + a) * BT
  static constexpr int kACol0 = kDCols;                     // the A slots follow the accumulators
  // A slots, counted in units (three stages' worth at most)
  static constexpr int kASlotsFit = (kTmemCols - kDCols) / kUnitCols;
  static constexpr int kASlots = kASlotsFit > 3 * kUnits ? 3 * kUnits : kASlotsFit;
  static_assert(kASlots >= 2 * kUnits, "need two stages of A slots so that conversion and MMA overlap");
  // mbarrier parity waits only tell "the phase with this parity is over", so a waiter must see every
  // phase of a barrier it waits on.  Unit u = g * kUnits + h (stage g, numbered across the tiles of
  // the CTA; h = the warpgroup's share) is filled by one fixed warpgroup of group g % kGroups and
  // consumed by issuer g % kIssuers; its barriers are number u % kABars with kABars a common
  // multiple of the slot count and of the unit periods of the groups and of the issuers (the slot
  // itself is u % kASlots): every barrier then always has the same producers and the same consumer,
  // and both pass through all of its phases.  The token ring does the same with kBBars (the
  // producer thread visits every token stage).
  static constexpr int kABars = lcm_c(lcm_c(kASlots, kGroups * kUnits), kIssuers * kUnits);
  static constexpr int kBBars = lcm_c(kBStages, kIssuers);
  // the running ring positions of the roles advance by one own stage at a time with a single
  // conditional wrap, and the units of one stage never straddle a wrap
  static_assert(kGroups * kUnits <= kASlots && kASlots % kUnits == 0 && kABars % kUnits == 0, "unit ring arithmetic");
  static_assert(kIssuers % MATS == 0 && kIssuers / MATS <= kBStages, "token ring arithmetic");
  static constexpr int kNumBars = 2 * kWStages + 2 * kBBars + 2 * kABars + 2 * kDBuf;
  static constexpr size_t kBarBytes = ((size_t)kNumBars * 8 + 64 + 127) / 128 * 128;   // + allocation slot, abort word
  // MXFP4 with narrow token tiles converts through a table in shared memory (see kLut below)
  static constexpr bool kLut = !INT4 && BT <= 64;
  static constexpr size_t kLutBytes = kLut ? 256 * 32 * 4 : 0;
  static constexpr size_t kSmemBytes = 1024 /*alignment slack*/ + (size_t)kWStages * kPackedStageBytes +
                                       (size_t)kBStages * kBStageBytes + (size_t)kWStages * kScaleStageBytes +
                                       kBarBytes + kLutBytes;
  static_assert(kSmemBytes <= 227 * 1024, "shared memory overcommitted");
};

// Kernel modes: which weights are streamed and what the epilogue does.
constexpr int kModeInt4 = 0;      // INT4 W4A16: rows = N, bf16 group scales by TMA, fp32 slot rows out
constexpr int kModeMxGateUp = 1;  // MXFP4 w13: a tile is 128 gate rows + the 128 matching up rows, the
                                  // two matrices alternate 256-K stages and accumulators; SwiGLU epilogue
constexpr int kModeMxDown = 2;    // MXFP4 w2: rows = hidden, bf16-rounded result x routing weight out; two 128-row
                                  // weight tiles per token tile like kModeInt4Pair: with K = ispp of a few
                                  // hundred a single-tile pass would be two stages long, and the per-tile work
                                  // (read-out, loop bookkeeping) would weigh as much as the stages themselves
constexpr int kModeInt4Pair = 3;  // INT4 with TWO 128-row weight tiles per token tile (they alternate
                                  // 256-K stages like gate/up): halves the token-tile traffic per flop
constexpr int kModeInt4GateUp = 4;  // INT4 w13 of a two-GEMM expert layer: gate rows and up rows alternate stages like
                                    // kModeMxGateUp, SwiGLU epilogue, bf16 activations out
constexpr bool mode_is_pair(int mode) { return mode == kModeInt4Pair || mode == kModeMxDown; }
constexpr bool mode_is_gate_up(int mode) { return mode == kModeMxGateUp || mode == kModeInt4GateUp; }
constexpr int mode_mats(int mode) { return (mode_is_gate_up(mode) || mode_is_pair(mode)) ? 2 : 1; }
constexpr bool mode_is_int4(int mode) { return mode == kModeInt4 || mode == kModeInt4Pair || mode == kModeInt4GateUp; }

struct TcParams {
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* num_post;
  const float* topk_w;
  float* scratch;               // [M*top_k, N] fp32 slot rows (INT4, MX down)
  int* status;
  int64_t numel;
  int N, K;                     // tile rows are taken from N rows per expert; K = contraction length
  int mul_w;
  int round_rows;               // INT4: round each weighted slot row to bf16 (the second GEMM of a two-GEMM layer,
                                // whose per-slot results the reference composition holds in bf16)
  // MXFP4 only
  const __nv_bfloat16* bias;    // b13 [E, 2*ispp] or b2 [E, hidden] or nullptr
  __nv_bfloat16* act;           // gate_up mode output: [positions, N] bf16 in the K-permuted order
  int rows_per_expert;          // 2*ispp (gate_up) or hidden (down)
  float limit;                  // SwiGLU clamp, <= 0 disables
  // Two GEMMs of one expert layer that overlap (see "block hand-over" at the kernel): the first
  // counts the finished read-outs of every token block in done_signal, the second waits until the
  // count of a block has reached done_target before it loads that block's activations.
  // what the routing may hold at most: a kernel that reads a value outside records status 3 and
  // skips the work instead of using it as an index
  int max_blocks;               // token blocks the routing buffers were sized for
  int num_experts;
  int32_t* done_signal;         // gate_up modes, or nullptr
  const int32_t* done_wait;     // the GEMM that consumes `act` as its tokens, or nullptr
  int done_target;
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

// ---- INT4 -> bf16 without a subtraction and with one shift per word --------------------------
// A bf16 bit pattern whose sign and upper seven exponent bits are zero reads as  m * 2^-133  for
// the 8-bit integer m in bits 7..0: the subnormals (exponent field 0) and the first binade
// (exponent field 1, implicit one worth 2^-126 = 128 * 2^-133) continue each other.  So the two
// low nibbles of each 16-bit half of a packed word are exact bf16 numbers in place, with no magic
// number to subtract again:  x & 0x000F000F = (nib * 2^-133),  x & 0x00F000F0 = (nib * 2^-129),
// and one shift by 8 brings the other two nibbles of each half down.  One fused multiply-add then
// gives  nib * s - 8 * s = (nib - 8) * s  with the single rounding of the reference
// (src/xkernels/ops/moe/w4a16.py:48-50): the product is exact inside the FMA and -8 * s is exact
// as a bf16 number.  Everything is kept 2^-30 smaller than the true weights so that the
// per-position multipliers s * 2^133 and s * 2^129 stay finite: multipliers s * 2^103 and
// s * 2^99, addend -s * 2^-27, and the epilogue multiplies the fp32 accumulators by 2^30, which
// is exact.  Exact for scales with 2^-96 <= |s| < 2^24 (and for s = 0); the host side refuses
// scale tensors outside that range.
constexpr bool kInt4NoSubtract = true;
constexpr uint32_t kMulLo = 0x73007300u;    // 2^103, twice: multiplier for nibbles at bits 3..0
constexpr uint32_t kMulHi = 0x71007100u;    // 2^99: nibbles at bits 7..4
constexpr uint32_t kMulAdd = 0xB200B200u;   // -2^-27 = -8 * 2^-30
constexpr float kInt4Unscale = 1073741824.f;  // 2^30
__device__ __forceinline__ uint32_t bf2_mul(uint32_t a, uint32_t b) {
  const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bf2_fma(uint32_t a, uint32_t b, uint32_t c) {
  const __nv_bfloat162 r = __hfma2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b),
                                   *reinterpret_cast<const __nv_bfloat162*>(&c));
  return *reinterpret_cast<const uint32_t*>(&r);
}

// ---- MXFP4: E2M1 code -> bf16 -------------------------------------------------------------
// The three magnitude bits (e1 e0 m) placed at bf16 bits 8..6 read as  e2m1 * 2^-126  (the code
// 0b001 = 0.5 lands on the bf16 subnormal 2^-127), the sign bit goes to bit 15.  One bf16 multiply
// by a power of two then gives the weight exactly.  The true factor 2^126 * 2^(s-127) does not fit
// bf16 for s > 128, so all weights are kept 2^-62 smaller than they are: the factor is 2^(s-63),
// a bf16 number for every e8m0 byte up to 190, and the epilogue multiplies the fp32 accumulators
// by 2^62, which is exact.  s = 0xFF decodes to 0 like in the reference
// (src/xkernels/ops/gather/mxfp4.py:60-66).  Exact for 57 <= s <= 190 (weights of magnitude
// 2^-70 ... 2^63 and above 2^-134 after scaling); smaller scales land on bf16 subnormals and lose
// bits far below anything an output can show; a scale byte in 191..254 (weights of 2^64 and
// more) is reported through the status word instead of being converted.
constexpr int kMxShift = 62;
constexpr float kMxUnscale = 4611686018427387904.f;   // 2^62
constexpr uint32_t kMxMaxScale = 190;
constexpr int kErrMxScaleRange = 2;                  // status code: an e8m0 scale byte in 191..254
constexpr int kErrBadRouting = 3;    // status code: a routing value read by a kernel was outside what the buffers can hold
__device__ __forceinline__ uint32_t mx_scale_factor(uint32_t s) {
  // exponent field of 2^(s - 1 - kMxShift), twice; 0 for the NaN code
  const uint32_t f = (s + (uint32_t)(126 - kMxShift)) * 0x00800080u;
  return s == 0xFFu ? 0u : f;
}
__device__ __forceinline__ uint32_t mx_pair(uint32_t mag_shifted, uint32_t sign_shifted, uint32_t c) {
  uint32_t t;
  asm("lop3.b32 %0, %1, 0x01C001C0, 0, 0xC0;" : "=r"(t) : "r"(mag_shifted));            // a & b
  asm("lop3.b32 %0, %0, %1, 0x80008000, 0xF8;" : "+r"(t) : "r"(sign_shifted));           // a | (b & c)
  return bf2_mul(t, c);
}
// The decode-sized MXFP4 tiles are bound by the integer pipe when they convert with shifts and masks
// (7 shifts + 8 logic operations per packed word on a half-rate pipe).  They convert through a table
// instead: one 32-bit entry per BYTE value = the two E2M1 codes of the byte as a bf16 pair (even k
// low), 256 entries, replicated for the 32 lanes so that lane l only ever reads bank l (entry b of
// lane l at word b * 32 + l: conflict-free whatever the data).  A byte then costs one shift, one
// logic operation (mask and merge with the lane's base address), one shared-memory load and one bf16
// multiply by the exact power of two 2^(s-127) -- no scaled accumulators, no scale range limit --
// and the weights come out in natural K order, so these tiles use no K permutation.
__device__ __forceinline__ uint32_t e2m1_bf16_bits(uint32_t code) {
  // magnitudes {0, .5, 1, 1.5, 2, 3, 4, 6} as bf16 bit patterns
  const uint32_t m = code & 7u;
  const uint32_t mag = (m == 0u) ? 0u : (m == 1u) ? 0x3F00u : 0x3F80u + ((m - 2u) << 6);
  return ((code & 8u) << 12) | mag;
}
// One packed word (8 codes) -> 4 registers in the nibble order (0,4),(1,5),(2,6),(3,7).
__device__ __forceinline__ void mx_word(uint32_t x, uint32_t c, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                        uint32_t& r3) {
  r0 = mx_pair(x << 6, x << 12, c);
  r1 = mx_pair(x << 2, x << 8, c);
  r2 = mx_pair(x >> 2, x << 4, c);
  r3 = mx_pair(x >> 6, x, c);
}

template <int BT, int MODE>
__global__ void __launch_bounds__((TcCfg<BT, mode_mats(MODE), mode_is_int4(MODE)>::kThreads), 1)
moe_tc_kernel(const __grid_constant__ CUtensorMap tm_packed, const __grid_constant__ CUtensorMap tm_scale,
               const __grid_constant__ CUtensorMap tm_tokens, const TcParams p) {
  using Cfg = TcCfg<BT, mode_mats(MODE), mode_is_int4(MODE)>;
  constexpr int kWStages = Cfg::kWStages;
  constexpr int kMatsC = mode_mats(MODE);
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                         ~uintptr_t(1023));
  unsigned char* s_packed = smem;                                         // kWStages x 16 KiB
  unsigned char* s_tokens = s_packed + kWStages * kPackedStageBytes;      // kBStages x 4 x [BT x 64] bf16
  unsigned char* s_scale = s_tokens + Cfg::kBStages * Cfg::kBStageBytes;  // kWStages x 2 KiB
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_scale + kWStages * kScaleStageBytes);
  uint64_t* w_full = bars;                       // [kWStages]
  uint64_t* w_empty = w_full + kWStages;         // [kWStages]
  uint64_t* b_full = w_empty + kWStages;         // [kBBars]
  uint64_t* b_empty = b_full + Cfg::kBBars;      // [kBBars]
  uint64_t* a_full = b_empty + Cfg::kBBars;      // [kABars]
  uint64_t* a_empty = a_full + Cfg::kABars;      // [kABars]
  uint64_t* d_full = a_empty + Cfg::kABars;      // [kDBuf]
  uint64_t* d_empty = d_full + Cfg::kDBuf;       // [kDBuf]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_empty + Cfg::kDBuf);
  int* abort_word = reinterpret_cast<int*>(tmem_slot + 1);
  uint32_t* lut = reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(bars) + Cfg::kBarBytes);   // [256][32] if kLut

  // broadcast so that the compiler knows the warp index is warp-uniform (tensor-memory addresses and
  // role branches then live in uniform registers)
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  Guard guard{abort_word, p.status};

  if (threadIdx.x == 0) {
    for (int i = 0; i < kWStages; ++i) { mbar_init(&w_full[i], 1); mbar_init(&w_empty[i], Cfg::kGroupWarps); }
    for (int i = 0; i < Cfg::kBBars; ++i) { mbar_init(&b_full[i], 1); mbar_init(&b_empty[i], kMatsC); }
    for (int i = 0; i < Cfg::kABars; ++i) { mbar_init(&a_full[i], Cfg::kGroupWarps / Cfg::kUnits); mbar_init(&a_empty[i], 1); }
    for (int i = 0; i < Cfg::kDBuf; ++i) { mbar_init(&d_full[i], Cfg::kIssuers); mbar_init(&d_empty[i], 4 * Cfg::kEpiWGs); }
    *abort_word = 0;
    mbar_fence_init();
  }
  // the token producer gets a warp of its own when the issuers leave one free (two threads of one warp
  // that both poll with back-off slow each other down); otherwise it shares the weight producer's
  constexpr int kCtrlWarps = Cfg::kCtrlWarps;
  constexpr int kTokWarp = kCtrlWarps - 1, kTokLane = 0;   // a warp of its own: two polling threads in one warp slow each other down
  if (Cfg::kLut) {   // byte -> (bf16 of the low code, bf16 of the high code), one copy per lane/bank
    for (int i = threadIdx.x; i < 256 * 32; i += Cfg::kThreads) {
      const uint32_t b = (uint32_t)i >> 5;
      lut[i] = e2m1_bf16_bits(b & 0xFu) | (e2m1_bf16_bits(b >> 4) << 16);
    }
  }
  if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
  if (warp == 0 && lane == 0) { prefetch_tensormap(&tm_packed); prefetch_tensormap(&tm_scale); }
  if (warp == kTokWarp && lane == kTokLane) prefetch_tensormap(&tm_tokens);
  // Block hand-over between the two GEMMs of an expert layer.  The second GEMM is launched as a
  // programmatic dependent of the first and does NOT wait for the first grid to complete: its CTAs
  // become resident as CTAs of the first exit (a CTA owns its SM), stream their weights at once and
  // wait per token block for the first GEMM's read-outs of that block (a counter per block, release
  // by the writer, acquire + async-proxy fence by the token producer before its TMA loads).  The
  // tail of the first GEMM, where most SMs have run out of tiles, is filled with tiles of the second.
  // Every CTA of the first GEMM is resident before any CTA of the second starts and never waits for
  // the second, so the wait cannot deadlock; it is bounded all the same.  The first GEMM lets its
  // dependents go only after its own wait for the kernels before it, so that what those wrote (the
  // routing) is visible to the second GEMM although it skips its wait; the counters are cleared
  // together with the status word by the memset that opens the fused call.
  const bool hand_over_first = mode_is_gate_up(MODE) && p.done_signal != nullptr;
  const bool hand_over_second = p.done_wait != nullptr;
  if (!hand_over_first) chain_trigger();   // the next kernel may be launched; it waits for this one's completion itself
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);   // (marks it warp-uniform)
  // everything above needed nothing from the kernels before this one (routing, gathered activations)
  if (!hand_over_second) chain_wait();
  if (hand_over_first) chain_trigger();

  // tile index t -> (token block, row tile); the row tile varies fastest so that CTAs that run
  // together share the token block and walk through one expert's weights
  const int n_tiles = p.N / (mode_is_pair(MODE) ? 2 * kTileRows : kTileRows);
  const int n_post = __ldcg(p.num_post);   // the routing was written by kernels this one may overlap: L2 loads, after the wait
  const bool routing_ok = n_post >= 0 && n_post <= p.max_blocks * BT;
  if (!routing_ok && threadIdx.x == 0) atomicCAS(p.status, 0, kErrBadRouting + (1 << 8));
  const int n_blocks = routing_ok ? n_post / BT : 0;
  const int total_tiles = n_blocks * n_tiles;   // the host checks that the worst case fits 31 bits
  const int k_stages = p.K / kStageK;   // 256-K stages per tile
  // "virtual" weight stages of a tile: two-matrix modes alternate the matrices stage by stage
  constexpr int kMats = mode_mats(MODE);
  const int v_stages = kMats * k_stages;
  // first weight row (in the [E * rows_per_expert] row space) of virtual stage vs of tile (b, nt)
  auto tile_row = [&](int b, int nt, int vs) -> int {
    int e = __ldcg(p.expert_ids + b);
    if ((unsigned)e >= (unsigned)p.num_experts) { atomicCAS(p.status, 0, kErrBadRouting + (2 << 8)); e = 0; }
    if (MODE == kModeInt4) return e * p.N + nt * kTileRows;
    if (MODE == kModeInt4Pair) return e * p.N + (2 * nt + (vs & 1)) * kTileRows;
    if (MODE == kModeMxDown) return e * p.rows_per_expert + (2 * nt + (vs & 1)) * kTileRows;
    return e * p.rows_per_expert + (vs & 1) * p.N + nt * kTileRows;  // gate rows, then up rows
  };

  if (warp == 0 && lane == 0) {
    // ---------------- weight producer ----------------
    {
      uint32_t st = 0, ph = 0;
      for (int t = (int)blockIdx.x; t < total_tiles && !guard.aborted(); t += (int)gridDim.x) {
        const int b = t / n_tiles, nt = t - b * n_tiles;
        for (int vs = 0; vs < v_stages; ++vs) {
          const int ks = vs / kMats;
          const int row0 = tile_row(b, nt, vs);
          if (!mbar_wait(&w_empty[st], ph ^ 1, guard, 1, kProdSleepNs)) break;
          if (mode_is_int4(MODE)) {
            mbar_expect_tx(&w_full[st], kPackedStageBytes + kScaleStageBytes);
            tma_load_2d(s_packed + st * kPackedStageBytes, &tm_packed, &w_full[st], ks * (kStageK / 2), row0);
            tma_load_2d(s_scale + st * kScaleStageBytes, &tm_scale, &w_full[st], ks * (kStageK / 32), row0);
          } else {  // e8m0 scales: 16 bytes per row = the scales of stages ks & ~1 and ks | 1
            mbar_expect_tx(&w_full[st], kPackedStageBytes + kScaleStageBytes);
            tma_load_2d(s_packed + st * kPackedStageBytes, &tm_packed, &w_full[st], ks * (kStageK / 2), row0);
            tma_load_2d(s_scale + st * kScaleStageBytes, &tm_scale, &w_full[st], (ks >> 1) * 16, row0);
          }
          if (++st == kWStages) { st = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == kTokWarp && lane == kTokLane) {
    // ---------------- token producer (diverged from lane 0; both make progress independently) ----------------
    {
      uint32_t st = 0, tb = 0;   // token stage slot and running number of the token stage
      int ready_b = -1;          // block hand-over: last block whose activations are known to be complete
      for (int t = (int)blockIdx.x; t < total_tiles && !guard.aborted(); t += (int)gridDim.x) {
        const int b = t / n_tiles;
        const int pos0 = b * BT;
        if (hand_over_second && b != ready_b) {   // block hand-over: the first GEMM's read-outs of block b
          uint64_t t0 = 0;
          bool ready = false;
          for (uint32_t i = 1; !ready; ++i) {
            int32_t seen;
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.done_wait + b) : "memory");
            if (seen >= p.done_target) { ready = true; break; }
            __nanosleep(200);
            if ((i & 15u) == 0u) {
              if (guard.aborted()) break;
              const uint64_t now = globaltimer_ns();
              if (t0 == 0) t0 = now;
              else if (now - t0 > kWaitBudgetNs) { guard.raise(kErrWaitTimeout + (9 << 8)); break; }
            }
          }
          if (!ready) break;
          asm volatile("fence.proxy.async;" ::: "memory");   // the TMA loads below read what generic stores wrote
          ready_b = b;
        }
        for (int ks = 0; ks < k_stages; ++ks) {
          // the slot's previous user was token stage tb - kBStages: wait for its readers' commits
          if (tb >= (uint32_t)Cfg::kBStages) {
            const uint32_t tp = tb - Cfg::kBStages;
            if (!mbar_wait(&b_empty[tp % Cfg::kBBars], (tp / Cfg::kBBars) & 1u, guard, 2, kProdSleepNs)) break;
          }
          const uint32_t bar = tb % Cfg::kBBars;
          mbar_expect_tx(&b_full[bar], Cfg::kBStageBytes);
#pragma unroll
          for (int j = 0; j < kSubs; ++j)
            tma_load_2d(s_tokens + st * Cfg::kBStageBytes + j * Cfg::kBSubBytes, &tm_tokens, &b_full[bar],
                        (ks * kSubs + j) * kSubK, pos0);
          if (++st == Cfg::kBStages) st = 0;
          ++tb;
        }
      }
    }
  } else if (warp >= 1 && warp < kCtrlWarps) {
    // ---------------- MMA issuers ----------------
    // Stage g (numbered across the tiles of this CTA) belongs to issuer g % kIssuers: it waits for
    // the A slot and the token stage, hands the weight stage back to the producer, issues the
    // sixteen M=128 N=BT K=16 MMAs into its own accumulator of the stage's matrix and commits.
    constexpr int kIssuers = Cfg::kIssuers;
    const uint32_t me = warp - 1;
    if ((kUniformIssuer || lane == 0) && me < (uint32_t)kIssuers) {
      const uint32_t leader = (lane == 0) ? 1u : 0u;
      // in the warp-uniform form every wait result is made uniform with a vote
      auto uni = [&](bool v) -> bool { return kUniformIssuer ? (__all_sync(0xffffffffu, v) != 0) : v; };
      constexpr uint32_t idesc = umma_idesc_bf16(kTileRows, BT);
      // This issuer's stages are g = me, me + kIssuers, ...; its ring positions advance with them
      // (no division in the loop: the issuing thread is on the critical path of every hand-off).
      constexpr uint32_t kDU = (uint32_t)(kIssuers * Cfg::kUnits);       // units per own-stage step
      constexpr uint32_t kDTB = (uint32_t)(kIssuers / kMats);            // token stages per own-stage step
      uint32_t aq0 = (me * Cfg::kUnits) % Cfg::kASlots;                  // A slot of the stage's first unit
      uint32_t ab0 = (me * Cfg::kUnits) % Cfg::kABars, acyc = 0;         // its barrier and the barrier ring's lap parity
      uint32_t bst = (me / kMats) % Cfg::kBStages;                       // token slot
      uint32_t bbar = (me / kMats) % Cfg::kBBars, bcyc = 0;              // token barrier and lap parity
      uint32_t it = 0, g0mod = 0;                                        // g0mod = (first stage of the tile) % kIssuers
      const uint32_t vsmod = (uint32_t)v_stages % kIssuers;
      for (int t = (int)blockIdx.x; t < total_tiles && uni(!guard.aborted()); t += (int)gridDim.x, ++it) {
        // accumulator set of this tile; its previous user must have been read out by every epilogue warp
        const uint32_t dbuf = it % Cfg::kDBuf, duse = it / Cfg::kDBuf;
        bool ok = uni(mbar_wait(&d_empty[dbuf], (duse & 1u) ^ 1u, guard, 8, 100));
        if (ok) tc_fence_after();
        uint32_t started = 0;   // bit m: this issuer has already written its accumulator of matrix m in this tile
        for (int vs = (int)(me >= g0mod ? me - g0mod : me + kIssuers - g0mod); vs < v_stages && ok; vs += kIssuers) {
          const int mat = vs % kMats;                       // which matrix this stage belongs to
          const int acc = (int)me;
          const uint32_t d_tmem = tmem_base + (uint32_t)(((int)dbuf * Cfg::kAccs + acc) * BT);
          const uint64_t b_desc = umma_desc_k_sw128(smem_u32(s_tokens + bst * Cfg::kBStageBytes));
          const bool fresh = ((started >> mat) & 1u) == 0;
          started |= 1u << mat;
#pragma unroll
          for (int h = 0; h < Cfg::kUnits; ++h) {
            ok = uni(mbar_wait(&a_full[ab0 + h], acyc, guard, 3, kIssSleepNs));
            if (!ok) break;
            if (h == 0) {
              ok = uni(mbar_wait(&b_full[bbar], bcyc, guard, 4));
              if (!ok) break;
            }
            tc_fence_after();
            const uint32_t a_tmem = tmem_base + Cfg::kACol0 + (aq0 + h) * Cfg::kUnitCols;
#pragma unroll
            for (int us = 0; us < Cfg::kUnitSubs; ++us) {
              const int sub = h * Cfg::kUnitSubs + us;
#pragma unroll
              for (int kk = 0; kk < kSubK / 16; ++kk)
                umma_ts_bf16_if(d_tmem, a_tmem + us * kSubCols + kk * 8,
                                b_desc + (uint64_t)((sub * Cfg::kBSubBytes) >> 4) + (uint64_t)(kk * 2), idesc,
                                (fresh && sub == 0 && kk == 0) ? 0u : 1u, leader);
            }
            tc_commit_if(&a_empty[ab0 + h], leader);
          }
          if (!ok) break;
          tc_commit_if(&b_empty[bbar], leader);   // kMats arrivals release the token stage
          // on to this issuer's next stage
          aq0 += kDU; if (aq0 >= (uint32_t)Cfg::kASlots) aq0 -= Cfg::kASlots;
          if (kDU >= (uint32_t)Cfg::kASlots && aq0 >= (uint32_t)Cfg::kASlots) aq0 -= Cfg::kASlots;
          ab0 += kDU; if (ab0 >= (uint32_t)Cfg::kABars) { ab0 -= Cfg::kABars; acyc ^= 1u; }
          // a two-matrix tile shares a token stage between the matrices: with kIssuers == kMats every
          // own stage is a new token stage; otherwise the step is kIssuers / kMats token stages
          bst += kDTB; if (bst >= (uint32_t)Cfg::kBStages) bst -= Cfg::kBStages;
          bbar += kDTB; if (bbar >= (uint32_t)Cfg::kBBars) { bbar -= Cfg::kBBars; bcyc ^= 1u; }
        }
        if (!ok) break;
        tc_commit_if(&d_full[dbuf], leader);
        g0mod += vsmod; if (g0mod >= (uint32_t)kIssuers) g0mod -= kIssuers;
      }
    }
  } else if (warp >= kCtrlWarps) {
    // ---------------- dequantisers + epilogue ----------------
    // Thread = weight row (the four warps of a warpgroup cover the four tensor-memory lane
    // quarters).  The sixteen warps form two groups of two warpgroups; stages (numbered g across
    // the tiles of the CTA) alternate between the groups, so that one group's barrier waits,
    // shared-memory loads and tensor-memory store drains overlap the other group's arithmetic.
    // Inside a group, warpgroup h converts the K slices 2h and 2h+1 (128 of the stage's 256 K) into
    // columns [64 h, 64 h + 64) of the stage's A slot, eight columns per tcgen05.st.
    const int wg = (warp - kCtrlWarps) >> 2;
    constexpr int kGroups = Cfg::kGroups, kChunks = Cfg::kChunks;
    const uint32_t grp = (uint32_t)wg / Cfg::kPartsPerStage;
    const int part = wg % Cfg::kPartsPerStage;   // which share of the stage's chunks this warpgroup converts
    const int quarter = warp & 3;              // tensor-memory lane quarter this warp may access
    const int row = quarter * 32 + lane;       // weight row inside the tile
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_packed_u32 = smem_u32(s_packed), s_scale_u32 = smem_u32(s_scale);
    const uint32_t lut_lane = smem_u32(lut) + (uint32_t)lane * 4u;   // this lane's column of the table
    // Epilogue of tile (b, nt) whose accumulators sit in set `dbuf` (use number `duse` of that
    // set).  It runs one weight stage into the NEXT tile (or after the last tile), so that the MMAs
    // it waits for have long finished and the pipeline never drains at a tile boundary.
    // Slot ids and routing weights of 16 token positions of block b: lane j holds position c0 + j
    // (padding positions carry the value numel).  Sixteen lanes load them side by side, and the first
    // group's are requested when the tile joins the read-out queue, two stages before they are used:
    // a read-out then never waits for global memory.
    auto load_cols = [&](int b, int c0, int32_t& slot, float& w) {
      slot = (lane < 16 && c0 < BT) ? __ldcg(p.sorted_ids + (int64_t)b * BT + c0 + lane) : -1;   // written by a kernel this one overlaps: no .nc load
      const bool live = slot >= 0 && slot < p.numel;
      w = (!mode_is_gate_up(MODE) && p.mul_w && live) ? __ldg(p.topk_w + slot) : 1.f;
    };
    auto run_epilogue = [&](int b, int nt, uint32_t dbuf, uint32_t duse, uint32_t tile_g0, int cg, int32_t my_slot,
                            float my_w) -> bool {
      const uint32_t d_base = tmem_base + lane_base + dbuf * (uint32_t)(Cfg::kAccs * BT);
      // which accumulators the tile's stages went to: stage vs -> issuer (g0 + vs) % kIssuers
      uint32_t valid = 0;
      if (Cfg::kLocked) {
        valid = (1u << kMats) - 1u;
      } else {
        for (int vs = 0; vs < v_stages && vs < Cfg::kIssuers; ++vs)
          valid |= 1u << ((tile_g0 + (uint32_t)vs) % Cfg::kIssuers);
      }
      if (!mbar_wait(&d_full[dbuf], duse & 1u, guard, 7)) return false;
      tc_fence_after();
      const int64_t n_glob = (int64_t)nt * (mode_is_pair(MODE) ? 2 * kTileRows : kTileRows) + row;
      float bias0 = 0.f, bias1 = 0.f;
      if (!mode_is_int4(MODE) && p.bias != nullptr) {
        int e_bias = __ldcg(p.expert_ids + b);
        if ((unsigned)e_bias >= (unsigned)p.num_experts) e_bias = 0;   // recorded by the weight producer
        const int64_t e_row = (int64_t)e_bias * p.rows_per_expert;
        bias0 = __bfloat162float(p.bias[e_row + n_glob]);
        if (MODE == kModeMxGateUp) bias1 = __bfloat162float(p.bias[e_row + p.N + n_glob]);
        if (MODE == kModeMxDown) bias1 = __bfloat162float(p.bias[e_row + n_glob + kTileRows]);
      }
      // this warpgroup's 16-column groups: cg, cg + kWGs, ...
#pragma unroll 1
      for (int c0 = cg * 16; c0 < BT; c0 += 16 * Cfg::kWGs) {
        // Everything below is skipped for padding positions, and a block of padding only costs the load.
        const int32_t cur_slot = my_slot;
        const float cur_w = my_w;
        if (c0 + 16 * Cfg::kWGs < BT) load_cols(b, c0 + 16 * Cfg::kWGs, my_slot, my_w);   // the next group's, in flight meanwhile
        const uint32_t live = __ballot_sync(0xffffffffu, cur_slot >= 0 && cur_slot < p.numel) & 0xFFFFu;
        if (live == 0u) continue;
        // acc = matrix 0 (INT4 / down: the only one; gate_up: gate; pair: first row tile), more = matrix 1,
        // each the sum of the accumulators that were written in this tile
        uint32_t acc[16], more[16];
#pragma unroll
        for (int q = 0; q < 16; ++q) { acc[q] = 0u; more[q] = 0u; }
#pragma unroll
        for (int a = 0; a < Cfg::kAccs; ++a) {
          if ((valid >> a) & 1u) {
            uint32_t part[16];
            tmem_ld_32x16(d_base + a * BT + c0, part);
            tmem_wait_ld();
            if (kMats == 2 && (a & 1)) {
#pragma unroll
              for (int q = 0; q < 16; ++q) more[q] = __float_as_uint(__uint_as_float(more[q]) + __uint_as_float(part[q]));
            } else {
#pragma unroll
              for (int q = 0; q < 16; ++q) acc[q] = __float_as_uint(__uint_as_float(acc[q]) + __uint_as_float(part[q]));
            }
          }
        }
        if (mode_is_gate_up(MODE)) {
          // acc = gate, more = up.  Rounding points of the reference
          // (src/xkernels/ops/moe/mxfp4_reference.py:92-100): gate_up to bf16, (+ bf16 bias, rounded),
          // fp32 clamp and silu(gate) * up, then bf16.  The activation goes out in the K order the
          // down GEMM's dequantiser produces: element j of a group of 8 at ((j & 3) << 1) | (j >> 2).
          const int64_t col = Cfg::kLut ? n_glob   // the table path of the next GEMM reads natural K order
                                        : ((n_glob & ~int64_t(7)) | (((n_glob & 3) << 1) | ((n_glob >> 2) & 1)));
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (!((live >> j) & 1u)) continue;          // warp-uniform
            constexpr float kUnscale = (MODE == kModeInt4GateUp) ? kInt4Unscale : (Cfg::kLut ? 1.f : kMxUnscale);
            float g = round_to_bf16(__uint_as_float(acc[j]) * kUnscale);   // exact: a power of two
            float u = round_to_bf16(__uint_as_float(more[j]) * kUnscale);
            if (p.bias != nullptr) { g = round_to_bf16(g + bias0); u = round_to_bf16(u + bias1); }
            if (p.limit > 0.f) { g = fminf(g, p.limit); u = fminf(fmaxf(u, -p.limit), p.limit); }
            const float silu = g / (1.f + expf(-g));
            p.act[((int64_t)b * BT + c0 + j) * p.N + col] = __float2bfloat16_rn(silu * u);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (!((live >> j) & 1u)) continue;          // warp-uniform
            const int32_t slot = __shfl_sync(0xffffffffu, cur_slot, j);
            const float w = __shfl_sync(0xffffffffu, cur_w, j);
            float v = __uint_as_float(acc[j]);
            if (mode_is_int4(MODE) && kInt4NoSubtract) v *= kInt4Unscale;   // exact: a power of two
            if (MODE == kModeMxDown) {  // reference rounds `down` to bf16, adds the bf16 bias, then x w
              v = round_to_bf16(Cfg::kLut ? v : v * kMxUnscale);
              if (p.bias != nullptr) v = round_to_bf16(v + bias0);
              if (p.mul_w) v = v * w;
            } else {
              if (p.mul_w) v = w * v;
              if (p.round_rows) v = round_to_bf16(v);
            }
            p.scratch[(int64_t)slot * p.N + n_glob] = v;
            if (mode_is_pair(MODE)) {  // the second weight tile: rows 128 further down
              float v2 = __uint_as_float(more[j]);
              if (MODE == kModeInt4Pair) {
                if (kInt4NoSubtract) v2 *= kInt4Unscale;
                if (p.mul_w) v2 = w * v2;
                if (p.round_rows) v2 = round_to_bf16(v2);
              } else {
                v2 = round_to_bf16(Cfg::kLut ? v2 : v2 * kMxUnscale);
                if (p.bias != nullptr) v2 = round_to_bf16(v2 + bias1);
                if (p.mul_w) v2 = v2 * w;
              }
              p.scratch[(int64_t)slot * p.N + n_glob + kTileRows] = v2;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      mbar_arrive_if(&d_empty[dbuf], (lane == 0) ? 1u : 0u);
      if (mode_is_gate_up(MODE) && p.done_signal != nullptr) {
        // this warp's part of block b is written (the __syncwarp above orders the other lanes' stores
        // before lane 0's release): one count per warp and tile, 4 * kEpiWGs per tile
        if (lane == 0) {
          __threadfence();
          asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(p.done_signal + b) : "memory");
        }
      }
      return true;
    };
    // Read-outs that are still due, oldest first (at most two wait at any time: a tile is read out
    // before its accumulator set is needed again, see below).
    struct Pending { int b, nt; uint32_t it, g0; int wait, cg; int32_t slot; float w; };
    Pending pq0{0, 0, 0, 0, 0, 0, -1, 1.f}, pq1{0, 0, 0, 0, 0, 0, -1, 1.f};
    int n_pend = 0;
    auto run_oldest = [&]() -> bool {
      const Pending e = pq0;
      pq0 = pq1;
      --n_pend;
      return run_epilogue(e.b, e.nt, e.it % Cfg::kDBuf, e.it / Cfg::kDBuf, e.g0, e.cg, e.slot, e.w);
    };
    uint32_t it = 0, g0 = 0;      // g0 = number of the tile's first stage
    // This group's stages are g = grp, grp + kGroups, ... whatever the tile boundaries, so its ring
    // positions advance by a fixed step per converted stage (no division in the loop).
    constexpr uint32_t kDU = (uint32_t)(kGroups * Cfg::kUnits);           // units per own-stage step
    const uint32_t u_first = grp * Cfg::kUnits + (Cfg::kUnits > 1 ? (uint32_t)part : 0u);
    uint32_t wst = grp % kWStages, wph = 0;                               // weight slot and its lap parity
    uint32_t aq = u_first % Cfg::kASlots;                                 // A slot of this warpgroup's unit
    uint32_t abar = u_first % Cfg::kABars, acyc = 0;                      // its barrier and the barrier ring's lap parity
    uint32_t n_own = 0;                                                   // own stages converted so far
    const uint32_t lead = (lane == 0) ? 1u : 0u;
    uint32_t g0mod = 0;                                                   // g0 % kGroups
    const uint32_t vsmod = (uint32_t)v_stages % kGroups;
    // (b, nt) of the tile advance with it: no division in the loop
    const int step_b = (int)gridDim.x / n_tiles, step_nt = (int)gridDim.x - step_b * n_tiles;
    int b = (int)blockIdx.x / n_tiles, nt = (int)blockIdx.x - b * n_tiles;
    for (int t = (int)blockIdx.x; t < total_tiles; t += (int)gridDim.x, ++it, g0 += (uint32_t)v_stages,
             b += step_b, nt += step_nt, b += (nt >= n_tiles ? 1 : 0), nt -= (nt >= n_tiles ? n_tiles : 0)) {
      bool ok = true;
      for (int vs = (int)(grp >= g0mod ? grp - g0mod : grp + kGroups - g0mod); vs < v_stages && ok; vs += kGroups) {
        if (!mbar_wait(&w_full[wst], wph, guard, 5)) { ok = false; break; }
        const uint32_t pk = s_packed_u32 + wst * kPackedStageBytes + row * 128;
        uint2 sw = make_uint2(0, 0);  // INT4: the kChunks bf16 group scales of this share; MXFP4: .x = its e8m0 bytes
        if (mode_is_int4(MODE)) {
          if (kChunks == 4) sw = lds64(s_scale_u32 + wst * kScaleStageBytes + row * 16 + part * 8);
          else sw.x = lds32(s_scale_u32 + wst * kScaleStageBytes + row * 16 + part * 4);
        } else {  // the kChunks e8m0 bytes of this share: this stage's half of the row's sixteen
          const uint32_t sa = s_scale_u32 + wst * kScaleStageBytes + row * 16 + (((vs / kMats) & 1) << 3) + part * kChunks;
          if (kChunks == 4) sw.x = lds32(sa);
          else sw.x = lds16(sa);
        }
        // 16-byte chunk = 32 weights = one scale group; this share is chunks kChunks * part ...
        uint4 w4[kChunks];
#pragma unroll
        for (int c = 0; c < kChunks; ++c) w4[c] = lds128(pk + (((part * kChunks + c) ^ (row & 7)) << 4));
        // This warp's share of the stage is in registers (the shared-memory unit executes a warp's
        // loads and the arrive in order, and the arrive has release semantics): one arrival per warp
        // of the group hands the stage back to the producer.
        __syncwarp();
        mbar_arrive_if(&w_empty[wst], lead);
        // the slot's previous user was the unit kASlots before this one: wait until its MMAs have completed
        if (n_own * kDU + u_first >= (uint32_t)Cfg::kASlots) {
          const bool same_lap = abar >= (uint32_t)Cfg::kASlots;
          const uint32_t eb = same_lap ? abar - Cfg::kASlots : abar + Cfg::kABars - Cfg::kASlots;
          if (!mbar_wait(&a_empty[eb], same_lap ? acyc : (acyc ^ 1u), guard, 6)) { ok = false; break; }
        }
        tc_fence_after();
        const uint32_t dst = tmem_base + lane_base + Cfg::kACol0 + aq * Cfg::kUnitCols +
                             (Cfg::kUnits > 1 ? 0 : part * (kChunks * 16));
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
          const uint32_t words[4] = {w4[c].x, w4[c].y, w4[c].z, w4[c].w};
          if (mode_is_int4(MODE)) {
            const uint32_t s01 = (c < 2) ? sw.x : sw.y;
            const uint32_t s2 = (c & 1) ? __byte_perm(s01, s01, 0x3232) : __byte_perm(s01, s01, 0x1010);
            if (kInt4NoSubtract) {
              const uint32_t m_lo = bf2_mul(s2, kMulLo), m_hi = bf2_mul(s2, kMulHi), add = bf2_mul(s2, kMulAdd);
#pragma unroll
              for (int wp = 0; wp < 2; ++wp) {  // two words = 16 weights = 8 columns
                const uint32_t x0 = words[2 * wp], x1 = words[2 * wp + 1];
                const uint32_t y0 = x0 >> 8, y1 = x1 >> 8;
                tmem_st_32x8(dst + c * 16 + wp * 8,
                             bf2_fma(x0 & 0x000F000Fu, m_lo, add), bf2_fma(x0 & 0x00F000F0u, m_hi, add),
                             bf2_fma(y0 & 0x000F000Fu, m_lo, add), bf2_fma(y0 & 0x00F000F0u, m_hi, add),
                             bf2_fma(x1 & 0x000F000Fu, m_lo, add), bf2_fma(x1 & 0x00F000F0u, m_hi, add),
                             bf2_fma(y1 & 0x000F000Fu, m_lo, add), bf2_fma(y1 & 0x00F000F0u, m_hi, add));
              }
            } else {
#pragma unroll
              for (int wp = 0; wp < 2; ++wp) {  // two words = 16 weights = 8 columns
                const uint32_t x0 = words[2 * wp], x1 = words[2 * wp + 1];
                tmem_st_32x8(dst + c * 16 + wp * 8,
                             dequant_pair(nib_pair(x0), s2), dequant_pair(nib_pair(x0 >> 4), s2),
                             dequant_pair(nib_pair(x0 >> 8), s2), dequant_pair(nib_pair(x0 >> 12), s2),
                             dequant_pair(nib_pair(x1), s2), dequant_pair(nib_pair(x1 >> 4), s2),
                             dequant_pair(nib_pair(x1 >> 8), s2), dequant_pair(nib_pair(x1 >> 12), s2));
              }
            }
          } else {
            const uint32_t sb = (sw.x >> (8 * c)) & 0xFFu;
            if (Cfg::kLut) {
              // 2^(sb - 127) as a bf16 pair: exponent field sb; byte 0 is the subnormal 2^-127, 0xFF decodes to 0
              uint32_t f = sb << 7;
              if (sb == 0u) f = 0x40u;
              if (sb == 0xFFu) f = 0u;
              const uint32_t cf = f * 0x00010001u;
#pragma unroll
              for (int wp = 0; wp < 2; ++wp) {
                uint32_t r[8];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                  const uint32_t x = words[2 * wp + h];
                  // entry of byte k of x for this lane: lut_lane + byte * 128 (bytes): one byte
                  // permute and one multiply-add each
                  r[4 * h + 0] = bf2_mul(lds32(__byte_perm(x, 0u, 0x4440u) * 128u + lut_lane), cf);
                  r[4 * h + 1] = bf2_mul(lds32(__byte_perm(x, 0u, 0x4441u) * 128u + lut_lane), cf);
                  r[4 * h + 2] = bf2_mul(lds32(__byte_perm(x, 0u, 0x4442u) * 128u + lut_lane), cf);
                  r[4 * h + 3] = bf2_mul(lds32(__byte_perm(x, 0u, 0x4443u) * 128u + lut_lane), cf);
                }
                tmem_st_32x8(dst + c * 16 + wp * 8, r[0], r[1], r[2], r[3], r[4], r[5], r[6], r[7]);
              }
              continue;
            }
            if (sb > kMxMaxScale && sb != 0xFFu) atomicCAS(p.status, 0, kErrMxScaleRange);   // never taken for sane weights
            const uint32_t cf = mx_scale_factor(sb);
#pragma unroll
            for (int wp = 0; wp < 2; ++wp) {
              uint32_t r[8];
              mx_word(words[2 * wp], cf, r[0], r[1], r[2], r[3]);
              mx_word(words[2 * wp + 1], cf, r[4], r[5], r[6], r[7]);
              tmem_st_32x8(dst + c * 16 + wp * 8, r[0], r[1], r[2], r[3], r[4], r[5], r[6], r[7]);
            }
          }
        }
        tmem_wait_st();          // warp-wide: every lane's stores have landed
        tc_fence_before();
        mbar_arrive_if(&a_full[abar], lead);
        // on to this group's next stage
        ++n_own;
        wst += kGroups; if (wst >= (uint32_t)kWStages) { wst -= kWStages; wph ^= 1u; }
        aq += kDU; if (aq >= (uint32_t)Cfg::kASlots) aq -= Cfg::kASlots;
        abar += kDU; if (abar >= (uint32_t)Cfg::kABars) { abar -= Cfg::kABars; acyc ^= 1u; }
        // read-outs whose delay has run out
        --pq0.wait; --pq1.wait;
        while (n_pend > 0 && pq0.wait <= 0 && ok) ok = run_oldest();
      }
      if (!ok) break;
      // Before this tile joins the queue: a tile must have been read out before the MMAs of the tile
      // kDBuf further on, which re-use its accumulator set, can start.  Reading it out no later than
      // here (before any stage of tile it + 1 is converted) keeps every converted stage consumable,
      // so the A slots can never fill up with stages that wait for a read-out.
      while (n_pend > 0 && (pq0.it + (uint32_t)Cfg::kDBuf <= it + 1u || n_pend == 2) && ok) ok = run_oldest();
      if (!ok) break;
      // is this warpgroup on read-out duty for this tile, and for which column group?
      const int cg = (Cfg::kEpiWGs == Cfg::kWGs) ? wg
                                                 : (int)(((uint32_t)wg + (uint32_t)Cfg::kWGs - (it * (uint32_t)Cfg::kColGroups) % (uint32_t)Cfg::kWGs) % (uint32_t)Cfg::kWGs);
      if (cg < Cfg::kColGroups || Cfg::kEpiWGs == Cfg::kWGs) {
        Pending e{b, nt, it, g0, Cfg::kDBuf >= 2 ? kEpiDelay : 1, cg, -1, 1.f};   // one set: the next tile's MMAs wait for it
        load_cols(b, cg * 16, e.slot, e.w);
        if (n_pend == 0) pq0 = e; else pq1 = e;
        ++n_pend;
      }
      g0mod += vsmod; if (g0mod >= (uint32_t)kGroups) g0mod -= kGroups;
    }
    while (n_pend > 0 && !guard.aborted()) {
      if (!run_oldest()) break;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------
// Activation gather: Ag[p, :] = A[sorted_ids[p] / top_k, :] with the nibble-order
// permutation (0,4,1,5,2,6,3,7) applied inside every group of 8 K elements.
// Padding positions are left untouched: their accumulator columns are never read.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gather_permute_kernel(const __nv_bfloat16* __restrict__ A, const int32_t* sorted_ids,
                      const int32_t* num_post, __nv_bfloat16* __restrict__ Ag, int64_t numel,
                      int K, int top_k, int permute, int64_t max_pad, int* __restrict__ status) {
  // The routing comes from the align kernel before this one, which may still be running when this
  // kernel starts.  It is read with L2 loads after the wait and through pointers that are NOT
  // `const __restrict__`: loads the compiler may treat as invariant (ld.global.nc) were seen to
  // deliver the value from before the align kernel's write (hoisted above the wait, or served from
  // the non-coherent cache).
  chain_wait();
  chain_trigger();
  int total = __ldcg(num_post);
  if (total < 0 || total > max_pad) {   // never with a routing the align stage wrote: recorded, nothing gathered
    if (threadIdx.x == 0 && blockIdx.x == 0) atomicCAS(status, 0, kErrBadRouting + (3 << 8));
    total = 0;
  }
  for (int64_t pos = blockIdx.x; pos < total; pos += gridDim.x) {
    const int32_t slot = __ldcg(sorted_ids + pos);
    if (slot < 0 || slot >= numel) continue;
    const uint4* src = reinterpret_cast<const uint4*>(A + (int64_t)(slot / top_k) * K);
    uint4* dst = reinterpret_cast<uint4*>(Ag + pos * K);
    for (int i = threadIdx.x; i < K / 8; i += blockDim.x) {
      const uint4 v = __ldg(src + i);  // elements e0..e7 as (e1:e0, e3:e2, e5:e4, e7:e6)
      if (!permute) { dst[i] = v; continue; }   // consumers that convert in natural K order
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
// Encoded maps are kept per (base, shape, box, type, swizzle): a serving loop calls with the same
// weights and workspace addresses every step, and an encode costs about as much host time as a launch.
// A map holds no device state, so a stale entry (memory freed and reused with another layout) is
// harmless: the key is everything the encoding depends on.
struct MapKey {
  const void* base; uint64_t rows, cols; uint32_t box_rows, box_cols; int dt, elem_bytes, swz;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows && box_cols == o.box_cols &&
           dt == o.dt && elem_bytes == o.elem_bytes && swz == o.swz;
  }
};
constexpr int kMapCacheSize = 64;
struct MapCache {
  std::mutex mu;
  MapKey keys[kMapCacheSize];
  CUtensorMap maps[kMapCacheSize];
  int used = 0, next = 0;
};
MapCache g_map_cache;

int make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t rows,
                uint64_t cols, uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swz, const char* what) {
  const MapKey key{base, rows, cols, box_rows, box_cols, (int)dt, elem_bytes, (int)swz};
  {
    std::lock_guard<std::mutex> lock(g_map_cache.mu);
    for (int i = 0; i < g_map_cache.used; ++i)
      if (g_map_cache.keys[i] == key) { *map = g_map_cache.maps[i]; return XKB_OK; }
  }
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
  {
    std::lock_guard<std::mutex> lock(g_map_cache.mu);
    const int slot = g_map_cache.used < kMapCacheSize ? g_map_cache.used++ : (g_map_cache.next++ % kMapCacheSize);
    g_map_cache.keys[slot] = key;
    g_map_cache.maps[slot] = *map;
  }
  return XKB_OK;
}

template <int BT, int MODE>
int launch_bt(const CUtensorMap& tmp, const CUtensorMap& tms, const CUtensorMap& tmt, const TcParams& prm,
              int64_t max_tiles, cudaStream_t stream) {
  using Cfg = TcCfg<BT, mode_mats(MODE), mode_is_int4(MODE)>;
  int dev = 0;
  XKB_CHECK_CUDA(cudaGetDevice(&dev));
  // once per (kernel instance, device): the shared-memory opt-in and the SM count
  static std::atomic<uint64_t> smem_set{0};
  static std::atomic<int> sm_count[64];
  const uint64_t bit = dev < 64 ? (1ull << dev) : 0ull;
  if (bit == 0 || (smem_set.load(std::memory_order_acquire) & bit) == 0) {
    XKB_CHECK_CUDA(cudaFuncSetAttribute(moe_tc_kernel<BT, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)Cfg::kSmemBytes));
    int n = 148;
    XKB_CHECK_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    if (bit != 0) {
      sm_count[dev].store(n, std::memory_order_relaxed);
      smem_set.fetch_or(bit, std::memory_order_release);
    }
  }
  int sms = 148;
  if (bit != 0) sms = sm_count[dev].load(std::memory_order_relaxed);
  else XKB_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  // one persistent CTA per SM (it owns all 512 tensor-memory columns), minus the SMs the caller
  // asked to keep free for kernels that should run beside this one (xkb_set_sm_margin)
  XKB_REQUIRE(max_tiles < (1ll << 31), "moe_tc_kernel: %lld tiles do not fit the kernel's 31-bit tile index", (long long)max_tiles);
  int64_t grid = (int64_t)sms - g_sm_margin.load(std::memory_order_relaxed);
  if (grid < 8) grid = 8;
  if (grid > max_tiles) grid = max_tiles;
  if (grid < 1) grid = 1;
  {
    GemmTimerScope timed(stream);
    XKB_CHECK_CUDA(launch_chained(moe_tc_kernel<BT, MODE>, dim3((unsigned)grid), dim3(Cfg::kThreads), Cfg::kSmemBytes,
                                  stream, tmp, tms, tmt, prm));
  }
  XKB_CHECK_LAUNCH("moe_tc_kernel");
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
  return 128;  // wide: 128 tokens x two 128-row weight tiles per CTA (one tile if N % 256 != 0)
}

// read-out warps that count per tile of the first GEMM: four per warpgroup on duty
static int hand_over_per_tile(int block) { return 4 * (block / 16 < 4 ? block / 16 : 4); }

int64_t int4_tc_workspace_bytes(int64_t numel, int64_t N, int64_t K, int E) {
  (void)N;
  // gathered activations for the largest token tile
  return align_up((numel + (int64_t)(E + 1) * 255) * K * 2, 256);
}

// one INT4 GEMM (tokens through `tm_tokens`) at the token tile the routing was aligned for
static int launch_int4_by_block(const CUtensorMap& tm_packed, const CUtensorMap& tm_scale, const CUtensorMap& tm_tokens,
                                const TcParams& prm, const Routing& r, int64_t N, cudaStream_t stream) {
  const int64_t max_tiles = r.max_blocks * (N / kTileRows);
  switch (r.block) {
    case 16: return launch_bt<16, kModeInt4>(tm_packed, tm_scale, tm_tokens, prm, max_tiles, stream);
    case 32: return launch_bt<32, kModeInt4>(tm_packed, tm_scale, tm_tokens, prm, max_tiles, stream);
    case 64: return launch_bt<64, kModeInt4>(tm_packed, tm_scale, tm_tokens, prm, max_tiles, stream);
    case 128:
      if (N % (2 * kTileRows) == 0)
        return launch_bt<128, kModeInt4Pair>(tm_packed, tm_scale, tm_tokens, prm, max_tiles / 2, stream);
      return launch_bt<128, kModeInt4>(tm_packed, tm_scale, tm_tokens, prm, max_tiles, stream);
    default: return fail(XKB_ERR_ARG, "int4 tcgen05 path: unsupported token tile %d", r.block);
  }
}

int launch_int4_tc(const void* A, const int32_t* packed, const void* scale, const Routing& r,
                   const float* topk_w, float* scratch, int64_t N, int64_t K, int E, int top_k, int mul_w,
                   void* tc_ws, int* status, cudaStream_t stream) {
  Carver carve(tc_ws);
  __nv_bfloat16* Ag = carve.take<__nv_bfloat16>(r.max_pad * K);

  int64_t gblocks = r.max_pad < 148 * 16 ? r.max_pad : 148 * 16;
  if (gblocks < 1) gblocks = 1;
  XKB_CHECK_CUDA(launch_chained(gather_permute_kernel, dim3((unsigned)gblocks), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(A),
                                                               r.sorted_ids, r.num_post, Ag, r.numel, (int)K,
                                                               top_k, 1, r.max_pad, status));
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
  prm.max_blocks = (int)r.max_blocks;
  prm.num_experts = E;
  prm.N = (int)N;
  prm.K = (int)K;
  prm.mul_w = mul_w;
  prm.round_rows = 0;
  prm.bias = nullptr;
  prm.act = nullptr;
  prm.rows_per_expert = (int)N;
  prm.limit = 0.f;
  prm.done_signal = nullptr;
  prm.done_wait = nullptr;
  prm.done_target = 0;
  return launch_int4_by_block(tm_packed, tm_scale, tm_tokens, prm, r, N, stream);
}

// ---------------------------------------------------------------------------
// INT4 two-GEMM expert layer: gate_up GEMM with fused SwiGLU, then the down GEMM whose weighted
// slot rows are rounded to bf16 (what the composition of the reference's ops holds between its
// second fused_moe_int4_w4a16 call and moe_sum_reduce).
// ---------------------------------------------------------------------------
bool int4_ffn_tc_supported(int a_dtype, int64_t M, int64_t hidden, int64_t inter, int E, int top_k, int group) {
  return a_dtype == XKB_BF16 && group == 32 && M > 0 && E > 0 && top_k > 0 && hidden > 0 && inter > 0 &&
         hidden % kStageK == 0 && inter % kStageK == 0 &&   // both are contraction lengths and tile-row counts
         (int64_t)E * 2 * inter < (1ll << 31) && (int64_t)E * hidden < (1ll << 31);
}

int launch_int4_ffn_tc(const void* A, const int32_t* w13, const void* s13, const int32_t* w2, const void* s2,
                       const Routing& r, const float* topk_w, __nv_bfloat16* act, float* scratch, int64_t hidden,
                       int64_t inter, int E, int top_k, float limit, void* tc_ws, int* status, cudaStream_t stream) {
  Carver carve(tc_ws);
  int32_t* done = r.block_counters != nullptr ? r.block_counters + r.counters_each : nullptr;   // block hand-over counters
  __nv_bfloat16* Ag = carve.take<__nv_bfloat16>(r.max_pad * hidden);
  int64_t gblocks = r.max_pad < 148 * 16 ? r.max_pad : 148 * 16;
  if (gblocks < 1) gblocks = 1;
  XKB_CHECK_CUDA(launch_chained(gather_permute_kernel, dim3((unsigned)gblocks), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(A), r.sorted_ids,
                                                               r.num_post, Ag, r.numel, (int)hidden, top_k, 1, r.max_pad, status));
  XKB_CHECK_LAUNCH("gather_permute_kernel");
  CUtensorMap tm_w13, tm_s13, tm_w2, tm_s2, tm_tok0, tm_tok1;
  int rc = make_map_2d(&tm_w13, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w13, (uint64_t)E * 2 * inter, (uint64_t)hidden / 2,
                       kTileRows, kStageK / 2, CU_TENSOR_MAP_SWIZZLE_128B, "w13 packed weights");
  if (rc != XKB_OK) return rc;
  rc = make_map_2d(&tm_s13, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, s13, (uint64_t)E * 2 * inter, (uint64_t)hidden / 32,
                   kTileRows, kStageK / 32, CU_TENSOR_MAP_SWIZZLE_NONE, "w13 group scales");
  if (rc != XKB_OK) return rc;
  rc = make_map_2d(&tm_w2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w2, (uint64_t)E * hidden, (uint64_t)inter / 2, kTileRows,
                   kStageK / 2, CU_TENSOR_MAP_SWIZZLE_128B, "w2 packed weights");
  if (rc != XKB_OK) return rc;
  rc = make_map_2d(&tm_s2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, s2, (uint64_t)E * hidden, (uint64_t)inter / 32,
                   kTileRows, kStageK / 32, CU_TENSOR_MAP_SWIZZLE_NONE, "w2 group scales");
  if (rc != XKB_OK) return rc;
  rc = make_map_2d(&tm_tok0, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Ag, (uint64_t)r.max_pad, (uint64_t)hidden,
                   (uint32_t)r.block, kSubK, CU_TENSOR_MAP_SWIZZLE_128B, "gathered activations");
  if (rc != XKB_OK) return rc;
  rc = make_map_2d(&tm_tok1, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, act, (uint64_t)r.max_pad, (uint64_t)inter,
                   (uint32_t)r.block, kSubK, CU_TENSOR_MAP_SWIZZLE_128B, "SwiGLU activations");
  if (rc != XKB_OK) return rc;

  TcParams prm;
  prm.sorted_ids = r.sorted_ids;
  prm.expert_ids = r.expert_ids;
  prm.num_post = r.num_post;
  prm.topk_w = topk_w;
  prm.status = status;
  prm.numel = r.numel;
  prm.max_blocks = (int)r.max_blocks;
  prm.num_experts = E;
  prm.bias = nullptr;
  prm.limit = limit;
  // gate_up + SwiGLU -> act
  prm.scratch = nullptr;
  prm.act = act;
  prm.N = (int)inter;
  prm.K = (int)hidden;
  prm.rows_per_expert = (int)(2 * inter);
  prm.mul_w = 0;
  prm.round_rows = 0;
  prm.done_signal = done;
  prm.done_wait = nullptr;
  prm.done_target = (int)(inter / kTileRows) * hand_over_per_tile(r.block);
  GemmTimerScope timed(stream);   // both GEMMs in one scope: they overlap
  const int64_t tiles0 = r.max_blocks * (inter / kTileRows);
  switch (r.block) {
    case 16: rc = launch_bt<16, kModeInt4GateUp>(tm_w13, tm_s13, tm_tok0, prm, tiles0, stream); break;
    case 32: rc = launch_bt<32, kModeInt4GateUp>(tm_w13, tm_s13, tm_tok0, prm, tiles0, stream); break;
    case 64: rc = launch_bt<64, kModeInt4GateUp>(tm_w13, tm_s13, tm_tok0, prm, tiles0, stream); break;
    case 128: rc = launch_bt<128, kModeInt4GateUp>(tm_w13, tm_s13, tm_tok0, prm, tiles0, stream); break;
    default: return fail(XKB_ERR_ARG, "int4 tcgen05 path: unsupported token tile %d", r.block);
  }
  if (rc != XKB_OK) return rc;
  // down: weighted slot rows, rounded to bf16
  prm.scratch = scratch;
  prm.act = nullptr;
  prm.N = (int)hidden;
  prm.K = (int)inter;
  prm.rows_per_expert = (int)hidden;
  prm.mul_w = 1;
  prm.round_rows = 1;
  prm.limit = 0.f;
  prm.done_signal = nullptr;
  prm.done_wait = done;
  return launch_int4_by_block(tm_w2, tm_s2, tm_tok1, prm, r, hidden, stream);
}

// ---------------------------------------------------------------------------
// MXFP4: gate_up GEMM with fused SwiGLU, then down GEMM, both on the same pipeline
// ---------------------------------------------------------------------------
bool mxfp4_tc_supported(int a_dtype, int64_t M, int64_t hidden, int64_t ispp, int E, int top_k) {
  return a_dtype == XKB_BF16 && M > 0 && E > 0 && top_k > 0 && hidden > 0 && ispp > 0 &&
         hidden % (2 * kStageK) == 0 && ispp % (2 * kStageK) == 0 &&   // contraction lengths and tile-row counts; a row's
                                                                        // e8m0 scales must be whole 16-byte TMA rows
         (int64_t)E * 2 * ispp < (1ll << 31) && (int64_t)E * hidden < (1ll << 31);
}

int mxfp4_tc_block(int64_t numel, int E) {
  // decode-sized batches: token tiles of 16; prefill-sized ones: 128 (gate and up then get one
  // MMA issuer each, like the row-tile pairs of the INT4 wide mode)
  const double avg = (double)numel / (E > 0 ? E : 1);
  return avg <= 48 ? 16 : 128;
}

int64_t mxfp4_tc_workspace_bytes(int64_t numel, int64_t hidden, int64_t ispp, int E) {
  (void)ispp;
  return align_up((numel + (int64_t)(E + 1) * 255) * hidden * 2, 256);  // gathered activations
}

int launch_mxfp4_tc(const void* A, const uint8_t* w13, const uint8_t* w13_scale, const uint8_t* w2,
                    const uint8_t* w2_scale, const void* b13, const void* b2, const Routing& r,
                    const float* topk_w, __nv_bfloat16* act, float* scratch, int64_t hidden, int64_t ispp,
                    int E, int top_k, float limit, int mul_w, void* tc_ws, int* status, cudaStream_t stream) {
  XKB_REQUIRE(r.block == 16 || r.block == 128, "mxfp4 tcgen05 path: unsupported token tile %d", r.block);
  XKB_REQUIRE(reinterpret_cast<uintptr_t>(w13_scale) % 16 == 0 && reinterpret_cast<uintptr_t>(w2_scale) % 16 == 0,
              "mxfp4 tcgen05 path: scale tensors must be 16-byte aligned");
  Carver carve(tc_ws);
  int32_t* done = r.block_counters != nullptr ? r.block_counters + r.counters_each : nullptr;   // block hand-over counters
  __nv_bfloat16* Ag = carve.take<__nv_bfloat16>(r.max_pad * hidden);
  int64_t gblocks = r.max_pad < 148 * 16 ? r.max_pad : 148 * 16;
  if (gblocks < 1) gblocks = 1;
  XKB_CHECK_CUDA(launch_chained(gather_permute_kernel, dim3((unsigned)gblocks), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(A),
                                                               r.sorted_ids, r.num_post, Ag, r.numel,
                                                               (int)hidden, top_k,
                                                               r.block == 16 ? 0 : 1,   // 16-token tiles convert through the table: natural K order
                                                               r.max_pad, status));
  XKB_CHECK_LAUNCH("gather_permute_kernel");

  CUtensorMap tm_w13, tm_w2, tm_tok0, tm_tok1, tm_s13, tm_s2;
  int rc = make_map_2d(&tm_w13, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w13, (uint64_t)E * 2 * ispp, (uint64_t)hidden / 2,
                       kTileRows, kStageK / 2, CU_TENSOR_MAP_SWIZZLE_128B, "w13");
  if (rc != XKB_OK) return rc;
  rc = make_map_2d(&tm_w2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w2, (uint64_t)E * hidden, (uint64_t)ispp / 2,
                   kTileRows, kStageK / 2, CU_TENSOR_MAP_SWIZZLE_128B, "w2");
  if (rc != XKB_OK) return rc;
  rc = make_map_2d(&tm_s13, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w13_scale, (uint64_t)E * 2 * ispp, (uint64_t)hidden / 32,
                   kTileRows, 16, CU_TENSOR_MAP_SWIZZLE_NONE, "w13 scales");
  if (rc != XKB_OK) return rc;
  rc = make_map_2d(&tm_s2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w2_scale, (uint64_t)E * hidden, (uint64_t)ispp / 32,
                   kTileRows, 16, CU_TENSOR_MAP_SWIZZLE_NONE, "w2 scales");
  if (rc != XKB_OK) return rc;
  rc = make_map_2d(&tm_tok0, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Ag, (uint64_t)r.max_pad, (uint64_t)hidden,
                   (uint32_t)r.block, kSubK, CU_TENSOR_MAP_SWIZZLE_128B, "gathered activations");
  if (rc != XKB_OK) return rc;
  rc = make_map_2d(&tm_tok1, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, act, (uint64_t)r.max_pad, (uint64_t)ispp,
                   (uint32_t)r.block, kSubK, CU_TENSOR_MAP_SWIZZLE_128B, "SwiGLU activations");
  if (rc != XKB_OK) return rc;

  TcParams prm;
  prm.sorted_ids = r.sorted_ids;
  prm.expert_ids = r.expert_ids;
  prm.num_post = r.num_post;
  prm.topk_w = topk_w;
  prm.status = status;
  prm.numel = r.numel;
  prm.max_blocks = (int)r.max_blocks;
  prm.num_experts = E;
  prm.mul_w = mul_w;
  prm.round_rows = 0;
  prm.limit = limit;
  // stage 0: gate_up + SwiGLU -> act
  prm.scratch = nullptr;
  prm.act = act;
  prm.N = (int)ispp;
  prm.K = (int)hidden;
  prm.rows_per_expert = (int)(2 * ispp);
  prm.bias = static_cast<const __nv_bfloat16*>(b13);
  prm.done_signal = done;
  prm.done_wait = nullptr;
  prm.done_target = (int)(ispp / kTileRows) * hand_over_per_tile(r.block);
  GemmTimerScope timed(stream);   // both GEMMs in one scope: they overlap
  int64_t max_tiles = r.max_blocks * (ispp / kTileRows);
  rc = r.block == 16 ? launch_bt<16, kModeMxGateUp>(tm_w13, tm_s13, tm_tok0, prm, max_tiles, stream)
                     : launch_bt<128, kModeMxGateUp>(tm_w13, tm_s13, tm_tok0, prm, max_tiles, stream);
  if (rc != XKB_OK) return rc;
  // stage 1: down -> fp32 slot rows
  prm.scratch = scratch;
  prm.act = nullptr;
  prm.N = (int)hidden;
  prm.K = (int)ispp;
  prm.rows_per_expert = (int)hidden;
  prm.bias = static_cast<const __nv_bfloat16*>(b2);
  prm.done_signal = nullptr;
  prm.done_wait = done;
  max_tiles = r.max_blocks * (hidden / kTileRows);
  // (hidden is a multiple of 512 here, so the row tiles pair up)
  return r.block == 16 ? launch_bt<16, kModeMxDown>(tm_w2, tm_s2, tm_tok1, prm, max_tiles / 2, stream)
                       : launch_bt<128, kModeMxDown>(tm_w2, tm_s2, tm_tok1, prm, max_tiles / 2, stream);
}

}  // namespace xkb

extern "C" int xkb_set_sm_margin(int sms) {
  if (sms < 0 || sms > 128) return xkb::fail(XKB_ERR_ARG, "xkb_set_sm_margin: %d outside [0,128]", sms);
  xkb::g_sm_margin.store(sms, std::memory_order_relaxed);
  return XKB_OK;
}

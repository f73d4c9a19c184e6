// FP16 / BF16 attention forward for sm_100a: TMA -> swizzled shared memory -> tcgen05.mma with
// accumulators in tensor memory, online softmax read straight out of tensor memory, P handed to the
// second MMA through tensor memory (no shared-memory or HBM round trip).
//
// Replaces the reference's mma.sync kernel (reference csrc/flash_attn/mma/kernel.cuh:18-201) and
// keeps its contract: scale 1/sqrt(D) folded into exp2 (mma/softmax.cuh:104-108), top-left causal
// mask "col > row" plus "col >= seqLenKV" (mma/softmax.cuh:136-138), KV head = Q head / group
// (params.cuh:25-27), fp32 accumulation of S and O, P rounded to the 16-bit input type before P.V
// while the row sum uses unrounded P (mma/softmax.cuh:107-108, mma/layout.cuh:87-97), a row whose
// sum is 0 yields 0 (mma/softmax.cuh:126), sequences without keys leave O untouched
// (mma/kernel.cuh:39-42).
//
// CTA = 16 warps:
//   warps 0-3   softmax for Q tile 0 (one thread per query row, 128 rows)
//   warps 4-7   softmax for Q tile 1 (when the CTA owns two Q tiles)
//   warps 8-11  epilogue: final 1/rowsum, conversion to the 16-bit type, stores O
//   warp  12    issues the tcgen05.mma of Q tile 0 (one thread)
//   warp  13    issues every TMA load (one thread)
//   warp  14    packed input: zeroes the V rows past a sequence's end; idle otherwise
//   warp  15    issues the tcgen05.mma of Q tile 1 (one thread)
//
// Tensor memory columns (fp32 words per lane; lane = query row of the tile):
//   [t*128, t*128+128)            S of Q tile t; the 16-bit P overwrites the first 64 columns
//   [256 + t*HDP, 256+(t+1)*HDP)  O of Q tile t (NT == 2, HDP == 128), or [128, 128+HDP) when NT == 1
//   HDP == 64: 192 columns per tile with S alternating between two positions (see Cfg::kRot), O at 384 + t*64
//
// Three CTA forms share this kernel body: two Q tiles per CTA and one CTA per SM (HDP 128; HDP 192 / 256 with one tile),
// one tile per CTA and two CTAs per SM (CfgSolo64, head dims 32 / 64), and clusters of two one-tile CTAs that share
// every K/V block through tcgen05.mma.cta_group::2 (CfgPair, head dims 192 / 256).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "ptx_sm100.cuh"
#include "tfa_common.cuh"

namespace tfa_b200 {

struct TcParams {
  void* O;
  const int* cuQ;
  const int* cuKV;
  int seqLenQ;    // fixed length, or max length for varlen
  int seqLenKV;
  int headsQ;
  int headsKV;
  int headDim;    // true head dim (<= HDP)
  int group;      // headsQ / headsKV
  int packShift;  // log2 of the number of Q heads interleaved into one 128-row tile
  int numPairs;   // query tile pairs per sequence (from the maximum length)
  int numUnits;   // Q head units (headsQ >> packShift)
  int numWork;    // numPairs * numUnits * batch
  int chunk;      // work index order: 0 = pair index fastest within a head; n > 0 = chunks of n (head unit, batch)
                  // entries, inside a chunk the pair index slowest (see make_work)
  int* workCounter;  // device counters, zero at launch: [0] next work item, [1] CTAs that have finished
  int causal;
  float scaleLog2;  // log2(e) / sqrt(headDim)
  int* status;      // device status word
  // packed variable-length input whose row totals the host does not know: the three tensor maps (Q, K, V), completed
  // on the device by patch_varlen_maps from cuQ[batch] / cuKV[batch]; nullptr = use the maps passed as kernel arguments
  const CUtensorMap* devMaps;
  int epoch;        // launch epoch (24 bits)
};

namespace tc {

constexpr int kBlockM = 128;  // query rows per tile = TMEM lanes
constexpr int kBlockN = 128;  // keys per KV block
constexpr int kThreads = 512;
constexpr int kIssuerB = 15;  // warp that issues the MMAs of Q tile 1 (warp 12 issues those of tile 0)
// Of every kEmuPeriod pairs of exponentials, the first kEmuCount are evaluated on the FMA pipe instead of the MUFU: pairs
// 0, 16, 32 and 48 of the 64 of a row and key block, i.e. the first pair of each 32-column quarter.  Measured on the
// benchmark shape (bf16 / fp16 non-causal, interleaved A/B of one build per pattern): none 961, 1 of 64 963, 2 of 64 991,
// 3 of 64 1071, **1 of 16 1187 / 1104**, 3 of 32 1043, 1 of 8 1055 / 1003, 1 of 4 942 TFLOP/s; the same four pairs moved
// to positions 8 or 15 of each quarter 1047 / 1073, all four in the first quarter 1014, five per block 1076.  The
// optimum is narrow and belongs to the instruction schedule the compiler finds for this exact mix (the FMA-pipe
// sequence is a long dependent chain that it hides behind the MUFU instructions of the pairs around it), not to a
// pipe-throughput model: by throughput alone 2-3 of 8 pairs would pay.
constexpr int kEmuPeriod = 16;
constexpr int kEmuCount = 1;
// Register split of the 64 K registers of an SM between the role groups (8 + 4 + 4 warps).
constexpr int kRegsSoftmax = 176;
constexpr int kRegsEpilogue = 96;
constexpr int kRegsIssue = 64;
// setmaxnreg only moves registers between the warps of one CTA: what the softmax warps gain must have been given up
// by the others, out of the allocation the CTA was launched with (registers per thread at launch = 64 K / threads,
// rounded down to a multiple of 8).  An increase that cannot be served blocks for ever, so this is checked here.
constexpr int kRegsAtLaunch = (65536 / kThreads) / 8 * 8;
static_assert(8 * kRegsSoftmax + 4 * kRegsEpilogue + 4 * kRegsIssue <= (kThreads / 32) * kRegsAtLaunch,
              "register budget: the CTA's launch allocation must cover every role's setmaxnreg value");
// Lazy-rescale threshold, log2 units.  Price in accuracy, measured on the benchmark shapes against fp64: the mean
// output error is 3-4 % above that of exact running maxima (and of the reference kernels), the maximum error within one
// unit in the last place of the output type.  With the exact maximum the largest weights of a row sit just below 1.0,
// at the top of a binade where the 16-bit P is most precise (the maximum itself is exactly 1.0); a stale reference
// value spreads them over the binade.  Threshold 0 restores the last 3 % and makes most blocks take the rescale path.
constexpr float kRescaleLog2 = 8.0f;
constexpr int kSubTileBytes = 128 * 128;  // 128 rows x 128 bytes (64 16-bit elements), one swizzle-128B slab

template <int HDP>
struct Cfg {
  static constexpr int kSub = HDP / 64;                  // 64-element slabs per row
  static constexpr int kTileBytes = kSub * kSubTileBytes;  // one 128-row tile of Q, K or V
  static constexpr int kNT = (HDP <= 128) ? 2 : 1;       // Q tiles per CTA
  // Q buffers per tile: with two, the Q tiles of the next work item load while the current item still computes.
  // HDP == 128 would have to give up a K/V ring stage for that (227 KB of shared memory): measured 12 % slower.
  static constexpr int kQBufs = (HDP == 64) ? 2 : 1;
  static constexpr int kStages = (HDP == 64) ? 6 : (HDP == 128) ? 4 : (HDP == 192) ? 3 : 2;
  static constexpr int kTmemCols = 512;
  // HDP == 64 leaves tensor memory to spare, which buys a second S position per tile: S of block j sits at
  // columns [0,128) (j even) or [64,192) (j odd) of the tile's 192-column region and P of block j in the 64 columns
  // that the next S does not cover ([0,64) or [128,192)).  Q.K^T of block j+1 can then be issued as soon as the
  // softmax has read S of block j, instead of after P.V of block j: the softmax never waits for the tensor pipe.
  static constexpr bool kRot = (HDP == 64);
  // HDP 192 / 256 run one Q tile per CTA, which leaves room for two full S buffers (columns [0,128) and [128,256)):
  // Q.K^T of block j+1 is issued before P.V of block j and overlaps the softmax of block j.
  static constexpr bool kDblS = (kNT == 1);
  static constexpr bool kTwoPos = kRot || kDblS;                           // S / P alternate between two positions
  static constexpr int kSPosStride = kRot ? 64 : (kDblS ? 128 : 0);        // column offset of S for odd blocks
  static constexpr int kPPosStride = kTwoPos ? 128 : 0;                    // column offset of P for odd blocks
  static constexpr int kSRegion = kRot ? 192 : (kDblS ? 256 : 128);        // columns per tile for S / P
  static constexpr int kOCol0 = kRot ? 384 : 256;
  static constexpr int kStageBytes = kTileBytes;         // one K/V ring stage
  static constexpr int kSmemBytes = kNT * kQBufs * kTileBytes + kStages * kStageBytes + 2048 /*barriers, scales*/ + 1024 /*align*/;
};

// Head dim <= 64, second form: ONE Q tile per CTA and TWO CTAs per SM (8 warps each: 4 softmax warps that also
// write the output, one MMA-issuing and one loading thread, two idle warps).  The two tiles of an SM then belong to different work
// items, so one CTA's item boundary (output, next item's first loads and scores) runs while the other CTA computes,
// instead of both tiles of one CTA standing at the same boundary.  Tensor memory: 256 columns per CTA - S rotating in
// 192 as above, O in the last 64.  Shared memory: two Q buffers and four K/V stages of 16 KB, 99 KB per CTA.
struct CfgSolo64 {
  static constexpr int kSub = 1;
  static constexpr int kTileBytes = kSubTileBytes;
  static constexpr int kNT = 1;
  static constexpr int kQBufs = 2;
  static constexpr int kStages = 4;
  static constexpr int kTmemCols = 256;
  static constexpr bool kRot = true;
  static constexpr bool kDblS = false;
  static constexpr bool kTwoPos = true;
  static constexpr int kSPosStride = 64;
  static constexpr int kPPosStride = 128;
  static constexpr int kSRegion = 192;
  static constexpr int kOCol0 = 192;
  static constexpr int kStageBytes = kTileBytes;
  static constexpr int kSmemBytes = kNT * kQBufs * kTileBytes + kStages * kStageBytes + 2048 + 1024;
};

// Head dims 192 / 256, pair form: a cluster of two CTAs on the two SMs of a TPC works on two neighbouring Q tiles of one
// head (one tile each) and shares every K/V block: the MMAs are issued by rank 0 with cta_group::2 (M = 256), which
// reads half of the B operand from each CTA's shared memory - keys [64 r, 64 r + 64) of the block for Q.K^T, half of
// the head dim for P.V.  Each CTA therefore loads half of every K and V block: half the L2 -> shared-memory traffic
// per FLOP of the one-tile form (which pulls 7-8 TB/s out of L2 at these head dims and is bound by it), and ring
// stages of 32 KB instead of 64 / 48 KB, i.e. room for four or five of them.  Tensor memory as in the one-tile form:
// two S buffers and O.  At head dim 192 each CTA's half of V is 96 columns, one and a half 64-element slabs: CTA r
// loads the slabs at head-dim offsets {0, 128} (r = 0) or {64, 160} (r = 1) and the MMA uses the first 96 columns, so
// that the O columns come out permuted in chunks of 32 (o_chunk_offset); the output pass undoes it.
template <int HDP>
struct CfgPair {
  static_assert(HDP == 192 || HDP == 256, "pair form: head dims 192 and 256");
  static constexpr int kSub = HDP / 64;
  static constexpr int kTileBytes = kSub * kSubTileBytes;  // one 128-row Q tile
  static constexpr int kNT = 1;
  static constexpr int kQBufs = 1;
  static constexpr int kStageBytes = 2 * kSubTileBytes;  // K: 64 keys x HDP (<= 32 KB); V: 128 keys x two 64-wide slabs
  static constexpr int kStages = (HDP == 256) ? 4 : 5;  // a fifth stage at 256 (exactly the 227 KB limit) measured no different
  static constexpr int kTmemCols = 512;
  static constexpr bool kRot = false;
  static constexpr bool kDblS = true;
  static constexpr bool kTwoPos = true;
  static constexpr int kSPosStride = 128;
  static constexpr int kPPosStride = 128;
  static constexpr int kSRegion = 256;
  static constexpr int kOCol0 = 256;
  static constexpr int kSmemBytes = kTileBytes + kStages * kStageBytes + 2048 + 1024;
};
// head-dim offset of the 32-column chunk ch of O (pair form; identity except at head dim 192, see CfgPair)
template <int HDP, bool kPair>
__host__ __device__ constexpr int o_chunk_offset(int ch) {
  if (kPair && HDP == 192) return ch == 0 ? 0 : ch == 1 ? 32 : ch == 2 ? 128 : ch == 3 ? 64 : ch == 4 ? 96 : 160;
  return ch * 32;
}
// head-dim offset of the slab a (0 / 1) of V that CTA `rank` of a pair loads
template <int HDP>
__device__ __forceinline__ int v_slab_offset(int rank, int a) {
  if (HDP == 192) return rank == 0 ? a * 128 : 64 + a * 96;
  return rank * 128 + a * 64;
}
constexpr int kThreadsSolo = 256;  // two whole warpgroups (setmaxnreg is a warpgroup-wide instruction); warps 6 and 7 idle

// Barrier slots (8 bytes each) inside the control block that follows the tiles.
// A parity wait can only tell "the phase in progress" from "the phase just completed": a waiter must never fall
// two phases behind its barrier.  Where a producer may legitimately run two uses ahead (Q tiles with two buffers,
// P in rotating-S mode) each buffer / position has its own barrier, whose next completion depends on the waiter.
enum Bar : int {
  kBarQFull = 0,       // [tile][Q buffer]  Q tile landed
  kBarQEmpty = 4,      // [tile][Q buffer]  last Q.K^T of the item finished: buffer may be overwritten (tcgen05.commit)
  kBarP0Ready = 8,     // [tile][S position] first half of P written (4 softmax warps; O already rescaled if needed)
  kBarP1Ready = 12,    // [tile][S position] second half of P written (4 softmax warps)
  kBarSFull = 44,      // [tile][S position]  S = Q.K^T finished (tcgen05.commit)
  kBarPvDone = 16,     // [tile][S position]  O += P.V finished (tcgen05.commit)
  kBarScaleFull = 20,  // [2]  softmax published the final row sums (once per tile and item)
  kBarTurn = 22,       // [2]  issue-turn token of the MMA thread of tile t
  kBarSFree = 24,      // [2]  softmax has read S into registers (rotating-S mode only)
  kBarOFree = 26,      // [2]  epilogue has read O of the item into registers (4 epilogue warps)
  kBarWorkFull = 28,   // [2]  loader published the next work item in slot k & 1
  kBarWorkEmpty = 30,  // [2]  every consumer has read the slot
  kBarKvFull = 32,     // [kStages <= 6]
  kBarKvEmpty = 38,    // [kStages <= 6]
  // pair form only
  kBarIdxFull = 48,    // [2]  rank 1: rank 0 has written the next work index into peerIdx[k & 1]
  kBarIdxEmpty = 50,   // [2]  rank 0: rank 1 has read peerIdx[k & 1]
  kBarOFreePair = 52,  // rank 0: the epilogue warps of both CTAs have read O of the item (8 arrivals)
  kNumBars = 54,
};

constexpr int kWorkConsumers = 14;  // 8 softmax warps + 4 epilogue warps + 2 MMA-issuing threads

// What the loader publishes about a work item: everything the other roles need, so that only one thread pays for
// the divisions of make_work (and does so while the previous item is still being computed).
struct WorkSlot {
  int idx;         // work item index; negative: no more work
  int sq, skv;
  int unit;
  long long qRow0;
  int qlo[2];
  int nblk[2];
  int nmax;
  int pad;
};

struct Ctl {
  uint64_t bars[kNumBars];
  float scale[2][kBlockM];
  uint32_t tmemBase;
  int failed;
  WorkSlot work[2];
  int peerIdx[2];  // pair form, rank 1: work indices handed over by rank 0
};

struct WaitCtx {
  volatile int* failed;
  int* status;
  int epoch;
};

// Bounded wait: gives up after ~2 s, records (epoch << 8 | site) and lets the caller continue so that
// every loop still terminates; later waits of the CTA return at once.
__device__ __forceinline__ void wait_bar(uint32_t bar, uint32_t parity, const WaitCtx& c, int site) {
  if (ptx::mbar_try_wait(bar, parity)) return;
  uint32_t spins = 0;
  uint64_t t0 = 0;
  while (!ptx::mbar_try_wait(bar, parity)) {
    if ((++spins & 0x3FF) == 0) {
      if (*c.failed) return;
      const uint64_t now = ptx::global_timer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > 2000000000ull) {
        *c.failed = 1;
        atomicExch(c.status, (c.epoch << 8) | site);
        return;
      }
    }
  }
}

// Same contract as wait_bar, with cluster-scope acquire: what the other CTA of a pair stored into this CTA's shared
// memory before its arrival is visible afterwards.
__device__ __forceinline__ void wait_bar_cluster(uint32_t bar, uint32_t parity, const WaitCtx& c, int site) {
  uint32_t spins = 0;
  uint64_t t0 = 0;
  while (!ptx::mbar_try_wait_cluster(bar, parity)) {
    if ((++spins & 0x3FF) == 0) {
      if (*c.failed) return;
      const uint64_t now = ptx::global_timer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > 2000000000ull) {
        *c.failed = 1;
        atomicExch(c.status, (c.epoch << 8) | site);
        return;
      }
    }
  }
}

// Same contract as wait_bar, polling with the non-blocking test_wait: lower wake-up latency, at the price of
// issue slots - used only by the single-thread MMA issuers, whose reaction time is on the critical path.
__device__ __forceinline__ void spin_bar(uint32_t bar, uint32_t parity, const WaitCtx& c, int site) {
  if (ptx::mbar_test_wait(bar, parity)) return;
  uint32_t spins = 0;
  uint64_t t0 = 0;
  while (!ptx::mbar_test_wait(bar, parity)) {
    if ((++spins & 0x3FFF) == 0) {
      if (*c.failed) return;
      const uint64_t now = ptx::global_timer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > 2000000000ull) {
        *c.failed = 1;
        atomicExch(c.status, (c.epoch << 8) | site);
        return;
      }
    }
  }
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Row maximum with NaN kept (max.f32 would drop it): a NaN score must poison its row, as it does in the reference,
// where it reaches the row sum through the exponential (reference csrc/flash_attn/mma/softmax.cuh:104-111).
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float fmax2(float a, float b) {
  float d;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
  return d;
}
// two-wide fp32 FMA / ADD on a register pair
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<const uint64_t&>(a)), "l"(reinterpret_cast<const uint64_t&>(b)),
        "l"(reinterpret_cast<const uint64_t&>(c)));
  return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<const uint64_t&>(a)), "l"(reinterpret_cast<const uint64_t&>(b)));
  return d;
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  float2 d;
  asm("mul.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<const uint64_t&>(a)), "l"(reinterpret_cast<const uint64_t&>(b)));
  return d;
}

__device__ __forceinline__ float2 fadd2_rm(float2 a, float2 b) {  // round toward -inf
  float2 d;
  asm("add.rm.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<const uint64_t&>(a)), "l"(reinterpret_cast<const uint64_t&>(b)));
  return d;
}

// exp2 on the FMA pipe for a pair of values (the MUFU unit is the co-bottleneck of this kernel: 16 ex2/clk/SM
// against 128x128 exponentials per tile-block).  x = floor(x) + f; 2^f by a minimax cubic with p(0) = 1 (max relative
// error 8.6e-5); 2^floor(x) by adding to the exponent field.  The magic constant 1.5*2^23 makes the low mantissa bits
// of t hold floor(x); x is clamped at -127.  The result feeds the 16-bit P: 8.6e-5 is far below bf16's rounding (2^-9)
// and, on one value in sixteen, adds 0.3 % to the rms error of an fp16 P (2^-12).  (A quartic, 2.9e-6, was measured for
// fp16: no difference in the output error - that is set by the stale row maxima, see kRescaleLog2 - and it does not get
// the schedule the cubic gets: 999 against 1104 TFLOP/s.)
__device__ __forceinline__ float2 ex2_fma2(float2 x) {
  const float kMagic = 12582912.f;
  x.x = fmaxf(x.x, -127.f);
  x.y = fmaxf(x.y, -127.f);
  const float2 t = fadd2_rm(x, make_float2(kMagic, kMagic));
  const float2 xi = fadd2(t, make_float2(-kMagic, -kMagic));
  const float2 f = ffma2(xi, make_float2(-1.f, -1.f), x);
  float2 p = ffma2(make_float2(0.07706704f, 0.07706704f), f, make_float2(0.22764499f, 0.22764499f));
  p = ffma2(p, f, make_float2(0.69511679f, 0.69511679f));
  p = ffma2(p, f, make_float2(1.f, 1.f));
  p.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23));
  p.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23));
  return p;
}

template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (kBf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

// Per-CTA work description, computed identically by every role.
struct Work {
  long long qRow0;   // first row of this sequence in Q/O (flattened [rows, H, D] view, used for the O stores)
  long long kvRow0;  // first row of this sequence in K/V
  // TMA coordinates.  Fixed length: tensors are described as [B, S, H, D], so rows past the end of a batch entry are
  // zero-filled by TMA exactly like the reference zero-fills them (reference csrc/flash_attn/mma/memory.cuh:52-59).
  // Packed variable length: one "batch entry" holding all rows; rows past a sequence end belong to the next sequence
  // and are masked (K) or weighted by P = 0 (V).
  int qRowTma, kvRowTma, batchTma;
  int sq, skv;
  int unit;          // Q head unit (packs 1 << packShift heads)
  int hkv;
  int qlo[2], qhi[2];  // sequence positions covered by each tile: [qlo, qhi)
  int nblk[2];         // KV blocks each tile consumes
  int nmax;
};

// Packed variable-length input, last key block of a sequence: overwrite the rows of the V tile that lie past the end
// of the sequence with zeros (they are the next sequence's, and P = 0 times a NaN or Inf stored there would still
// poison O; the reference zero-fills rows past a sequence end, reference csrc/flash_attn/mma/memory.cuh:52-59).  One
// warp, four key rows per lane, once the tile has landed.  K needs nothing: its columns are masked whatever they hold.
template <int kSub>
__device__ __forceinline__ void zero_v_tail(uint32_t tileAddr, int lane, int tail) {
  for (int row = lane; row < kBlockN; row += 32) {
    if (row >= tail) {  // key rows [tail, 128) of the block are not this sequence's
      const uint32_t rowAddr = tileAddr + (uint32_t)(row * 128);
#pragma unroll
      for (int a = 0; a < kSub; a++) {
#pragma unroll
        for (int q = 0; q < 8; q++) {
          asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(rowAddr + a * kSubTileBytes + q * 16), "r"(0u) : "memory");
        }
      }
    }
  }
  ptx::fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's reads
  __syncwarp();
}

// Work item idx -> (query tile pair, Q head unit, batch entry).  Two orders.  Pair index fastest: CTAs running at the
// same time work on the same head and share its K/V through L2 (all items cost the same when nothing is causal).
// Causal: the cost of an item grows with its pair index, so inside a chunk of p.chunk consecutive (head unit, batch)
// entries the items are handed out heaviest first (pair index slowest, descending) - the longest-processing-time-first
// rule, which leaves only light items for the end of the launch; neighbouring indices are then the Q heads of one KV
// group, which still share K/V, and the host sizes the chunk so that the K/V of its heads stay resident in L2.
template <int NT, bool kVarlen>
__device__ __forceinline__ bool make_work(const TcParams& p, int idx, Work& w) {
  int pr, rest;
  if (p.chunk > 0) {
    const int per = p.numWork / p.numPairs;  // (head unit, batch) entries
    const int chunkItems = p.chunk * p.numPairs;
    const int c = idx / chunkItems;
    const int within = idx - c * chunkItems;
    const int width = min(p.chunk, per - c * p.chunk);  // the last chunk may be narrower
    pr = within / width;
    rest = c * p.chunk + (within - pr * width);
  } else {
    pr = idx % p.numPairs;
    rest = idx / p.numPairs;
  }
  const int pairIdx = p.causal ? (p.numPairs - 1 - pr) : pr;
  w.unit = rest % p.numUnits;
  const int b = rest / p.numUnits;
  if constexpr (kVarlen) {
    const int q0 = p.cuQ[b], q1 = p.cuQ[b + 1], k0 = p.cuKV[b], k1 = p.cuKV[b + 1];
    w.qRow0 = q0;
    w.sq = q1 - q0;
    w.kvRow0 = k0;
    w.skv = k1 - k0;
    w.qRowTma = q0;
    w.kvRowTma = k0;
    w.batchTma = 0;
  } else {
    w.sq = p.seqLenQ;
    w.skv = p.seqLenKV;
    w.qRow0 = (long long)b * p.seqLenQ;
    w.kvRow0 = (long long)b * p.seqLenKV;
    w.qRowTma = 0;
    w.kvRowTma = 0;
    w.batchTma = b;
  }
  const int rows = kBlockM >> p.packShift;  // sequence positions per tile
  const int seq0 = pairIdx * NT * rows;
  w.nmax = 0;
  w.nblk[0] = w.nblk[1] = 0;
  if (seq0 >= w.sq || w.skv <= 0) return false;
  w.hkv = (w.unit << p.packShift) / p.group;
  const int nTotal = (w.skv + kBlockN - 1) / kBlockN;
#pragma unroll
  for (int t = 0; t < 2; t++) {
    w.qlo[t] = seq0 + t * rows;
    w.qhi[t] = min(w.qlo[t] + rows, w.sq);
    int n = 0;
    if (t < NT && w.qlo[t] < w.sq) {
      n = p.causal ? min(nTotal, (w.qhi[t] + kBlockN - 1) / kBlockN) : nTotal;
    }
    w.nblk[t] = n;
    w.nmax = max(w.nmax, n);
  }
  return true;
}

// Persistent kernel: gridDim.x CTAs (one per SM) pull work items from a global counter until it runs out, so the
// prologue of the next item (Q/K/V loads, first Q.K^T) overlaps the epilogue of the current one.  Every mbarrier keeps
// running across items; each role tracks phases with its own running counters.
// kMode: 0 fixed length, 1 packed variable-length input (cu_seqlens), 2 fixed length where no score is ever masked
// (not causal, key length a multiple of the 128-key block).  Separate instantiations, because code that a path never
// executes still costs it when it sits in the softmax loop (measured: the variable-length code 4-5 % of the
// fixed-length speed; the masking code 8 % at head dim 64 and nothing at 128 / 256, so mode 2 is only built for
// the 64 kernel).
constexpr int kModeFixed = 0, kModeVarlen = 1, kModeFixedNoMask = 2;
// kHD: the head dim the MMAs are shaped for.  The tiles in shared memory are always HDP wide (64-element slabs, TMA
// zero-fills past the true head dim); with kHD < HDP (32 in the 64-wide kernel, 96 in the 128-wide one) Q.K^T stops
// after kHD / 16 k-steps, P.V produces kHD output columns, and the rescale and output passes touch kHD columns.
// kPair: the CTA-pair form of head dims 192 / 256 (CfgPair): launched as clusters of two, fixed-length input only.
template <int HDP, bool kBf16, int kMode, bool kSolo = false, int kHD = HDP, bool kPair = false>
__global__ void __launch_bounds__(kSolo ? kThreadsSolo : kThreads, kSolo ? 2 : 1)
fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const TcParams p) {
  static_assert(!kSolo || HDP == 64, "the one-tile, two-CTAs-per-SM form exists for padded head dim 64 only");
  static_assert(kHD == HDP || (HDP == 64 && kHD == 32) || (HDP == 128 && kHD == 96), "MMA head dim");
  static_assert(!kPair || (HDP >= 192 && kMode == kModeFixed && !kSolo), "pair form: head dims 192 / 256, fixed length");
  using C = typename std::conditional<kPair, CfgPair<(kPair ? HDP : 256)>,
                                      typename std::conditional<kSolo, CfgSolo64, Cfg<HDP>>::type>::type;
  constexpr int NT = C::kNT;
  // warp roles: softmax warps [0, 4 * NT'), epilogue warps, the two MMA-issuing warps, the loading warp
  constexpr int kSoftmaxWarps = kSolo ? 4 : 8;
  constexpr int kEpilogueEnd = kSolo ? 4 : 12;  // epilogue warps are [kSoftmaxWarps, kEpilogueEnd): none in the solo form
  constexpr int kIssueWarpA = kSolo ? 4 : 12, kIssueWarpB = kSolo ? -1 : kIssuerB, kLoadWarp = kSolo ? 5 : 13;
  constexpr bool kVarlen = (kMode == kModeVarlen);
  // Packed input has one more role: a warp that is idle otherwise (14, or 6 in the one-tile form) zeroes the V rows
  // past a sequence's end and takes part in every "first half of P ready" barrier, so that no P.V can start before
  // the rows are clean.  Kept out of the softmax warps: the same code inside their block loop, executed once per
  // sequence and tile, cost the packed kernel 4-5 % on every block.
  constexpr int kHelpWarp = kSolo ? 6 : 14;
  constexpr int kConsumers = (kSolo ? 5 : kWorkConsumers) + (kVarlen ? 1 : 0);  // roles that read every work item
  constexpr int NS = C::kStages;
  static_assert(NS <= 6, "barrier slots");
  // One-tile forms: a ring stage's "free" barrier completes exactly when the MMAs that read the stage have finished,
  // i.e. when S of that K block (resp. O += P.V of that V block) is ready, and one issuing thread feeds the tensor
  // pipe, which idles while that thread executes a tcgen05.commit (~120-150 clocks each).  So the softmax and output
  // warps wait on the ring barriers themselves (they can work out every block's ring position from the running load
  // count) and the issuing thread commits twice per block instead of four times.  With two tiles per CTA a stage is
  // free only when both tiles are done with it, which says nothing about one tile's S, so they keep their own barriers.
  // Not with a ring of two stages (head dim 256, one-tile form): there K of block j + 1 re-uses the stage of K of block
  // j and its Q.K^T is issued before P.V of block j, so the stage's barrier could complete a second time before a slow
  // softmax warp has looked at it once, and a parity wait cannot tell the two apart.  From three stages on, whatever
  // re-uses a stage is consumed at or after P.V of the block whose scores the waiting warp is about to produce.
  constexpr bool kRingSig = (NT == 1 && NS >= 3);
  static_assert(!kRingSig || C::kTwoPos, "one-tile forms alternate S between two positions");

  extern __shared__ uint8_t smemRaw[];
  const uint32_t rawAddr = ptx::smem_u32(smemRaw);
  const uint32_t tileAddr = (rawAddr + 1023u) & ~1023u;  // swizzle-128B slabs need 1024-byte alignment
  uint8_t* smem = smemRaw + (tileAddr - rawAddr);
  const uint32_t sQ = tileAddr;
  const uint32_t sKV = tileAddr + NT * C::kQBufs * C::kTileBytes;
  Ctl* ctl = reinterpret_cast<Ctl*>(smem + NT * C::kQBufs * C::kTileBytes + NS * C::kStageBytes);
  const uint32_t barBase = ptx::smem_u32(&ctl->bars[0]);
  auto bar = [&](int slot) { return barBase + 8u * (uint32_t)slot; };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // pair form: rank in the cluster of two, and this CTA's / rank 0's barrier block seen through the cluster window
  uint32_t rank = 0, barBase0 = barBase, barBasePeer = barBase;
  if constexpr (kPair) {
    rank = ptx::cluster_ctarank();
    barBase0 = ptx::mapa(barBase, 0);
    barBasePeer = ptx::mapa(barBase, rank ^ 1u);
  }
  auto bar0 = [&](int slot) { return barBase0 + 8u * (uint32_t)slot; };  // the barrier of rank 0 (cluster address)
  (void)barBasePeer;
  (void)bar0;

  if (threadIdx.x == 0) {
    for (int t = 0; t < 2; t++) {
      for (int u = 0; u < 2; u++) {
        ptx::mbar_init(bar(kBarQFull + 2 * t + u), 1);
        ptx::mbar_init(bar(kBarQEmpty + 2 * t + u), 1);
        // pair form: the softmax warps of both CTAs; packed input: the four softmax warps and the V-tail warp
        ptx::mbar_init(bar(kBarP0Ready + 2 * t + u), kPair ? 8 : (kVarlen ? 5 : 4));
        ptx::mbar_init(bar(kBarP1Ready + 2 * t + u), kPair ? 8 : 4);
        ptx::mbar_init(bar(kBarSFull + 2 * t + u), 1);
        ptx::mbar_init(bar(kBarPvDone + 2 * t + u), 1);
      }
      ptx::mbar_init(bar(kBarTurn + t), 1);
      ptx::mbar_init(bar(kBarSFree + t), 4);
      ptx::mbar_init(bar(kBarScaleFull + t), 4);
      ptx::mbar_init(bar(kBarOFree + t), 4);
      ptx::mbar_init(bar(kBarWorkFull + t), 1);
      ptx::mbar_init(bar(kBarWorkEmpty + t), kConsumers);
      ptx::mbar_init(bar(kBarIdxFull + t), 1);
      ptx::mbar_init(bar(kBarIdxEmpty + t), 1);
    }
    ptx::mbar_init(bar(kBarOFreePair), 8);
    for (int s = 0; s < NS; s++) {
      ptx::mbar_init(bar(kBarKvFull + s), 1);
      ptx::mbar_init(bar(kBarKvEmpty + s), 2);  // one arrival per MMA-issuing thread
    }
    ctl->failed = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == kIssueWarpA) {
    if constexpr (kPair) {
      ptx::tmem_alloc_pair(ptx::smem_u32(&ctl->tmemBase), C::kTmemCols);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(ptx::smem_u32(&ctl->tmemBase), C::kTmemCols);
      ptx::tmem_relinquish();
    }
  }
  // tensor maps: the kernel arguments, or (packed input with totals only known on the device) maps in global memory
  const CUtensorMap* mapQ = &tmQ;
  const CUtensorMap* mapK = &tmK;
  const CUtensorMap* mapV = &tmV;
  if constexpr (kVarlen) {
    if (p.devMaps != nullptr) {
      mapQ = p.devMaps;
      mapK = p.devMaps + 1;
      mapV = p.devMaps + 2;
    }
  }
  if (warp == kLoadWarp && lane == 0) {
    if (kVarlen && p.devMaps != nullptr) {
      ptx::tensormap_acquire(mapQ);
      ptx::tensormap_acquire(mapK);
      ptx::tensormap_acquire(mapV);
    } else {
      ptx::prefetch_tensormap(mapQ);
      ptx::prefetch_tensormap(mapK);
      ptx::prefetch_tensormap(mapV);
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if constexpr (kPair) ptx::cluster_sync();  // the other CTA's barriers are initialised before anyone arrives on them
  ptx::tc_fence_after();
  const uint32_t tmem = ctl->tmemBase;
  const WaitCtx wc{&ctl->failed, p.status, p.epoch};

  // Every consumer of work items (8 softmax warps, 4 epilogue warps, 2 MMA threads) reads item k from slot k & 1
  // and frees the slot; a negative index ends the loop.
  auto fetchWork = [&](int k, Work& w) -> int {
    wait_bar(bar(kBarWorkFull + (k & 1)), (k >> 1) & 1, wc, 20);
    // plain loads: the barrier wait above is an acquire and a compiler-level memory fence, and fields that a role
    // does not use cost it neither a load nor a register
    const WorkSlot* ws = &ctl->work[k & 1];
    w.sq = ws->sq;
    w.skv = ws->skv;
    w.unit = ws->unit;
    w.qRow0 = ws->qRow0;
    w.qlo[0] = ws->qlo[0];
    w.qlo[1] = ws->qlo[1];
    w.nblk[0] = ws->nblk[0];
    w.nblk[1] = ws->nblk[1];
    w.nmax = ws->nmax;
    return ws->idx;
  };

  if (warp < kSoftmaxWarps) {
    // ================================================================ softmax
    ptx::setmaxnreg_inc<kRegsSoftmax>();
    const int t = warp >> 2;
    const int r = threadIdx.x & 127;
    const uint32_t tRegion = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(t * C::kSRegion);
    const float c = p.scaleLog2;
    int it = 0;      // blocks of this tile processed so far, over all work items (phase of the per-block barriers)
    int items = 0;   // work items in which this tile was active
    int ldBase = 0;  // K/V ring loads of all earlier items (packed variable-length input only, see below)
    for (int k = 0;; k++) {
      Work w;
      const int idx = fetchWork(k, w);
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(bar(kBarWorkEmpty + (k & 1)));
      if (idx < 0 || *wc.failed) break;
      if (w.nmax == 0) continue;
      const int ldItem = ldBase;
      if constexpr (kRingSig) ldBase += 2 * w.nmax;
      (void)ldItem;
      if (t >= NT || w.nblk[t] == 0) continue;
      const int qpos = w.qlo[t] + (r >> p.packShift);
      float m = -INFINITY, l = 0.f;
      const int n = w.nblk[t];
      for (int j = 0; j < n; j++, it++) {
        if constexpr (kRingSig) {  // ring order K0 | K1 V0 | K2 V1 | ...: K of block j is load 2 j - 1 of the item (K0: 0)
          const int g = ldItem + (j == 0 ? 0 : 2 * j - 1);
          wait_bar(bar(kBarKvEmpty + g % NS), (g / NS) & 1, wc, 1);
        } else {
          wait_bar(bar(kBarSFull + 2 * t + (C::kTwoPos ? (it & 1) : 0)), (C::kTwoPos ? (it >> 1) : it) & 1, wc, 1);
        }
        ptx::tc_fence_after();
        uint32_t v[4][32];
        const uint32_t tS = tRegion + (uint32_t)((it & 1) * C::kSPosStride);   // S of this block
        const uint32_t tP = tRegion + (uint32_t)((it & 1) * C::kPPosStride);   // where its P goes
        const int pSlot = C::kTwoPos ? (it & 1) : 0;  // which P barrier pair
#pragma unroll
        for (int q = 0; q < 4; q++) ptx::tmem_ld_32x32b_x32(tS + q * 32, v[q]);
        ptx::tmem_wait_ld();
#pragma unroll
        for (int q = 0; q < 4; q++) ptx::tmem_ld_fence(v[q]);
        if constexpr (C::kRot) {  // S is in registers: the next Q.K^T may overwrite it
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(bar(kBarSFree + t));
        }

        const int kbase = j * kBlockN;
        const bool needMask = (kMode != kModeFixedNoMask) &&
                              ((kbase + kBlockN > w.skv) || (p.causal && (kbase + kBlockN - 1 > w.qlo[t])));
        if (needMask) {
          int lim = w.skv - kbase;                         // columns [0, lim) are real keys
          if (p.causal) lim = min(lim, qpos - kbase + 1);  // ... that are not in the future
#pragma unroll
          for (int q = 0; q < 4; q++) {
#pragma unroll
            for (int i = 0; i < 32; i++) {
              if (q * 32 + i >= lim) v[q][i] = 0xff800000u;  // -inf
            }
          }
        }
        // Exponentials of one 32-key quarter: 16 pairs -> 16 packed 16-bit words, plus their (unrounded) sum.
        const float2 c2 = make_float2(c, c);
        auto expQuarter = [&](const uint32_t(&vq)[32], float negMc, uint32_t(&dst)[16], float2& sum, const int quarter) {
          const float2 negMc2 = make_float2(negMc, negMc);
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float2 x = make_float2(__uint_as_float(vq[i]), __uint_as_float(vq[i + 1]));
            x = ffma2(x, c2, negMc2);
            if (((quarter * 16 + (i >> 1)) % kEmuPeriod) < kEmuCount) {  // compile-time pattern: this pair goes to the FMA pipe
              x = ex2_fma2(x);
            } else {
              x.x = ex2(x.x);
              x.y = ex2(x.y);
            }
            sum = fadd2(sum, x);
            dst[i >> 1] = pack2<kBf16>(x.x, x.y);
          }
        };
        uint32_t pkA[16], pkB[16];

        // row max: four independent chains of 3-input max
        float mx4[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
          mx4[q] = fmax2(__uint_as_float(v[q][0]), __uint_as_float(v[q][1]));
#pragma unroll
          for (int i = 2; i < 32; i += 2) mx4[q] = fmax3(mx4[q], __uint_as_float(v[q][i]), __uint_as_float(v[q][i + 1]));
        }
        const float mx = fmax2(fmax2(mx4[0], mx4[1]), fmax2(mx4[2], mx4[3]));  // NaN if any score of the row is
        // Lazy rescale: keep the old reference max while the new one exceeds it by less than kRescaleLog2 in
        // the exp2 domain (P then grows up to 2^kRescaleLog2, harmless in fp32 sums and 16-bit P); the
        // result is unchanged because O and the row sum stay relative to the same reference value.
        float mNew = fmaxf(m, mx);
        const bool grow = (m != -INFINITY) && ((mNew - m) * c > kRescaleLog2);
        if (__any_sync(0xffffffffu, grow)) {
          // Rare: some row of this warp moves its reference max.  Rescale that row's O in tensor memory (rows
          // that keep their max multiply by 1) once the previous P.V has landed; P.V of this block waits for
          // the P0 arrival below, so it sees the rescaled accumulator.  (A parity wait is only meaningful for the
          // phase in progress or the one just completed: P.V of block it-2 finished before S of this block was
          // produced, and P.V of this block cannot start before this warp arrives.)
          const float scale = grow ? ex2((m - mNew) * c) : 1.f;
          if constexpr (kRingSig) {  // V of block j - 1 is load 2 j of the item (j >= 1 here: block 0 never rescales)
            const int g = ldItem + 2 * j;
            wait_bar(bar(kBarKvEmpty + g % NS), (g / NS) & 1, wc, 5);
          } else {
            wait_bar(bar(kBarPvDone + 2 * t + (C::kTwoPos ? ((it - 1) & 1) : 0)),
                     (C::kTwoPos ? ((it - 1) >> 1) : (it - 1)) & 1, wc, 5);
          }
          ptx::tc_fence_after();
          const uint32_t tO = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(C::kOCol0 + t * HDP);
#pragma unroll 1
          for (int ch = 0; ch < kHD / 16; ch++) {  // 16 columns at a time: the scores of this block stay in registers
            uint32_t o[16];
            ptx::tmem_ld_32x32b_x16(tO + ch * 16, o);
            ptx::tmem_wait_ld();
            ptx::tmem_ld_fence(o);
#pragma unroll
            for (int i = 0; i < 16; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * scale);
            ptx::tmem_st_32x32b_x16(tO + ch * 16, o);
          }
          ptx::tmem_wait_st();
          l *= scale;
        }
        if (m != -INFINITY && !grow) mNew = m;
        const float mUse = (mNew == -INFINITY) ? 0.f : mNew;
        m = mNew;

        // A NaN score makes every exponential of the row NaN (the pairs evaluated on the FMA pipe clamp their
        // argument and would turn a NaN of their own into 0), hence the row sum and the output row.
        const float negMc = (mx != mx) ? mx : -mUse * c;
        float2 sum2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int half = 0; half < 2; half++) {
          if (half == 0) {
            expQuarter(v[0], negMc, pkA, sum2, 0);
            expQuarter(v[1], negMc, pkB, sum2, 1);
          } else {
            expQuarter(v[2], negMc, pkA, sum2, 2);
            expQuarter(v[3], negMc, pkB, sum2, 3);
          }
          ptx::tmem_st_32x32b_x16(tP + half * 32, pkA);
          ptx::tmem_st_32x32b_x16(tP + half * 32 + 16, pkB);
          ptx::tmem_wait_st();
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if constexpr (kPair) {  // the issuing thread of rank 0 waits for both CTAs' halves of the 256-row P
              ptx::mbar_arrive_cluster(bar0((half == 0 ? kBarP0Ready : kBarP1Ready) + 2 * t + pSlot));
            } else {
              ptx::mbar_arrive(bar((half == 0 ? kBarP0Ready : kBarP1Ready) + 2 * t + pSlot));
            }
          }
        }
        l += sum2.x + sum2.y;
      }
      if constexpr (kSolo) {
        // This warp is also the epilogue of its 32 rows: wait for the last P.V of the item, read O, release the
        // accumulator to the next item, normalise, convert and store.  Meanwhile the SM's other CTA keeps computing.
        const int gLast = ldItem + 2 * w.nmax - 1;  // the item's last load is V of its last block
        wait_bar(bar(kBarKvEmpty + gLast % NS), (gLast / NS) & 1, wc, 7);
        ptx::tc_fence_after();
        const float inv = (l > 0.f) ? (1.f / l) : 0.f;
        const int gp = 1 << p.packShift;
        const int head = (w.unit << p.packShift) + (r & (gp - 1));
        const bool valid = qpos < w.sq;
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.O) +
                                              ((w.qRow0 + qpos) * p.headsQ + head) * (long long)p.headDim);
        const uint32_t tO = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(C::kOCol0 + t * HDP);
#pragma unroll
        for (int ch = 0; ch < kHD / 32; ch++) {
          uint32_t o[32];
          ptx::tmem_ld_32x32b_x32(tO + ch * 32, o);
          ptx::tmem_wait_ld();
          ptx::tmem_ld_fence(o);
          if (ch == kHD / 32 - 1) {
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar(kBarOFree + t));
          }
          if (valid && ch * 32 < p.headDim) {
#pragma unroll
            for (int g = 0; g < 4; g++) {
              uint4 q;
              q.x = pack2<kBf16>(__uint_as_float(o[g * 8 + 0]) * inv, __uint_as_float(o[g * 8 + 1]) * inv);
              q.y = pack2<kBf16>(__uint_as_float(o[g * 8 + 2]) * inv, __uint_as_float(o[g * 8 + 3]) * inv);
              q.z = pack2<kBf16>(__uint_as_float(o[g * 8 + 4]) * inv, __uint_as_float(o[g * 8 + 5]) * inv);
              q.w = pack2<kBf16>(__uint_as_float(o[g * 8 + 6]) * inv, __uint_as_float(o[g * 8 + 7]) * inv);
              dst[ch * 4 + g] = q;
            }
          }
        }
        items++;
        continue;
      }
      // final row sums for the epilogue; the slot is free once the epilogue of the previous item has released O
      if (items > 0) wait_bar(bar(kBarOFree + t), (items - 1) & 1, wc, 3);
      ctl->scale[t][r] = l;
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(bar(kBarScaleFull + t));
      items++;
    }
  } else if (warp < kEpilogueEnd) {
    // ================================================================ epilogue
    ptx::setmaxnreg_dec<kRegsEpilogue>();
    const int r = threadIdx.x & 127;
    const uint32_t laneOff = (uint32_t)((warp & 3) * 32) << 16;
    const int gp = 1 << p.packShift;
    int items[2] = {0, 0};    // work items in which tile t was active
    int pvTotal[2] = {0, 0};  // blocks of tile t issued so far
    int ldBase = 0;           // K/V ring loads of all earlier items
    for (int k = 0;; k++) {
      Work w;
      const int idx = fetchWork(k, w);
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(bar(kBarWorkEmpty + (k & 1)));
      if (idx < 0 || *wc.failed) break;
      if (w.nmax == 0) continue;
      const int gLast = ldBase + 2 * w.nmax - 1;  // the item's last load: V of its last block
      ldBase += 2 * w.nmax;
      (void)gLast;
#pragma unroll
      for (int t = 0; t < NT; t++) {
        const int n = w.nblk[t];
        if (n == 0) continue;
        pvTotal[t] += n;
        wait_bar(bar(kBarScaleFull + t), items[t] & 1, wc, 6);
        const float l = ctl->scale[t][r];
        // Last P.V of the item.  Valid as a parity wait: the softmax published its row sums after storing the
        // last P, i.e. after all earlier P.V of the tile, and the next item's P.V waits for kBarOFree below.
        // (with two S positions P.V of block X-1 may still be running at this point: its barrier is the other one)
        const int lastBlk = pvTotal[t] - 1;
        if constexpr (kRingSig) {
          wait_bar(bar(kBarKvEmpty + gLast % NS), (gLast / NS) & 1, wc, 7);
        } else {
          wait_bar(bar(kBarPvDone + 2 * t + (C::kTwoPos ? (lastBlk & 1) : 0)), (C::kTwoPos ? (lastBlk >> 1) : lastBlk) & 1, wc, 7);
        }
        ptx::tc_fence_after();
        const float inv = (l > 0.f) ? (1.f / l) : 0.f;
        const int qpos = w.qlo[t] + (r >> p.packShift);
        const int head = (w.unit << p.packShift) + (r & (gp - 1));
        const bool valid = qpos < w.sq;
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.O) +
                                              ((w.qRow0 + qpos) * p.headsQ + head) * (long long)p.headDim);
        const uint32_t tO = tmem + laneOff + (uint32_t)(C::kOCol0 + t * HDP);
#pragma unroll
        for (int ch = 0; ch < kHD / 32; ch++) {
          uint32_t o[32];
          ptx::tmem_ld_32x32b_x32(tO + ch * 32, o);
          ptx::tmem_wait_ld();
          ptx::tmem_ld_fence(o);
          if (ch == kHD / 32 - 1) {  // O is in registers: the next item's first P.V may overwrite the accumulator
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              ptx::mbar_arrive(bar(kBarOFree + t));
              if constexpr (kPair) ptx::mbar_arrive_cluster(bar0(kBarOFreePair));
            }
          }
          const int hdOff = o_chunk_offset<HDP, kPair>(ch);  // a constant once the loop is unrolled
          if (valid && hdOff < p.headDim) {
#pragma unroll
            for (int g = 0; g < 4; g++) {
              uint4 q;
              q.x = pack2<kBf16>(__uint_as_float(o[g * 8 + 0]) * inv, __uint_as_float(o[g * 8 + 1]) * inv);
              q.y = pack2<kBf16>(__uint_as_float(o[g * 8 + 2]) * inv, __uint_as_float(o[g * 8 + 3]) * inv);
              q.z = pack2<kBf16>(__uint_as_float(o[g * 8 + 4]) * inv, __uint_as_float(o[g * 8 + 5]) * inv);
              q.w = pack2<kBf16>(__uint_as_float(o[g * 8 + 6]) * inv, __uint_as_float(o[g * 8 + 7]) * inv);
              dst[hdOff / 8 + g] = q;
            }
          }
        }
        items[t]++;
      }
    }
  } else {
    ptx::setmaxnreg_dec<kRegsIssue>();
    if ((warp == kIssueWarpA || warp == kIssueWarpB) && lane == 0) {
      // ============================================================== MMA issue
      const int fmt = kBf16 ? 1 : 0;
      // pair form: M = 256 over the two CTAs
      const uint32_t idQK = ptx::instr_desc_f16(fmt, kPair ? 2 * kBlockM : kBlockM, kBlockN, 0, 0);
      const uint32_t idPV = ptx::instr_desc_f16(fmt, kPair ? 2 * kBlockM : kBlockM, kHD, 0, 1);
      // K-major operands (Q, K): rows of 128 bytes, 8-row groups 1024 bytes apart.
      const uint64_t descK = ptx::smem_desc_sw128(16, 1024);
      // MN-major operand (V, head dim contiguous): 64-wide slabs kTileBytes/kSub apart, 8-key groups 1024 bytes apart.
      const uint64_t descV = ptx::smem_desc_sw128(kSubTileBytes, 1024);
      const uint32_t kHi = (uint32_t)(descK >> 32), vHi = (uint32_t)(descV >> 32);
      const uint32_t kLoT = (uint32_t)descK, vLoT = (uint32_t)descV;  // LBO field; start address added below
      // Issue helpers.  The tensor pipe overlaps at most one MMA with the issuing thread's next instructions, so
      // everything between two tcgen05.mma costs tensor time: per MMA there is one 32-bit add on a descriptor word.
      const int t = (warp != kIssueWarpA) ? 1 : 0;
      const uint32_t qLo0 = kLoT | ((sQ + (uint32_t)t * C::kQBufs * C::kTileBytes) >> 4);
      uint32_t qLo = qLo0;  // Q buffer of the current item
      const uint32_t dRegion = tmem + (uint32_t)(t * C::kSRegion);
      const uint32_t dO = tmem + (uint32_t)(C::kOCol0 + t * HDP);
      auto issueQK = [&](int blk, uint32_t kAddr, int part) {  // part 0 / 1: first / second half of the k-steps
        const uint32_t kLo = kLoT | (kAddr >> 4);
        const uint32_t dS = dRegion + (uint32_t)((blk & 1) * C::kSPosStride);
#pragma unroll
        for (int k2 = 0; k2 < kHD / 32; k2++) {
          const int kk = part * (kHD / 32) + k2;
          const uint32_t off = (uint32_t)((kk >> 2) * kSubTileBytes + (kk & 3) * 32) >> 4;
          if constexpr (kPair) {  // this CTA's K slabs hold 64 keys: half the slab stride
            const uint32_t offB = (uint32_t)((kk >> 2) * (kSubTileBytes / 2) + (kk & 3) * 32) >> 4;
            ptx::mma_ss_lohi_pair(dS, qLo + off, kHi, kLo + offB, kHi, idQK, kk > 0 ? 1u : 0u);
          } else {
            ptx::mma_ss_lohi(dS, qLo + off, kHi, kLo + off, kHi, idQK, kk > 0 ? 1u : 0u);
          }
        }
      };
      // completion of everything issued so far -> barrier (pair form: the same barrier in both CTAs)
      auto commit = [&](uint32_t b) {
        if constexpr (kPair) {
          ptx::tc_commit_pair(b, 3);
        } else {
          ptx::tc_commit(b);
        }
      };
      auto issuePV = [&](int blk, uint32_t vAddr, uint32_t firstAcc, int half) {  // firstAcc: accumulate flag of k-step 0
        const uint32_t vLo = vLoT | (vAddr >> 4);
        const uint32_t aP = dRegion + (uint32_t)((blk & 1) * C::kPPosStride);
#pragma unroll
        for (int k4 = 0; k4 < kBlockN / 32; k4++) {
          const int kk = half * (kBlockN / 32) + k4;
          if constexpr (kPair) {
            ptx::mma_ts_lohi_pair(dO, aP + kk * 8, vLo + ((kk * 2048) >> 4), vHi, idPV, kk == 0 ? firstAcc : 1u);
          } else {
            ptx::mma_ts_lohi(dO, aP + kk * 8, vLo + ((kk * 2048) >> 4), vHi, idPV, kk == 0 ? firstAcc : 1u);
          }
        }
      };

      // One issuing thread per Q tile (warp 12: tile 0, warp kIssuerB: tile 1).  Every wait and commit costs the
      // issuing thread ~100 clocks during which it feeds nothing to the tensor pipe; with two issuers the other
      // tile's MMAs fill those gaps.  Both threads walk the same ring of K/V loads; a stage is free again after two
      // arrivals: a tcgen05.commit from each tile that used the block, and for a tile that did not use it (causal:
      // the last block belongs to tile 1 alone; one-tile head dims: tile 1 never) one from the loader when it issues
      // the load.  A thread therefore never waits for a block it does not need, and the loader's arrival cannot be
      // counted for the stage's previous use because the loader has waited for that phase before re-using the stage.
      auto release = [&](int stage, bool used) {
        if (used) commit(bar(kBarKvEmpty + stage));
      };
      // The two issuers take strict turns (A: tile 0, B: tile 1, A, B, ...), which keeps the two tiles in
      // anti-phase: one tile's softmax runs while the other tile's MMAs run.  Without the turn token the two
      // tiles drift into lock-step and share both the MUFU and the tensor pipe at the same time.  Turn g of A
      // needs turn g-1 of B, turn g of B needs turn g of A; a thread does its data waits before asking for the
      // token and releases ring stages after passing it on, so those latencies overlap the other thread's issue.
      const uint32_t myTurn = bar(kBarTurn + t), otherTurn = bar(kBarTurn + (t ^ 1));
      int turn = 0;  // turns taken so far by this thread (same count on both threads)
      int ld = 0;    // KV-ring loads consumed so far (K0 V0 K1 V1 ... of every item)
      int it = 0;    // blocks of this tile issued so far
      int qc = 0;    // work items in which this tile was active
      for (int k = 0;; k++) {
        Work w;
        const int idx = fetchWork(k, w);
        ptx::mbar_arrive(bar(kBarWorkEmpty + (k & 1)));
        if (idx < 0 || *wc.failed) break;
        if (w.nmax == 0) continue;
        // pair form: rank 1 issues nothing (its loop only keeps the work slots and counters moving)
        const int n = (t < NT && !(kPair && rank != 0)) ? w.nblk[t] : 0;
        qLo = qLo0 + (uint32_t)((qc % C::kQBufs) * (C::kTileBytes >> 4));
        const bool dual = (NT == 2) && !C::kTwoPos && w.nblk[0] > 0 && w.nblk[1] > 0;
        // The token covers the blocks both tiles have.  Past those (causal: tile 1 has one block more) the thread
        // that still has work runs free and the other one moves on to the next item, whose first Q.K^T and softmax
        // then overlap the last, unpaired block of this one instead of waiting behind it.
        const int nTok = dual ? min(w.nblk[0], w.nblk[1]) : 0;
        // The first Q.K^T of an item is issued without the token: tile 0 then starts the next item while tile 1 is
        // still in the last block of this one, which also re-creates the phase offset between the tiles.
        bool tok = false;
        auto takeTurn = [&]() {
          if (!tok) return;
          if (t == 0) {
            if (turn > 0) spin_bar(myTurn, (turn - 1) & 1, wc, 16);
          } else {
            spin_bar(myTurn, turn & 1, wc, 17);
          }
        };
        auto passTurn = [&]() {
          if (tok) {
            ptx::mbar_arrive(otherTurn);
            turn++;
          }
        };
        {
          const int s0 = ld % NS;
          const uint32_t ph0 = (ld / NS) & 1;
          if (n > 0) {
            wait_bar(bar(kBarKvFull + s0), ph0, wc, 8);
            wait_bar(bar(kBarQFull + 2 * t + (qc % C::kQBufs)), (qc / C::kQBufs) & 1, wc, 9);
            ptx::tc_fence_after();
          }
          takeTurn();
          if (n > 0) {
            issueQK(it, sKV + s0 * C::kStageBytes, 0);
            issueQK(it, sKV + s0 * C::kStageBytes, 1);
            if constexpr (kRingSig) {
              release(s0, true);  // doubles as "S of block 0 is ready"
            } else {
              commit(bar(kBarSFull + 2 * t + (C::kTwoPos ? (it & 1) : 0)));
            }
            if (n == 1) commit(bar(kBarQEmpty + 2 * t + (qc % C::kQBufs)));  // Q tile no longer needed
          }
          passTurn();
          if constexpr (!kRingSig) release(s0, n > 0);
          ld++;
        }
        for (int j = 0; j < w.nmax; j++) {
          const bool hasNext = (j + 1 < w.nmax);
          // Ring order follows consumption order.  One S position: K0 | V0 K1 | V1 K2 | ...  Two S positions (the
          // next scores are issued before P.V): K0 | K1 V0 | K2 V1 | ...
          int sV, sK;
          uint32_t phV, phK;
          if constexpr (C::kTwoPos) {
            sK = ld % NS;
            phK = (ld / NS) & 1;
            if (hasNext) ld++;
            sV = ld % NS;
            phV = (ld / NS) & 1;
            ld++;
          } else {
            sV = ld % NS;
            phV = (ld / NS) & 1;
            ld++;
            sK = ld % NS;
            phK = (ld / NS) & 1;
          }
          const int blk = it + j;  // running index of block j of this tile
          tok = (j < nTok);
          if constexpr (C::kTwoPos) {
            // two S positions: the next scores first (rotating S: they wait for the softmax to have read the
            // current ones, whose columns they partly overwrite; two full buffers: the target buffer was last
            // read by P.V of block j-1, issued earlier by this thread), then P.V of the current block
            if (j + 1 < n) {
              wait_bar(bar(kBarKvFull + sK), phK, wc, 12);
              if constexpr (C::kRot) wait_bar(bar(kBarSFree + t), blk & 1, wc, 18);
              ptx::tc_fence_after();
              issueQK(blk + 1, sKV + sK * C::kStageBytes, 0);
              issueQK(blk + 1, sKV + sK * C::kStageBytes, 1);
              if constexpr (kRingSig) {
                release(sK, true);  // the stage is free when these MMAs finish, which is when S of block j + 1 is ready
              } else {
                commit(bar(kBarSFull + 2 * t + ((blk + 1) & 1)));
              }
              if (j + 2 == n) commit(bar(kBarQEmpty + 2 * t + (qc % C::kQBufs)));
            }
            if (j < n) {
              wait_bar(bar(kBarKvFull + sV), phV, wc, 10);
              if (j == 0 && qc > 0) wait_bar(bar(kPair ? kBarOFreePair : kBarOFree + t), (qc - 1) & 1, wc, 19);
              wait_bar(bar(kBarP0Ready + 2 * t + (blk & 1)), (blk >> 1) & 1, wc, 11);
              ptx::tc_fence_after();
              issuePV(blk, sKV + sV * C::kStageBytes, j == 0 ? 0u : 1u, 0);
              wait_bar(bar(kBarP1Ready + 2 * t + (blk & 1)), (blk >> 1) & 1, wc, 15);
              ptx::tc_fence_after();
              issuePV(blk, sKV + sV * C::kStageBytes, 1u, 1);
              if constexpr (kRingSig) {
                release(sV, true);  // ... and likewise "O += P.V of block j has finished"
              } else {
                commit(bar(kBarPvDone + 2 * t + (blk & 1)));
              }
            }
            if constexpr (!kRingSig) {
              if (hasNext) release(sK, j + 1 < n);
              release(sV, j < n);
            }
            continue;
          }
          bool p1Ready = false;
          if (j < n) {
            wait_bar(bar(kBarKvFull + sV), phV, wc, 10);
            if (j + 1 < n) wait_bar(bar(kBarKvFull + sK), phK, wc, 12);
            if (j == 0 && qc > 0) wait_bar(bar(kBarOFree + t), (qc - 1) & 1, wc, 19);
            spin_bar(bar(kBarP0Ready + 2 * t), blk & 1, wc, 11);
            p1Ready = ptx::mbar_test_wait(bar(kBarP1Ready + 2 * t), blk & 1);
          }
          takeTurn();
          // The token is passed on while a few MMAs of this turn are still to be issued: the other thread needs
          // ~150 clocks to see it, and its first MMAs then queue behind the rest of this turn instead of finding
          // the tensor pipe idle.  MMAs of the two tiles touch disjoint tensor memory, so interleaving is harmless.
          if (j < n) {
            ptx::tc_fence_after();
            issuePV(blk, sKV + sV * C::kTileBytes, j == 0 ? 0u : 1u, 0);
            if (!p1Ready) {
              spin_bar(bar(kBarP1Ready + 2 * t), blk & 1, wc, 15);
              ptx::tc_fence_after();
            }
            issuePV(blk, sKV + sV * C::kTileBytes, 1u, 1);
            if (j + 1 < n) {
              issueQK(blk + 1, sKV + sK * C::kTileBytes, 0);
              passTurn();
              issueQK(blk + 1, sKV + sK * C::kTileBytes, 1);
              ptx::tc_commit(bar(kBarSFull + 2 * t));
              if (j + 2 == n) ptx::tc_commit(bar(kBarQEmpty + 2 * t + (qc % C::kQBufs)));
            } else {
              passTurn();
            }
            ptx::tc_commit(bar(kBarPvDone + 2 * t));
          } else {
            passTurn();
          }
          release(sV, j < n);
          if (hasNext) {
            release(sK, j + 1 < n);
            ld++;
          }
        }
        it += n;
        if (n > 0) qc++;
      }
    } else if (warp == kLoadWarp && lane == 0) {
      // ============================================================== work distribution + TMA loads
      const int gp = 1 << p.packShift;
      int ld = 0;            // KV-ring loads issued so far
      int qc[2] = {0, 0};    // Q loads issued so far per tile
      // Takes the next work index, works out its description and publishes both in slot k & 1 (free once every
      // consumer has read item k - 2 from it).  Returns false when the work has run out.
      Work wq[2];
      auto publish = [&](int k) -> bool {
        if (k >= 2) wait_bar(bar(kBarWorkEmpty + (k & 1)), ((k >> 1) - 1) & 1, wc, 21);
        Work& w = wq[k & 1];
        // indices whose tile pair lies past the end of a short sequence (packed variable-length input) are
        // dropped here: nobody else hears of them
        int idx;
        if constexpr (kPair) {
          // A work item is two neighbouring Q tiles (make_work with two tiles per item), one per CTA.  Rank 0 takes
          // the index and hands it over through rank 1's shared memory (a mailbox per slot parity, full / empty
          // barriers); both then work out the same description and keep their own tile of it as tile 0.
          if (rank == 0) {
            do {
              idx = atomicAdd(p.workCounter, 1);
              if (idx >= p.numWork || *reinterpret_cast<volatile int*>(&ctl->failed)) idx = -1;
            } while (idx >= 0 && !make_work<2, kVarlen>(p, idx, w));
            if (k >= 2) wait_bar(bar(kBarIdxEmpty + (k & 1)), ((k >> 1) - 1) & 1, wc, 26);
            ptx::st_cluster_u32(ptx::mapa(ptx::smem_u32(&ctl->peerIdx[k & 1]), 1), (uint32_t)idx);
            ptx::mbar_arrive_cluster_release(barBasePeer + 8u * (uint32_t)(kBarIdxFull + (k & 1)));
          } else {
            wait_bar_cluster(bar(kBarIdxFull + (k & 1)), (k >> 1) & 1, wc, 27);
            idx = *reinterpret_cast<volatile int*>(&ctl->peerIdx[k & 1]);
            if (*reinterpret_cast<volatile int*>(&ctl->failed)) idx = -1;
            ptx::mbar_arrive_cluster(barBasePeer + 8u * (uint32_t)(kBarIdxEmpty + (k & 1)));
            if (idx >= 0) make_work<2, kVarlen>(p, idx, w);
          }
          if (idx >= 0) {
            // Both tiles run every key block of the item in one M = 256 MMA.  A tile whose rows lie past the end of
            // the sequence, or (causal) whose last block is entirely in the future, computes on zero-filled or fully
            // masked scores and stores nothing for them.
            w.qlo[0] = w.qlo[rank];
            w.qhi[0] = w.qhi[rank];
            w.nblk[0] = w.nmax;
            w.nblk[1] = 0;
          }
        } else {
          do {
            idx = atomicAdd(p.workCounter, 1);
            if (idx >= p.numWork || *reinterpret_cast<volatile int*>(&ctl->failed)) idx = -1;
          } while (idx >= 0 && !make_work<NT, kVarlen>(p, idx, w));
        }
        volatile WorkSlot* ws = &ctl->work[k & 1];
        ws->idx = idx;
        ws->sq = w.sq;
        ws->skv = w.skv;
        ws->unit = w.unit;
        ws->qRow0 = w.qRow0;
        ws->qlo[0] = w.qlo[0];
        ws->qlo[1] = w.qlo[1];
        ws->nblk[0] = w.nblk[0];
        ws->nblk[1] = w.nblk[1];
        ws->nmax = w.nmax;
        ptx::mbar_arrive(bar(kBarWorkFull + (k & 1)));  // release: the stores above are visible to whoever waits
        return idx >= 0;
      };
      bool more = publish(0);
      for (int k = 0; more; k++) {
        // Item k + 1 is taken and published two blocks before the end of this item's loads: by then this thread is
        // only waiting for ring stages, and nobody waits for the atomic round trip and the divisions between two
        // items.  (Doing it right after the first loads of the item, when the ring is still filling, cost 6 %.)
        bool nextDone = false;
        const Work& w = wq[k & 1];
        // The Q tiles of this item cannot land in shared memory before the previous item's last Q.K^T has
        // finished; pulling them into L2 now shortens that exposed load at the item boundary.
#pragma unroll
        for (int t = 0; t < NT; t++) {
          if (w.nblk[t] == 0 || qc[t] == 0 || C::kQBufs > 1) continue;
#pragma unroll
          for (int a = 0; a < C::kSub; a++) ptx::tma_prefetch_4d(mapQ, a * 64, w.unit * gp, w.qRowTma + w.qlo[t], w.batchTma);
        }
        auto loadQ = [&](int t) {
          if (t >= NT || w.nblk[t] == 0) return;
          // buffer qc % kQBufs was last used by item qc - kQBufs of this tile
          const int qb = qc[t] % C::kQBufs, qUse = qc[t] / C::kQBufs;  // buffer and how often it was used before
          if (qUse > 0) wait_bar(bar(kBarQEmpty + 2 * t + qb), (qUse - 1) & 1, wc, 22);
          const uint32_t qDst = sQ + (t * C::kQBufs + qb) * C::kTileBytes;
          if constexpr (kPair) {  // rank 0's barrier counts the Q tiles of both CTAs
            if (rank == 0) ptx::mbar_arrive_expect_tx(bar(kBarQFull + 2 * t + qb), 2 * C::kTileBytes);
#pragma unroll
            for (int a = 0; a < C::kSub; a++) {
              ptx::tma_load_4d_pair(qDst + a * kSubTileBytes, mapQ, bar0(kBarQFull + 2 * t + qb), a * 64, w.unit * gp,
                                    w.qRowTma + w.qlo[t], w.batchTma);
            }
          } else {
            ptx::mbar_arrive_expect_tx(bar(kBarQFull + 2 * t + qb), C::kTileBytes);
#pragma unroll
            for (int a = 0; a < C::kSub; a++) {
              ptx::tma_load_4d(qDst + a * kSubTileBytes, mapQ, bar(kBarQFull + 2 * t + qb), a * 64, w.unit * gp,
                               w.qRowTma + w.qlo[t], w.batchTma);
            }
          }
          qc[t]++;
        };
        // Order: Q of tile 0, the first K block, Q of tile 1, everything else.  Tile 0 finishes an item first (causal:
        // one block earlier), so its Q buffer is free while tile 1 still computes; its first Q.K^T of this item then
        // needs only these two loads and overlaps the end of the previous item.
        loadQ(0);
        const int numLoads = 2 * w.nmax;
        for (int i = 0; i < numLoads; i++, ld++) {
          if (i == 1) loadQ(1);
          if (i == numLoads - 4 && !nextDone) {
            more = publish(k + 1);
            nextDone = true;
          }
          const int s = ld % NS;
          if (ld >= NS) wait_bar(bar(kBarKvEmpty + s), ((ld / NS) - 1) & 1, wc, 14);
          if constexpr (!kPair) ptx::mbar_arrive_expect_tx(bar(kBarKvFull + s), C::kTileBytes);
          bool isV;
          int blkIdx;
          if constexpr (C::kTwoPos) {  // K0 | K1 V0 | K2 V1 | ... | V(last)
            if (i == 0) {
              isV = false;
              blkIdx = 0;
            } else if (i == numLoads - 1) {
              isV = true;
              blkIdx = w.nmax - 1;
            } else {
              isV = (i & 1) == 0;
              blkIdx = isV ? (i - 2) / 2 : (i + 1) / 2;
            }
          } else {  // K0 | V0 K1 | V1 K2 | ...
            isV = (i & 1) != 0;
            blkIdx = i >> 1;
          }
          const CUtensorMap* tm = isV ? mapV : mapK;
          const int row = w.kvRowTma + blkIdx * kBlockN;
          if constexpr (kPair) {
            // This CTA's half of the block, counted on rank 0's barrier together with the other half.
            // K: keys [64 rank, 64 rank + 64), all of the head dim (the K map's box is 64 rows high);
            // V: all 128 keys, two 64-wide slabs of the head dim (v_slab_offset).
            const uint32_t dst = sKV + s * C::kStageBytes;
            if (isV) {
              if (rank == 0) ptx::mbar_arrive_expect_tx(bar(kBarKvFull + s), 2 * 2 * kSubTileBytes);
#pragma unroll
              for (int a = 0; a < 2; a++) {
                ptx::tma_load_4d_pair(dst + a * kSubTileBytes, tm, bar0(kBarKvFull + s), v_slab_offset<HDP>((int)rank, a), w.hkv,
                                      row, w.batchTma);
              }
            } else {
              if (rank == 0) ptx::mbar_arrive_expect_tx(bar(kBarKvFull + s), C::kTileBytes);
#pragma unroll
              for (int a = 0; a < C::kSub; a++) {
                ptx::tma_load_4d_pair(dst + a * (kSubTileBytes / 2), tm, bar0(kBarKvFull + s), a * 64, w.hkv,
                                      row + (int)rank * (kBlockN / 2), w.batchTma);
              }
            }
          } else {
#pragma unroll
            for (int a = 0; a < C::kSub; a++) {
              ptx::tma_load_4d(sKV + s * C::kTileBytes + a * kSubTileBytes, tm, bar(kBarKvFull + s), a * 64, w.hkv, row,
                               w.batchTma);
            }
          }
          // the stage-free arrival of every tile that will not touch this block
#pragma unroll
          for (int t = 0; t < 2; t++) {
            if (t >= NT || blkIdx >= w.nblk[t]) ptx::mbar_arrive(bar(kBarKvEmpty + s));
          }
        }
        if (!nextDone) more = publish(k + 1);
      }
    } else if (kVarlen && warp == kHelpWarp) {
      // ============================================================== packed input: V rows past a sequence's end
      int ldBase = 0;         // K/V ring loads of all earlier items
      int cnt[2] = {0, 0};    // blocks of tile t so far, over all items (phase of its P-ready barriers)
      for (int k = 0;; k++) {
        Work w;
        const int idx = fetchWork(k, w);
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(bar(kBarWorkEmpty + (k & 1)));
        if (idx < 0 || *wc.failed) break;
        if (w.nmax == 0) continue;
        const int ldv = ldBase + 2 * w.nmax - 1;  // the item's last load is V of its last block
        ldBase += 2 * w.nmax;
        const int nTotal = (w.skv + kBlockN - 1) / kBlockN;
        const int tail = w.skv - (nTotal - 1) * kBlockN;  // keys of the sequence in its last block
        for (int j = 0; j < w.nmax; j++) {
          if (j == nTotal - 1 && tail < kBlockN) {  // some tile of this item reaches the ragged last block
            // First wait until the scores of this block exist for a tile that has it: K of the block has then been
            // consumed, so the ring is at most one use of V's stage behind and the parity wait below asks for the phase
            // in progress or the one just completed.  (Straight after the previous block's barrier the ring may be two
            // uses behind, and a parity wait for a phase two ahead returns at once.)
            const int tz = (j < w.nblk[0]) ? 0 : 1;
            if constexpr (kRingSig) {
              const int g = (ldv - (2 * w.nmax - 1)) + (j == 0 ? 0 : 2 * j - 1);
              wait_bar(bar(kBarKvEmpty + g % NS), (g / NS) & 1, wc, 24);
            } else {
              wait_bar(bar(kBarSFull + 2 * tz + (C::kTwoPos ? (cnt[tz] & 1) : 0)), (C::kTwoPos ? (cnt[tz] >> 1) : cnt[tz]) & 1, wc, 24);
            }
            wait_bar(bar(kBarKvFull + ldv % NS), (ldv / NS) & 1, wc, 25);
            zero_v_tail<C::kSub>(sKV + (uint32_t)((ldv % NS) * C::kStageBytes), lane, tail);
          }
          // one arrival per tile and block, then wait for the phase to complete before the next arrival on the same
          // barrier: two arrivals of this warp must never fall into one phase
#pragma unroll
          for (int t = 0; t < NT; t++) {
            if (j < w.nblk[t] && lane == 0) ptx::mbar_arrive(bar(kBarP0Ready + 2 * t + (C::kTwoPos ? (cnt[t] & 1) : 0)));
          }
#pragma unroll
          for (int t = 0; t < NT; t++) {
            if (j < w.nblk[t]) {
              wait_bar(bar(kBarP0Ready + 2 * t + (C::kTwoPos ? (cnt[t] & 1) : 0)), (C::kTwoPos ? (cnt[t] >> 1) : cnt[t]) & 1, wc, 31);
              cnt[t]++;
            }
          }
        }
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) {
    // The last CTA to get here puts both counters back to zero for the next launch that uses them.  Every CTA's
    // fetches from the work counter precede its arrival on the done counter (same CTA, separated by the barrier above).
    __threadfence();
    if (atomicAdd(p.workCounter + 1, 1) == (int)gridDim.x - 1) {
      // Every CTA stops at its first index past the end, so the work counter must now read numWork + gridDim.x.
      // Anything else means another launch used the same counters at the same time (the host hands out a pair per
      // stream and per captured launch precisely to rule that out): report it rather than return a result with rows
      // that nobody computed.
      const int taken = *reinterpret_cast<volatile int*>(p.workCounter);
      const int takers = kPair ? (int)gridDim.x / 2 : (int)gridDim.x;  // pair form: rank 0 of each pair takes indices
      if (taken != p.numWork + takers && *wc.failed == 0) atomicExch(p.status, (p.epoch << 8) | 30);
      p.workCounter[0] = 0;
      p.workCounter[1] = 0;
    }
  }
  // pair form: neither CTA leaves (or frees tensor memory) while the other may still reach into its shared memory
  // or have MMAs of the pair in flight
  if constexpr (kPair) ptx::cluster_sync();
  if (warp == kIssueWarpA) {
    if (*wc.failed) __nanosleep(200000);  // a wait gave up: let whatever is still in flight drain before freeing
    ptx::tc_fence_after();
    if constexpr (kPair) {
      ptx::tmem_dealloc_pair(tmem, C::kTmemCols);
    } else {
      ptx::tmem_dealloc(tmem, C::kTmemCols);
    }
  }
}

}  // namespace tc
}  // namespace tfa_b200

// Split-KV attention forward for short query blocks (decode shapes), fp16 / bf16, sm_100a.
//
// The reference has no such path: with seqQ = 1 its grid is one CTA per (batch, Q head) walking every KV tile and
// every Q head of a GQA group re-reads the same K/V (reference csrc/flash_attn/launcher.cuh:32,
// params.cuh:25-27).  This path is bound by HBM bandwidth - K and V are read exactly once - so it is organised
// around memory parallelism, not around the tcgen05 pipe:
//   * the (seqQ x group) query rows that share one KV head (at most 16) form one 16-row MMA tile, so a KV head is
//     streamed once for all of its Q heads;
//   * the key range is split over gridDim.x CTAs so that B x Hkv x splits fills the 148 SMs several times;
//   * each CTA streams 64-key K and V blocks through a 3-stage cp.async ring (16-byte chunks, XOR-swizzled so that
//     ldmatrix is conflict-free); each of its 4 warps owns 16 keys of a block with its own online softmax
//     (mma.sync m16n8k16, fp32 accumulate: the tensor work is negligible next to the memory stream);
//   * warps are merged through shared memory, splits through a small fp32 scratch buffer and a combine kernel.
// Numerical contract as in the main kernel (reference csrc/flash_attn/mma/softmax.cuh:67-138): scale 1/sqrt(D)
// folded into exp2, top-left causal mask, "col >= seqLenKV" mask, P rounded to the 16-bit type before P.V, row sum
// from unrounded P, empty rows give 0.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>

#include <mutex>

#include "../../include/tinyfa_b200.h"
#include "build_config.cuh"
#include "tfa_common.cuh"

namespace tfa_b200 {
namespace decode {

constexpr int kThreads = 128;
constexpr int kBlockKeys = 64;
constexpr int kStages = 3;
constexpr int kRows = 16;  // query rows per CTA (MMA M)

struct Params {
  const void* Q;
  const void* K;
  const void* V;
  void* O;          // final output (16-bit)
  float* partO;     // [splits][totalQRows][Hq][D] normalised partial outputs (splits > 1)
  float* partLse;   // [splits][totalQRows][Hq]   log2-domain log-sum-exp of each partial
  const int* cuQ;
  const int* cuKV;
  int seqLenQ;
  int seqLenKV;
  int headsQ;
  int headsKV;
  int group;
  int causal;
  int splits;
  int keysPerSplit;  // multiple of kBlockKeys
  long long totalQ;  // rows of Q (for the partial buffers' stride)
  float scaleLog2;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
template <bool kBf16>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (kBf16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
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

// Byte offset of 16-byte chunk `c` of row `r` in a tile whose rows hold D 16-bit elements.
// Rows are D * 2 bytes and contiguous, so which banks a row starts on depends on D: for D = 64, 128, 192, 256 every
// row starts on bank 0 and chunk c is exchanged with c ^ (r & 7) (stays inside its group of eight chunks); for D = 32
// and 96 (64- and 192-byte rows) rows alternate between the two halves of the 128-byte bank line and the chunk is
// exchanged inside its group of four, c ^ ((r >> 1) & 3).  Either way the eight rows of an ldmatrix hit eight
// different 16-byte bank groups.
template <int D>
__device__ __forceinline__ uint32_t swz(int r, int c) {
  if constexpr (D == 32 || D == 96) {
    return (uint32_t)(r * (D * 2) + ((c ^ ((r >> 1) & 3)) << 4));
  } else {
    return (uint32_t)(r * (D * 2) + ((c ^ (r & 7)) << 4));
  }
}

// 64 keys x D of one KV head -> one stage; keys >= keyEnd are zero-filled.
template <int D>
__device__ __forceinline__ void load_block(uint32_t smemDst, const uint16_t* base, long long rowStride, long long key0,
                                           long long keyEnd) {
  constexpr int kChunksPerRow = D / 8;
  constexpr int kChunks = kBlockKeys * kChunksPerRow;
#pragma unroll
  for (int i = 0; i < kChunks / kThreads; i++) {
    const int idx = threadIdx.x + i * kThreads;
    const int r = idx / kChunksPerRow, c = idx % kChunksPerRow;
    const bool valid = (key0 + r) < keyEnd;
    const uint16_t* src = base + (valid ? (key0 + r) * rowStride + c * 8 : 0);
    cp_async16(smemDst + swz<D>(r, c), src, valid);
  }
}

template <int D, bool kBf16>
__global__ void __launch_bounds__(kThreads) fwd_splitkv_kernel(const Params p) {
  constexpr int kTileBytes = kBlockKeys * D * 2;
  constexpr int kNT = D / 8;  // 8-wide output column tiles
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sBase = static_cast<uint32_t>(__cvta_generic_to_shared(smem));

  const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  long long qRow0, kvRow0;
  int sq, skv;
  if (p.cuQ != nullptr) {
    qRow0 = p.cuQ[b];
    sq = p.cuQ[b + 1] - p.cuQ[b];
    kvRow0 = p.cuKV[b];
    skv = p.cuKV[b + 1] - p.cuKV[b];
  } else {
    sq = p.seqLenQ;
    skv = p.seqLenKV;
    qRow0 = (long long)b * sq;
    kvRow0 = (long long)b * skv;
  }
  if (sq <= 0) return;
  if (skv <= 0 && p.splits == 1) return;  // nothing to write; with splits > 1 the partials must still be defined
  const int nRows = sq * p.group;  // <= 16 by dispatch
  int keyEnd = skv;
  if (p.causal) keyEnd = min(keyEnd, sq);  // top-left causal: key j needs j <= i <= sq-1
  // keysPerSplit comes from the caller's maximum key length, which only sizes the launch: the last split runs to
  // the real end of the sequence, so an understated maximum loses no keys (the reference derives its key loop from
  // the actual length as well, reference csrc/flash_attn/params.cuh:156-163).
  const int key0 = split * p.keysPerSplit;
  const int key1 = (split == p.splits - 1) ? keyEnd : min(key0 + p.keysPerSplit, keyEnd);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;

  const long long qStride = (long long)p.headsQ * D;
  const long long kvStride = (long long)p.headsKV * D;
  const uint16_t* gK = reinterpret_cast<const uint16_t*>(p.K) + kvRow0 * kvStride + (long long)hkv * D;
  const uint16_t* gV = reinterpret_cast<const uint16_t*>(p.V) + kvRow0 * kvStride + (long long)hkv * D;

  // rows of this thread's fragments: r0 = g, r1 = g + 8; row r <-> (query position r / group, head hkv*group + r % group)
  const int rowA = g, rowB = g + 8;
  const int qposA = rowA / p.group, qposB = rowB / p.group;
  const int headA = hkv * p.group + rowA % p.group, headB = hkv * p.group + rowB % p.group;
  const bool validA = rowA < nRows, validB = rowB < nRows;

  float o[kNT][4];
#pragma unroll
  for (int i = 0; i < kNT; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;

  const int nBlocks = (key1 > key0) ? (key1 - key0 + kBlockKeys - 1) / kBlockKeys : 0;
  if (nBlocks > 0) {
    // Q fragments (A operand), loaded once straight from global memory.
    uint32_t qf[D / 16][4];
    {
      const uint16_t* gQ = reinterpret_cast<const uint16_t*>(p.Q);
      const uint16_t* qa = gQ + (qRow0 + qposA) * qStride + (long long)headA * D;
      const uint16_t* qb = gQ + (qRow0 + qposB) * qStride + (long long)headB * D;
#pragma unroll
      for (int ks = 0; ks < D / 16; ks++) {
        const int c0 = ks * 16 + 2 * tig;
        qf[ks][0] = validA ? *reinterpret_cast<const uint32_t*>(qa + c0) : 0u;
        qf[ks][1] = validB ? *reinterpret_cast<const uint32_t*>(qb + c0) : 0u;
        qf[ks][2] = validA ? *reinterpret_cast<const uint32_t*>(qa + c0 + 8) : 0u;
        qf[ks][3] = validB ? *reinterpret_cast<const uint32_t*>(qb + c0 + 8) : 0u;
      }
    }
    const float c = p.scaleLog2;

#pragma unroll
    for (int s = 0; s < kStages - 1; s++) {
      if (s < nBlocks) {
        load_block<D>(sBase + s * 2 * kTileBytes, gK, kvStride, key0 + s * kBlockKeys, key1);
        load_block<D>(sBase + s * 2 * kTileBytes + kTileBytes, gV, kvStride, key0 + s * kBlockKeys, key1);
      }
      cp_async_commit();
    }
    for (int blk = 0; blk < nBlocks; blk++) {
      {
        const int nb = blk + kStages - 1;
        if (nb < nBlocks) {
          const int s = nb % kStages;
          load_block<D>(sBase + s * 2 * kTileBytes, gK, kvStride, key0 + nb * kBlockKeys, key1);
          load_block<D>(sBase + s * 2 * kTileBytes + kTileBytes, gV, kvStride, key0 + nb * kBlockKeys, key1);
        }
        cp_async_commit();
      }
      cp_async_wait<kStages - 1>();
      __syncthreads();
      const uint32_t sK = sBase + (blk % kStages) * 2 * kTileBytes;
      const uint32_t sV = sK + kTileBytes;
      const int kb = key0 + blk * kBlockKeys + warp * 16;  // first key of this warp's 16-key slice
      if (kb < key1) {
        // ---- S = Q K^T for 16 rows x 16 keys
        float sc[2][4];
#pragma unroll
        for (int n = 0; n < 2; n++) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ks++) {
          // matrices: (keys 0-7, dims lo), (keys 0-7, dims hi), (keys 8-15, dims lo), (keys 8-15, dims hi)
          const int r = warp * 16 + (lane & 7) + ((lane >> 4) << 3);
          const int ch = ks * 2 + ((lane >> 3) & 1);
          uint32_t kf[4];
          ldmatrix_x4(sK + swz<D>(r, ch), kf);
          mma16816<kBf16>(sc[0], qf[ks], kf[0], kf[1]);
          mma16816<kBf16>(sc[1], qf[ks], kf[2], kf[3]);
        }
        // ---- mask (tail of the key range, top-left causal)
        const bool needMask = (kb + 16 > key1) || p.causal;
        if (needMask) {
#pragma unroll
          for (int n = 0; n < 2; n++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
              const int key = kb + n * 8 + 2 * tig + (e & 1);
              const int qpos = (e < 2) ? qposA : qposB;
              if (key >= key1 || (p.causal && key > qpos)) sc[n][e] = -INFINITY;
            }
          }
        }
        // ---- online softmax for rows g (A) and g+8 (B)
        float mxA = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
        float mxB = fmaxf(fmaxf(sc[0][2], sc[0][3]), fmaxf(sc[1][2], sc[1][3]));
        mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
        mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
        mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
        mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
        const float mnA = fmaxf(mA, mxA), mnB = fmaxf(mB, mxB);
        const float muA = (mnA == -INFINITY) ? 0.f : mnA, muB = (mnB == -INFINITY) ? 0.f : mnB;
        const float scA = (mA == -INFINITY) ? 0.f : ex2((mA - muA) * c);
        const float scB = (mB == -INFINITY) ? 0.f : ex2((mB - muB) * c);
        mA = mnA;
        mB = mnB;
        float pA[4], pB[4];
#pragma unroll
        for (int n = 0; n < 2; n++) {
          pA[n * 2 + 0] = ex2(fmaf(sc[n][0], c, -muA * c));
          pA[n * 2 + 1] = ex2(fmaf(sc[n][1], c, -muA * c));
          pB[n * 2 + 0] = ex2(fmaf(sc[n][2], c, -muB * c));
          pB[n * 2 + 1] = ex2(fmaf(sc[n][3], c, -muB * c));
        }
        lA = lA * scA + (pA[0] + pA[1] + pA[2] + pA[3]);  // per-thread partial, reduced over the quad at the end
        lB = lB * scB + (pB[0] + pB[1] + pB[2] + pB[3]);
        uint32_t pf[4];
        pf[0] = pack2<kBf16>(pA[0], pA[1]);
        pf[1] = pack2<kBf16>(pB[0], pB[1]);
        pf[2] = pack2<kBf16>(pA[2], pA[3]);
        pf[3] = pack2<kBf16>(pB[2], pB[3]);
        // ---- O = O * scale + P V
#pragma unroll
        for (int nt = 0; nt < kNT; nt += 2) {
          // matrices (transposed on load): (keys 0-7, dims nt), (keys 8-15, dims nt), (keys 0-7, dims nt+1), (keys 8-15, dims nt+1)
          const int r = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
          const int ch = nt + (lane >> 4);
          uint32_t vf[4];
          ldmatrix_x4_trans(sV + swz<D>(r, ch), vf);
          o[nt][0] *= scA;
          o[nt][1] *= scA;
          o[nt][2] *= scB;
          o[nt][3] *= scB;
          o[nt + 1][0] *= scA;
          o[nt + 1][1] *= scA;
          o[nt + 1][2] *= scB;
          o[nt + 1][3] *= scB;
          mma16816<kBf16>(o[nt], pf, vf[0], vf[1]);
          mma16816<kBf16>(o[nt + 1], pf, vf[2], vf[3]);
        }
      }
      __syncthreads();
    }
    cp_async_wait<0>();
  }

  // ---- merge the four warps (each saw a disjoint quarter of the keys) through shared memory
  lA += __shfl_xor_sync(0xffffffffu, lA, 1);
  lA += __shfl_xor_sync(0xffffffffu, lA, 2);
  lB += __shfl_xor_sync(0xffffffffu, lB, 1);
  lB += __shfl_xor_sync(0xffffffffu, lB, 2);
  float* sO = reinterpret_cast<float*>(smem);          // [4][16][D]
  float* sM = sO + 4 * kRows * D;                        // [4][16]
  float* sL = sM + 4 * kRows;                            // [4][16]
  __syncthreads();
  if (tig == 0) {
    sM[warp * kRows + rowA] = mA;
    sM[warp * kRows + rowB] = mB;
    sL[warp * kRows + rowA] = lA;
    sL[warp * kRows + rowB] = lB;
  }
#pragma unroll
  for (int nt = 0; nt < kNT; nt++) {
    const int col = nt * 8 + 2 * tig;
    *reinterpret_cast<float2*>(sO + (warp * kRows + rowA) * D + col) = make_float2(o[nt][0], o[nt][1]);
    *reinterpret_cast<float2*>(sO + (warp * kRows + rowB) * D + col) = make_float2(o[nt][2], o[nt][3]);
  }
  __syncthreads();
  const float c = p.scaleLog2;
  for (int idx = threadIdx.x; idx < kRows * (D / 4); idx += kThreads) {
    const int r = idx / (D / 4), c4 = idx % (D / 4);
    if (r >= nRows) continue;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; w++) m = fmaxf(m, sM[w * kRows + r]);
    float l = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < 4; w++) {
      const float mw = sM[w * kRows + r];
      const float f = (mw == -INFINITY) ? 0.f : ex2((mw - m) * c);
      l += sL[w * kRows + r] * f;
      const float4 v = *reinterpret_cast<const float4*>(sO + (w * kRows + r) * D + c4 * 4);
      acc.x += v.x * f;
      acc.y += v.y * f;
      acc.z += v.z * f;
      acc.w += v.w * f;
    }
    const float inv = (l > 0.f) ? (1.f / l) : 0.f;
    acc.x *= inv;
    acc.y *= inv;
    acc.z *= inv;
    acc.w *= inv;
    const int qpos = r / p.group, head = hkv * p.group + r % p.group;
    const long long orow = (qRow0 + qpos) * p.headsQ + head;
    if (p.splits == 1) {
      uint2 out;
      out.x = pack2<kBf16>(acc.x, acc.y);
      out.y = pack2<kBf16>(acc.z, acc.w);
      *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(p.O) + orow * D + c4 * 4) = out;
    } else {
      const long long prow = (long long)split * p.totalQ * p.headsQ + orow;
      *reinterpret_cast<float4*>(p.partO + prow * D + c4 * 4) = acc;
      if (c4 == 0) p.partLse[prow] = (l > 0.f) ? (m * c + log2f(l)) : -INFINITY;
    }
  }
}

// O[row] = sum_s 2^(lse_s - M) O_s / sum_s 2^(lse_s - M); one thread per 4 output elements.
template <int D, bool kBf16>
__global__ void combine_kernel(const float* __restrict__ partO, const float* __restrict__ partLse, void* O,
                               long long rows /* totalQ * Hq */, int splits, const int* cuQ, const int* cuKV, int batch,
                               int headsQ) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * (D / 4)) return;
  const long long row = idx / (D / 4);
  const int c4 = (int)(idx % (D / 4));
  // packed input: rows past the last sequence (a Q tensor longer than cu_seqlens_q[batch]) have no partials
  if (cuQ != nullptr && row / headsQ >= cuQ[batch]) return;
  float M = -INFINITY;
  for (int s = 0; s < splits; s++) M = fmaxf(M, partLse[(long long)s * rows + row]);
  if (M == -INFINITY) return;  // no keys at all for this row: leave O untouched
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float wsum = 0.f;
  for (int s = 0; s < splits; s++) {
    const float lse = partLse[(long long)s * rows + row];
    if (lse == -INFINITY) continue;
    const float w = exp2f(lse - M);
    const float4 v = *reinterpret_cast<const float4*>(partO + ((long long)s * rows + row) * D + c4 * 4);
    acc.x += w * v.x;
    acc.y += w * v.y;
    acc.z += w * v.z;
    acc.w += w * v.w;
    wsum += w;
  }
  const float inv = 1.f / wsum;
  uint2 out;
  out.x = pack2<kBf16>(acc.x * inv, acc.y * inv);
  out.y = pack2<kBf16>(acc.z * inv, acc.w * inv);
  *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(O) + row * D + c4 * 4) = out;
  (void)cuKV;
}

template <int D, bool kBf16>
int launch(const FwdProblem& pr, int splits, float* partO, float* partLse) {
  constexpr int kTileBytes = kBlockKeys * D * 2;
  constexpr int kPipeBytes = kStages * 2 * kTileBytes;
  constexpr int kMergeBytes = (4 * kRows * D + 8 * kRows) * (int)sizeof(float);
  constexpr int kSmem = kPipeBytes > kMergeBytes ? kPipeBytes : kMergeBytes;
  auto kernel = fwd_splitkv_kernel<D, kBf16>;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return kCudaError;
  static std::once_flag once[64];
  static cudaError_t attrErr[64];
  std::call_once(once[device], [&] {
    attrErr[device] = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  });
  if (attrErr[device] != cudaSuccess) {
    set_error_string("cudaFuncSetAttribute(%d bytes): %s", kSmem, cudaGetErrorString(attrErr[device]));
    return kCudaError;
  }
  Params p;
  p.Q = pr.Q;
  p.K = pr.K;
  p.V = pr.V;
  p.O = pr.O;
  p.partO = partO;
  p.partLse = partLse;
  p.cuQ = pr.cuQ;
  p.cuKV = pr.cuKV;
  p.seqLenQ = pr.seqLenQ;
  p.seqLenKV = pr.seqLenKV;
  p.headsQ = pr.headsQ;
  p.headsKV = pr.headsKV;
  p.group = pr.headsQ / pr.headsKV;
  p.causal = pr.causal;
  p.splits = splits;
  const int blocks = (pr.seqLenKV + kBlockKeys - 1) / kBlockKeys;
  p.keysPerSplit = ((blocks + splits - 1) / splits) * kBlockKeys;
  p.totalQ = pr.totalQ;
  p.scaleLog2 = (float)(1.4426950408889634 / sqrt((double)D));
  dim3 grid((unsigned)splits, (unsigned)pr.headsKV, (unsigned)pr.batch);
  kernel<<<grid, kThreads, kSmem, pr.stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess && splits > 1) {
    const long long rows = pr.totalQ * pr.headsQ;
    const long long threads = rows * (D / 4);
    combine_kernel<D, kBf16><<<(unsigned)((threads + 255) / 256), 256, 0, pr.stream>>>(
        partO, partLse, pr.O, rows, splits, pr.cuQ, pr.cuKV, pr.batch, pr.headsQ);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    set_error_string("split-KV kernel launch failed: %s", cudaGetErrorString(e));
    return kCudaError;
  }
  return kOk;
}

}  // namespace decode

bool splitkv_applicable(const FwdProblem& p) {
  if (p.dtype != kFp16 && p.dtype != kBf16) return false;
  if (!dtype_compiled(p.dtype) || !head_dim_compiled(p.headDim)) return false;  // left out at build time
  const int group = p.headsQ / p.headsKV;
  return (long long)p.seqLenQ * group <= decode::kRows && p.seqLenKV >= 256;
}

// Number of key-range splits.  The kernel runs two CTAs per SM; what costs time is a grid that is slightly larger than
// a whole number of such waves (batch 8 x 8 KV heads with 5 splits = 320 CTAs on 296 slots: 256 us, with 4 or 8
// splits 190 us), while splitting itself costs 20-25 % in partials and the combine pass once there are enough
// (batch, KV head) pairs to fill the GPU without it (batch 64: 7.1 TB/s unsplit, 6.8 with 2-4 splits).  So: no split
// from one full wave of pairs on, otherwise as many splits as fit two waves exactly or just under, at most 32
// (measured at 32768 keys, 8 KV heads, batch 1 / 4 / 8 / 16: 60 / 121 / 196 / 331 us; best seen 60 / 114 / 188 / 331),
// at least 256 keys per split.
int splitkv_num_splits(const FwdProblem& p, int numSMs) {
  const long long base = (long long)p.batch * p.headsKV;
  const long long slots = 2LL * numSMs;
  if (base >= slots) return 1;
  long long splits = (2 * slots) / base;
  if (splits > 32) splits = 32;
  const long long maxSplits = (p.seqLenKV + 255) / 256;
  if (splits > maxSplits) splits = maxSplits;
  if (splits < 1) splits = 1;
  return (int)splits;
}

size_t splitkv_scratch_floats(const FwdProblem& p, int splits) {
  if (splits <= 1) return 0;
  const size_t rows = (size_t)p.totalQ * p.headsQ;
  return (size_t)splits * rows * (p.headDim + 1);
}

// partO = scratch, partLse = scratch + splits*rows*D
int launch_fwd_splitkv(const FwdProblem& p, int splits, float* scratch) {
  const size_t rows = (size_t)p.totalQ * p.headsQ;
  float* partO = scratch;
  float* partLse = scratch ? scratch + (size_t)splits * rows * p.headDim : nullptr;
  const bool bf = (p.dtype == kBf16);
#define TFA_DECODE_CASE(D)                                                                   \
  case D:                                                                                    \
    if (bf) {                                                                                \
      if constexpr (TFA_HAVE_BF16) return decode::launch<D, true>(p, splits, partO, partLse);  \
    } else {                                                                                 \
      if constexpr (TFA_HAVE_FP16) return decode::launch<D, false>(p, splits, partO, partLse); \
    }                                                                                        \
    return kBadDtype;
  (void)bf; (void)partO; (void)partLse;
  switch (p.headDim) {
#if TFA_HAVE_HD32
    TFA_DECODE_CASE(32)
#endif
#if TFA_HAVE_HD64
    TFA_DECODE_CASE(64)
#endif
#if TFA_HAVE_HD96
    TFA_DECODE_CASE(96)
#endif
#if TFA_HAVE_HD128
    TFA_DECODE_CASE(128)
#endif
#if TFA_HAVE_HD192
    TFA_DECODE_CASE(192)
#endif
#if TFA_HAVE_HD256
    TFA_DECODE_CASE(256)
#endif
    default:
      return kBadHeadDim;
  }
#undef TFA_DECODE_CASE
}

}  // namespace tfa_b200

// ---------------------------------------------------------------------------------------------------------------
// Allocation-free variant of the split-KV path.
//
// Who needs it: serving processes that give all device memory to their own planner at start-up (a fixed KV-cache
// budget, nothing left for the driver to hand out later) and latency-critical decode loops in which a driver
// allocation may stall or fail.  For them the fp32 partial results of the key-range splits live in the fixed array
// below instead of a stream-ordered allocation.  The price: every GPU that loads this library carries the array
// (TFA_B200_NOALLOC_SCRATCH_FLOATS floats) until the process exits, and all calls share it.
namespace tfa_b200 {
namespace decode {

static __device__ __align__(256) float g_static_scratch[TFA_B200_NOALLOC_SCRATCH_FLOATS];

// Device address of g_static_scratch on the current device.  In host code the symbol's name is only a handle, not
// a device pointer, so the address is fetched once per device with cudaGetSymbolAddress (that device current).
static int static_scratch_ptr(float** out) {
  static std::mutex mutex;
  static float* cached[64] = {nullptr};
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= 64) {
    set_error_string("cudaGetDevice: %s", cudaGetErrorString(e));
    return kCudaError;
  }
  std::lock_guard<std::mutex> lock(mutex);
  if (cached[device] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_error_string("cudaGetSymbolAddress(static split-KV scratch) on device %d: %s", device, cudaGetErrorString(e));
      return kCudaError;
    }
    cached[device] = static_cast<float*>(p);
  }
  *out = cached[device];
  return kOk;
}

}  // namespace decode
}  // namespace tfa_b200

extern "C" int tfa_b200_fwd_decode_noalloc(const void* Q, const void* K, const void* V, void* O, int dtype,
                                           int batchSize, int seqLenQ, int seqLenKV, int numHeadsQ, int numHeadsKV,
                                           int headDim, int isCausal, int numSplits, void* stream) {
  using namespace tfa_b200;
  int rc = validate_common(Q, K, V, O, dtype, batchSize, seqLenQ, seqLenKV, numHeadsQ, numHeadsKV, headDim);
  if (rc != kOk) return rc;
  if (batchSize == 0 || seqLenQ == 0 || seqLenKV == 0) return kOk;
  if ((rc = check_device()) != kOk) return rc;
  FwdProblem p;
  p.Q = Q;
  p.K = K;
  p.V = V;
  p.O = O;
  p.cuQ = nullptr;
  p.cuKV = nullptr;
  p.dtype = dtype;
  p.batch = batchSize;
  p.seqLenQ = seqLenQ;
  p.seqLenKV = seqLenKV;
  p.totalQ = (long long)batchSize * seqLenQ;
  p.totalKV = (long long)batchSize * seqLenKV;
  p.headsQ = numHeadsQ;
  p.headsKV = numHeadsKV;
  p.headDim = headDim;
  p.causal = isCausal ? 1 : 0;
  p.stream = static_cast<cudaStream_t>(stream);
  if (!splitkv_applicable(p)) {
    set_error_string("tfa_b200_fwd_decode_noalloc handles fp16/bf16, seqLenQ * (Hq/Hkv) <= 16 and "
                     "seqLenKV >= 256 only (got dtype %d, headDim %d, seqLenQ %d, group %d, seqLenKV %d)",
                     dtype, headDim, seqLenQ, numHeadsQ / numHeadsKV, seqLenKV);
    return kBadArgument;
  }
  int device = 0, sms = 148;
  if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  int splits = (numSplits > 0) ? numSplits : splitkv_num_splits(p, sms);
  const int maxSplits = (seqLenKV + decode::kBlockKeys - 1) / decode::kBlockKeys;
  if (splits > maxSplits) splits = maxSplits;
  const size_t need = splitkv_scratch_floats(p, splits);
  if (need > (size_t)TFA_B200_NOALLOC_SCRATCH_FLOATS) {
    set_error_string("split-KV partials need %zu floats (%d splits x %lld rows x (%d + 1)) but the built-in scratch holds "
                     "%zu; use fewer splits or tfa_b200_fwd",
                     need, splits, (long long)p.totalQ * numHeadsQ, headDim, (size_t)TFA_B200_NOALLOC_SCRATCH_FLOATS);
    return kTooLarge;
  }
  float* scratch = nullptr;
  if ((rc = decode::static_scratch_ptr(&scratch)) != kOk) return rc;
  // Every (split, row) partial that the combine kernel reads is written by the split kernel of the same call, so
  // nothing in the array has to start at zero and contents left by an earlier call are never consumed.
  return launch_fwd_splitkv(p, splits, need > 0 ? scratch : nullptr);
}

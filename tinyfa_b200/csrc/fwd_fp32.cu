// FP32 attention forward on CUDA cores (true fp32 FMAs, no TF32), for sm_100a.
//
// Takes the place of the reference's FMA kernel for DType = float (reference
// csrc/flash_attn/fma/kernel.cuh:83-240) with the same contract: inputs and accumulators are fp32
// (fma/gemm.cuh:94-98, 162-166), scale 1/sqrt(D) folded into exp2, top-left causal mask and
// "col >= seqLenKV" mask (fma/softmax.cuh:97-99), row sum 0 -> output 0 (fma/softmax.cuh:76),
// sequences without keys leave O untouched (fma/kernel.cuh:116-119).
//
// One CTA (2 * BR threads: 128 for BR = 64, 256 for BR = 128) owns BR query rows of one (batch, Q head) and streams
// 64-key blocks.  Thread (ty, tx) = (tid / 8, tid % 8) owns RPT = 4 rows; in S it owns the 8 columns tx + 8*i, in O
// the float4 chunks tx + 8*i of the head dim.  K and V blocks are staged with 16-byte cp.async into
// padded rows (row stride D + 4 floats keeps the float4 reads of 8 neighbouring threads on distinct
// banks); V(j) streams in under S(j) and K(j+1) under P.V(j).
#include <cuda_runtime.h>
#include <math.h>

#include <mutex>

#include "build_config.cuh"
#include "tfa_common.cuh"

namespace tfa_b200 {

int device_num_sms(int device);  // c_abi.cu
int option_fp32_t8();             // c_abi.cu: 8 x 8 thread-tile form of the fp32 kernel at head dim 128

struct Fp32Params {
  const float* Q;
  const float* K;
  const float* V;
  float* O;
  const int* cuQ;
  const int* cuKV;
  int seqLenQ;
  int seqLenKV;
  int headsQ;
  int headsKV;
  int group;
  int causal;
  float scaleLog2;
};

namespace fp32 {

constexpr int kRowsPerThread = 4;
[[maybe_unused]] constexpr int kBC = 64;

__device__ __forceinline__ void cp_async16(float* smemDst, const float* gmemSrc, bool valid) {
  const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smemDst));
  const int bytes = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmemSrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// rows [row0, row0 + ROWS) of one head -> smem tile with row stride LD; rows >= rowEnd are zero-filled.
// Two fp32 FMAs per instruction (fma.rn.f32x2 on a register pair): the FMA pipe is no faster for it, but the kernel
// spends half as many issue slots on arithmetic, which leaves room for the shared-memory loads next to them.
// Measured against the scalar form (B2 S2048 H16): +12 % at D = 96, +5 % at 128, +11 % at 192, but -3 % at 32 / 64 and
// -11 % at 256 (the second set of partial sums spills), so only those three head dims use it.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(reinterpret_cast<unsigned long long&>(d))
      : "l"(reinterpret_cast<const unsigned long long&>(a)), "l"(reinterpret_cast<const unsigned long long&>(b)),
        "l"(reinterpret_cast<const unsigned long long&>(c)));
  return d;
}
template <int D>
constexpr bool use_packed_fma() {
  return D == 96 || D == 128 || D == 192;
}

template <int D, int ROWS, int LD, int NTHREADS>
__device__ __forceinline__ void load_tile(float* sm, const float* base, long long row0, long long rowEnd,
                                          long long rowStride) {
  constexpr int kChunks = ROWS * (D / 4);
  for (int i = threadIdx.x; i < kChunks; i += NTHREADS) {
    const int r = i / (D / 4), c = i % (D / 4);
    const bool valid = (row0 + r) < rowEnd;
    const float* src = base + (valid ? (row0 + r) : row0) * rowStride + c * 4;
    cp_async16(sm + r * LD + c * 4, valid ? src : base, valid);
  }
}

template <int D, int BR>
__global__ void __launch_bounds__(BR * 8 / kRowsPerThread) fwd_fp32_kernel(const Fp32Params p) {
  constexpr int kThreads = BR * 8 / kRowsPerThread;
  constexpr int LD = D + 4;
  constexpr int LDP = kBC + 4;
  constexpr int RPT = kRowsPerThread;
  constexpr int NCH = D / 32;
  extern __shared__ float4 smemF4[];
  float* sQ = reinterpret_cast<float*>(smemF4);
  float* sK = sQ + BR * LD;
  float* sV = sK + kBC * LD;
  float* sP = sV + kBC * LD;

  const int b = blockIdx.z, h = blockIdx.y;
  const int hkv = h / p.group;
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
  const int numTilesQ = gridDim.x;
  const int tileIdx = p.causal ? (numTilesQ - 1 - (int)blockIdx.x) : (int)blockIdx.x;
  const int q0 = tileIdx * BR;
  if (q0 >= sq || skv <= 0) return;
  const int qEnd = min(q0 + BR, sq);
  int nblk = (skv + kBC - 1) / kBC;
  if (p.causal) nblk = min(nblk, (qEnd + kBC - 1) / kBC);

  const long long qStride = (long long)p.headsQ * D;
  const long long kvStride = (long long)p.headsKV * D;
  const float* gQ = p.Q + (long long)h * D;
  const float* gK = p.K + (long long)hkv * D;
  const float* gV = p.V + (long long)hkv * D;

  const int ty = threadIdx.x >> 3, tx = threadIdx.x & 7;

  load_tile<D, BR, LD, kThreads>(sQ, gQ, qRow0 + q0, qRow0 + sq, qStride);
  load_tile<D, kBC, LD, kThreads>(sK, gK, kvRow0, kvRow0 + skv, kvStride);
  cp_async_commit();

  float o[RPT][NCH][4];
  float m[RPT], l[RPT];
#pragma unroll
  for (int r = 0; r < RPT; r++) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int i = 0; i < NCH; i++) {
      o[r][i][0] = o[r][i][1] = o[r][i][2] = o[r][i][3] = 0.f;
    }
  }
  const float c = p.scaleLog2;

  for (int j = 0; j < nblk; j++) {
    const int kbase = j * kBC;
    load_tile<D, kBC, LD, kThreads>(sV, gV, kvRow0 + kbase, kvRow0 + skv, kvStride);
    cp_async_commit();
    cp_async_wait<1>();  // Q and K(j) have landed
    __syncthreads();

    // ---- S = Q K^T for rows ty*RPT.., columns tx + 8*i
    float s[RPT][8];
    if constexpr (use_packed_fma<D>()) {
      // each score is accumulated as two partial sums (even and odd head-dim elements) held in one register pair, so
      // that one packed FMA covers two elements of the dot product
      float2 acc[RPT][8];
#pragma unroll
      for (int r = 0; r < RPT; r++) {
#pragma unroll
        for (int i = 0; i < 8; i++) acc[r][i] = make_float2(0.f, 0.f);
      }
#pragma unroll 4
      for (int d4 = 0; d4 < D / 4; d4++) {
        float4 q[RPT];
#pragma unroll
        for (int r = 0; r < RPT; r++) q[r] = *reinterpret_cast<const float4*>(sQ + (ty * RPT + r) * LD + d4 * 4);
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const float4 k = *reinterpret_cast<const float4*>(sK + (tx + 8 * i) * LD + d4 * 4);
#pragma unroll
          for (int r = 0; r < RPT; r++) {
            acc[r][i] = ffma2(make_float2(q[r].x, q[r].y), make_float2(k.x, k.y), acc[r][i]);
            acc[r][i] = ffma2(make_float2(q[r].z, q[r].w), make_float2(k.z, k.w), acc[r][i]);
          }
        }
      }
#pragma unroll
      for (int r = 0; r < RPT; r++) {
#pragma unroll
        for (int i = 0; i < 8; i++) s[r][i] = acc[r][i].x + acc[r][i].y;
      }
    } else {
  #pragma unroll
      for (int r = 0; r < RPT; r++) {
  #pragma unroll
        for (int i = 0; i < 8; i++) s[r][i] = 0.f;
      }
  #pragma unroll 4
      for (int d4 = 0; d4 < D / 4; d4++) {
        float4 q[RPT];
  #pragma unroll
        for (int r = 0; r < RPT; r++) q[r] = *reinterpret_cast<const float4*>(sQ + (ty * RPT + r) * LD + d4 * 4);
  #pragma unroll
        for (int i = 0; i < 8; i++) {
          const float4 k = *reinterpret_cast<const float4*>(sK + (tx + 8 * i) * LD + d4 * 4);
  #pragma unroll
          for (int r = 0; r < RPT; r++) {
            s[r][i] = fmaf(q[r].x, k.x, s[r][i]);
            s[r][i] = fmaf(q[r].y, k.y, s[r][i]);
            s[r][i] = fmaf(q[r].z, k.z, s[r][i]);
            s[r][i] = fmaf(q[r].w, k.w, s[r][i]);
          }
        }
      }
    }

    // ---- mask + online softmax
    const bool needMask = (kbase + kBC > skv) || (p.causal && (kbase + kBC - 1 > q0));
#pragma unroll
    for (int r = 0; r < RPT; r++) {
      const int qpos = q0 + ty * RPT + r;
      if (needMask) {
        int lim = skv - kbase;
        if (p.causal) lim = min(lim, qpos - kbase + 1);
#pragma unroll
        for (int i = 0; i < 8; i++) {
          if (tx + 8 * i >= lim) s[r][i] = -INFINITY;
        }
      }
      float mx = s[r][0];
#pragma unroll
      for (int i = 1; i < 8; i++) mx = fmaxf(mx, s[r][i]);
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      const float mNew = fmaxf(m[r], mx);
      const float mUse = (mNew == -INFINITY) ? 0.f : mNew;
      const float scale = (m[r] == -INFINITY) ? 0.f : ex2((m[r] - mUse) * c);
      m[r] = mNew;
      const float negMc = -mUse * c;
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const float pv = ex2(fmaf(s[r][i], c, negMc));
        sum += pv;
        sP[(ty * RPT + r) * LDP + tx + 8 * i] = pv;
      }
      l[r] = l[r] * scale + sum;  // per-thread partial row sum, reduced over tx at the end
#pragma unroll
      for (int i = 0; i < NCH; i++) {
        o[r][i][0] *= scale;
        o[r][i][1] *= scale;
        o[r][i][2] *= scale;
        o[r][i][3] *= scale;
      }
    }

    cp_async_wait<0>();  // V(j) has landed
    __syncthreads();     // ... and P is visible, and nobody still reads K(j)
    if (j + 1 < nblk) {
      load_tile<D, kBC, LD, kThreads>(sK, gK, kvRow0 + kbase + kBC, kvRow0 + skv, kvStride);
    }
    cp_async_commit();

    // ---- O += P V
#pragma unroll 2
    for (int c4 = 0; c4 < kBC / 4; c4++) {
      float pr[RPT][4];
#pragma unroll
      for (int r = 0; r < RPT; r++) {
        const float4 t = *reinterpret_cast<const float4*>(sP + (ty * RPT + r) * LDP + c4 * 4);
        pr[r][0] = t.x;
        pr[r][1] = t.y;
        pr[r][2] = t.z;
        pr[r][3] = t.w;
      }
#pragma unroll
      for (int cc = 0; cc < 4; cc++) {
#pragma unroll
        for (int i = 0; i < NCH; i++) {
          const float4 v = *reinterpret_cast<const float4*>(sV + (c4 * 4 + cc) * LD + (tx + 8 * i) * 4);
#pragma unroll
          for (int r = 0; r < RPT; r++) {
            if constexpr (use_packed_fma<D>()) {
              const float2 pp = make_float2(pr[r][cc], pr[r][cc]);
              const float2 lo = ffma2(pp, make_float2(v.x, v.y), make_float2(o[r][i][0], o[r][i][1]));
              const float2 hi = ffma2(pp, make_float2(v.z, v.w), make_float2(o[r][i][2], o[r][i][3]));
              o[r][i][0] = lo.x;
              o[r][i][1] = lo.y;
              o[r][i][2] = hi.x;
              o[r][i][3] = hi.y;
            } else {
              o[r][i][0] = fmaf(pr[r][cc], v.x, o[r][i][0]);
              o[r][i][1] = fmaf(pr[r][cc], v.y, o[r][i][1]);
              o[r][i][2] = fmaf(pr[r][cc], v.z, o[r][i][2]);
              o[r][i][3] = fmaf(pr[r][cc], v.w, o[r][i][3]);
            }
          }
        }
      }
    }
    __syncthreads();  // P and V(j) are free again
  }
  cp_async_wait<0>();

  // ---- normalise and store
#pragma unroll
  for (int r = 0; r < RPT; r++) {
    float sum = l[r];
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    sum += __shfl_xor_sync(0xffffffffu, sum, 4);
    const float inv = (sum > 0.f) ? (1.f / sum) : 0.f;
    const int qpos = q0 + ty * RPT + r;
    if (qpos < sq) {
      float* dst = p.O + (qRow0 + qpos) * qStride + (long long)h * D;
#pragma unroll
      for (int i = 0; i < NCH; i++) {
        float4 v;
        v.x = o[r][i][0] * inv;
        v.y = o[r][i][1] * inv;
        v.z = o[r][i][2] * inv;
        v.w = o[r][i][3] * inv;
        *reinterpret_cast<float4*>(dst + (tx + 8 * i) * 4) = v;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Second form of the fp32 kernel: "warp owns rows, lane owns columns"; used for head dim 256.
//
// A warp owns 8 query rows and a lane owns every 32nd key of a block: the Q operand of a step is one address for the
// whole warp (a broadcast), the K operand a conflict-free full-width load; in P.V the roles swap (P[row][key] is the
// broadcast, V[key][lane's dims] the full-width load).  Per lane 8 x BC/32 scores and 8 x D/32 output elements, i.e. far
// fewer registers than the thread-tile form above needs at large head dims (179 against 255 at D = 256), which is
// where it wins: 37.5 against 32.0 TFLOP/s at B2 S2048 H16 D256.  At D <= 192 it loses (D = 128: 35 against 46): the
// broadcast loads are not as cheap as one shared-memory cycle, and with 8 + BC/32 loads per 8 x BC/32 x 4 FMAs the
// kernel is as shared-memory-bound as the other form.  P goes through shared memory, but each warp reads back only the
// rows it wrote.  The contract is the one stated at the top of this file.
template <int D, int BC>
__global__ void __launch_bounds__(256) fwd_fp32_lane_kernel(const Fp32Params p) {
  constexpr int kThreads = 256;
  constexpr int BR = 64;            // query rows per CTA
  constexpr int R = 8;              // ... per warp
  constexpr int C = BC / 32;        // keys per lane and block: lane, lane + 32, ...
  constexpr int VW = (D % 128 == 0) ? 4 : (D % 64 == 0) ? 2 : 1;  // floats per vector of the lane's share of O / V
  constexpr int NV = D / (32 * VW);                               // such vectors per lane: dims lane*VW + 32*VW*i
  constexpr int LD = D + 4;
  constexpr int LDP = BC + 4;
  extern __shared__ float4 smemF4[];
  float* sQ = reinterpret_cast<float*>(smemF4);
  float* sK = sQ + BR * LD;
  float* sV = sK + BC * LD;
  float* sP = sV + BC * LD;

  const int b = blockIdx.z, h = blockIdx.y;
  const int hkv = h / p.group;
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
  const int numTilesQ = gridDim.x;
  const int tileIdx = p.causal ? (numTilesQ - 1 - (int)blockIdx.x) : (int)blockIdx.x;  // heavy causal tiles first
  const int q0 = tileIdx * BR;
  if (q0 >= sq || skv <= 0) return;
  const int qEnd = min(q0 + BR, sq);
  int nblk = (skv + BC - 1) / BC;
  if (p.causal) nblk = min(nblk, (qEnd + BC - 1) / BC);

  const long long qStride = (long long)p.headsQ * D;
  const long long kvStride = (long long)p.headsKV * D;
  const float* gQ = p.Q + (long long)h * D;
  const float* gK = p.K + (long long)hkv * D;
  const float* gV = p.V + (long long)hkv * D;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = warp * R;  // first row of this warp inside the tile

  load_tile<D, BR, LD, kThreads>(sQ, gQ, qRow0 + q0, qRow0 + sq, qStride);
  load_tile<D, BC, LD, kThreads>(sK, gK, kvRow0, kvRow0 + skv, kvStride);
  cp_async_commit();

  float o[R][NV * VW];
  float m[R], l[R];
#pragma unroll
  for (int r = 0; r < R; r++) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int i = 0; i < NV * VW; i++) o[r][i] = 0.f;
  }
  const float c = p.scaleLog2;

  for (int j = 0; j < nblk; j++) {
    const int kbase = j * BC;
    load_tile<D, BC, LD, kThreads>(sV, gV, kvRow0 + kbase, kvRow0 + skv, kvStride);
    cp_async_commit();
    cp_async_wait<1>();  // Q and K(j) have landed
    __syncthreads();

    // ---- S = Q K^T: rows row0 .. row0+7, keys lane + 32*i
    float s[R][C];
#pragma unroll
    for (int r = 0; r < R; r++) {
#pragma unroll
      for (int i = 0; i < C; i++) s[r][i] = 0.f;
    }
#pragma unroll 2
    for (int d4 = 0; d4 < D / 4; d4++) {
      float4 k[C];
#pragma unroll
      for (int i = 0; i < C; i++) k[i] = *reinterpret_cast<const float4*>(sK + (lane + 32 * i) * LD + d4 * 4);
#pragma unroll
      for (int r = 0; r < R; r++) {
        const float4 q = *reinterpret_cast<const float4*>(sQ + (row0 + r) * LD + d4 * 4);  // one address per warp
#pragma unroll
        for (int i = 0; i < C; i++) {
          s[r][i] = fmaf(q.x, k[i].x, s[r][i]);
          s[r][i] = fmaf(q.y, k[i].y, s[r][i]);
          s[r][i] = fmaf(q.z, k[i].z, s[r][i]);
          s[r][i] = fmaf(q.w, k[i].w, s[r][i]);
        }
      }
    }

    // ---- mask + online softmax; every lane ends up with the row's maximum, the row sum stays split over the lanes
    const bool needMask = (kbase + BC > skv) || (p.causal && (kbase + BC - 1 > q0));
#pragma unroll
    for (int r = 0; r < R; r++) {
      const int qpos = q0 + row0 + r;
      if (needMask) {
        int lim = skv - kbase;
        if (p.causal) lim = min(lim, qpos - kbase + 1);
#pragma unroll
        for (int i = 0; i < C; i++) {
          if (lane + 32 * i >= lim) s[r][i] = -INFINITY;
        }
      }
      float mx = s[r][0];
#pragma unroll
      for (int i = 1; i < C; i++) mx = fmaxf(mx, s[r][i]);
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float mNew = fmaxf(m[r], mx);
      const float mUse = (mNew == -INFINITY) ? 0.f : mNew;
      const float scale = (m[r] == -INFINITY) ? 0.f : ex2((m[r] - mUse) * c);
      m[r] = mNew;
      const float negMc = -mUse * c;
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < C; i++) {
        const float pv = ex2(fmaf(s[r][i], c, negMc));
        sum += pv;
        sP[(row0 + r) * LDP + lane + 32 * i] = pv;
      }
      l[r] = l[r] * scale + sum;
#pragma unroll
      for (int i = 0; i < NV * VW; i++) o[r][i] *= scale;
    }

    cp_async_wait<0>();  // V(j) has landed
    __syncthreads();     // ... for everybody, nobody still reads K(j), and this warp's P rows are visible to its lanes
    if (j + 1 < nblk) {
      load_tile<D, BC, LD, kThreads>(sK, gK, kvRow0 + kbase + BC, kvRow0 + skv, kvStride);
    }
    cp_async_commit();

    // ---- O += P V: P[row][key] is one address per warp, V[key][lane's dims] the full-width load
#pragma unroll 2
    for (int k4 = 0; k4 < BC / 4; k4++) {
      float4 pr[R];
#pragma unroll
      for (int r = 0; r < R; r++) pr[r] = *reinterpret_cast<const float4*>(sP + (row0 + r) * LDP + k4 * 4);
#pragma unroll
      for (int kk = 0; kk < 4; kk++) {
        float v[NV * VW];
#pragma unroll
        for (int i = 0; i < NV; i++) {
          const float* src = sV + (k4 * 4 + kk) * LD + lane * VW + 32 * VW * i;
          if constexpr (VW == 4) {
            const float4 t = *reinterpret_cast<const float4*>(src);
            v[i * 4 + 0] = t.x;
            v[i * 4 + 1] = t.y;
            v[i * 4 + 2] = t.z;
            v[i * 4 + 3] = t.w;
          } else if constexpr (VW == 2) {
            const float2 t = *reinterpret_cast<const float2*>(src);
            v[i * 2 + 0] = t.x;
            v[i * 2 + 1] = t.y;
          } else {
            v[i] = *src;
          }
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
          const float pw = (kk == 0) ? pr[r].x : (kk == 1) ? pr[r].y : (kk == 2) ? pr[r].z : pr[r].w;
#pragma unroll
          for (int i = 0; i < NV * VW; i++) o[r][i] = fmaf(pw, v[i], o[r][i]);
        }
      }
    }
    __syncthreads();  // V(j) and P are free again
  }
  cp_async_wait<0>();

  // ---- normalise and store: lane writes its dims of each of the warp's rows
#pragma unroll
  for (int r = 0; r < R; r++) {
    float sum = l[r];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    const float inv = (sum > 0.f) ? (1.f / sum) : 0.f;
    const int qpos = q0 + row0 + r;
    if (qpos < sq) {
      float* dst = p.O + (qRow0 + qpos) * qStride + (long long)h * D;
#pragma unroll
      for (int i = 0; i < NV; i++) {
        float* d = dst + lane * VW + 32 * VW * i;
        if constexpr (VW == 4) {
          *reinterpret_cast<float4*>(d) = make_float4(o[r][i * 4] * inv, o[r][i * 4 + 1] * inv, o[r][i * 4 + 2] * inv,
                                                      o[r][i * 4 + 3] * inv);
        } else if constexpr (VW == 2) {
          *reinterpret_cast<float2*>(d) = make_float2(o[r][i * 2] * inv, o[r][i * 2 + 1] * inv);
        } else {
          *d = o[r][i] * inv;
        }
      }
    }
  }
}

template <int D, int BC>
int launch_lane(const FwdProblem& pr) {
  constexpr int LD = D + 4;
  constexpr int kSmem = (64 * LD + 2 * BC * LD + 64 * (BC + 4)) * (int)sizeof(float);
  static_assert(kSmem <= 227 * 1024, "shared memory");
  auto kernel = fwd_fp32_lane_kernel<D, BC>;
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
  Fp32Params p;
  p.Q = static_cast<const float*>(pr.Q);
  p.K = static_cast<const float*>(pr.K);
  p.V = static_cast<const float*>(pr.V);
  p.O = static_cast<float*>(pr.O);
  p.cuQ = pr.cuQ;
  p.cuKV = pr.cuKV;
  p.seqLenQ = pr.seqLenQ;
  p.seqLenKV = pr.seqLenKV;
  p.headsQ = pr.headsQ;
  p.headsKV = pr.headsKV;
  p.group = pr.headsQ / pr.headsKV;
  p.causal = pr.causal;
  p.scaleLog2 = (float)(1.4426950408889634 / sqrt((double)D));
  dim3 grid((unsigned)((pr.seqLenQ + 63) / 64), (unsigned)pr.headsQ, (unsigned)pr.batch);
  kernel<<<grid, 256, kSmem, pr.stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error_string("fp32 kernel launch failed: %s", cudaGetErrorString(e));
    return kCudaError;
  }
  return kOk;
}

// ---------------------------------------------------------------------------------------------------------------
// 8 x 8 thread-tile form (D = 128): 128 query rows x 128 keys per block, 256 threads.  Thread (ty, tx) = (tid / 16,
// tid % 16) owns rows 8 ty .. 8 ty + 7; in S the 8 columns tx + 16 i, in O the float4 chunks tx and tx + 16 of the head
// dim.  Both products then fetch 16 values per 64 FMAs (the 4 x 8 form: 12 per 32 and 20 per 64), which is what takes
// the kernel off the shared-memory roofline: a 16-byte shared-memory load is served a quarter warp at a time whatever
// addresses coincide, so the only way to fewer shared-memory cycles per FMA is more FMAs per loaded value.
//   * Q is transposed once per CTA (sQT[d][row]) and P is written transposed (sPT[key][row]), so that two neighbouring
//     rows form a register pair: one fma.rn.f32x2 covers rows r, r + 1 against a duplicated K (V) value - no second
//     set of partial sums, 64 + 64 accumulators per thread.
//   * P is written over the K block it came from (a barrier between the two products), so three 66 KB buffers do:
//     Q^T, K / P^T, V.  V(j) streams in under Q.K^T(j); K(j + 1) can only be requested after P.V(j) and is waited for at
//     the top of the next block (about 1 of 20 us per block exposed; a 96-key variant with a P^T buffer of its own, which
//     hides that load, measured 1 % slower).
// Measured at B2 S4096 H32: 46.4 -> 49.4 TFLOP/s non-causal, 41.8 -> 44.4 causal; shared-memory data pipe 77 % -> 52 %
// busy, FMA pipe 65 % -> 70 %; 255 registers, so the SM runs these 8 warps and no more, and what is left is latency that
// two warps per scheduler do not cover.
template <int D>
__global__ void __launch_bounds__(256, 1) fwd_fp32_t8_kernel(const Fp32Params p) {
  static_assert(D == 128, "8 x 8 form: head dim 128");
  constexpr int BR = 128, BC = 128, kThreads = 256;
  constexpr int NC = BC / 16;  // score columns per thread
  constexpr int LDQ = BR + 4;  // sQT row pitch (a row of sQT holds one head-dim element of all 128 query rows)
  constexpr int LD = D + 4;    // K / V row pitch
  constexpr int LDP = BR + 4;  // sPT row pitch (a row holds one key's weights for all 128 query rows)
  extern __shared__ float4 smemF4[];
  float* sQT = reinterpret_cast<float*>(smemF4);
  float* sK = sQT + D * LDQ;
  float* sV = sK + BC * LD;
  float* sPT = sK;  // aliased: P^T of block j overwrites K(j) once every warp is done with Q.K^T
  static_assert(BC * LDP <= BC * LD, "P^T fits the K buffer");

  const int b = blockIdx.z, h = blockIdx.y;
  const int hkv = h / p.group;
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
  const int numTilesQ = gridDim.x;
  const int tileIdx = p.causal ? (numTilesQ - 1 - (int)blockIdx.x) : (int)blockIdx.x;
  const int q0 = tileIdx * BR;
  if (q0 >= sq || skv <= 0) return;
  const int qEnd = min(q0 + BR, sq);
  int nblk = (skv + BC - 1) / BC;
  if (p.causal) nblk = min(nblk, (qEnd + BC - 1) / BC);

  const long long qStride = (long long)p.headsQ * D;
  const long long kvStride = (long long)p.headsKV * D;
  const float* gQ = p.Q + (long long)h * D;
  const float* gK = p.K + (long long)hkv * D;
  const float* gV = p.V + (long long)hkv * D;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const int r0 = ty * 8;

  // K(0) on its way, then Q transposed into shared memory (lanes walk rows: the transposed stores hit 32 banks)
  load_tile<D, BC, LD, kThreads>(sK, gK, kvRow0, kvRow0 + skv, kvStride);
  cp_async_commit();
  for (int i = threadIdx.x; i < BR * (D / 4); i += kThreads) {
    const int row = i % BR, d4 = i / BR;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (q0 + row < sq) v = *reinterpret_cast<const float4*>(gQ + (qRow0 + q0 + row) * qStride + d4 * 4);
    sQT[(d4 * 4 + 0) * LDQ + row] = v.x;
    sQT[(d4 * 4 + 1) * LDQ + row] = v.y;
    sQT[(d4 * 4 + 2) * LDQ + row] = v.z;
    sQT[(d4 * 4 + 3) * LDQ + row] = v.w;
  }

  float2 o[4][8];  // [row pair][head-dim column]: .x = row r0 + 2 rp, .y = the next row
  float m[8], l[8];
#pragma unroll
  for (int r = 0; r < 8; r++) {
    m[r] = -INFINITY;
    l[r] = 0.f;
  }
#pragma unroll
  for (int rp = 0; rp < 4; rp++) {
#pragma unroll
    for (int cidx = 0; cidx < 8; cidx++) o[rp][cidx] = make_float2(0.f, 0.f);
  }
  const float c = p.scaleLog2;

  for (int j = 0; j < nblk; j++) {
    const int kbase = j * BC;
    cp_async_wait<0>();  // K(j) has landed (and, for j = 0, nothing else is outstanding)
    __syncthreads();     // ... for every thread; Q^T is visible; nobody still reads V(j - 1) or P^T(j - 1)
    load_tile<D, BC, LD, kThreads>(sV, gV, kvRow0 + kbase, kvRow0 + skv, kvStride);
    cp_async_commit();

    // ---- S = Q K^T: rows r0 .. r0 + 7 as four register pairs, columns tx + 16 i
    float2 acc[4][NC];
#pragma unroll
    for (int rp = 0; rp < 4; rp++) {
#pragma unroll
      for (int i = 0; i < NC; i++) acc[rp][i] = make_float2(0.f, 0.f);
    }
#pragma unroll 1
    for (int d4 = 0; d4 < D / 4; d4++) {
      float4 qa[4], qb[4];
#pragma unroll
      for (int dd = 0; dd < 4; dd++) {
        qa[dd] = *reinterpret_cast<const float4*>(sQT + (d4 * 4 + dd) * LDQ + r0);
        qb[dd] = *reinterpret_cast<const float4*>(sQT + (d4 * 4 + dd) * LDQ + r0 + 4);
      }
#pragma unroll
      for (int i = 0; i < NC; i++) {
        const float4 k = *reinterpret_cast<const float4*>(sK + (tx + 16 * i) * LD + d4 * 4);
        const float kv[4] = {k.x, k.y, k.z, k.w};
#pragma unroll
        for (int dd = 0; dd < 4; dd++) {
          const float2 kd = make_float2(kv[dd], kv[dd]);
          acc[0][i] = ffma2(make_float2(qa[dd].x, qa[dd].y), kd, acc[0][i]);
          acc[1][i] = ffma2(make_float2(qa[dd].z, qa[dd].w), kd, acc[1][i]);
          acc[2][i] = ffma2(make_float2(qb[dd].x, qb[dd].y), kd, acc[2][i]);
          acc[3][i] = ffma2(make_float2(qb[dd].z, qb[dd].w), kd, acc[3][i]);
        }
      }
    }
    __syncthreads();  // every warp is done with K(j): its buffer becomes P^T(j)

    // ---- mask + online softmax; P^T written as two float4 per column (8 consecutive rows)
    const bool needMask = (kbase + BC > skv) || (p.causal && (kbase + BC - 1 > q0));
    float scale[8], negMc[8];
#pragma unroll
    for (int r = 0; r < 8; r++) {
      const int qpos = q0 + r0 + r;
      int lim = BC;
      if (needMask) {
        lim = skv - kbase;
        if (p.causal) lim = min(lim, qpos - kbase + 1);
      }
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < NC; i++) {
        float sv = (r & 1) ? acc[r >> 1][i].y : acc[r >> 1][i].x;
        if (needMask && tx + 16 * i >= lim) sv = -INFINITY;
        if (r & 1) {
          acc[r >> 1][i].y = sv;
        } else {
          acc[r >> 1][i].x = sv;
        }
        mx = fmaxf(mx, sv);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      const float mNew = fmaxf(m[r], mx);
      const float mUse = (mNew == -INFINITY) ? 0.f : mNew;
      scale[r] = (m[r] == -INFINITY) ? 0.f : ex2((m[r] - mUse) * c);
      m[r] = mNew;
      negMc[r] = -mUse * c;
    }
    float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < NC; i++) {
      float pv[8];
#pragma unroll
      for (int r = 0; r < 8; r++) {
        const float sv = (r & 1) ? acc[r >> 1][i].y : acc[r >> 1][i].x;
        pv[r] = ex2(fmaf(sv, c, negMc[r]));
        sum[r] += pv[r];
      }
      float* dst = sPT + (tx + 16 * i) * LDP + r0;
      *reinterpret_cast<float4*>(dst) = make_float4(pv[0], pv[1], pv[2], pv[3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(pv[4], pv[5], pv[6], pv[7]);
    }
#pragma unroll
    for (int r = 0; r < 8; r++) l[r] = l[r] * scale[r] + sum[r];  // per-thread partial row sums, reduced over tx at the end
#pragma unroll
    for (int rp = 0; rp < 4; rp++) {
      const float2 sc = make_float2(scale[2 * rp], scale[2 * rp + 1]);
#pragma unroll
      for (int cidx = 0; cidx < 8; cidx++) {
        o[rp][cidx].x *= sc.x;
        o[rp][cidx].y *= sc.y;
      }
    }

    cp_async_wait<0>();  // V(j) has landed
    __syncthreads();     // ... and P^T(j) is visible

    // ---- O += P V: per key two float4 of P^T (8 rows) and two float4 of V (8 head-dim columns)
#pragma unroll 4
    for (int key = 0; key < BC; key++) {
      const float4 pa = *reinterpret_cast<const float4*>(sPT + key * LDP + r0);
      const float4 pb = *reinterpret_cast<const float4*>(sPT + key * LDP + r0 + 4);
      const float4 va = *reinterpret_cast<const float4*>(sV + key * LD + tx * 4);
      const float4 vb = *reinterpret_cast<const float4*>(sV + key * LD + 64 + tx * 4);
      const float vv[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
#pragma unroll
      for (int cidx = 0; cidx < 8; cidx++) {
        const float2 vd = make_float2(vv[cidx], vv[cidx]);
        o[0][cidx] = ffma2(make_float2(pa.x, pa.y), vd, o[0][cidx]);
        o[1][cidx] = ffma2(make_float2(pa.z, pa.w), vd, o[1][cidx]);
        o[2][cidx] = ffma2(make_float2(pb.x, pb.y), vd, o[2][cidx]);
        o[3][cidx] = ffma2(make_float2(pb.z, pb.w), vd, o[3][cidx]);
      }
    }
    __syncthreads();  // P^T(j) and V(j) are free again
    if (j + 1 < nblk) load_tile<D, BC, LD, kThreads>(sK, gK, kvRow0 + kbase + BC, kvRow0 + skv, kvStride);
    cp_async_commit();
  }
  cp_async_wait<0>();

  // ---- normalise and store
#pragma unroll
  for (int r = 0; r < 8; r++) {
    float sum = l[r];
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    sum += __shfl_xor_sync(0xffffffffu, sum, 4);
    sum += __shfl_xor_sync(0xffffffffu, sum, 8);
    const float inv = (sum > 0.f) ? (1.f / sum) : 0.f;
    const int qpos = q0 + r0 + r;
    if (qpos < sq) {
      float* dst = p.O + (qRow0 + qpos) * qStride + (long long)h * D;
      const int rp = r >> 1;
      float4 a, bq;
      if (r & 1) {
        a = make_float4(o[rp][0].y * inv, o[rp][1].y * inv, o[rp][2].y * inv, o[rp][3].y * inv);
        bq = make_float4(o[rp][4].y * inv, o[rp][5].y * inv, o[rp][6].y * inv, o[rp][7].y * inv);
      } else {
        a = make_float4(o[rp][0].x * inv, o[rp][1].x * inv, o[rp][2].x * inv, o[rp][3].x * inv);
        bq = make_float4(o[rp][4].x * inv, o[rp][5].x * inv, o[rp][6].x * inv, o[rp][7].x * inv);
      }
      *reinterpret_cast<float4*>(dst + tx * 4) = a;
      *reinterpret_cast<float4*>(dst + 64 + tx * 4) = bq;
    }
  }
}

template <int D>
int launch_t8(const FwdProblem& pr) {
  constexpr int kSmem = (D * (128 + 4) + 2 * 128 * (D + 4)) * (int)sizeof(float);
  auto kernel = fwd_fp32_t8_kernel<D>;
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
  Fp32Params p;
  p.Q = static_cast<const float*>(pr.Q);
  p.K = static_cast<const float*>(pr.K);
  p.V = static_cast<const float*>(pr.V);
  p.O = static_cast<float*>(pr.O);
  p.cuQ = pr.cuQ;
  p.cuKV = pr.cuKV;
  p.seqLenQ = pr.seqLenQ;
  p.seqLenKV = pr.seqLenKV;
  p.headsQ = pr.headsQ;
  p.headsKV = pr.headsKV;
  p.group = pr.headsQ / pr.headsKV;
  p.causal = pr.causal;
  p.scaleLog2 = (float)(1.4426950408889634 / sqrt((double)D));
  dim3 grid((unsigned)((pr.seqLenQ + 127) / 128), (unsigned)pr.headsQ, (unsigned)pr.batch);
  kernel<<<grid, 256, kSmem, pr.stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error_string("fp32 kernel launch failed: %s", cudaGetErrorString(e));
    return kCudaError;
  }
  return kOk;
}

template <int D, int BR>
int launch(const FwdProblem& pr) {
  constexpr int LD = D + 4;
  constexpr int kSmem = (BR * LD + 2 * kBC * LD + BR * (kBC + 4)) * (int)sizeof(float);
  auto kernel = fwd_fp32_kernel<D, BR>;
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
  Fp32Params p;
  p.Q = static_cast<const float*>(pr.Q);
  p.K = static_cast<const float*>(pr.K);
  p.V = static_cast<const float*>(pr.V);
  p.O = static_cast<float*>(pr.O);
  p.cuQ = pr.cuQ;
  p.cuKV = pr.cuKV;
  p.seqLenQ = pr.seqLenQ;
  p.seqLenKV = pr.seqLenKV;
  p.headsQ = pr.headsQ;
  p.headsKV = pr.headsKV;
  p.group = pr.headsQ / pr.headsKV;
  p.causal = pr.causal;
  p.scaleLog2 = (float)(1.4426950408889634 / sqrt((double)D));
  dim3 grid((unsigned)((pr.seqLenQ + BR - 1) / BR), (unsigned)pr.headsQ, (unsigned)pr.batch);
  kernel<<<grid, BR * 8 / kRowsPerThread, kSmem, pr.stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error_string("fp32 kernel launch failed: %s", cudaGetErrorString(e));
    return kCudaError;
  }
  return kOk;
}

}  // namespace fp32

int launch_fwd_fp32(const FwdProblem& pr) {
#if TFA_HAVE_FP32
  switch (pr.headDim) {
#if TFA_HAVE_HD32
    case 32:
      return fp32::launch<32, 64>(pr);
#endif
#if TFA_HAVE_HD64
    case 64:
      return fp32::launch<64, 64>(pr);
#endif
#if TFA_HAVE_HD96
    case 96:
      return fp32::launch<96, 64>(pr);
#endif
#if TFA_HAVE_HD128
    case 128:
      // The 64-row form fits one 4-warp CTA per SM only (119 KB of shared memory); with 128 rows and 256 threads an SM
      // runs 8 warps and every K/V block serves twice as many rows: +18 % at B2 S4096 H32 (39 -> 46 TFLOP/s).  Small
      // problems keep the 64-row form, which makes twice as many CTAs.
      {
        int device = 0;
        cudaGetDevice(&device);
        const long long ctas128 = (long long)((pr.seqLenQ + 127) / 128) * pr.headsQ * pr.batch;
        const int t8 = option_fp32_t8();  // 0 never, 1 for large problems (the default), 2 always (tests)
        if (t8 == 2) return fp32::launch_t8<128>(pr);
        if (ctas128 >= 3LL * device_num_sms(device)) {
          return t8 != 0 ? fp32::launch_t8<128>(pr) : fp32::launch<128, 128>(pr);
        }
      }
      return fp32::launch<128, 64>(pr);
#endif
#if TFA_HAVE_HD192
    case 192:
      return fp32::launch<192, 64>(pr);
#endif
#if TFA_HAVE_HD256
    case 256:
      // the warp-rows / lane-columns form: 37.5 against 32.0 TFLOP/s at B2 S2048 H16 (the thread-tile form sits at 255
      // registers there); at every other head dim the thread-tile form is the faster one (128: 46 against 35)
      return fp32::launch_lane<256, 64>(pr);
#endif
    default:
      break;
  }
  set_error_string("TinyFA: fp32 kernel for headDim %d was not compiled into this library", pr.headDim);
  return kBadHeadDim;
#else
  set_error_string("TinyFA: fp32 kernels were not compiled into this library (TFA_TARGET_DTYPE build switch)");
  return kBadDtype;
#endif
}

}  // namespace tfa_b200

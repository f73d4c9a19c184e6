// Host launcher for one (padded head dim, dtype) instantiation of the tcgen05 attention kernel.
// Compiled once per pair with -DTFA_HDP=<64|128|192|256> -DTFA_BF16=<0|1> so that the instantiations
// build in parallel (the reference splits its instantiations the same way, one translation unit per
// dtype and architecture: reference csrc/flash_attn/kernels/tfa_fwd_*_sm8x.cu).
//
// Takes the place of the reference's host launcher (reference csrc/flash_attn/launcher.cuh:28-99):
// it derives the grid from the problem sizes, opts in to large dynamic shared memory and launches on
// the caller's stream; in addition it encodes the three TMA descriptors the kernel needs.
#include <cstdio>
#include <mutex>

#include "fwd_tc.cuh"

#ifndef TFA_HDP
#error "compile with -DTFA_HDP=<64|128|192|256>"
#endif
#ifndef TFA_BF16
#error "compile with -DTFA_BF16=<0|1>"
#endif

namespace tfa_b200 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_tiled();  // c_abi.cu
int* device_status_word(int device);  // c_abi.cu: per-device status word (device memory)
int next_epoch();                     // c_abi.cu
int* device_work_counter(int device, cudaStream_t stream, int* rc, CUtensorMap** maps);  // c_abi.cu
int launch_patch_varlen_maps(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, CUtensorMap* out,
                             const int* cuQ, const int* cuKV, int batch, cudaStream_t stream);  // c_abi.cu
int device_num_sms(int device);       // c_abi.cu
int option_narrow_mma();              // c_abi.cu: MMAs shaped for head dims 32 / 96 inside the 64- / 128-wide kernels
int option_solo64();                  // c_abi.cu: one-tile CTAs, two per SM, for head dims 32 / 64
int option_work_order();              // c_abi.cu: -1 auto, 0 pair index fastest, n > 0 chunk width
int option_pair_cta();                // c_abi.cu: head dims 192 / 256 in clusters of two CTAs that share K/V

#define TFA_CAT3(a, b, c) a##b##c
#define TFA_NAME(hdp, bf) TFA_CAT3(launch_fwd_tc_hdp##hdp, _bf, bf)
#define TFA_NAME2(hdp, bf) TFA_NAME(hdp, bf)

// [batches, rows, heads, headDim] tensor, 16-bit elements (packed varlen: batches = 1, rows = total);
// box = 64 elements x boxHeads x boxRows x 1, 128-byte swizzle; out-of-range elements read as zero.
static int make_map(CUtensorMap* m, const void* base, long long batches, long long rows, int heads, int headDim,
                    int boxHeads, int boxRows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return kCudaError;
  cuuint64_t dims[4] = {(cuuint64_t)headDim, (cuuint64_t)heads, (cuuint64_t)rows, (cuuint64_t)batches};
  cuuint64_t strides[3] = {(cuuint64_t)headDim * 2, (cuuint64_t)heads * headDim * 2,
                           (cuuint64_t)rows * heads * headDim * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)boxHeads, (cuuint32_t)boxRows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(m, TFA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error_string("cuTensorMapEncodeTiled failed with CUresult %d (batches=%lld rows=%lld heads=%d headDim=%d box=%d,%d)",
                     (int)r, batches, rows, heads, headDim, boxHeads, boxRows);
    return kCudaError;
  }
  return kOk;
}

int TFA_NAME2(TFA_HDP, TFA_BF16)(const FwdProblem& pr, int packShift) {
  using C = tc::Cfg<TFA_HDP>;
  const bool varlen = (pr.cuQ != nullptr);
  constexpr bool kBf = (TFA_BF16 != 0);
  auto kernel = varlen ? tc::fwd_tc_kernel<TFA_HDP, kBf, tc::kModeVarlen> : tc::fwd_tc_kernel<TFA_HDP, kBf, tc::kModeFixed>;
  bool solo = false;  // one Q tile per CTA, two CTAs per SM (padded head dim 64 only)
  int kNT = C::kNT, smemBytes = C::kSmemBytes, threads = tc::kThreads;
#if TFA_HDP == 128
  // head dim 96 has MMAs of its own shape in the 128-wide kernel (6 of 8 k-steps, 96 output columns)
  if (pr.headDim == 96 && option_narrow_mma() != 0) {
    kernel = varlen ? tc::fwd_tc_kernel<128, kBf, tc::kModeVarlen, false, 96> : tc::fwd_tc_kernel<128, kBf, tc::kModeFixed, false, 96>;
  }
#endif
#if TFA_HDP == 64
  // nothing to mask: not causal, and the key length fills its last 128-key block
  const bool noMask = !varlen && !pr.causal && pr.seqLenKV % tc::kBlockN == 0;
  if (noMask) kernel = tc::fwd_tc_kernel<64, kBf, tc::kModeFixedNoMask>;
  solo = option_solo64() != 0;
  if (solo) {
    const bool narrow = (pr.headDim == 32 && option_narrow_mma() != 0);  // head dim 32: 2 of 4 k-steps, 32 output columns
    if (narrow) {
      kernel = varlen ? tc::fwd_tc_kernel<64, kBf, tc::kModeVarlen, true, 32>
                      : (noMask ? tc::fwd_tc_kernel<64, kBf, tc::kModeFixedNoMask, true, 32>
                                : tc::fwd_tc_kernel<64, kBf, tc::kModeFixed, true, 32>);
    } else {
      kernel = varlen ? tc::fwd_tc_kernel<64, kBf, tc::kModeVarlen, true>
                      : (noMask ? tc::fwd_tc_kernel<64, kBf, tc::kModeFixedNoMask, true>
                                : tc::fwd_tc_kernel<64, kBf, tc::kModeFixed, true>);
    }
    kNT = 1;
    smemBytes = tc::CfgSolo64::kSmemBytes;
    threads = tc::kThreadsSolo;
  }
#endif

  bool pair = false;  // clusters of two CTAs, one Q tile each, K/V shared (head dims 192 / 256, fixed length)
#if TFA_HDP >= 192
  // Measured (fp16, H16, batch x length = 16 K tokens, 600-800-launch loops, one-tile form -> pair form): head dim 256
  // non-causal S256 500 -> 497, S512 672 -> 789, S1024 791 -> 1010, S2048 872 -> 1168, S8192 957 -> 1244 TFLOP/s; causal
  // S512 444 -> 432, S1024 611 -> 673, S1536 702 -> 813, S2048 760 -> 896; head dim 192 non-causal S2048 1023 -> 1013,
  // S8192 1098 -> 1119, causal S2048 826 -> 764, S8192 1009 -> 1007 (three ring stages already keep its one-tile form
  // fed).  Causal pairs pay for the fully masked last block of their first tile and, with short sequences, for item
  // boundaries that are twice as heavy; "auto" is head dim 256 only, and its causal problems from 1024 query rows.
  const int pairOpt = option_pair_cta();
  const bool pairAuto = (TFA_HDP == 256) && (!pr.causal || pr.seqLenQ >= 1024);
  pair = !varlen && pr.seqLenQ > (tc::kBlockM >> packShift) && (pairOpt > 0 || (pairOpt < 0 && pairAuto));
  if (pair) {
    kernel = tc::fwd_tc_kernel<TFA_HDP, kBf, tc::kModeFixed, false, TFA_HDP, true>;
    kNT = 2;  // a work item is the two tiles of a pair
    smemBytes = tc::CfgPair<TFA_HDP>::kSmemBytes;
  }
#endif

  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return kCudaError;
  static std::once_flag once[64];
  static cudaError_t attrErr[64];
  if (device < 0 || device >= 64) return kBadArgument;
  std::call_once(once[device], [&] {
    auto bigAttr = [&](auto k) {
      if (attrErr[device] != cudaSuccess) return;
      attrErr[device] = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    };
    attrErr[device] = cudaSuccess;
    bigAttr(tc::fwd_tc_kernel<TFA_HDP, kBf, tc::kModeFixed>);
    bigAttr(tc::fwd_tc_kernel<TFA_HDP, kBf, tc::kModeVarlen>);
#if TFA_HDP >= 192
    if (attrErr[device] == cudaSuccess) {
      attrErr[device] = cudaFuncSetAttribute(tc::fwd_tc_kernel<TFA_HDP, kBf, tc::kModeFixed, false, TFA_HDP, true>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, tc::CfgPair<TFA_HDP>::kSmemBytes);
    }
#endif
#if TFA_HDP == 128
    bigAttr(tc::fwd_tc_kernel<128, kBf, tc::kModeFixed, false, 96>);
    bigAttr(tc::fwd_tc_kernel<128, kBf, tc::kModeVarlen, false, 96>);
#endif
#if TFA_HDP == 64
    bigAttr(tc::fwd_tc_kernel<64, kBf, tc::kModeFixedNoMask>);
    // the two-CTAs-per-SM form: 99 KB each, and the largest shared-memory carve-out so that two fit
    auto soloAttr = [&](auto k) {
      if (attrErr[device] != cudaSuccess) return;
      attrErr[device] = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::CfgSolo64::kSmemBytes);
      if (attrErr[device] == cudaSuccess) {
        attrErr[device] = cudaFuncSetAttribute(k, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
      }
    };
    soloAttr(tc::fwd_tc_kernel<64, kBf, tc::kModeFixed, true>);
    soloAttr(tc::fwd_tc_kernel<64, kBf, tc::kModeVarlen, true>);
    soloAttr(tc::fwd_tc_kernel<64, kBf, tc::kModeFixedNoMask, true>);
    soloAttr(tc::fwd_tc_kernel<64, kBf, tc::kModeFixed, true, 32>);
    soloAttr(tc::fwd_tc_kernel<64, kBf, tc::kModeVarlen, true, 32>);
    soloAttr(tc::fwd_tc_kernel<64, kBf, tc::kModeFixedNoMask, true, 32>);
#endif
  });
  if (attrErr[device] != cudaSuccess) {
    set_error_string("cudaFuncSetAttribute(%d bytes): %s", C::kSmemBytes, cudaGetErrorString(attrErr[device]));
    return kCudaError;
  }

  const int gp = 1 << packShift;
  const int rowsPerTile = tc::kBlockM >> packShift;
  CUtensorMap tmQ, tmK, tmV;
  int rc;
  const long long nb = varlen ? 1 : pr.batch;
  // packed input with unknown totals: placeholder extent, completed on the device before the kernel runs
  const bool devMaps = varlen && (pr.totalQ < 0 || pr.totalKV < 0);
  const long long rowsQ = varlen ? (devMaps ? 1 : pr.totalQ) : pr.seqLenQ;
  const long long rowsKV = varlen ? (devMaps ? 1 : pr.totalKV) : pr.seqLenKV;
  if ((rc = make_map(&tmQ, pr.Q, nb, rowsQ, pr.headsQ, pr.headDim, gp, rowsPerTile)) != kOk) return rc;
  // pair form: each CTA loads 64 of a block's 128 keys
  if ((rc = make_map(&tmK, pr.K, nb, rowsKV, pr.headsKV, pr.headDim, 1, pair ? tc::kBlockN / 2 : tc::kBlockN)) != kOk) return rc;
  if ((rc = make_map(&tmV, pr.V, nb, rowsKV, pr.headsKV, pr.headDim, 1, tc::kBlockN)) != kOk) return rc;

  TcParams p;
  p.O = pr.O;
  p.cuQ = pr.cuQ;
  p.cuKV = pr.cuKV;
  p.seqLenQ = pr.seqLenQ;
  p.seqLenKV = pr.seqLenKV;
  p.headsQ = pr.headsQ;
  p.headsKV = pr.headsKV;
  p.headDim = pr.headDim;
  p.group = pr.headsQ / pr.headsKV;
  p.packShift = packShift;
  const int seqPerCta = kNT * rowsPerTile;
  p.numPairs = (pr.seqLenQ + seqPerCta - 1) / seqPerCta;
  p.causal = pr.causal;
  p.scaleLog2 = (float)(1.4426950408889634 / sqrt((double)pr.headDim));
  p.status = device_status_word(device);
  p.epoch = next_epoch();
  if (p.status == nullptr) return kCudaError;
  p.numUnits = pr.headsQ / gp;
  const long long numWork = (long long)p.numPairs * p.numUnits * pr.batch;
  if (numWork > 0x7FFFFFFFll) {
    set_error_string("too many work items (%lld)", numWork);
    return kTooLarge;
  }
  p.numWork = (int)numWork;
  // Causal problems: heaviest query tile pairs first inside chunks of (head unit, batch) entries.  A chunk is as wide
  // as the KV heads whose K and V fit a quarter of the L2 (32 MB) together, and at least wide enough to hold two
  // items per SM.  Option "work_order": -1 this rule, 0 pair index fastest, n > 0 chunks of n entries.
  const int order = option_work_order();
  p.chunk = 0;
  if (order > 0) {
    const long long per = (long long)p.numUnits * pr.batch;
    p.chunk = (int)(order < per ? order : per);
  } else if (order < 0 && pr.causal) {
    const long long kvPerHead = 4ll * pr.seqLenKV * pr.headDim;  // K and V of one KV head, 16-bit elements
    const int unitsPerKvHead = (p.group >> packShift) > 0 ? (p.group >> packShift) : 1;
    long long heads = (32ll << 20) / (kvPerHead > 0 ? kvPerHead : 1);
    if (heads < 1) heads = 1;
    long long width = heads * unitsPerKvHead;
    // two items per worker: a worker is a CTA, or in the pair form a cluster of two
    const long long workers = pair ? device_num_sms(device) / 2 : device_num_sms(device);
    const long long minWidth = (2ll * workers + p.numPairs - 1) / p.numPairs;
    if (width < minWidth) width = minWidth;
    const long long per = (long long)p.numUnits * pr.batch;
    if (width > per) width = per;
    // equal chunks: a narrow last chunk would start its heaviest items when everything else is about to finish
    const long long chunks = (per + width / 2) / width > 0 ? (per + width / 2) / width : 1;
    p.chunk = (int)((per + chunks - 1) / chunks);
  }
  int rcCounter = kCudaError;
  CUtensorMap* slotMaps = nullptr;
  p.workCounter = device_work_counter(device, pr.stream, &rcCounter, &slotMaps);
  if (p.workCounter == nullptr) return rcCounter;
  p.devMaps = nullptr;
  if (devMaps) {
    if ((rc = launch_patch_varlen_maps(tmQ, tmK, tmV, slotMaps, pr.cuQ, pr.cuKV, pr.batch, pr.stream)) != kOk) return rc;
    p.devMaps = slotMaps;
  }

  // persistent: one CTA per SM (512 tensor-memory columns and ~200 KB of shared memory each), or two of the small form
  const long long slots = (long long)device_num_sms(device) * (solo ? 2 : 1);
  const int ctas = (int)(numWork < slots ? numWork : slots);
  cudaError_t e;
  if (pair) {
    // one cluster of two CTAs per work item in flight; as many clusters as the device runs at once
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = (size_t)smemBytes;
    cfg.stream = pr.stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    static int maxClusters[64] = {0};
    if (maxClusters[device] == 0) {
      cfg.gridDim = dim3((unsigned)(2 * (device_num_sms(device) / 2)));
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();
        n = device_num_sms(device) / 2;
      }
      maxClusters[device] = n;
    }
    const long long clusters = numWork < maxClusters[device] ? numWork : maxClusters[device];
    cfg.gridDim = dim3((unsigned)(2 * clusters));
    e = cudaLaunchKernelEx(&cfg, kernel, tmQ, tmK, tmV, p);
  } else {
    kernel<<<dim3((unsigned)ctas), threads, smemBytes, pr.stream>>>(tmQ, tmK, tmV, p);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    set_error_string("kernel launch failed: %s", cudaGetErrorString(e));
    return kCudaError;
  }
  return kOk;
}


}  // namespace tfa_b200

// extern "C" boundary of libtinyfa_b200.so: argument validation, run-time dispatch on
// (dtype, head dim) and the per-device bookkeeping the kernels need.
//
// Takes the place of the reference's dispatch macros TFA_DISPATCH_KERNEL / TFA_DISPATCH_ARCH /
// TFA_DISPATCH_HEAD_DIM (reference csrc/flash_attn/flash_api.cuh:27-41, config.cuh:86-100, 276-333):
// where the reference turns (compute capability, head dim, causal) into template arguments and aborts
// on an unsupported head dim, this file requires compute capability 10.x and returns status codes.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <thread>
#include <unordered_map>

#include "../../include/tinyfa_b200.h"
#include "build_config.cuh"
#include "ptx_sm100.cuh"
#include "tfa_common.cuh"

namespace tfa_b200 {

// ---- instantiations (fwd_tc_inst.cu, one object per pair)
// Only the (padded head dim, dtype) pairs selected at build time exist as objects.
#define TFA_DECLARE_TC(HDP)                                                               \
  int launch_fwd_tc_hdp##HDP##_bf0(const FwdProblem&, int);                               \
  int launch_fwd_tc_hdp##HDP##_bf1(const FwdProblem&, int);                               \
  static inline int tc_call_hdp##HDP(const FwdProblem& p, int packShift, bool bf16) {     \
    (void)p; (void)packShift;                                                             \
    if (bf16) {                                                                           \
      if constexpr (TFA_HAVE_BF16) return launch_fwd_tc_hdp##HDP##_bf1(p, packShift);     \
    } else {                                                                              \
      if constexpr (TFA_HAVE_FP16) return launch_fwd_tc_hdp##HDP##_bf0(p, packShift);     \
    }                                                                                     \
    return kBadDtype;                                                                     \
  }
#if TFA_HAVE_HDP64
TFA_DECLARE_TC(64)
#endif
#if TFA_HAVE_HDP128
TFA_DECLARE_TC(128)
#endif
#if TFA_HAVE_HDP192
TFA_DECLARE_TC(192)
#endif
#if TFA_HAVE_HDP256
TFA_DECLARE_TC(256)
#endif
#undef TFA_DECLARE_TC

// ---- split-KV path for short query blocks (fwd_decode.cu)
bool splitkv_applicable(const FwdProblem& p);
int splitkv_num_splits(const FwdProblem& p, int numSMs);
size_t splitkv_scratch_floats(const FwdProblem& p, int splits);
int launch_fwd_splitkv(const FwdProblem& p, int splits, float* scratch);

static thread_local char g_err[512] = "";

void set_error_string(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

static std::atomic<int> g_optPackGqa{-1};
static std::atomic<int> g_optSplitKv{-1};  // -1 auto, 0 never, n > 0 force n splits when applicable
static std::atomic<int> g_optWorkOrder{-1};  // -1 auto, 0 pair index fastest, n > 0 heaviest first in chunks of n
static std::atomic<int> g_epoch{1};

int option_work_order() { return g_optWorkOrder.load(); }
static std::atomic<int> g_optNarrowMma{1};
int option_narrow_mma() { return g_optNarrowMma.load(); }
static std::atomic<int> g_optSolo64{1};  // head dims 32 / 64: one-tile CTAs, two per SM (measured 4-10 % faster than the two-tile form)
int option_solo64() { return g_optSolo64.load(); }
static std::atomic<int> g_optPairCta{-1};  // head dims 192 / 256, fixed length: clusters of two CTAs sharing every K/V block (-1 auto)
int option_pair_cta() { return g_optPairCta.load(); }
static std::atomic<int> g_optFp32T8{1};  // fp32, head dim 128, large problems: the 8 x 8 thread-tile form
int option_fp32_t8() { return g_optFp32T8.load(); }

int next_epoch() { return (g_epoch.fetch_add(1) & 0x7FFFFF) + 1; }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess) return (EncodeTiledFn) nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  if (fn == nullptr) set_error_string("cuTensorMapEncodeTiled is not available from the driver");
  return fn;
}

// One small block of ints per device, allocated on first use and kept for the life of the process: word 0 is the
// status word, followed by (work, done) counter pairs of the persistent kernel.  Both counters of a pair are zero
// whenever no launch that uses them is running, because the last CTA of a launch to finish puts them back to zero
// (no memset on the launch path).  Launches that may run at the same time must not share a pair, so:
//   - an eager launch takes the pair of its stream (launches on one stream run one after the other); the per-thread
//     default stream is one handle for many streams and is told apart by the calling thread;
//   - a launch that is being captured into a CUDA graph takes a pair of its own that is never handed out again: the
//     graph may later be replayed on any stream, next to anything.
// kStreamPairs distinct streams and kCapturePairs captured launches per device are supported; past that the call
// returns TFA_B200_TOO_LARGE instead of sharing a pair (two kernels on one pair would steal each other's work items).
constexpr int kStreamPairs = 1024;
constexpr int kCapturePairs = 3072;
static std::mutex g_devMutex;
static int* g_statusWord[64] = {nullptr};
static int g_devChecked[64] = {0};  // 0 = unknown, 1 = cc 10.x, -1 = other
struct StreamKey {
  cudaStream_t stream;
  std::thread::id thread;  // only for the per-thread default stream
  bool operator==(const StreamKey& o) const { return stream == o.stream && thread == o.thread; }
};
struct StreamKeyHash {
  size_t operator()(const StreamKey& k) const {
    return std::hash<void*>()(static_cast<void*>(k.stream)) ^ (std::hash<std::thread::id>()(k.thread) * 1000003u);
  }
};
static std::unordered_map<StreamKey, int, StreamKeyHash> g_streamPair[64];
static int g_capturePairsUsed[64] = {0};
// Beside every counter pair: room for three tensor maps (Q, K, V) that a launch completes on the device when the
// host does not know the packed tensors' row totals (patch_varlen_maps below).  Same sharing rule as the counters.
static CUtensorMap* g_mapBlock[64] = {nullptr};

static int* device_block_locked(int device) {
  if (device < 0 || device >= 64) return nullptr;
  if (g_statusWord[device] == nullptr) {
    int* p = nullptr;
    const size_t bytes = sizeof(int) * (1 + 2 * (kStreamPairs + kCapturePairs));
    if (cudaMalloc(&p, bytes) != cudaSuccess || cudaMemset(p, 0, bytes) != cudaSuccess) {
      set_error_string("could not allocate the device status word: %s", cudaGetErrorString(cudaGetLastError()));
      return nullptr;
    }
    CUtensorMap* maps = nullptr;
    if (cudaMalloc(&maps, sizeof(CUtensorMap) * 3 * (kStreamPairs + kCapturePairs)) != cudaSuccess) {
      set_error_string("could not allocate the device tensor-map block: %s", cudaGetErrorString(cudaGetLastError()));
      cudaFree(p);
      return nullptr;
    }
    g_statusWord[device] = p;
    g_mapBlock[device] = maps;
  }
  return g_statusWord[device];
}

int* device_status_word(int device) {
  std::lock_guard<std::mutex> lock(g_devMutex);
  return device_block_locked(device);
}

// (work, done) counter pair for one launch on `stream`; see above.  *rc receives the status when nullptr is returned.
int* device_work_counter(int device, cudaStream_t stream, int* rc, CUtensorMap** maps) {
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) {
    set_error_string("cudaStreamIsCapturing: %s", cudaGetErrorString(cudaGetLastError()));
    *rc = kCudaError;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_devMutex);
  int* base = device_block_locked(device);
  if (base == nullptr) {
    *rc = kCudaError;
    return nullptr;
  }
  if (cap != cudaStreamCaptureStatusNone) {
    if (g_capturePairsUsed[device] >= kCapturePairs) {
      set_error_string("more than %d launches of this library captured into CUDA graphs on device %d", kCapturePairs, device);
      *rc = kTooLarge;
      return nullptr;
    }
    const int slot = kStreamPairs + g_capturePairsUsed[device]++;
    if (maps != nullptr) *maps = g_mapBlock[device] + 3 * slot;
    return base + 1 + 2 * slot;
  }
  StreamKey key{stream, stream == cudaStreamPerThread ? std::this_thread::get_id() : std::thread::id()};
  auto& table = g_streamPair[device];
  auto it = table.find(key);
  if (it == table.end()) {
    if ((int)table.size() >= kStreamPairs) {
      set_error_string("more than %d distinct streams used with this library on device %d", kStreamPairs, device);
      *rc = kTooLarge;
      return nullptr;
    }
    it = table.emplace(key, (int)table.size()).first;
  }
  if (maps != nullptr) *maps = g_mapBlock[device] + 3 * it->second;
  return base + 1 + 2 * it->second;
}

// Completes the tensor maps of a packed variable-length launch on the device: the three maps arrive as kernel
// arguments with a placeholder row count, the real counts are cuQ[batch] and cuKV[batch] (the reference reads its
// lengths on the device as well, reference csrc/flash_attn/params.cuh:89-94).  One warp; the maps go to `out` in
// global memory, from where the attention kernel of the same stream uses them.
__global__ void patch_varlen_maps(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                                  const __grid_constant__ CUtensorMap mv, CUtensorMap* out, const int* cuQ,
                                  const int* cuKV, int batch) {
  __shared__ alignas(128) CUtensorMap sm[3];
  const int lane = threadIdx.x;
  const CUtensorMap* src[3] = {&mq, &mk, &mv};
#pragma unroll
  for (int i = 0; i < 3; i++) reinterpret_cast<uint32_t*>(&sm[i])[lane] = reinterpret_cast<const uint32_t*>(src[i])[lane];
  __syncwarp();
  if (lane == 0) {
    const int rowsQ = cuQ[batch], rowsKV = cuKV[batch];
    // an extent of zero is not a valid tensor map; with no rows the attention kernel finds no work and loads nothing
    ptx::tensormap_set_dim2(ptx::smem_u32(&sm[0]), (uint32_t)(rowsQ > 0 ? rowsQ : 1));
    ptx::tensormap_set_dim2(ptx::smem_u32(&sm[1]), (uint32_t)(rowsKV > 0 ? rowsKV : 1));
    ptx::tensormap_set_dim2(ptx::smem_u32(&sm[2]), (uint32_t)(rowsKV > 0 ? rowsKV : 1));
  }
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 3; i++) ptx::tensormap_publish(out + i, ptx::smem_u32(&sm[i]));
}

int launch_patch_varlen_maps(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, CUtensorMap* out,
                             const int* cuQ, const int* cuKV, int batch, cudaStream_t stream) {
  patch_varlen_maps<<<1, 32, 0, stream>>>(mq, mk, mv, out, cuQ, cuKV, batch);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error_string("tensor-map patch kernel launch failed: %s", cudaGetErrorString(e));
    return kCudaError;
  }
  return kOk;
}

// Stream-ordered scratch for the split-KV partials comes from a pool of this library's own, one per device, that
// keeps its memory across synchronisations (release threshold = max): with the default pool every call that
// follows a device synchronise would pay a fresh device allocation (~200 us, measured).
static cudaMemPool_t g_scratchPool[64] = {nullptr};
static cudaMemPool_t scratch_pool(int device) {
  std::lock_guard<std::mutex> lock(g_devMutex);
  if (device < 0 || device >= 64) return nullptr;
  if (g_scratchPool[device] == nullptr) {
    cudaMemPoolProps props;
    memset(&props, 0, sizeof(props));
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = device;
    cudaMemPool_t pool = nullptr;
    if (cudaMemPoolCreate(&pool, &props) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    unsigned long long keep = ~0ull;
    cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    g_scratchPool[device] = pool;
  }
  return g_scratchPool[device];
}

int device_num_sms(int device) {
  static int cached[64] = {0};
  if (device < 0 || device >= 64) return 148;
  if (cached[device] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
    cached[device] = n;
  }
  return cached[device];
}

int check_device() {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) {
    set_error_string("cudaGetDevice: %s", cudaGetErrorString(e));
    return kCudaError;
  }
  if (device < 0 || device >= 64) return kBadArgument;
  std::lock_guard<std::mutex> lock(g_devMutex);
  if (g_devChecked[device] == 0) {
    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    if (e != cudaSuccess) {
      set_error_string("cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
      return kCudaError;
    }
    g_devChecked[device] = (major == 10) ? 1 : -1;
  }
  if (g_devChecked[device] != 1) {
    set_error_string("device %d is not compute capability 10.x; this library contains sm_100a code only", device);
    return kWrongDevice;
  }
  return kOk;
}

static bool head_dim_ok(int d) { return d == 32 || d == 64 || d == 96 || d == 128 || d == 192 || d == 256; }

// A (dtype, padded head dim) kernel that the build left out: same message style as an unsupported head dim.
static int not_compiled(const FwdProblem& p) {
  set_error_string("TinyFA: kernel for dtype code %d, headDim %d was not compiled into this library "
                   "(TFA_TARGET_HEADDIM_<N> / TFA_TARGET_DTYPE build switches)", p.dtype, p.headDim);
  return dtype_compiled(p.dtype) ? kBadHeadDim : kBadDtype;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int pick_pack_shift(const FwdProblem& p) {
  const int group = p.headsQ / p.headsKV;
  int shift = 0;
  while (((group >> (shift + 1)) << (shift + 1)) == group && (1 << (shift + 1)) <= 128) shift++;  // pow-2 part
  const int opt = g_optPackGqa.load();
  if (opt == 0 || shift == 0) return 0;
  if (opt == 1) return shift;
  // auto: short query blocks share one tile across the group's heads; so do causal problems of any length - with the
  // heads of a group interleaved, the two tiles of a work item cover 128 >> shift positions each inside one 128-key
  // block and therefore run the same number of key blocks (one head per tile: tile 1 has one block more and tile 0
  // idles for it).  Measured on causal Hq32 / Hkv8 hd128: +2.0 % (B4 S8192), +2.6 % (B2 S4096), +3.6 % (B8 S2048);
  // non-causal: no difference, tiles stay one head wide there.
  return (p.seqLenQ < 128 || p.causal) ? shift : 0;
}

static int num_sms() {
  static int cached[64] = {0};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
  if (cached[device] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
    cached[device] = n;
  }
  return cached[device];
}

// Short query blocks: stream K/V once for all Q heads of a KV head and split the key range over CTAs.  The partial
// results live in a stream-ordered scratch allocation that is released behind the combine kernel.
static int dispatch_splitkv(const FwdProblem& p, int splits) {
  const size_t floats = splitkv_scratch_floats(p, splits);
  float* scratch = nullptr;
  if (floats > 0) {
    int device = 0;
    cudaGetDevice(&device);
    cudaMemPool_t pool = scratch_pool(device);
    cudaError_t e = (pool != nullptr)
                        ? cudaMallocFromPoolAsync(reinterpret_cast<void**>(&scratch), floats * sizeof(float), pool, p.stream)
                        : cudaMallocAsync(reinterpret_cast<void**>(&scratch), floats * sizeof(float), p.stream);
    if (e != cudaSuccess) {
      set_error_string("cudaMallocAsync(%zu bytes) for split-KV partials: %s", floats * sizeof(float),
                       cudaGetErrorString(e));
      return kCudaError;
    }
  }
  const int rc = launch_fwd_splitkv(p, splits, scratch);
  if (scratch != nullptr) cudaFreeAsync(scratch, p.stream);
  return rc;
}

static int dispatch(const FwdProblem& p) {
  if (p.dtype == kFp32) return launch_fwd_fp32(p);
  const int optSplit = g_optSplitKv.load();
  if (optSplit != 0 && p.totalQ >= 0 && splitkv_applicable(p)) {
    int splits = (optSplit > 0) ? optSplit : splitkv_num_splits(p, num_sms());
    const int maxSplits = (p.seqLenKV + 63) / 64;
    if (splits > maxSplits) splits = maxSplits;
    return dispatch_splitkv(p, splits);
  }
  const bool bf = (p.dtype == kBf16);
  const int ps = pick_pack_shift(p);
  switch (p.headDim) {
    case 32:
    case 64:
#if TFA_HAVE_HDP64
      return tc_call_hdp64(p, ps, bf);
#else
      break;
#endif
    case 96:
    case 128:
#if TFA_HAVE_HDP128
      return tc_call_hdp128(p, ps, bf);
#else
      break;
#endif
    case 192:
#if TFA_HAVE_HDP192
      return tc_call_hdp192(p, ps, bf);
#else
      break;
#endif
    case 256:
#if TFA_HAVE_HDP256
      return tc_call_hdp256(p, ps, bf);
#else
      break;
#endif
    default:
      return kBadHeadDim;
  }
  (void)ps;
  (void)bf;
  return not_compiled(p);
}

int validate_common(const void* Q, const void* K, const void* V, void* O, int dtype, int batch, int sq, int skv,
                           int hq, int hkv, int d) {
  if (dtype != kFp16 && dtype != kBf16 && dtype != kFp32) {
    set_error_string("unsupported dtype code %d (1 = fp16, 2 = bf16, 3 = fp32)", dtype);
    return kBadDtype;
  }
  if (!head_dim_ok(d)) {
    set_error_string("TinyFA: unsupported headDim: %d", d);
    return kBadHeadDim;
  }
  if (!dtype_compiled(dtype)) {
    set_error_string("TinyFA: dtype code %d was not compiled into this library (TFA_TARGET_DTYPE build switch)", dtype);
    return kBadDtype;
  }
  if (!head_dim_compiled(d)) {
    set_error_string("TinyFA: headDim %d was not compiled into this library (TFA_TARGET_HEADDIM_%d build switch)", d, d);
    return kBadHeadDim;
  }
  if (batch < 0 || sq < 0 || skv < 0 || hq <= 0 || hkv <= 0) {
    set_error_string("negative size or non-positive head count (batch=%d seqQ=%d seqKV=%d Hq=%d Hkv=%d)", batch, sq,
                     skv, hq, hkv);
    return kBadArgument;
  }
  if (hq % hkv != 0) {
    set_error_string("numHeadsQ (%d) must be divisible by numHeadsKV (%d)", hq, hkv);
    return kBadArgument;
  }
  if (batch > 65535 || hq > 65535) {
    set_error_string("batchSize and numHeadsQ are limited to 65535 (grid dimensions)");
    return kTooLarge;
  }
  if (batch > 0 && sq > 0 && (Q == nullptr || O == nullptr || (skv > 0 && (K == nullptr || V == nullptr)))) {
    set_error_string("null tensor pointer");
    return kBadArgument;
  }
  if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(O)) {
    set_error_string("Q, K, V and O must be 16-byte aligned");
    return kBadArgument;
  }
  return kOk;
}

}  // namespace tfa_b200

using namespace tfa_b200;

extern "C" int tfa_b200_fwd(const void* Q, const void* K, const void* V, void* O, int dtype, int batchSize,
                            int seqLenQ, int seqLenKV, int numHeadsQ, int numHeadsKV, int headDim, int isCausal,
                            void* stream) {
  int rc = validate_common(Q, K, V, O, dtype, batchSize, seqLenQ, seqLenKV, numHeadsQ, numHeadsKV, headDim);
  if (rc != kOk) return rc;
  if (batchSize == 0 || seqLenQ == 0 || seqLenKV == 0) return kOk;  // nothing to write
  if ((long long)batchSize * seqLenQ > 0x7FFFFFFFll || (long long)batchSize * seqLenKV > 0x7FFFFFFFll) {
    set_error_string("batchSize * seqLen must stay below 2^31 rows");
    return kTooLarge;
  }
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
  return dispatch(p);
}

extern "C" int tfa_b200_fwd_varlen(const void* Q, const void* K, const void* V, void* O, const int* cuSeqLensQ,
                                   const int* cuSeqLensKV, int dtype, int batchSize, int maxSeqLenQ, int maxSeqLenKV,
                                   long long totalQ, long long totalKV, int numHeadsQ, int numHeadsKV, int headDim,
                                   int isCausal, void* stream) {
  int rc = validate_common(Q, K, V, O, dtype, batchSize, maxSeqLenQ, maxSeqLenKV, numHeadsQ, numHeadsKV, headDim);
  if (rc != kOk) return rc;
  if (batchSize == 0 || maxSeqLenQ == 0 || maxSeqLenKV == 0) return kOk;
  if (cuSeqLensQ == nullptr || cuSeqLensKV == nullptr) {
    set_error_string("null cu_seqlens pointer");
    return kBadArgument;
  }
  if ((rc = check_device()) != kOk) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // Totals the caller does not know (the reference signature has none): the tensor-core path completes its tensor
  // maps on the device from cu_seqlens[batch]; nothing is read back and the call stays asynchronous.
  if (totalQ < 0 || totalKV < 0) totalQ = totalKV = -1;
  if (totalQ == 0 || totalKV == 0) return kOk;
  if (totalQ > 0x7FFFFFFFll || totalKV > 0x7FFFFFFFll) return kTooLarge;
  FwdProblem p;
  p.Q = Q;
  p.K = K;
  p.V = V;
  p.O = O;
  p.cuQ = cuSeqLensQ;
  p.cuKV = cuSeqLensKV;
  p.dtype = dtype;
  p.batch = batchSize;
  p.seqLenQ = maxSeqLenQ;
  p.seqLenKV = maxSeqLenKV;
  p.totalQ = totalQ;
  p.totalKV = totalKV;
  p.headsQ = numHeadsQ;
  p.headsKV = numHeadsKV;
  p.headDim = headDim;
  p.causal = isCausal ? 1 : 0;
  p.stream = s;
  return dispatch(p);
}

extern "C" int tfa_b200_head_dim_supported(int headDim) { return head_dim_compiled(headDim) ? 1 : 0; }

extern "C" const char* tfa_b200_last_error_string(void) { return g_err; }

extern "C" int tfa_b200_device_status(int* site) {
  if (site != nullptr) *site = 0;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return kCudaError;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    set_error_string("cudaDeviceSynchronize: %s", cudaGetErrorString(e));
    return kCudaError;
  }
  int* word = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_devMutex);
    if (device >= 0 && device < 64) word = g_statusWord[device];
  }
  if (word == nullptr) return kOk;  // no kernel of this library has run on this device yet
  int v = 0;
  if (cudaMemcpy(&v, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return kCudaError;
  if (v == 0) return kOk;
  cudaMemset(word, 0, sizeof(int));
  if (site != nullptr) *site = v & 0xFF;
  if ((v & 0xFF) == 30) {
    set_error_string("two launches used one pair of work counters at the same time (launch epoch %d): results of both "
                     "are incomplete", v >> 8);
  } else {
    set_error_string("a kernel gave up on a bounded wait (site %d, launch epoch %d)", v & 0xFF, v >> 8);
  }
  return kDeviceTimeout;
}

extern "C" int tfa_b200_set_option(const char* name, int value) {
  if (name == nullptr) return kBadArgument;
  if (strcmp(name, "pack_gqa") == 0) {
    g_optPackGqa.store(value < 0 ? -1 : (value ? 1 : 0));
    return kOk;
  }
  if (strcmp(name, "split_kv") == 0) {
    g_optSplitKv.store(value < 0 ? -1 : value);
    return kOk;
  }
  if (strcmp(name, "narrow_mma") == 0) {
    g_optNarrowMma.store(value ? 1 : 0);
    return kOk;
  }
  if (strcmp(name, "solo64") == 0) {
    g_optSolo64.store(value ? 1 : 0);
    return kOk;
  }
  if (strcmp(name, "fp32_t8") == 0) {
    g_optFp32T8.store(value < 0 ? 1 : (value > 2 ? 2 : value));
    return kOk;
  }
  if (strcmp(name, "pair_cta") == 0) {
    g_optPairCta.store(value < 0 ? -1 : (value ? 1 : 0));
    return kOk;
  }
  if (strcmp(name, "work_order") == 0) {
    g_optWorkOrder.store(value < 0 ? -1 : value);
    return kOk;
  }
  set_error_string("unknown option '%s'", name);
  return kBadArgument;
}

extern "C" const char* tfa_b200_version(void) { return "tinyfa_b200 0.1 (sm_100a)"; }

/*
 * C ABI of the B200-native attention-forward library (libtinyfa_b200.so).
 *
 * This is the drop-in boundary for the reference's forward path: each entry point below names the
 * reference interface it stands in for.  Plain pointers and sizes only; all tensor pointers are
 * DEVICE pointers owned by the caller; work is enqueued asynchronously on `stream` (a cudaStream_t
 * passed as void*, NULL = the legacy default stream); the library keeps no handle.
 *
 * dtype codes (reference csrc/binding/flash_attn_binding.cu:22): 1 = fp16, 2 = bf16, 3 = fp32.
 * Every function returning int returns 0 on success or one of the TFA_B200_* codes.
 *
 * Streams and CUDA graphs: the first call on a device creates a few KB of per-device state (a status word, work
 * counters and tensor-map slots, shared-memory opt-in of the kernels, a scratch pool) with synchronous calls; make it
 * outside a stream capture.  After that a forward call only enqueues kernels on `stream` (the split-KV path of
 * tfa_b200_fwd also a stream-ordered allocation and free; tfa_b200_fwd_decode_noalloc none), so it can be captured
 * into a CUDA graph and replayed.  The persistent kernel hands out its work through a pair of device counters that two
 * launches must not use at the same time: eager launches take the pair of their stream (up to 1024 distinct streams
 * per device; the per-thread default stream counts once per calling thread), every captured launch takes a pair of
 * its own for good (up to 3072 per device), past either limit the call returns TFA_B200_TOO_LARGE.  So eager launches
 * on any streams and replays of captured graphs can run side by side; the one thing to avoid is instantiating one
 * captured graph twice and running both executables at the same time.  Should two launches share a pair all the same,
 * tfa_b200_device_status reports it (site 30).
 */
#ifndef TINYFA_B200_H_
#define TINYFA_B200_H_

#ifdef __cplusplus
extern "C" {
#endif

#define TFA_B200_OK 0
#define TFA_B200_BAD_DTYPE 1
#define TFA_B200_BAD_HEAD_DIM 2
#define TFA_B200_BAD_ARGUMENT 3
#define TFA_B200_CUDA_ERROR 4
#define TFA_B200_WRONG_DEVICE 5
#define TFA_B200_TOO_LARGE 6
#define TFA_B200_DEVICE_TIMEOUT 7

/*
 * Fixed-length forward.  Replaces tfa::flashAttn<DType> (reference csrc/flash_attn/flash_api.cuh:43-50)
 * and the explicit instantiations impl::runFwd<Arch,DType,HD,Causal> it dispatches to
 * (flash_api.cuh:17-19, csrc/flash_attn/launcher.cuh:68-81).
 *   Q, O : [batchSize, seqLenQ,  numHeadsQ,  headDim]   K, V : [batchSize, seqLenKV, numHeadsKV, headDim]
 * dense row-major, 16-byte aligned.  Scale is 1/sqrt(headDim); causal masking is top-left aligned
 * (key j visible to query i iff j <= i).  O is written for every query row when seqLenKV > 0 and is
 * left untouched when seqLenKV == 0 (reference csrc/flash_attn/mma/kernel.cuh:39-42).
 */
int tfa_b200_fwd(const void* Q, const void* K, const void* V, void* O, int dtype, int batchSize, int seqLenQ,
                 int seqLenKV, int numHeadsQ, int numHeadsKV, int headDim, int isCausal, void* stream);

/*
 * Packed variable-length forward.  Replaces tfa::flashAttnVarLen<DType> (reference
 * csrc/flash_attn/flash_api.cuh:52-60) and impl::runFwdVarlen (launcher.cuh:83-99).
 *   Q, O : [totalQ, numHeadsQ, headDim]   K, V : [totalKV, numHeadsKV, headDim]
 *   cuSeqLensQ / cuSeqLensKV : int32 [batchSize + 1] prefix sums, DEVICE pointers.
 * maxSeqLenQ / maxSeqLenKV only size the launch, as in the reference (launcher.cuh:94-98).
 * totalQ / totalKV are the row counts of the packed tensors (= cuSeqLens[batchSize]); the reference signature does
 * not carry them, so a caller that only has the reference's arguments passes -1 for both.  The call stays
 * asynchronous either way, as the reference's is (launcher.cuh:83-99): with -1 a one-warp kernel on `stream` reads the
 * two totals from cuSeqLens on the device and completes the tensor maps there; nothing is copied back to the host.
 */
int tfa_b200_fwd_varlen(const void* Q, const void* K, const void* V, void* O, const int* cuSeqLensQ,
                        const int* cuSeqLensKV, int dtype, int batchSize, int maxSeqLenQ, int maxSeqLenKV,
                        long long totalQ, long long totalKV, int numHeadsQ, int numHeadsKV, int headDim,
                        int isCausal, void* stream);

/* Replaces tfa::isHeadDimCompiled (reference csrc/flash_attn/config.cuh:102-131): 1 for 32/64/96/128/192/256. */
int tfa_b200_head_dim_supported(int headDim);

/*
 * Human-readable text for the last non-zero status returned on the calling thread.  Stands in for the
 * reference's stderr messages (reference csrc/flash_attn/utils.cuh:17-24, config.cuh:95-98).
 */
const char* tfa_b200_last_error_string(void);

/*
 * Synchronises the current device and reports whether any kernel of this library gave up on one of its
 * bounded waits since the last call (TFA_B200_DEVICE_TIMEOUT) or 0.  *site, when not NULL, receives the
 * code of the wait that gave up.  The reference never checks its launches (launcher.cuh:39); this is an
 * addition for tests and health checks.
 */
int tfa_b200_device_status(int* site);

/*
 * Tuning / debugging knobs (process-wide).  No counterpart in the reference, whose tile table is fixed
 * at compile time (csrc/flash_attn/config.cuh:133-272).
 *   "pack_gqa" -1/0/1  interleave the Q heads of a KV group into one 128-row tile: auto (short query blocks and
 *                      causal problems) / never / always
 *   "split_kv" -1/0/n  split-KV path for short query blocks (seqQ * group <= 16): auto / never / exactly n splits
 *   "narrow_mma" 0/1   head dims 32 / 96: MMAs of the padded width (64 / 128) / MMAs shaped for the head dim (the default)
 *   "solo64" 0/1       head dims 32 / 64: two-tile CTAs, one per SM / one-tile CTAs, two per SM (the default)
 *   "fp32_t8" 0/1/2    fp32, head dim 128: 4 x 8 thread tiles always / 8 x 8 thread tiles for problems of at least three
 *                      CTAs per SM (the default) / 8 x 8 always
 *   "pair_cta" -1/0/1  head dims 192 / 256, fixed-length input: clusters of two CTAs that work on two neighbouring query
 *                      tiles and share every K/V block through one MMA over both SMs (tcgen05 cta_group::2):
 *                      auto (head dim 256: non-causal, and causal from 1024 query rows; head dim 192: never, its
 *                      one-tile form measures as fast) / never / wherever it applies.  Results are bit-identical to
 *                      the one-tile form.
 *   "work_order" -1/0/n  order in which the persistent kernel hands out (query tile pair, head, batch) items:
 *                      auto (causal: heaviest pairs first inside chunks of heads whose K/V fit a quarter of L2;
 *                      otherwise pair index fastest) / pair index fastest / heaviest first in chunks of n heads
 * Returns TFA_B200_BAD_ARGUMENT for an unknown name.
 */
int tfa_b200_set_option(const char* name, int value);

const char* tfa_b200_version(void);

/*
 * Allocation-free decode forward.  No counterpart in the reference (which has neither a split-KV path nor any
 * scratch memory).  Same tensors, layouts and result as tfa_b200_fwd, restricted to what the split-KV kernel
 * handles: fp16 / bf16, every supported headDim, seqLenQ * (numHeadsQ / numHeadsKV) <= 16, seqLenKV >= 256.
 *
 * For callers that cannot let a library allocate: engines that hand all device memory to their own planner at
 * start-up, and decode loops that must not risk a stalling or failing driver allocation.  tfa_b200_fwd keeps the
 * partial results of its key-range splits in a stream-ordered allocation; this entry point keeps them in a fixed
 * array inside the library image, TFA_B200_NOALLOC_SCRATCH_FLOATS floats (16 MiB) per GPU that loads the library,
 * held until the process exits.  It calls no cudaMalloc / cudaFree / allocating routine of any kind.
 *
 * numSplits: 0 lets the library choose, n > 0 asks for n key-range splits.  The partials need
 * numSplits * batchSize * seqLenQ * numHeadsQ * (headDim + 1) floats (none for one split); a call that needs more
 * than the array holds returns TFA_B200_TOO_LARGE and launches nothing.
 *
 * The first call on each device resolves the array's device address (cudaGetSymbolAddress, with that device
 * current); make that first call before starting any stream capture.  All calls on a device share the one array:
 * calls whose kernels can overlap on the GPU (different streams without ordering) race on it - serialise them.
 * The array keeps the last call's partials; nothing in it needs to be zero and nothing stale is ever read.
 */
#define TFA_B200_NOALLOC_SCRATCH_FLOATS (4u * 1024u * 1024u)
int tfa_b200_fwd_decode_noalloc(const void* Q, const void* K, const void* V, void* O, int dtype, int batchSize,
                                int seqLenQ, int seqLenKV, int numHeadsQ, int numHeadsKV, int headDim, int isCausal,
                                int numSplits, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TINYFA_B200_H_ */

// TEST / BENCHMARK INFRASTRUCTURE ONLY - never linked into the product library.
//
// extern "C" wrapper around the UNMODIFIED reference templates tfa::flashAttn<T> and
// tfa::flashAttnVarLen<T> (reference csrc/flash_attn/flash_api.cuh:43-60).  The reference
// sources are compiled where they lie (see oracle/Makefile, target ref_gpu); nothing of
// them is copied.  The result, oracle/_ref/libtinyfa_ref.so, is the "reference kernels
// compiled for sm_100a" comparator: on a cc 10.0 device the reference's own dispatcher
// takes its SM8x tile table (reference csrc/flash_attn/config.cuh:311-317), which is what
// -DTFA_TARGET_SM=89 pins at compile time.
//
// dtype codes follow the reference binding (csrc/binding/flash_attn_binding.cu:22):
// 1 = fp16, 2 = bf16, 3 = fp32.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "flash_attn/flash_api.cuh"

extern "C" int tfa_ref_fwd(const void* Q, const void* K, const void* V, void* O, int dtype, int batchSize,
                           int seqLenQ, int seqLenKV, int numHeadsQ, int numHeadsKV, int headDim, int isCausal,
                           void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!tfa::isHeadDimCompiled(headDim)) return 2;
  switch (dtype) {
    case 1:
      tfa::flashAttn<__half>((const __half*)Q, (const __half*)K, (const __half*)V, (__half*)O, batchSize, seqLenQ,
                             seqLenKV, numHeadsQ, numHeadsKV, headDim, isCausal != 0, s);
      return 0;
    case 2:
      tfa::flashAttn<__nv_bfloat16>((const __nv_bfloat16*)Q, (const __nv_bfloat16*)K, (const __nv_bfloat16*)V,
                                    (__nv_bfloat16*)O, batchSize, seqLenQ, seqLenKV, numHeadsQ, numHeadsKV, headDim,
                                    isCausal != 0, s);
      return 0;
#ifdef TFA_REF_HAS_FP32
    case 3:
      tfa::flashAttn<float>((const float*)Q, (const float*)K, (const float*)V, (float*)O, batchSize, seqLenQ,
                            seqLenKV, numHeadsQ, numHeadsKV, headDim, isCausal != 0, s);
      return 0;
#endif
    default:
      return 1;
  }
}

extern "C" int tfa_ref_fwd_varlen(const void* Q, const void* K, const void* V, void* O, const int* cuQ,
                                  const int* cuKV, int dtype, int batchSize, int maxSeqLenQ, int maxSeqLenKV,
                                  int numHeadsQ, int numHeadsKV, int headDim, int isCausal, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!tfa::isHeadDimCompiled(headDim)) return 2;
  switch (dtype) {
    case 1:
      tfa::flashAttnVarLen<__half>((const __half*)Q, (const __half*)K, (const __half*)V, (__half*)O, cuQ, cuKV,
                                   batchSize, maxSeqLenQ, maxSeqLenKV, numHeadsQ, numHeadsKV, headDim, isCausal != 0,
                                   s);
      return 0;
    case 2:
      tfa::flashAttnVarLen<__nv_bfloat16>((const __nv_bfloat16*)Q, (const __nv_bfloat16*)K, (const __nv_bfloat16*)V,
                                          (__nv_bfloat16*)O, cuQ, cuKV, batchSize, maxSeqLenQ, maxSeqLenKV, numHeadsQ,
                                          numHeadsKV, headDim, isCausal != 0, s);
      return 0;
#ifdef TFA_REF_HAS_FP32
    case 3:
      tfa::flashAttnVarLen<float>((const float*)Q, (const float*)K, (const float*)V, (float*)O, cuQ, cuKV, batchSize,
                                  maxSeqLenQ, maxSeqLenKV, numHeadsQ, numHeadsKV, headDim, isCausal != 0, s);
      return 0;
#endif
    default:
      return 1;
  }
}

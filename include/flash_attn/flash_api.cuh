// Drop-in replacement for the reference's public header, to be included under the same name
// ("flash_attn/flash_api.cuh", reference csrc/flash_attn/flash_api.cuh).  The two templates keep the
// reference's names, namespace, parameter order, types and defaults (flash_api.cuh:43-50 and :52-60) and
// tfa::isHeadDimCompiled keeps its signature (reference csrc/flash_attn/config.cuh:102-131); the bodies forward
// to the C ABI of libtinyfa_b200.so (tinyfa_b200.h) instead of dispatching to template instantiations.
//
// Error behaviour mirrors the reference: the functions return void; an unsupported head dim or a failed CUDA
// call prints to stderr and aborts (reference config.cuh:95-98, utils.cuh:17-24).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <type_traits>

#include "../tinyfa_b200.h"

namespace tfa {

using FP32 = float;
using FP16 = __half;
using BF16 = __nv_bfloat16;

namespace detail {

template <typename DType>
constexpr int dtypeCode() {
  static_assert(std::is_same_v<DType, float> || std::is_same_v<DType, __half> || std::is_same_v<DType, __nv_bfloat16>,
                "tfa::flashAttn supports float, __half and __nv_bfloat16");
  return std::is_same_v<DType, __half> ? 1 : (std::is_same_v<DType, __nv_bfloat16> ? 2 : 3);
}

inline void checkStatus(int status) {
  if (status != TFA_B200_OK) {
    fprintf(stderr, "TinyFA (B200): status %d: %s\n", status, tfa_b200_last_error_string());
    abort();
  }
}

}  // namespace detail

inline bool isHeadDimCompiled(int headDim) { return tfa_b200_head_dim_supported(headDim) != 0; }

template <typename DType>
void flashAttn(const DType* Q, const DType* K, const DType* V, DType* O, int batchSize, int seqLenQ, int seqLenKV,
               int numHeadsQ, int numHeadsKV, int headDim, bool isCausal = false, cudaStream_t stream = nullptr) {
  detail::checkStatus(tfa_b200_fwd(Q, K, V, O, detail::dtypeCode<DType>(), batchSize, seqLenQ, seqLenKV, numHeadsQ,
                                   numHeadsKV, headDim, isCausal ? 1 : 0, stream));
}

template <typename DType>
void flashAttnVarLen(const DType* Q, const DType* K, const DType* V, DType* O, const int* cuSeqLensQ,
                     const int* cuSeqLensKV, int batchSize, int maxSeqLenQ, int maxSeqLenKV, int numHeadsQ,
                     int numHeadsKV, int headDim, bool isCausal = false, cudaStream_t stream = nullptr) {
  // The reference signature carries no row totals: -1 lets the library read them from cuSeqLens on the device.
  detail::checkStatus(tfa_b200_fwd_varlen(Q, K, V, O, cuSeqLensQ, cuSeqLensKV, detail::dtypeCode<DType>(), batchSize,
                                          maxSeqLenQ, maxSeqLenKV, -1, -1, numHeadsQ, numHeadsKV, headDim,
                                          isCausal ? 1 : 0, stream));
}

}  // namespace tfa

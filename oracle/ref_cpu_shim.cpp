// TEST / BENCHMARK INFRASTRUCTURE ONLY - never linked into the product library.
//
// extern "C" wrapper around the reference's own naive CPU attention,
// tfa::test::cpuAttentionFixedLen / cpuAttentionVarLen (reference tests/cpp/cpu_reference.h:14-66, 68-129).
// The header is included from where the reference lies; nothing of it is copied.  Built by
// oracle/Makefile (target ref_cpu) into oracle/_ref/libtinyfa_refcpu.so.
//
// The reference functions are single-threaded loops over (batch, head, row).  Every (batch, Q head)
// pair is independent, so to use all host cores this shim repacks one (batch, Q head) slice at a
// time into a dense [1, S, 1, D] problem and calls the UNCHANGED reference function on it from an
// OpenMP loop: the arithmetic executed for each output element is the reference's own, in the
// reference's own order.
#ifdef _OPENMP
#include <omp.h>
#endif

#include <algorithm>
#include <cstring>
#include <vector>

#include "cpu_reference.h"

extern "C" int tfa_refcpu_num_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

namespace {

// rows [row0, row0+n) of head h from a [rows, H, D] tensor -> dense [n, D]
void gatherHead(const float* src, float* dst, long row0, int n, int H, int h, int D) {
  for (int r = 0; r < n; r++) {
    std::memcpy(dst + (long)r * D, src + ((row0 + r) * H + h) * (long)D, sizeof(float) * D);
  }
}

void scatterHead(const float* src, float* dst, long row0, int n, int H, int h, int D) {
  for (int r = 0; r < n; r++) {
    std::memcpy(dst + ((row0 + r) * H + h) * (long)D, src + (long)r * D, sizeof(float) * D);
  }
}

}  // namespace

// Whole problem in one call of the reference function (single thread) - used to pin the port.
extern "C" void tfa_refcpu_fixed(const float* Q, const float* K, const float* V, float* O, int batchSize,
                                 int seqLenQ, int seqLenKV, int numHeadsQ, int numHeadsKV, int headDim,
                                 int isCausal) {
  tfa::test::cpuAttentionFixedLen(Q, K, V, O, batchSize, seqLenQ, seqLenKV, numHeadsQ, numHeadsKV, headDim,
                                  isCausal != 0);
}

extern "C" void tfa_refcpu_varlen(const float* Q, const float* K, const float* V, float* O, const int* cuQ,
                                  const int* cuKV, int batchSize, int numHeadsQ, int numHeadsKV, int headDim,
                                  int isCausal) {
  tfa::test::cpuAttentionVarLen(Q, K, V, O, cuQ, cuKV, batchSize, numHeadsQ, numHeadsKV, headDim, isCausal != 0);
}

// Multi-threaded: one reference call per (batch, Q head) slice.  qRows > 0 limits the work to the
// first qRows query rows of every sequence (a bounded sample for timing); 0 means all rows.
extern "C" void tfa_refcpu_fixed_mt(const float* Q, const float* K, const float* V, float* O, int batchSize,
                                    int seqLenQ, int seqLenKV, int numHeadsQ, int numHeadsKV, int headDim,
                                    int isCausal, int qRows) {
  const int group = numHeadsQ / numHeadsKV;
  const int nq = (qRows > 0) ? std::min(qRows, seqLenQ) : seqLenQ;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int b = 0; b < batchSize; b++) {
    for (int h = 0; h < numHeadsQ; h++) {
      std::vector<float> q((size_t)nq * headDim), k((size_t)seqLenKV * headDim), v((size_t)seqLenKV * headDim),
          o((size_t)nq * headDim);
      gatherHead(Q, q.data(), (long)b * seqLenQ, nq, numHeadsQ, h, headDim);
      gatherHead(K, k.data(), (long)b * seqLenKV, seqLenKV, numHeadsKV, h / group, headDim);
      gatherHead(V, v.data(), (long)b * seqLenKV, seqLenKV, numHeadsKV, h / group, headDim);
      tfa::test::cpuAttentionFixedLen(q.data(), k.data(), v.data(), o.data(), 1, nq, seqLenKV, 1, 1, headDim,
                                      isCausal != 0);
      scatterHead(o.data(), O, (long)b * seqLenQ, nq, numHeadsQ, h, headDim);
    }
  }
}

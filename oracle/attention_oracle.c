/*
 * TEST INFRASTRUCTURE ONLY.  CPU restatement of the attention forward that the reference
 * computes; used as the checker by tests/, by the smoke run and by the benchmark's CPU
 * baseline leg.  The product library never links, loads or calls this file.
 *
 * Algorithm followed (reference file:line):
 *   - layouts, GQA head map hq / (Hq/Hkv), scale 1/sqrt(D), top-left causal "key j > query i
 *     is masked":                      tests/cpp/cpu_reference.h:14-66 (fixed), :68-129 (varlen)
 *   - the same contract on the device: csrc/flash_attn/params.cuh:25-27, 49-68, 97-116;
 *     csrc/flash_attn/mma/softmax.cuh:136-138 (mask), :113-132 (row sum 0 -> output 0)
 *
 * Two arithmetic variants:
 *   tfa_oracle_*_f32  - float arithmetic in exactly the reference CPU code's operation order
 *                       (masked score -1e9f, max, exp, divide by the sum, then P.V), so that it can
 *                       be pinned bit-for-bit against the reference's own cpu_reference.h;
 *   tfa_oracle_*_f64  - the same mathematics in double (masked keys skipped), the
 *                       "fp64 naive softmax(QK^T/sqrt(d))V" that error bounds are stated against.
 *
 * Parity pin: tests/test_oracle.py checks the f32 variant bit-exactly against golden vectors
 * produced by the reference's cpu_reference.h (tests/golden/make_golden.py) and, when
 * oracle/_ref/libtinyfa_refcpu.so is present, against that library directly.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

int tfa_oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* One (sequence, Q head) slice in float, reference operation order (cpu_reference.h:23-62). */
static void slice_f32(const float* Q, const float* K, const float* V, float* O, long qRow0, long kvRow0, int seqLenQ,
                      int seqLenKV, int numHeadsQ, int numHeadsKV, int hq, int hkv, int headDim, int isCausal,
                      int qBegin, int qEnd, float* scores) {
  const float scale = 1.0f / sqrtf((float)headDim);
  (void)seqLenQ;
  for (int qi = qBegin; qi < qEnd; qi++) {
    const float* q = Q + ((qRow0 + qi) * numHeadsQ + hq) * (long)headDim;
    float maxScore = -1e9f;
    for (int kj = 0; kj < seqLenKV; kj++) {
      if (isCausal && kj > qi) {
        scores[kj] = -1e9f;
      } else {
        const float* k = K + ((kvRow0 + kj) * numHeadsKV + hkv) * (long)headDim;
        float dot = 0.0f;
        for (int d = 0; d < headDim; d++) dot += q[d] * k[d];
        scores[kj] = dot * scale;
      }
      maxScore = scores[kj] > maxScore ? scores[kj] : maxScore;
    }
    float sumExp = 0.0f;
    for (int kj = 0; kj < seqLenKV; kj++) {
      scores[kj] = expf(scores[kj] - maxScore);
      sumExp += scores[kj];
    }
    for (int kj = 0; kj < seqLenKV; kj++) scores[kj] /= sumExp;
    float* o = O + ((qRow0 + qi) * numHeadsQ + hq) * (long)headDim;
    for (int d = 0; d < headDim; d++) {
      float val = 0.0f;
      for (int kj = 0; kj < seqLenKV; kj++) {
        val += scores[kj] * V[((kvRow0 + kj) * numHeadsKV + hkv) * (long)headDim + d];
      }
      o[d] = val;
    }
  }
}

/* One (sequence, Q head) slice in double; masked keys are skipped; empty rows give 0. */
static void slice_f64(const float* Q, const float* K, const float* V, double* O, long qRow0, long kvRow0,
                      int seqLenKV, int numHeadsQ, int numHeadsKV, int hq, int hkv, int headDim, int isCausal,
                      int qBegin, int qEnd, double* scores, double* acc) {
  const double scale = 1.0 / sqrt((double)headDim);
  for (int qi = qBegin; qi < qEnd; qi++) {
    const float* q = Q + ((qRow0 + qi) * numHeadsQ + hq) * (long)headDim;
    int nk = seqLenKV;
    if (isCausal && qi + 1 < nk) nk = qi + 1;
    double maxScore = -INFINITY;
    for (int kj = 0; kj < nk; kj++) {
      const float* k = K + ((kvRow0 + kj) * numHeadsKV + hkv) * (long)headDim;
      double dot = 0.0;
      for (int d = 0; d < headDim; d++) dot += (double)q[d] * (double)k[d];
      scores[kj] = dot * scale;
      if (scores[kj] > maxScore) maxScore = scores[kj];
    }
    double sumExp = 0.0;
    for (int d = 0; d < headDim; d++) acc[d] = 0.0;
    for (int kj = 0; kj < nk; kj++) {
      const double p = exp(scores[kj] - maxScore);
      sumExp += p;
      const float* v = V + ((kvRow0 + kj) * numHeadsKV + hkv) * (long)headDim;
      for (int d = 0; d < headDim; d++) acc[d] += p * (double)v[d];
    }
    double* o = O + ((qRow0 + qi) * numHeadsQ + hq) * (long)headDim;
    const double inv = sumExp > 0.0 ? 1.0 / sumExp : 0.0;
    for (int d = 0; d < headDim; d++) o[d] = acc[d] * inv;
  }
}

/*
 * Fixed length: Q,O [B,Sq,Hq,D], K,V [B,Skv,Hkv,D] (cpu_reference.h:33-34,55,58).
 * qRows > 0 restricts the work to query rows [0, qRows) of every sequence (timing sample).
 */
void tfa_oracle_fixed_f32(const float* Q, const float* K, const float* V, float* O, int batchSize, int seqLenQ,
                          int seqLenKV, int numHeadsQ, int numHeadsKV, int headDim, int isCausal, int qRows) {
  const int group = numHeadsQ / numHeadsKV;
  const int qEnd = (qRows > 0 && qRows < seqLenQ) ? qRows : seqLenQ;
#pragma omp parallel
  {
    float* scores = (float*)malloc(sizeof(float) * (size_t)(seqLenKV > 0 ? seqLenKV : 1));
#pragma omp for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < batchSize; b++) {
      for (int hq = 0; hq < numHeadsQ; hq++) {
        slice_f32(Q, K, V, O, (long)b * seqLenQ, (long)b * seqLenKV, seqLenQ, seqLenKV, numHeadsQ, numHeadsKV, hq,
                  hq / group, headDim, isCausal, 0, qEnd, scores);
      }
    }
    free(scores);
  }
}

void tfa_oracle_fixed_f64(const float* Q, const float* K, const float* V, double* O, int batchSize, int seqLenQ,
                          int seqLenKV, int numHeadsQ, int numHeadsKV, int headDim, int isCausal, int qRows) {
  const int group = numHeadsQ / numHeadsKV;
  const int qEnd = (qRows > 0 && qRows < seqLenQ) ? qRows : seqLenQ;
#pragma omp parallel
  {
    double* scores = (double*)malloc(sizeof(double) * (size_t)(seqLenKV > 0 ? seqLenKV : 1));
    double* acc = (double*)malloc(sizeof(double) * (size_t)headDim);
#pragma omp for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < batchSize; b++) {
      for (int hq = 0; hq < numHeadsQ; hq++) {
        slice_f64(Q, K, V, O, (long)b * seqLenQ, (long)b * seqLenKV, seqLenKV, numHeadsQ, numHeadsKV, hq,
                  hq / group, headDim, isCausal, 0, qEnd, scores, acc);
      }
    }
    free(scores);
    free(acc);
  }
}

/*
 * Packed variable length: Q,O [totalQ,Hq,D], K,V [totalKV,Hkv,D]; sequence b owns rows
 * cu[b] .. cu[b+1]-1 (cpu_reference.h:74-83,96-97,118,121).
 */
void tfa_oracle_varlen_f32(const float* Q, const float* K, const float* V, float* O, const int* cuQ, const int* cuKV,
                           int batchSize, int numHeadsQ, int numHeadsKV, int headDim, int isCausal) {
  const int group = numHeadsQ / numHeadsKV;
  int maxKV = 1;
  for (int b = 0; b < batchSize; b++) {
    if (cuKV[b + 1] - cuKV[b] > maxKV) maxKV = cuKV[b + 1] - cuKV[b];
  }
#pragma omp parallel
  {
    float* scores = (float*)malloc(sizeof(float) * (size_t)maxKV);
#pragma omp for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < batchSize; b++) {
      for (int hq = 0; hq < numHeadsQ; hq++) {
        const int sq = cuQ[b + 1] - cuQ[b], skv = cuKV[b + 1] - cuKV[b];
        slice_f32(Q, K, V, O, cuQ[b], cuKV[b], sq, skv, numHeadsQ, numHeadsKV, hq, hq / group, headDim, isCausal, 0,
                  sq, scores);
      }
    }
    free(scores);
  }
}

void tfa_oracle_varlen_f64(const float* Q, const float* K, const float* V, double* O, const int* cuQ,
                           const int* cuKV, int batchSize, int numHeadsQ, int numHeadsKV, int headDim,
                           int isCausal) {
  const int group = numHeadsQ / numHeadsKV;
  int maxKV = 1;
  for (int b = 0; b < batchSize; b++) {
    if (cuKV[b + 1] - cuKV[b] > maxKV) maxKV = cuKV[b + 1] - cuKV[b];
  }
#pragma omp parallel
  {
    double* scores = (double*)malloc(sizeof(double) * (size_t)maxKV);
    double* acc = (double*)malloc(sizeof(double) * (size_t)headDim);
#pragma omp for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < batchSize; b++) {
      for (int hq = 0; hq < numHeadsQ; hq++) {
        const int sq = cuQ[b + 1] - cuQ[b], skv = cuKV[b + 1] - cuKV[b];
        slice_f64(Q, K, V, O, cuQ[b], cuKV[b], skv, numHeadsQ, numHeadsKV, hq, hq / group, headDim, isCausal, 0, sq,
                  scores, acc);
      }
    }
    free(scores);
    free(acc);
  }
}

/*
 * kron_oracle.c -- CPU restatement of the reference's GeMKM / GeKMM algorithm.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the parity checker of the test-suite
 * and the "port" CPU baseline of the benchmark; no product code path may call it.
 *
 * Parity status: PINNED.  tests/test_oracle.py checks this restatement against
 * (a) the unmodified reference x86 backend built by oracle/build_ref.sh, where
 * that library is present, and (b) golden vectors under tests/golden/ that were
 * produced by that same reference library (tests/golden/make_golden.py).
 *
 * Algorithm (the reference's sliced multiply):
 *   - factors are applied from the last to the first
 *     (src/kmm/kmmalgo.cpp:172-214, loop "for i = n-1 .. 0");
 *   - one step with factor F (P x Q) maps a row of K' values to K'/P*Q values:
 *       out[q*(K'/P) + s] = sum_p in[s*P + p] * F[p][q]
 *     (src/kernels/cuda/global-store.cuh:248-256; serial form in
 *     tests/testBase.h:256-276), p ascending;
 *   - alpha and beta*Y enter on the step that consumes factor 0
 *     (src/handle/handle.cpp:190, tests/testBase.h:276-280);
 *   - operand access rules (include/fastkron.h:206-231):
 *       MKM  X[m,k] = opX==N ? X[m*K+k] : X[k*M+m];  F[p,q] = opF==N ? F[p*Q+q] : F[q*P+p];
 *            Z[m,l] = Z[m*L+l]
 *       KMM  X[m,k] = opX==N ? X[k*M+m] : X[m*K+k];  F[p,q] = opF==N ? F[q*P+p] : F[p*Q+q];
 *            Z[m,l] = Z[l*M+m]
 *   - the forward variants keep the matrix after each step; intermediate i-1 is
 *     the matrix after factors N-1..i, M x cols row-major for MKM and cols x M for
 *     KMM (src/kmm/kmmalgo.cpp:100-110, tests/testBase.h:277-279,311-313).
 *
 * The *_T versions compute in the element type (like the reference kernels);
 * the *_exact versions accumulate in long double / double and are used to judge
 * which of two fp32 results is closer to the truth.
 */
#include <stdint.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define OP_N 1
#define OP_T 2

#define DEFINE_ORACLE(NAME, T, ACC)                                                          \
int NAME(int isKmm, uint32_t M, uint32_t N, const uint32_t* Ps, const uint32_t* Qs,          \
         const T* X, int opX, const T* const* Fs, int opF, T* Z, double alpha, double beta,  \
         const T* Y, T* const* inter) {                                                      \
  uint64_t K = 1, L = 1, maxCols = 1;                                                        \
  for (uint32_t i = 0; i < N; i++) { K *= Ps[i]; L *= Qs[i]; }                               \
  {                                                                                          \
    uint64_t c = K; maxCols = K;                                                             \
    for (int i = (int)N - 1; i >= 0; i--) { c = c / Ps[i] * Qs[i]; if (c > maxCols) maxCols = c; } \
  }                                                                                          \
  const int xRowMajor = isKmm ? (opX == OP_T) : (opX == OP_N);                               \
  const int fPMajor   = isKmm ? (opF == OP_T) : (opF == OP_N);                               \
  int failed = 0;                                                                            \
  _Pragma("omp parallel")                                                                    \
  {                                                                                          \
    ACC* cur = (ACC*)malloc(sizeof(ACC) * maxCols);                                          \
    ACC* nxt = (ACC*)malloc(sizeof(ACC) * maxCols);                                          \
    if (!cur || !nxt) { failed = 1; }                                                        \
    _Pragma("omp for schedule(static)")                                                      \
    for (int64_t m = 0; m < (int64_t)M; m++) {                                               \
      if (failed) continue;                                                                  \
      for (uint64_t k = 0; k < K; k++)                                                       \
        cur[k] = (ACC)(xRowMajor ? X[(uint64_t)m * K + k] : X[k * (uint64_t)M + m]);         \
      uint64_t cols = K;                                                                     \
      for (int i = (int)N - 1; i >= 0; i--) {                                                \
        const uint32_t P = Ps[i], Q = Qs[i];                                                 \
        const uint64_t S = cols / P;                                                         \
        const T* F = Fs[i];                                                                  \
        for (uint32_t q = 0; q < Q; q++) {                                                   \
          for (uint64_t s = 0; s < S; s++) {                                                 \
            ACC acc = 0;                                                                     \
            for (uint32_t p = 0; p < P; p++) {                                               \
              const ACC f = (ACC)(fPMajor ? F[(uint64_t)p * Q + q] : F[(uint64_t)q * P + p]); \
              acc += cur[s * P + p] * f;                                                     \
            }                                                                                \
            nxt[(uint64_t)q * S + s] = acc;                                                  \
          }                                                                                  \
        }                                                                                    \
        cols = S * Q;                                                                        \
        if (i > 0 && inter && inter[i - 1]) {                                                \
          T* I = inter[i - 1];                                                               \
          for (uint64_t c = 0; c < cols; c++) {                                              \
            if (isKmm) I[c * (uint64_t)M + m] = (T)nxt[c];                                   \
            else       I[(uint64_t)m * cols + c] = (T)nxt[c];                                \
          }                                                                                  \
        }                                                                                    \
        ACC* t = cur; cur = nxt; nxt = t;                                                    \
      }                                                                                      \
      for (uint64_t l = 0; l < L; l++) {                                                     \
        const uint64_t zi = isKmm ? l * (uint64_t)M + m : (uint64_t)m * L + l;               \
        ACC v = (ACC)alpha * cur[l];                                                         \
        if (beta != 0.0 && Y) v += (ACC)beta * (ACC)Y[zi];                                   \
        Z[zi] = (T)v;                                                                        \
      }                                                                                      \
    }                                                                                        \
    free(cur); free(nxt);                                                                    \
  }                                                                                          \
  return failed;                                                                             \
}

DEFINE_ORACLE(oracle_gekmm_f32, float, float)
DEFINE_ORACLE(oracle_gekmm_f64, double, double)
DEFINE_ORACLE(oracle_gekmm_f32_exact, float, double)
DEFINE_ORACLE(oracle_gekmm_f64_exact, double, long double)

/*
 * fastkron.h -- C ABI of the B200-native GeMKM / GeKMM engine.
 *
 * The declarations below reproduce, symbol for symbol and argument for argument,
 * the public interface of abhijangda/fastkron (include/fastkron.h:27-628 in that
 * project) so that programs and bindings written against it link against this
 * library without change.  Enum values are part of the ABI and are identical.
 * The implementation behind the interface is new: a host planner plus
 * hand-written sm_100a kernels (see fastkron_b200/csrc).
 *
 * Operation
 *   GeMKM:  Z = alpha * op(X) * (op(F1) (x) ... (x) op(FN)) + beta * Y
 *           op(X) is M x K (K = prod Ps), op(Fi) is Ps[i] x Qs[i],
 *           Y and Z are M x L (L = prod Qs), everything row-major.
 *   GeKMM:  Z = alpha * (op(F1) (x) ... (x) op(FN)) * op(X) + beta * Y
 *           op(Fi) is Qs[i] x Ps[i], op(X) is K x M, Y and Z are L x M.
 *   fastKronOp_T on an operand means its buffer holds the transpose of the
 *   row-major operand (i.e. the operand stored column-major).
 *
 * Only the CUDA backend exists in this library.  Requests for any other
 * backend are answered with an error code; nothing is computed on the host.
 */
#pragma once

#include <stdint.h>
#include <stddef.h>
#include <stdio.h>
#include <stdlib.h>

/* Caller-side convenience: abort the program on a non-success return code.
 * (reference: include/fastkron.h:9-17) */
#define FastKronCHECK(cmd) do {                                   \
  fastKronError e_ = (cmd);                                       \
  if (e_ != fastKronSuccess) {                                    \
    printf("Failed: FastKron error %s:%d at %s:%d \n",            \
           fastKronGetErrorString(e_), (int)e_, __FILE__, __LINE__); \
    exit(EXIT_FAILURE);                                           \
  }                                                               \
} while (0)

/* reference: include/fastkron.h:27-30 */
enum fastKronOp {
  fastKronOp_N = 1,   /* buffer is the row-major operand               */
  fastKronOp_T = 2    /* buffer is the transpose of the row-major operand */
};

/* reference: include/fastkron.h:42-48 */
enum fastKronBackend {
  fastKronBackend_NONE = 1 << 0,
  fastKronBackend_X86  = 1 << 1,
  fastKronBackend_ARM  = 1 << 2,
  fastKronBackend_CUDA = 1 << 3,
  fastKronBackend_HIP  = 1 << 4
};

/* reference: include/fastkron.h:57-61 */
enum fastKronOptions {
  fastKronOptionsNone      = 1 << 0,
  fastKronOptionsUseFusion = 1 << 1,  /* allow several factors per kernel     */
  fastKronOptionsTune      = 1 << 2,  /* time candidate plans on first use    */
  /* Not in the reference.  Opt-in: fp32 passes with 64x64 / 128x128 factors run on the TF32
   * tensor cores (operands read with a 10-bit mantissa, fp32 accumulation); results then
   * agree with fp32 only to a few 1e-3 of the row maximum.  Also switched on by the
   * environment variable FASTKRON_TF32=1.  Off by default. */
  fastKronOptionsTF32      = 1 << 3,
  /* Not in the reference.  Opt-in: fp32 passes with 64x64 factors run on the tensor cores with
   * every operand split into two TF32 numbers and three products per fp32 product (fp32
   * accumulation); results agree with the default fp32 kernels to about 1e-6 of the row
   * maximum.  Also switched on by FASTKRON_TF32=3.  Off by default; wins over TF32 when both
   * are set. */
  fastKronOptionsTF32x3    = 1 << 4
};

/* reference: include/fastkron.h:74-82 */
enum fastKronError {
  fastKronSuccess             = 0,
  fastKronBackendNotAvailable = 1,
  fastKronInvalidMemoryAccess = 2,
  fastKronKernelNotFound      = 3,
  fastKronInvalidArgument     = 4,
  fastKronInvalidKMMProblem   = 5,
  fastKronOtherError          = 6
};

#ifdef __cplusplus
extern "C" {
#endif

#ifndef __cplusplus
typedef enum fastKronOp fastKronOp;
typedef enum fastKronBackend fastKronBackend;
typedef enum fastKronError fastKronError;
#endif

/* Opaque library context.  A handle is used by one host thread at a time. */
typedef void* fastKronHandle;

/* ---- library information (reference: include/fastkron.h:95-121) ---------- */
const char* fastKronVersion();
const char* fastKronCUDAArchs();
const char* fastKronGetErrorString(fastKronError err);
/* Bitwise OR of the fastKronBackend values compiled into this library. */
uint32_t    fastKronGetBackends();

/* ---- handle life cycle (reference: include/fastkron.h:123-204) ----------- */
/* Create a handle for the OR-ed `backends`.  A backend that this library does
 * not contain yields fastKronInvalidArgument (the handle is still written). */
fastKronError fastKronInit(fastKronHandle* handle, uint32_t backends);
fastKronError fastKronInitAllBackends(fastKronHandle* handle);
fastKronError fastKronSetOptions(fastKronHandle handle, uint32_t options);
void          fastKronDestroy(fastKronHandle handle);
/* `ptrToStream` points to a cudaStream_t; all later work is enqueued there. */
fastKronError fastKronInitCUDA(fastKronHandle handle, void* ptrToStream);
fastKronError fastKronInitHIP(fastKronHandle handle, void* ptrToStream);
fastKronError fastKronInitX86(fastKronHandle handle);
fastKronError fastKronSetStream(fastKronHandle handle, fastKronBackend backend,
                                void* ptrToStream);

/* ---- sizes (reference: include/fastkron.h:249-251) ------------------------ */
/* Number of elements of the result and of EACH temporary buffer. */
fastKronError gekmmSizes(fastKronHandle handle, uint32_t M, uint32_t N,
                         uint32_t Ps[], uint32_t Qs[],
                         size_t* yElems, size_t* tmpElems);

/* The argument lists of the product functions differ only in the element type, so they
 * are written once as macros (T = float for the s-, double for the d- functions).
 * Order and meaning are the reference's.  Common rules: Fs is a HOST array of N device
 * pointers; X and Fs are never written; calls enqueue work on the handle's stream and
 * return without synchronising. */

/* GeMKM arguments (reference: include/fastkron.h:284-296): M rows, N factors of shape
 * Ps[i] x Qs[i]; temp1 must not be NULL; temp2 may be NULL unless Z aliases Y or Z is
 * smaller than a temporary -- with temp2 NULL the library uses Z as its second scratch, so Z
 * must then hold the tmpElems that gekmmSizes reports, which exceeds M*L whenever an
 * intermediate is wider than the result (shrinking factors, P > Q).  The library cannot see
 * the size of Z and does not check this. */
#define FASTKRON_GEMKM_ARGS(T)                                                    \
  fastKronHandle handle, fastKronBackend backend,                                 \
  uint32_t M, uint32_t N, uint32_t Ps[], uint32_t Qs[],                           \
  const T* X, fastKronOp opX, const T* const Fs[], fastKronOp opFs,               \
  T* Z, T alpha, T beta, const T* Y, T* temp1, T* temp2

/* GeKMM arguments (reference: include/fastkron.h:329-341); note Qs before Ps and the
 * factors before X. */
#define FASTKRON_GEKMM_ARGS(T)                                                    \
  fastKronHandle handle, fastKronBackend backend,                                 \
  uint32_t N, uint32_t Qs[], uint32_t Ps[], uint32_t M,                           \
  const T* const Fs[], fastKronOp opFs, const T* X, fastKronOp opX,               \
  T* Z, T alpha, T beta, const T* Y, T* temp1, T* temp2

fastKronError sgemkm(FASTKRON_GEMKM_ARGS(float));
fastKronError dgemkm(FASTKRON_GEMKM_ARGS(double));
fastKronError sgekmm(FASTKRON_GEKMM_ARGS(float));
fastKronError dgekmm(FASTKRON_GEKMM_ARGS(double));

/* Strided-batched forms (reference: include/fastkron.h:384-449).  Batch b uses
 * X + b*strideX, Fs[i] + b*strideF[i], Z + b*strideZ, Y + b*strideY (strides in elements;
 * 0 shares the operand across the batch).  Each temporary holds batchCount * tmpElems. */
#define FASTKRON_GEMKM_SB_ARGS(T)                                                 \
  fastKronHandle handle, fastKronBackend backend,                                 \
  uint32_t M, uint32_t N, uint32_t Ps[], uint32_t Qs[],                           \
  const T* X, fastKronOp opX, uint64_t strideX,                                   \
  const T* const Fs[], fastKronOp opFs, uint64_t strideF[],                       \
  T* Z, uint64_t strideZ, T alpha, T beta, uint32_t batchCount,                   \
  const T* Y, uint64_t strideY, T* temp1, T* temp2
#define FASTKRON_GEKMM_SB_ARGS(T)                                                 \
  fastKronHandle handle, fastKronBackend backend,                                 \
  uint32_t N, uint32_t Qs[], uint32_t Ps[], uint32_t M,                           \
  const T* const Fs[], fastKronOp opFs, uint64_t strideF[],                       \
  const T* X, fastKronOp opX, uint64_t strideX,                                   \
  T* Z, uint64_t strideZ, T alpha, T beta, uint32_t batchCount,                   \
  const T* Y, uint64_t strideY, T* temp1, T* temp2

fastKronError sgemkmStridedBatched(FASTKRON_GEMKM_SB_ARGS(float));
fastKronError dgemkmStridedBatched(FASTKRON_GEMKM_SB_ARGS(double));
fastKronError sgekmmStridedBatched(FASTKRON_GEKMM_SB_ARGS(float));
fastKronError dgekmmStridedBatched(FASTKRON_GEKMM_SB_ARGS(double));

/* Forward variants keeping every intermediate (reference: include/fastkron.h:470-628):
 * alpha = 1, beta = 0.  Intermediates[i-1] receives the matrix obtained after the factors
 * N-1 .. i have been applied (i = N-1 .. 1), in the reference's sliced-multiply column
 * order; gekmmSizesForward reports its element count in intermediateElems[i-1]. */
fastKronError gekmmSizesForward(fastKronHandle handle, uint32_t M, uint32_t N,
                                uint32_t Ps[], uint32_t Qs[],
                                size_t* yElems, size_t* intermediateElems);

#define FASTKRON_MKM_FWD_ARGS(T)                                                  \
  fastKronHandle handle, fastKronBackend backend,                                 \
  uint32_t M, uint32_t N, uint32_t Ps[], uint32_t Qs[],                           \
  const T* X, fastKronOp opX, const T* const Fs[], fastKronOp opFs,               \
  T* Z, T* Intermediates[]
#define FASTKRON_KMM_FWD_ARGS(T)                                                  \
  fastKronHandle handle, fastKronBackend backend,                                 \
  uint32_t N, uint32_t Qs[], uint32_t Ps[], uint32_t M,                           \
  const T* const Fs[], fastKronOp opFs, const T* X, fastKronOp opX,               \
  T* Z, T* Intermediates[]
#define FASTKRON_MKM_FWD_SB_ARGS(T)                                               \
  fastKronHandle handle, fastKronBackend backend,                                 \
  uint32_t M, uint32_t N, uint32_t Ps[], uint32_t Qs[],                           \
  const T* X, fastKronOp opX, uint64_t strideX,                                   \
  const T* const Fs[], fastKronOp opFs, uint64_t strideF[],                       \
  T* Z, uint64_t strideZ, uint32_t batchCount,                                    \
  T* Intermediates[], uint64_t strideIntermediates[]
#define FASTKRON_KMM_FWD_SB_ARGS(T)                                               \
  fastKronHandle handle, fastKronBackend backend,                                 \
  uint32_t N, uint32_t Qs[], uint32_t Ps[], uint32_t M,                           \
  const T* const Fs[], fastKronOp opFs, uint64_t strideF[],                       \
  const T* X, fastKronOp opX, uint64_t strideX,                                   \
  T* Z, uint64_t strideZ, uint32_t batchCount,                                    \
  T* Intermediates[], uint64_t strideIntermediates[]

fastKronError smkmForward(FASTKRON_MKM_FWD_ARGS(float));
fastKronError dmkmForward(FASTKRON_MKM_FWD_ARGS(double));
fastKronError skmmForward(FASTKRON_KMM_FWD_ARGS(float));
fastKronError dkmmForward(FASTKRON_KMM_FWD_ARGS(double));
fastKronError smkmForwardStridedBatched(FASTKRON_MKM_FWD_SB_ARGS(float));
fastKronError dmkmForwardStridedBatched(FASTKRON_MKM_FWD_SB_ARGS(double));
fastKronError skmmForwardStridedBatched(FASTKRON_KMM_FWD_SB_ARGS(float));
fastKronError dkmmForwardStridedBatched(FASTKRON_KMM_FWD_SB_ARGS(double));

/* ---- GeMKM without caller-provided temporaries -------------------------------------
 * This function has no counterpart in the reference.  It is sgemkm for callers that
 * may not allocate device memory (code inside another framework's fixed memory plan,
 * processes where allocation after start-up is forbidden): the two temporaries come
 * from a static buffer inside the library, FASTKRON_NOALLOC_MAX_TEMP_ELEMS floats each,
 * resident on every GPU that loads the library.  Problems whose gekmmSizes() tmpElems
 * exceeds that are rejected with fastKronInvalidArgument.  The first call on a device
 * looks up the buffer's address and should be made before any stream capture.  All
 * calls on one device share the buffer: calls that can overlap on the GPU race.  The
 * handle must have been given a stream with fastKronInitCUDA; the device that was
 * current then must be current now. */
#define FASTKRON_NOALLOC_MAX_TEMP_ELEMS (2u << 20)
fastKronError sgemkmNoAlloc(fastKronHandle handle,
                            uint32_t M, uint32_t N, uint32_t Ps[], uint32_t Qs[],
                            const float* X, fastKronOp opX,
                            const float* const Fs[], fastKronOp opFs,
                            float* Z, float alpha, float beta, const float* Y);

#ifdef __cplusplus
}
#endif

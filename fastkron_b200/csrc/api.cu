// extern "C" entry points of include/fastkron.h.  Each marshals its arguments
// into a Problem + CallOperands and hands them to the Engine, mirroring what the
// reference's src/fastkron.cpp:19-402 does with KMMProblem/FastKronHandle.

#include "engine.h"
#include "gemm_table.h"
#include "fastkron.h"

#include <string.h>
#include <stdlib.h>

using namespace fkb;

#ifndef FKB_VERSION
#define FKB_VERSION "1.1.0"
#endif

static inline Engine* E(fastKronHandle h) { return reinterpret_cast<Engine*>(h); }

extern "C" {

const char* fastKronVersion() { return FKB_VERSION "+CUDA12.9+sm_100a"; }

const char* fastKronCUDAArchs() { return "100a"; }

// Same strings as the reference (src/fastkron.cpp:44-61), plus a text for
// fastKronInvalidKMMProblem, for which the reference returns NULL.
const char* fastKronGetErrorString(fastKronError err) {
  switch (err) {
    case fastKronSuccess:             return "Operation successfull";
    case fastKronBackendNotAvailable: return "Requested backend is not available";
    case fastKronInvalidMemoryAccess: return "Illegal memory access";
    case fastKronKernelNotFound:      return "Kernel to execute the problem not found";
    case fastKronInvalidArgument:     return "An argument to the function is invalid";
    case fastKronInvalidKMMProblem:   return "Invalid Kronecker matrix multiplication problem";
    case fastKronOtherError:          return "Unknown error occurred";
    default:                          return nullptr;
  }
}

uint32_t fastKronGetBackends() { return fastKronBackend_CUDA; }

fastKronError fastKronInit(fastKronHandle* handle, uint32_t backends) {
  if (!handle) return fastKronInvalidArgument;
  Engine* e = new Engine(backends);
  *handle = reinterpret_cast<fastKronHandle>(e);
  uint32_t opts = fastKronOptionsUseFusion;
  const char* tune = getenv("FASTKRON_TUNE");
  if (tune && tune[0] == '1') opts |= fastKronOptionsTune;
  e->setOptions(opts);
  if ((backends & fastKronGetBackends()) != backends) return fastKronInvalidArgument;
  return fastKronSuccess;
}

fastKronError fastKronInitAllBackends(fastKronHandle* handle) {
  return fastKronInit(handle, fastKronGetBackends());
}

fastKronError fastKronSetOptions(fastKronHandle handle, uint32_t options) {
  if (!handle) return fastKronInvalidArgument;
  E(handle)->setOptions(options);
  return fastKronSuccess;
}

void fastKronDestroy(fastKronHandle handle) { delete E(handle); }

fastKronError fastKronInitCUDA(fastKronHandle handle, void* ptrToStream) {
  if (!handle) return fastKronInvalidArgument;
  return E(handle)->initCUDA(ptrToStream);
}

fastKronError fastKronInitHIP(fastKronHandle handle, void*) {
  if (!handle) return fastKronInvalidArgument;
  return fastKronBackendNotAvailable;
}

fastKronError fastKronInitX86(fastKronHandle handle) {
  if (!handle) return fastKronInvalidArgument;
  return fastKronBackendNotAvailable;
}

fastKronError fastKronSetStream(fastKronHandle handle, fastKronBackend backend, void* ptrToStream) {
  if (!handle || !ptrToStream) return fastKronInvalidArgument;
  if (!E(handle)->hasBackend(backend) || backend != fastKronBackend_CUDA) return fastKronBackendNotAvailable;
  return E(handle)->setStream(ptrToStream);
}

}  // extern "C"

// ---- marshalling helpers ----------------------------------------------------

static bool fillProblem(Problem* pr, MMType mm, DType dt, uint32_t M, uint32_t N,
                        const uint32_t* Ps, const uint32_t* Qs, fastKronOp opX, fastKronOp opF) {
  if (N == 0 || N > (uint32_t)kMaxFactors || !Ps || !Qs) return false;
  pr->mm = mm; pr->dt = dt; pr->M = M; pr->N = N; pr->opX = opX; pr->opF = opF;
  for (uint32_t i = 0; i < N; i++) { pr->P[i] = Ps[i]; pr->Q[i] = Qs[i]; }
  return true;
}

static bool validOp(fastKronOp o) { return o == fastKronOp_N || o == fastKronOp_T; }

template <typename T>
static fastKronError gemm(fastKronHandle h, fastKronBackend backend, MMType mm, uint32_t M, uint32_t N,
                          const uint32_t* Ps, const uint32_t* Qs, const T* X, fastKronOp opX,
                          const T* const Fs[], fastKronOp opFs, T* Z, T alpha, T beta, const T* Y,
                          T* temp1, T* temp2, uint32_t batch, uint64_t strideX, const uint64_t* strideF,
                          uint64_t strideZ, uint64_t strideY) {
  if (!h) return fastKronInvalidArgument;
  Engine* e = E(h);
  // reference: src/handle/handle.cpp:116-122
  if (Z == nullptr || temp1 == nullptr || !e->hasBackend(backend)) return fastKronInvalidArgument;
  if (backend != fastKronBackend_CUDA) return fastKronBackendNotAvailable;
  if (!validOp(opX) || !validOp(opFs)) return fastKronInvalidArgument;
  Problem pr;
  if (!fillProblem(&pr, mm, sizeof(T) == 4 ? DType::F32 : DType::F64, M, N, Ps, Qs, opX, opFs))
    return fastKronInvalidArgument;
  pr.batch = batch;
  CallOperands ops;
  ops.X = X; ops.Fs = reinterpret_cast<const void* const*>(Fs); ops.Z = Z; ops.Y = Y;
  ops.temp1 = temp1; ops.temp2 = temp2; ops.alpha = (double)alpha; ops.beta = (double)beta;
  ops.strideX = strideX; ops.strideZ = strideZ; ops.strideY = strideY; ops.strideF = strideF;
  if (batch > 1 && !strideF) return fastKronInvalidArgument;
  return e->run(pr, ops);
}

template <typename T>
static fastKronError forward(fastKronHandle h, fastKronBackend backend, MMType mm, uint32_t M, uint32_t N,
                             const uint32_t* Ps, const uint32_t* Qs, const T* X, fastKronOp opX,
                             const T* const Fs[], fastKronOp opFs, T* Z, T* inter[], uint32_t batch,
                             uint64_t strideX, const uint64_t* strideF, uint64_t strideZ,
                             const uint64_t* strideI) {
  if (!h) return fastKronInvalidArgument;
  Engine* e = E(h);
  if (Z == nullptr || !e->hasBackend(backend)) return fastKronInvalidArgument;
  if (backend != fastKronBackend_CUDA) return fastKronBackendNotAvailable;
  if (!validOp(opX) || !validOp(opFs)) return fastKronInvalidArgument;
  Problem pr;
  if (!fillProblem(&pr, mm, sizeof(T) == 4 ? DType::F32 : DType::F64, M, N, Ps, Qs, opX, opFs))
    return fastKronInvalidArgument;
  pr.batch = batch;
  pr.forward = true;
  CallOperands ops;
  ops.X = X; ops.Fs = reinterpret_cast<const void* const*>(Fs); ops.Z = Z;
  ops.intermediates = reinterpret_cast<void* const*>(inter);
  ops.strideX = strideX; ops.strideZ = strideZ; ops.strideF = strideF; ops.strideI = strideI;
  if (batch > 1 && !strideF) return fastKronInvalidArgument;
  return e->run(pr, ops);
}

extern "C" {

// Both size queries describe the problem as an MKM, like the reference
// (src/fastkron.cpp:126-142); the counts are the same for KMM.
fastKronError gekmmSizes(fastKronHandle handle, uint32_t M, uint32_t N, uint32_t Ps[], uint32_t Qs[],
                         size_t* yElems, size_t* tmpElems) {
  if (!handle) return fastKronInvalidArgument;
  Problem pr;
  if (!fillProblem(&pr, MMType::MKM, DType::F32, M, N, Ps, Qs, fastKronOp_N, fastKronOp_N))
    return fastKronInvalidArgument;
  fastKronError e = E(handle)->sizes(pr, yElems, tmpElems);
  if (e == fastKronSuccess && E(handle)->mg) mgAdjustSizes(E(handle)->mg, pr, yElems, tmpElems);
  return e;
}
fastKronError gekmmSizesForward(fastKronHandle handle, uint32_t M, uint32_t N, uint32_t Ps[],
                                uint32_t Qs[], size_t* yElems, size_t* intermediateElems) {
  if (!handle) return fastKronInvalidArgument;
  Problem pr;
  if (!fillProblem(&pr, MMType::MKM, DType::F32, M, N, Ps, Qs, fastKronOp_N, fastKronOp_N))
    return fastKronInvalidArgument;
  return E(handle)->sizesForward(pr, yElems, intermediateElems);
}

#define FKB_GEMKM(name, T)                                                                         \
  fastKronError name(fastKronHandle handle, fastKronBackend backend, uint32_t M, uint32_t N,       \
                     uint32_t Ps[], uint32_t Qs[], const T* X, fastKronOp opX, const T* const Fs[], \
                     fastKronOp opFs, T* Z, T alpha, T beta, const T* Y, T* temp1, T* temp2) {     \
    return gemm<T>(handle, backend, MMType::MKM, M, N, Ps, Qs, X, opX, Fs, opFs, Z, alpha, beta, Y, \
                   temp1, temp2, 1, 0, nullptr, 0, 0);                                             \
  }
#define FKB_GEKMM(name, T)                                                                         \
  fastKronError name(fastKronHandle handle, fastKronBackend backend, uint32_t N, uint32_t Qs[],    \
                     uint32_t Ps[], uint32_t M, const T* const Fs[], fastKronOp opFs, const T* X,  \
                     fastKronOp opX, T* Z, T alpha, T beta, const T* Y, T* temp1, T* temp2) {      \
    return gemm<T>(handle, backend, MMType::KMM, M, N, Ps, Qs, X, opX, Fs, opFs, Z, alpha, beta, Y, \
                   temp1, temp2, 1, 0, nullptr, 0, 0);                                             \
  }
FKB_GEMKM(sgemkm, float)
FKB_GEMKM(dgemkm, double)
FKB_GEKMM(sgekmm, float)
FKB_GEKMM(dgekmm, double)

#define FKB_GEMKM_SB(name, T)                                                                      \
  fastKronError name(fastKronHandle handle, fastKronBackend backend, uint32_t M, uint32_t N,       \
                     uint32_t Ps[], uint32_t Qs[], const T* X, fastKronOp opX, uint64_t strideX,   \
                     const T* const Fs[], fastKronOp opFs, uint64_t strideF[], T* Z,               \
                     uint64_t strideZ, T alpha, T beta, uint32_t batchCount, const T* Y,           \
                     uint64_t strideY, T* temp1, T* temp2) {                                       \
    return gemm<T>(handle, backend, MMType::MKM, M, N, Ps, Qs, X, opX, Fs, opFs, Z, alpha, beta, Y, \
                   temp1, temp2, batchCount, strideX, strideF, strideZ, strideY);                  \
  }
#define FKB_GEKMM_SB(name, T)                                                                      \
  fastKronError name(fastKronHandle handle, fastKronBackend backend, uint32_t N, uint32_t Qs[],    \
                     uint32_t Ps[], uint32_t M, const T* const Fs[], fastKronOp opFs,              \
                     uint64_t strideF[], const T* X, fastKronOp opX, uint64_t strideX, T* Z,       \
                     uint64_t strideZ, T alpha, T beta, uint32_t batchCount, const T* Y,           \
                     uint64_t strideY, T* temp1, T* temp2) {                                       \
    return gemm<T>(handle, backend, MMType::KMM, M, N, Ps, Qs, X, opX, Fs, opFs, Z, alpha, beta, Y, \
                   temp1, temp2, batchCount, strideX, strideF, strideZ, strideY);                  \
  }
FKB_GEMKM_SB(sgemkmStridedBatched, float)
FKB_GEMKM_SB(dgemkmStridedBatched, double)
FKB_GEKMM_SB(sgekmmStridedBatched, float)
FKB_GEKMM_SB(dgekmmStridedBatched, double)

#define FKB_MKM_FWD(name, T)                                                                       \
  fastKronError name(fastKronHandle handle, fastKronBackend backend, uint32_t M, uint32_t N,       \
                     uint32_t Ps[], uint32_t Qs[], const T* X, fastKronOp opX, const T* const Fs[], \
                     fastKronOp opFs, T* Z, T* Intermediates[]) {                                  \
    return forward<T>(handle, backend, MMType::MKM, M, N, Ps, Qs, X, opX, Fs, opFs, Z,             \
                      Intermediates, 1, 0, nullptr, 0, nullptr);                                   \
  }
#define FKB_KMM_FWD(name, T)                                                                       \
  fastKronError name(fastKronHandle handle, fastKronBackend backend, uint32_t N, uint32_t Qs[],    \
                     uint32_t Ps[], uint32_t M, const T* const Fs[], fastKronOp opFs, const T* X,  \
                     fastKronOp opX, T* Z, T* Intermediates[]) {                                   \
    return forward<T>(handle, backend, MMType::KMM, M, N, Ps, Qs, X, opX, Fs, opFs, Z,             \
                      Intermediates, 1, 0, nullptr, 0, nullptr);                                   \
  }
FKB_MKM_FWD(smkmForward, float)
FKB_MKM_FWD(dmkmForward, double)
FKB_KMM_FWD(skmmForward, float)
FKB_KMM_FWD(dkmmForward, double)

#define FKB_MKM_FWD_SB(name, T)                                                                    \
  fastKronError name(fastKronHandle handle, fastKronBackend backend, uint32_t M, uint32_t N,       \
                     uint32_t Ps[], uint32_t Qs[], const T* X, fastKronOp opX, uint64_t strideX,   \
                     const T* const Fs[], fastKronOp opFs, uint64_t strideF[], T* Z,               \
                     uint64_t strideZ, uint32_t batchCount, T* Intermediates[],                    \
                     uint64_t strideIntermediates[]) {                                             \
    return forward<T>(handle, backend, MMType::MKM, M, N, Ps, Qs, X, opX, Fs, opFs, Z,             \
                      Intermediates, batchCount, strideX, strideF, strideZ, strideIntermediates);  \
  }
#define FKB_KMM_FWD_SB(name, T)                                                                    \
  fastKronError name(fastKronHandle handle, fastKronBackend backend, uint32_t N, uint32_t Qs[],    \
                     uint32_t Ps[], uint32_t M, const T* const Fs[], fastKronOp opFs,              \
                     uint64_t strideF[], const T* X, fastKronOp opX, uint64_t strideX, T* Z,       \
                     uint64_t strideZ, uint32_t batchCount, T* Intermediates[],                    \
                     uint64_t strideIntermediates[]) {                                             \
    return forward<T>(handle, backend, MMType::KMM, M, N, Ps, Qs, X, opX, Fs, opFs, Z,             \
                      Intermediates, batchCount, strideX, strideF, strideZ, strideIntermediates);  \
  }
FKB_MKM_FWD_SB(smkmForwardStridedBatched, float)
FKB_MKM_FWD_SB(dmkmForwardStridedBatched, double)
FKB_KMM_FWD_SB(skmmForwardStridedBatched, float)
FKB_KMM_FWD_SB(dkmmForwardStridedBatched, double)

// ---- measurement helpers used by bench.py (not part of the reference ABI) ---------
// Number of kernels this library has launched in this process.
unsigned long long fkbLaunchCount() { return Engine::launchCount(); }
// Bracket every pass with CUDA events on the handle's stream (on != 0).
int fkbSetProfiling(fastKronHandle handle, int on) {
  if (!handle) return (int)fastKronInvalidArgument;
  E(handle)->setProfiling(on != 0);
  return 0;
}
// Durations (ms) and kernel kinds (0 generic, 1 tile, 2 gemm) of the passes recorded
// since the last call; synchronises on the recorded events.  Returns the count.
int fkbGetPassTimes(fastKronHandle handle, float* ms, int* kinds, int maxN) {
  if (!handle || !ms) return -1;
  return E(handle)->passTimes(ms, kinds, maxN);
}

// Tuner hook (fastkron_b200/tune.py): cap the fusion depth of every plan made afterwards by
// this process (0 = none).  Cached plans of existing handles are not revisited.
void fkbSetMaxFuse(int cap) { setMaxFuseOverride(cap); }

// Health check for callers of the TMA-staged kernels: every wait on a transfer barrier in this
// library is time-bounded (about two seconds); a wait that gives up makes its CTA return without
// writing its tiles and raises a per-device flag.  Call after synchronising the stream:
// fastKronSuccess when no wait ever gave up on the current device, fastKronOtherError otherwise
// (the results of the affected call are then incomplete).
extern "C" int fkbGemmTmaTimeouts();
extern "C" int fkbGemmTcTimeouts();
extern "C" int fkbTileTmaTimeouts();
fastKronError fkbDeviceStatus() {
  const int a = fkbGemmTmaTimeouts(), b = fkbGemmTcTimeouts(), c = fkbTileTmaTimeouts();
  if (a < 0 || b < 0 || c < 0) return fastKronBackendNotAvailable;
  return (a | b | c) ? fastKronOtherError : fastKronSuccess;
}

// Measurement hook: while set, every plan made by this process runs all passes on the
// one-thread-per-output kernel.  Cached plans of existing handles are not revisited.
void fkbSetForceGeneric(int on) { setForceGenericOverride(on != 0); }

// Measurement hook: smallest factor (elements, P*Q) that plans made afterwards give to the
// any-shape tiled kernel instead of the one-thread-per-output kernel; 0 restores the default rule.
void fkbSetAnyMinElems(int elems) { gAnyMinElems = elems > 0 ? elems : 0; }

// ---- introspection used by the host-side tests (not part of the reference ABI) --
// Writes the textual plan of a problem into buf; returns the number of passes
// or a negative fastKronError.
int fkbDescribePlan(int isKmm, int isDouble, uint32_t M, uint32_t N, const uint32_t* Ps,
                    const uint32_t* Qs, int opX, int opF, int forwardMode, int haveTemp2, int fusion,
                    int align, char* buf, size_t bufLen) {
  Problem pr;
  if (!fillProblem(&pr, isKmm ? MMType::KMM : MMType::MKM, isDouble ? DType::F64 : DType::F32, M, N,
                   Ps, Qs, (fastKronOp)opX, (fastKronOp)opF))
    return -(int)fastKronInvalidArgument;
  pr.forward = forwardMode != 0;
  if (pr.mm == MMType::KMM && pr.M == 1) {
    pr.mm = MMType::MKM; pr.opX = fastKronOp_N;
    pr.opF = (pr.opF == fastKronOp_N) ? fastKronOp_T : fastKronOp_N;
  }
  PlanOptions po;
  po.haveT2 = haveTemp2 != 0; po.fusion = fusion != 0; po.align = align;
  Plan plan;
  fastKronError e = makePlan(pr, po, &plan);
  if (e != fastKronSuccess) return -(int)e;
  const std::string s = plan.describe();
  if (buf && bufLen) {
    const size_t n = s.size() < bufLen - 1 ? s.size() : bufLen - 1;
    memcpy(buf, s.data(), n);
    buf[n] = 0;
  }
  return (int)plan.passes.size();
}

}  // extern "C"

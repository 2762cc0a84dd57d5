// sgemkmNoAlloc: GeMKM for callers that are not allowed to allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a
// product: code running inside another framework's memory plan (a caching allocator
// whose pool is already carved up, an inference server that fixes its device
// footprint at start-up), or real-time / safety-partitioned processes in which
// allocation after initialisation is forbidden.  sgemkm needs two temporaries that
// such a caller cannot provide.  This entry point takes them from a fixed buffer that
// is part of the library image instead: a file-scope __device__ array, present once on
// every GPU that loads the library and held until the process exits.
//
// Rules that follow from the buffer being shared and static:
//   * limit: each temporary holds at most FASTKRON_NOALLOC_MAX_TEMP_ELEMS floats
//     (what gekmmSizes reports as tmpElems); larger problems are rejected with
//     fastKronInvalidArgument and a message on stderr, nothing is launched;
//   * the first call on a device resolves the buffer's device address (one
//     cudaGetSymbolAddress with that device current); make that first call before any
//     stream capture begins;
//   * every call on a device uses the same buffer: two calls whose kernels can overlap
//     on the GPU (different streams, different handles) race on it -- serialise them;
//   * the buffer keeps whatever the previous call left there.  No kernel of this
//     library reads a temporary before the same call has written it, so nothing has to
//     be cleared.
// The function itself calls no cudaMalloc / cudaFree or other allocating routine.
#include <stdio.h>

#include "engine.h"
#include "fastkron.h"

using namespace fkb;

namespace {

constexpr size_t kMaxTmp = FASTKRON_NOALLOC_MAX_TEMP_ELEMS;

// temp1 = first half, temp2 = second half
static __device__ __align__(256) float gNoAllocScratch[2 * kMaxTmp];

// Device address of gNoAllocScratch per device ordinal.  The symbol's name is only a
// host-side handle: kernels must be given the address cudaGetSymbolAddress returns for
// the device that is current.
float* gScratchAddr[kMaxDevices] = {nullptr};

}  // namespace

extern "C" fastKronError sgemkmNoAlloc(fastKronHandle handle, uint32_t M, uint32_t N, uint32_t Ps[],
                                       uint32_t Qs[], const float* X, fastKronOp opX,
                                       const float* const Fs[], fastKronOp opFs, float* Z, float alpha,
                                       float beta, const float* Y) {
  if (!handle || !Ps || !Qs || N == 0 || N > (uint32_t)kMaxFactors) return fastKronInvalidArgument;
  Engine* e = reinterpret_cast<Engine*>(handle);
  if (!e->hasBackend(fastKronBackend_CUDA) || !e->cudaReady()) return fastKronBackendNotAvailable;
  if ((opX != fastKronOp_N && opX != fastKronOp_T) || (opFs != fastKronOp_N && opFs != fastKronOp_T))
    return fastKronInvalidArgument;

  Problem pr;
  pr.mm = MMType::MKM; pr.dt = DType::F32; pr.M = M; pr.N = N; pr.opX = opX; pr.opF = opFs;
  for (uint32_t i = 0; i < N; i++) { pr.P[i] = Ps[i]; pr.Q[i] = Qs[i]; }
  size_t yElems = 0, tmpElems = 0;
  fastKronError err = e->sizes(pr, &yElems, &tmpElems);
  if (err != fastKronSuccess) return err;
  if (tmpElems > kMaxTmp) {
    fprintf(stderr,
            "sgemkmNoAlloc: problem needs temporaries of %zu elements, the static scratch holds %zu "
            "(FASTKRON_NOALLOC_MAX_TEMP_ELEMS); use sgemkm with caller-provided temporaries\n",
            tmpElems, kMaxTmp);
    return fastKronInvalidArgument;
  }

  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return fastKronOtherError;
  // The handle's stream belongs to the device that was current at fastKronInitCUDA; the scratch
  // address is per device, so the two must agree.
  if (dev != e->device()) {
    fprintf(stderr, "sgemkmNoAlloc: current device %d is not the handle's device %d\n", dev, e->device());
    return fastKronInvalidArgument;
  }
  if (gScratchAddr[dev] == nullptr) {
    // once per device, with that device current
    float* p = nullptr;
    const cudaError_t ce = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), gNoAllocScratch);
    if (ce != cudaSuccess || p == nullptr) {
      fprintf(stderr, "sgemkmNoAlloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(ce));
      return fastKronOtherError;
    }
    gScratchAddr[dev] = p;
  }

  CallOperands ops;
  ops.X = X; ops.Fs = reinterpret_cast<const void* const*>(Fs); ops.Z = Z; ops.Y = Y;
  ops.temp1 = gScratchAddr[dev];
  ops.temp2 = gScratchAddr[dev] + kMaxTmp;
  ops.alpha = (double)alpha; ops.beta = (double)beta;
  return e->run(pr, ops);
}

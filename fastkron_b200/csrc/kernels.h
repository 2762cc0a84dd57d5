// Launch interface between the host planner and the device kernels.
#pragma once

#include <cuda_runtime.h>

#include "fk_common.h"

namespace fkb {

// Everything a kernel launcher needs besides the Pass itself.
struct LaunchCtx {
  cudaStream_t stream = nullptr;
  DType  dt = DType::F32;
  const void* src = nullptr;      // pass input
  void*       dst = nullptr;      // pass output
  const void* Y   = nullptr;      // epilogue operand (may be null when beta == 0)
  const void* F[kMaxGroup] = {nullptr};   // device pointers of factors f0 .. f0+nf-1
  int64_t fsP = 1, fsQ = 1;       // factor element (p,q) at p*fsP + q*fsQ
  double alpha = 1.0, beta = 0.0; // applied only when pass.epilogue
  int smCount = 148;
};

// Each returns fastKronKernelNotFound when the pass does not fit the kernel
// family (the caller then falls back to the generic kernel), or a CUDA failure
// mapped to a fastKronError.
fastKronError launchGeneric(const Pass& ps, const LaunchCtx& cx);
fastKronError launchTile(const Pass& ps, const LaunchCtx& cx);
fastKronError launchGemm(const Pass& ps, const LaunchCtx& cx);

// True when launchTile / launchGemm have an instantiation for the pass; used
// by the planner's caller to downgrade a pass to Generic up front.
bool tileSupported(DType dt, uint32_t P, int nf, int tileB);
bool gemmSupported(DType dt, uint32_t P, uint32_t Q, uint64_t B);

inline fastKronError cudaToFk(cudaError_t e) {
  if (e == cudaSuccess) return fastKronSuccess;
  if (e == cudaErrorIllegalAddress) return fastKronInvalidMemoryAccess;
  if (e == cudaErrorInvalidValue || e == cudaErrorInvalidConfiguration) return fastKronInvalidArgument;
  return fastKronOtherError;
}

}  // namespace fkb

// Launch interface between the host planner and the device kernels.
#pragma once

#include <cuda_runtime.h>

#include "fk_common.h"

namespace fkb {

// Output redirection of a pass whose result is redistributed over several GPUs (the
// all-to-all of the column-sharded multi-GPU path, fused into the producing kernel's
// stores).  With chunk n = m*aLoc + a, output row (n, q) and trailing position b:
//   address = base[q / qPer] + m*sM + a*sA + (q % qPer)*sQ + zOff + b
// base[d] is a buffer on GPU d, reached with plain peer stores.  parts == 0: off.
constexpr int kMaxParts = 8;
struct Scatter {
  int parts = 0;
  void* base[kMaxParts] = {nullptr};
  unsigned long long qPer = 1, aLoc = 1;
  long long sM = 0, sA = 0, sQ = 0, zOff = 0;
};

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
  Scatter scatter;                // only honoured by the Generic and Gemm launchers
  // Gemm launcher only: input rows split as [outer][chunk][pSplit][B] (see GemmArgs)
  unsigned pSplit = 0;
  unsigned long long pOuter = 0, nStride = 0;
  // Gemm launcher: opt-in tensor-core kernels for fp32 passes: 0 off, 1 TF32 operands
  // (fastKronOptionsTF32), 3 split TF32 with fp32-level results (fastKronOptionsTF32x3)
  int tf32 = 0;
  // Strided batch in ONE launch (the reference batches in grid.z, src/kernels/gpu_kmmkernel.h:124-144):
  // entry e of `batch` reads src + e*bsX, writes dst + e*bsZ, uses Y + e*bsY and factor k at
  // F[k] + e*bsF[k] (element strides; 0 = shared).  Honoured by the generic, any-shape and
  // tile pass kernels (passBatchCapable); the engine loops over entries for the others.
  uint32_t batch = 1;
  uint64_t bsX = 0, bsZ = 0, bsY = 0;
  uint64_t bsF[kMaxGroup] = {0};
};

// True when the kernel that runs `ps` takes a strided batch in one launch.
inline bool passBatchCapable(const Pass& ps) {
  if (ps.kind == KernelKind::Generic) return true;
  if (ps.kind == KernelKind::Gemm) return ps.variant == 3;
  return ps.kind == KernelKind::Tile && ps.variant == 0;
}

// Each returns fastKronKernelNotFound when the pass does not fit the kernel
// family (the caller then falls back to the generic kernel), or a CUDA failure
// mapped to a fastKronError.
fastKronError launchGeneric(const Pass& ps, const LaunchCtx& cx);
fastKronError launchTile(const Pass& ps, const LaunchCtx& cx);
fastKronError launchGemm(const Pass& ps, const LaunchCtx& cx);
fastKronError launchGemmTf32(const Pass& ps, const LaunchCtx& cx);   // only reached through launchGemm
fastKronError launchGemmAny(const Pass& ps, const LaunchCtx& cx);    // any shape, strides, alignment (through launchGemm)

// True when launchTile / launchGemm have an instantiation for the pass; used
// by the planner's caller to downgrade a pass to Generic up front.
bool tileSupported(DType dt, uint32_t P, int nf, int tileB);
bool gemmSupported(DType dt, uint32_t P, uint32_t Q, uint64_t B);

// Function attributes (the opt-in to more than 48 KB of dynamic shared memory) and occupancy
// answers belong to one device: a launcher that caches them keeps one slot per device ordinal,
// indexed by the device that is current at the launch.
constexpr int kMaxDevices = 64;
inline int currentDeviceSlot() {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess) { cudaGetLastError(); return 0; }
  return (d >= 0 && d < kMaxDevices) ? d : 0;
}

inline fastKronError cudaToFk(cudaError_t e) {
  if (e == cudaSuccess) return fastKronSuccess;
  if (e == cudaErrorIllegalAddress) return fastKronInvalidMemoryAccess;
  if (e == cudaErrorInvalidValue || e == cudaErrorInvalidConfiguration) return fastKronInvalidArgument;
  return fastKronOtherError;
}

}  // namespace fkb

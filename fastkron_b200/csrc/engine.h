// The engine behind a fastKronHandle: options, stream, plan cache and the code
// that walks a plan and launches its passes.
#pragma once

#include <stdlib.h>

#include <cuda_runtime.h>

#include <map>
#include <string>
#include <vector>

#include "fk_common.h"
#include "kernels.h"

namespace fkb {

struct MgState;   // multi-GPU context, defined in mg.cu
// Per-device result / temporary element counts once a handle is distributed.
void mgAdjustSizes(const MgState* mg, const Problem& pr, size_t* yElems, size_t* tmpElems);
void mgDestroy(MgState* mg);

// Operands of one (possibly strided-batched) call, element type erased.
struct CallOperands {
  const void* X = nullptr;
  const void* const* Fs = nullptr;   // host array of N device pointers
  void* Z = nullptr;
  const void* Y = nullptr;
  void* temp1 = nullptr;
  void* temp2 = nullptr;
  void* const* intermediates = nullptr;     // forward variants: N-1 device pointers
  double alpha = 1.0, beta = 0.0;
  // batch strides in elements (ignored when batch == 1)
  uint64_t strideX = 0, strideZ = 0, strideY = 0;
  const uint64_t* strideF = nullptr;
  const uint64_t* strideI = nullptr;
};

class Engine {
 public:
  explicit Engine(uint32_t backends);
  ~Engine();

  uint32_t backends() const { return backends_; }
  bool hasBackend(uint32_t b) const { return (backends_ & b) != 0; }
  void setOptions(uint32_t o) { options_ = o; }
  uint32_t options() const { return options_; }

  fastKronError initCUDA(void* ptrToStream);
  fastKronError setStream(void* ptrToStream);
  bool cudaReady() const { return cudaReady_; }
  cudaStream_t stream() const { return stream_; }
  int device() const { return device_; }       // device that was current at initCUDA
  // SMs of the handle's device; persistent kernels size their grids from it.
  int smCount() const { return smCount_; }
  // Tensor-core mode of fp32 large-factor passes: 3 (split TF32, fp32-level results) with
  // fastKronOptionsTF32x3 on the handle or FASTKRON_TF32=3 in the environment, 1 (TF32 operands)
  // with fastKronOptionsTF32 or FASTKRON_TF32=1, else 0.  The environment is read once.
  int tf32Mode() const {
    static const int env = [] { const char* e = getenv("FASTKRON_TF32"); return e && e[0] == '3' ? 3 : (e && e[0] == '1' ? 1 : 0); }();
    if (env == 3 || (options_ & fastKronOptionsTF32x3) != 0) return 3;
    return (env == 1 || (options_ & fastKronOptionsTF32) != 0) ? 1 : 0;
  }

  // Result / temporary element counts (per batch entry).
  fastKronError sizes(const Problem& pr, size_t* yElems, size_t* tmpElems) const;
  fastKronError sizesForward(const Problem& pr, size_t* yElems, size_t* interElems) const;

  // Plan and enqueue one call on the handle's stream.
  fastKronError run(Problem pr, const CallOperands& ops);

  // Enqueue the passes of `plan` on `stream`: for one batch entry, or (batch > 1) for all
  // entries at once, every pass one launch with the batch as a grid dimension; tmpElems is
  // then the distance between the entries' temporaries.
  fastKronError execute(const Problem& pr, const Plan& plan, const CallOperands& ops,
                        cudaStream_t stream, int smCount, uint32_t batch = 1, size_t tmpElems = 0);

  float timePlan(const Problem& pr, const Plan& plan, const CallOperands& ops);

  // Launch one pass (with fallback to the generic kernel and optional event timing).
  fastKronError launchPass(const Pass& ps, const LaunchCtx& cx);

  MgState* mg = nullptr;

  // Optional per-pass timing: when enabled, execute() brackets every kernel launch
  // with events on the launching stream; passTimes() synchronises and reads them.
  void setProfiling(bool on) { profiling_ = on; }
  int passTimes(float* ms, int* kinds, int maxN);
  static unsigned long long launchCount();

 private:
  bool profiling_ = false;
  std::vector<cudaEvent_t> evPool_;
  std::vector<int> evKinds_;
  size_t evUsed_ = 0;
  uint32_t backends_;
  uint32_t options_ = fastKronOptionsUseFusion;
  bool cudaReady_ = false;
  cudaStream_t stream_ = nullptr;
  int device_ = 0;
  int smCount_ = 148;
  std::map<std::string, Plan> planCache_;
};

// Factor element strides for (mm, opF): element (p,q) at p*fsP + q*fsQ.
inline void factorStrides(MMType mm, fastKronOp opF, uint32_t P, uint32_t Q, int64_t* fsP, int64_t* fsQ) {
  const bool pMajor = (mm == MMType::MKM) ? (opF == fastKronOp_N) : (opF == fastKronOp_T);
  if (pMajor) { *fsP = Q; *fsQ = 1; } else { *fsP = 1; *fsQ = P; }
}

}  // namespace fkb

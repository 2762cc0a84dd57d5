// Multi-GPU entry points of include/fastkronMg.h (work in progress: the
// distributed engine is not wired yet, every call reports that).
#include "engine.h"
#include "fastkronMg.h"

namespace fkb {
struct MgState { int gpus = 1, gm = 1, gk = 1; };
void mgAdjustSizes(const MgState* mg, const Problem&, size_t* yElems, size_t* tmpElems) {
  const size_t div = (size_t)mg->gm * mg->gk;
  *yElems /= div; *tmpElems /= div;
}
void mgDestroy(MgState* mg) { delete mg; }
}  // namespace fkb

extern "C" {
fastKronError fastKronMgInitCUDA(fastKronHandle, void*, int, int, int, int) { return fastKronBackendNotAvailable; }
fastKronError fastKronMgSGEMM(fastKronHandle, const uint32_t, void*[], void*[], void*[], uint32_t, uint32_t,
                              uint32_t, uint32_t[], uint32_t[], void*[], void*[], void*) {
  return fastKronBackendNotAvailable;
}
fastKronError fastKronMgAllocX(fastKronHandle, void*[], void*, uint32_t, uint32_t) { return fastKronBackendNotAvailable; }
fastKronError fastKronMgGatherY(fastKronHandle, void*[], void*, uint32_t, uint32_t, uint32_t, uint32_t[], uint32_t[]) {
  return fastKronBackendNotAvailable;
}
}

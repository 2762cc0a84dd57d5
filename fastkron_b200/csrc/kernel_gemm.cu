// Placeholder until the large-factor kernel lands: reports "no kernel" so the
// engine falls back to the generic pass.
#include "kernels.h"
namespace fkb {
bool gemmSupported(DType, uint32_t, uint32_t, uint64_t) { return false; }
fastKronError launchGemm(const Pass&, const LaunchCtx&) { return fastKronKernelNotFound; }
}

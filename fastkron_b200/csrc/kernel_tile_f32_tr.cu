// Instantiation unit: transposing tile kernels for float.
#include "kernel_tile_launch.cuh"
namespace fkb {
template fastKronError launchTileTr<float, 1>(const Pass&, const LaunchCtx&);
template fastKronError launchTileTr<float, 2>(const Pass&, const LaunchCtx&);
}

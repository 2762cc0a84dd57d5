// Instantiation unit: transposing tile kernels for double.
#include "kernel_tile_launch.cuh"
namespace fkb {
template fastKronError launchTileTr<double, 1>(const Pass&, const LaunchCtx&);
template fastKronError launchTileTr<double, 2>(const Pass&, const LaunchCtx&);
}

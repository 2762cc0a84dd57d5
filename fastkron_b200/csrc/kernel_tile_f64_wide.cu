// Instantiation unit: tile kernels for double, wide layout.
#include "kernel_tile_launch.cuh"
namespace fkb {
template fastKronError launchTileTW<double, true>(const Pass&, const LaunchCtx&);
}

// Instantiation unit: tile kernels for double, narrow layout.
#include "kernel_tile_launch.cuh"
namespace fkb {
template fastKronError launchTileTW<double, false>(const Pass&, const LaunchCtx&);
}

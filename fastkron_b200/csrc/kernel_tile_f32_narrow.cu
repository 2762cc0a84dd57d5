// Instantiation unit: tile kernels for float, narrow layout.
#include "kernel_tile_launch.cuh"
namespace fkb {
template fastKronError launchTileTW<float, false>(const Pass&, const LaunchCtx&);
}

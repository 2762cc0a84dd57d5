// Instantiation unit: tile kernels for float, wide layout.
#include "kernel_tile_launch.cuh"
namespace fkb {
template fastKronError launchTileTW<float, true>(const Pass&, const LaunchCtx&);
}

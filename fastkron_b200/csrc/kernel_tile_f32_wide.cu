// Instantiation unit: tile kernels for float, wide layout (the TMA-staged ones live here).
#include "kernel_tile_launch.cuh"
namespace fkb {
template fastKronError launchTileTW<float, true>(const Pass&, const LaunchCtx&);

int tileTmaTimeouts() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, gTileTmaTimeouts, sizeof(int)) != cudaSuccess) { cudaGetLastError(); return -1; }
  return v;
}
}

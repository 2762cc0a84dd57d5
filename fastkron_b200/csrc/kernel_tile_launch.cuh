// Host launcher for the tile kernels, templated on element type and layout so
// that each (type, layout) pair compiles in its own translation unit.
#pragma once

#include "kernel_tile.cuh"
#include "tile_table.h"

namespace fkb {

template <typename T, int P, int NF, bool WIDE>
static fastKronError launchTileOne(const Pass& ps, const LaunchCtx& cx) {
  constexpr int BT = WIDE ? (int)(128 / sizeof(T)) : 1;
  constexpr int G = ipow(P, NF);
  constexpr int SUB = G * BT;
  constexpr size_t es = sizeof(T);

  TileArgs<T> a;
  a.X = (const T*)cx.src; a.Z = (T*)cx.dst; a.Y = (const T*)cx.Y;
  for (int k = 0; k < NF; k++) a.F[k] = (const T*)cx.F[k];
  a.fsP = cx.fsP; a.fsQ = cx.fsQ;
  a.B = ps.B;
  a.tilesPerChunk = WIDE ? ps.B / BT : 1;
  const unsigned long long chunks = ps.M * ps.A;
  a.numSub = chunks * a.tilesPerChunk;
  a.alpha = (T)cx.alpha; a.beta = (T)cx.beta; a.epilogue = ps.epilogue ? 1 : 0;
  if (a.numSub == 0) return fastKronSuccess;

  // super-tile of about 32 KB (64 KB for P = 32, whose thread items are larger),
  // shrunk while the grid would leave SMs idle
  const size_t target = (P == 32 ? 64 : 32) * 1024;
  long long R = ps.tileR > 1 ? ps.tileR : (long long)(target / (SUB * es));
  if (R < 1) R = 1;
  if (WIDE && R > kTileMaxR) R = kTileMaxR;      // wide sub-tiles keep a table of bases
  while (R > 1 && (a.numSub + R - 1) / R < (unsigned long long)cx.smCount * 4) R >>= 1;
  a.R = (int)R;

  const size_t smem = (size_t)R * SUB * es + (size_t)NF * P * P * es + kTileMaxR * sizeof(unsigned long long);
  auto kern = tilePassKernel<T, P, NF, WIDE>;
  static bool attrSet = false;
  if (!attrSet) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return cudaToFk(e);
    attrSet = true;
  }
  if (smem > 200 * 1024) return fastKronKernelNotFound;
  unsigned long long supers = (a.numSub + R - 1) / R;
  const unsigned long long cap = (unsigned long long)cx.smCount * 16;
  if (supers > cap) supers = cap;
  kern<<<(unsigned)supers, kTileThreads, smem, cx.stream>>>(a);
  return cudaToFk(cudaGetLastError());
}

template <typename T, bool WIDE>
fastKronError launchTileTW(const Pass& ps, const LaunchCtx& cx) {
  const uint32_t P = ps.P[0];
  const int nf = ps.nf;
#define FKB_DISPATCH(p, n) if (P == p && nf == n) return launchTileOne<T, p, n, WIDE>(ps, cx);
  if constexpr (WIDE) { FKB_TILE_WIDE(FKB_DISPATCH) } else { FKB_TILE_NARROW(FKB_DISPATCH) }
#undef FKB_DISPATCH
  return fastKronKernelNotFound;
}

}  // namespace fkb

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
  static bool attrSetDev[kMaxDevices] = {false};
  bool& attrSet = attrSetDev[currentDeviceSlot()];
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

// ---- transposing variant (narrow table, TR = 1 or 2) ------------------------------------
template <typename T, int P, int NF, int TR>
static fastKronError launchTileTrOne(const Pass& ps, const LaunchCtx& cx) {
  constexpr int G = ipow(P, NF);
  constexpr size_t es = sizeof(T);
  TileTrArgs<T> a;
  a.X = (const T*)cx.src; a.Z = (T*)cx.dst; a.Y = (const T*)cx.Y;
  for (int k = 0; k < NF; k++) a.F[k] = (const T*)cx.F[k];
  a.fsP = cx.fsP; a.fsQ = cx.fsQ;
  a.M = ps.M; a.A = ps.A;
  a.alpha = (T)cx.alpha; a.beta = (T)cx.beta; a.epilogue = ps.epilogue ? 1 : 0;
  // rows per super-tile: 32 (128-byte runs on the m-contiguous side) while the tile stays
  // within 64 KB, fewer for large groups; then as many leading chunks as fit in ~32 KB
  int mT = 32;
  while (mT > 4 && (size_t)mT * G * es > 64 * 1024) mT >>= 1;
  if ((size_t)mT * G * es > 64 * 1024) return fastKronKernelNotFound;
  int aT = 1;
  while (aT * 2 * mT <= kTileMaxR && (size_t)aT * 2 * mT * G * es <= 32 * 1024 && (unsigned long long)aT * 2 <= ps.A) aT *= 2;
  a.mT = mT; a.aT = aT;
  a.mBlocks = (ps.M + mT - 1) / mT;
  a.numSuper = a.mBlocks * ((ps.A + aT - 1) / aT);
  if (a.numSuper == 0) return fastKronSuccess;
  const size_t smem = (size_t)mT * aT * G * es + (size_t)NF * P * P * es + 2 * kTileMaxR * sizeof(unsigned long long);
  auto kern = tileTransposeKernel<T, P, NF, TR>;
  static bool attrSetDev[kMaxDevices] = {false};
  bool& attrSet = attrSetDev[currentDeviceSlot()];
  if (!attrSet) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    if (e != cudaSuccess) return cudaToFk(e);
    attrSet = true;
  }
  unsigned long long grid = a.numSuper;
  const unsigned long long cap = (unsigned long long)cx.smCount * 16;
  if (grid > cap) grid = cap;
  kern<<<(unsigned)grid, kTileThreads, smem, cx.stream>>>(a);
  return cudaToFk(cudaGetLastError());
}

template <typename T, int TR>
fastKronError launchTileTr(const Pass& ps, const LaunchCtx& cx) {
  const uint32_t P = ps.P[0];
  const int nf = ps.nf;
#define FKB_DISPATCH(p, n) if (P == p && nf == n) return launchTileTrOne<T, p, n, TR>(ps, cx);
  FKB_TILE_NARROW(FKB_DISPATCH)
#undef FKB_DISPATCH
  return fastKronKernelNotFound;
}


}  // namespace fkb

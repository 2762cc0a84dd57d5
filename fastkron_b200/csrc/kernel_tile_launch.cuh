// Host launcher for the tile kernels, templated on element type and layout so
// that each (type, layout) pair compiles in its own translation unit.
#pragma once

#include <cuda.h>            // CUtensorMap (type only; the encoder is fetched at run time)
#include <string.h>
#include <stdlib.h>

#include "kernel_tile.cuh"
#include "tile_table.h"
#include "tile_db.h"

namespace fkb {

// cuTensorMapEncodeTiled from the driver, without linking libcuda.
typedef CUresult (*TileEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline TileEncodeFn tileMapEncoder() {
  static TileEncodeFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<TileEncodeFn>(p);
    else
      cudaGetLastError();
  }
  return fn;
}

// Tensor map over a wide pass's input viewed as [entries][chunks][G][B] fp32 (entries of a
// strided batch `bsX` elements apart; 1 entry otherwise), box {32, min(G, 256), 1, 1}.
inline bool encodeTileMap(TileTmaMap* out, const void* X, unsigned long long chunks, unsigned G, unsigned long long B,
                          unsigned batch, unsigned long long bsX) {
  static_assert(sizeof(CUtensorMap) <= sizeof(TileTmaMap), "tensor map size");
  TileEncodeFn enc = tileMapEncoder();
  if (!enc || B > 0xFFFFFFFFull || chunks > 0x7FFFFFFFull || (B * 4) % 16 != 0) return false;
  if (batch > 1 && ((bsX * 4) % 16 != 0 || bsX == 0)) return false;
  const cuuint64_t dims[4] = {B, G, chunks, batch};
  const cuuint64_t strides[3] = {B * 4, (cuuint64_t)G * B * 4, batch > 1 ? bsX * 4 : (cuuint64_t)chunks * G * B * 4};
  const cuuint32_t box[4] = {32, G < 256 ? G : 256, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(X), dims, strides, box,
             estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename T, int P, int NF, bool WIDE, bool TMA, int MINB = kTileMinBlocks, int NBUF = 2>
static fastKronError launchTileKernel(const TileArgs<T>& a, const TileTmaMap& tm, const TileTmaMap& tmOut, size_t smem,
                                      unsigned long long supers, const LaunchCtx& cx) {
  auto kern = tilePassKernel<T, P, NF, WIDE, TMA, MINB, NBUF>;
  // per device: the shared-memory opt-in, and the occupancy for the last tile size seen
  static bool attrSetDev[kMaxDevices] = {false};
  static size_t occSmemDev[kMaxDevices] = {0};
  static int occDev[kMaxDevices] = {0};
  const int dev = currentDeviceSlot();
  if (!attrSetDev[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return cudaToFk(e);
    attrSetDev[dev] = true;
  }
  if (occSmemDev[dev] != smem || occDev[dev] < 1) {
    int q = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&q, kern, kTileThreads, smem) != cudaSuccess || q < 1) {
      cudaGetLastError();
      return fastKronKernelNotFound;
    }
    occSmemDev[dev] = smem; occDev[dev] = q;
  }
  const int n = occDev[dev];
  unsigned long long grid = (unsigned long long)cx.smCount * n;
  if (grid > supers) grid = supers;
  kern<<<(unsigned)grid, kTileThreads, smem, cx.stream>>>(a, tm, tmOut);
  return cudaToFk(cudaGetLastError());
}

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

  // tile size, ring depth and CTAs per SM of this kernel: the swept table, or the tuner's override
  const TileTune tn = tileTuneFor(sizeof(T) == 4 ? DType::F32 : DType::F64, P, NF, WIDE);
  const size_t target = (size_t)tn.kb * 1024;
  long long R = (long long)(target / (SUB * es));
  if (R < 1) R = 1;
  if (WIDE && R > kTileMaxR) R = kTileMaxR;      // wide sub-tiles keep a table of bases
  // shrunk while the grid would leave SMs idle
  while (R > 1 && ((a.numSub + R - 1) / R) * cx.batch < (unsigned long long)cx.smCount * 3) R >>= 1;
  a.R = (int)R;

  const size_t smem = (size_t)tn.nbuf * R * SUB * es + (size_t)NF * P * P * es + 2 * kTileMaxR * sizeof(unsigned long long);
  if (smem > 200 * 1024) return fastKronKernelNotFound;
  a.supersPerEntry = (a.numSub + R - 1) / R;
  a.batch = cx.batch; a.bsX = cx.bsX; a.bsZ = cx.bsZ; a.bsY = cx.bsY;
  a.batchedF = 0;
  for (int k = 0; k < NF; k++) { a.bsF[k] = cx.bsF[k]; if (cx.batch > 1 && cx.bsF[k] != 0) a.batchedF = 1; }
  if (cx.batch > 1 && (((cx.bsX | cx.bsZ | cx.bsY) * es) % 16) != 0) return fastKronKernelNotFound;
  const unsigned long long supers = a.supersPerEntry * a.batch;
  TileTmaMap tm, tmOut;
  memset(&tm, 0, sizeof(tm));
  memset(&tmOut, 0, sizeof(tmOut));
  a.bulkOut = 0;
  if constexpr (WIDE && sizeof(T) == 4) {
    // TMA staging needs the ring (its point is to overlap the next tile's transfer)
    if (tn.nbuf == 2 && tn.tma && encodeTileMap(&tm, a.X, chunks, (unsigned)G, a.B, a.batch, a.bsX)) {
      // no epilogue arithmetic: the tiles leave by bulk tensor stores as well
      if (!a.epilogue && encodeTileMap(&tmOut, a.Z, chunks, (unsigned)G, a.B, a.batch, a.bsZ)) a.bulkOut = 1;
      if (tn.minb >= 4) return launchTileKernel<T, P, NF, WIDE, true, 4, 2>(a, tm, tmOut, smem, supers, cx);
      return launchTileKernel<T, P, NF, WIDE, true, 3, 2>(a, tm, tmOut, smem, supers, cx);
    }
  }
  if (tn.nbuf == 1) {
    if (tn.minb >= 6) return launchTileKernel<T, P, NF, WIDE, false, 6, 1>(a, tm, tmOut, smem, supers, cx);
    return launchTileKernel<T, P, NF, WIDE, false, 4, 1>(a, tm, tmOut, smem, supers, cx);
  }
  if (tn.minb >= 4) return launchTileKernel<T, P, NF, WIDE, false, 4, 2>(a, tm, tmOut, smem, supers, cx);
  return launchTileKernel<T, P, NF, WIDE, false, 3, 2>(a, tm, tmOut, smem, supers, cx);
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
  {
    // the m-contiguous side can move 16-byte vectors when rows come in whole, aligned groups
    constexpr int VEC = 16 / (int)sizeof(T);
    const void* mSide = TR == 1 ? (const void*)cx.dst : cx.src;
    const bool yOk = TR != 1 || cx.Y == nullptr || ((uintptr_t)cx.Y & 15) == 0;
    a.vecM = (ps.M % VEC == 0 && mT % VEC == 0 && ((uintptr_t)mSide & 15) == 0 && yOk) ? 1 : 0;
  }
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

// Host launcher of the large-factor kernels (kernel_gemm.cuh).
#include "kernel_gemm.cuh"
#include "gemm_table.h"

#include <string.h>

#include <stdlib.h>

namespace fkb {

// cuTensorMapEncodeTiled from the driver, without linking libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn tensorMapEncoder() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      cudaGetLastError();
  }
  return fn;
}

// Tensor map over the pass input viewed as [chunks][P][B], box = one stage [1][PC][TJ].
template <typename T>
static bool encodeInputMap(CUtensorMap* tm, const void* X, unsigned long long chunks, unsigned P, unsigned long long B,
                           unsigned TJ, unsigned PC) {
  EncodeTiledFn enc = tensorMapEncoder();
  if (!enc || B > 0xFFFFFFFFull || chunks > 0xFFFFFFFFull || (B * sizeof(T)) % 16 != 0) return false;
  const cuuint64_t dims[3] = {B, P, chunks};
  const cuuint64_t strides[2] = {B * sizeof(T), (cuuint64_t)P * B * sizeof(T)};
  const cuuint32_t box[3] = {TJ, PC, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = sizeof(T) == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT64;
  return enc(tm, dt, 3, const_cast<void*>(X), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool gemmSupported(DType dt, uint32_t P, uint32_t Q, uint64_t B) { return gemmEligible(dt, P, Q, B); }

template <typename T, int P, int Q, int TJ, int PC, int STAGES, int MQ, int MJ, bool XT, int UNR, int MINB, bool PACK = false>
static fastKronError launchGemmOne(const Pass& ps, const LaunchCtx& cx, int mode) {
  using C = GemmCfg<T, P, Q, TJ, PC, STAGES, MQ, MJ, XT>;
  GemmArgs<T> a;
  a.X = (const T*)cx.src; a.Z = (T*)cx.dst; a.Y = (const T*)cx.Y; a.F = (const T*)cx.F[0];
  a.fsP = cx.fsP; a.fsQ = cx.fsQ;
  a.numChunks = ps.M * ps.A;
  a.B = ps.B;
  a.mode = mode;
  a.tilesPerChunk = 1;
  if (mode == 0) { a.tilesPerChunk = ps.B / TJ; a.numTiles = a.numChunks * a.tilesPerChunk; }
  else if (mode == 1) { const unsigned long long per = TJ / ps.B; a.numTiles = (a.numChunks + per - 1) / per; }
  else { a.numTiles = (a.numChunks + TJ - 1) / TJ; }
  a.alpha = (T)cx.alpha; a.beta = (T)cx.beta; a.epilogue = ps.epilogue ? 1 : 0;
  a.sc = cx.scatter;
  a.pSplit = cx.pSplit; a.pOuter = cx.pOuter; a.nStride = cx.nStride;
  if (a.pSplit != 0 && mode != 0) return fastKronKernelNotFound;
  if (a.numTiles == 0) return fastKronSuccess;
  if (a.numTiles >= (1ull << 31) / C::NCH) return fastKronKernelNotFound;   // 32-bit tile counters

  auto kern = gemmPassKernel<T, P, Q, TJ, PC, STAGES, MQ, MJ, XT, UNR, MINB, PACK>;
  static int ctasPerSmDev[kMaxDevices] = {0};
  int& ctasPerSm = ctasPerSmDev[currentDeviceSlot()];
  if (ctasPerSm == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM);
    if (e != cudaSuccess) return cudaToFk(e);
    int n = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, C::THREADS, C::SMEM);
    if (e != cudaSuccess || n < 1) return e != cudaSuccess ? cudaToFk(e) : fastKronKernelNotFound;
    ctasPerSm = n;
  }
  CUtensorMap tmap;
  memset(&tmap, 0, sizeof(tmap));
  a.useTma = 0;
  if (!XT && mode == 0 && a.pSplit == 0 && TJ <= 256 && PC <= 256 &&
      encodeInputMap<T>(&tmap, a.X, a.numChunks, P, a.B, TJ, PC))
    a.useTma = 1;
  unsigned long long grid = (unsigned long long)cx.smCount * ctasPerSm;
  if (grid > a.numTiles) grid = a.numTiles;
  kern<<<(unsigned)grid, C::THREADS, C::SMEM, cx.stream>>>(a, tmap);
  return cudaToFk(cudaGetLastError());
}

// Tile shapes per factor size, from a sweep on B200.  fp32 64x64 runs 128-thread CTAs, three
// per SM (variants that spill or hold fewer CTAs lose 10-15%).  The packed-FMA inner loop
// (fma.rn.f32x2) wins where the scalar loop was short of issue slots: the contiguous-
// contraction layout (+4%) and 128x128, where it makes an 8x16 block per thread on a
// 256-wide tile the best shape (+8%); the plain 64x64 pass measured the same either way
// and stays scalar.
static fastKronError launchGemmFixed(const Pass& ps, const LaunchCtx& cx);

// The fixed-shape kernels where they apply, the any-shape kernel otherwise.
fastKronError launchGemm(const Pass& ps, const LaunchCtx& cx) {
  if (ps.variant != 3) {
    const fastKronError e = launchGemmFixed(ps, cx);
    if (e != fastKronKernelNotFound) return e;
  }
  return launchGemmAny(ps, cx);
}

static fastKronError launchGemmFixed(const Pass& ps, const LaunchCtx& cx) {
  if (ps.nf != 1 || ps.xsB != 1 || ps.zsB != 1) return fastKronKernelNotFound;
  const uint32_t P = ps.P[0], Q = ps.Q[0];
  if (!gemmEligible(cx.dt, P, Q, ps.B)) return fastKronKernelNotFound;
  // dense [chunks][P][B] -> [chunks][Q][B] only
  if (ps.xsG != (int64_t)ps.B || ps.zsG != (int64_t)ps.B || ps.xsA != (int64_t)(P * ps.B) || ps.zsA != (int64_t)(Q * ps.B)) return fastKronKernelNotFound;
  if (ps.M > 1 && (ps.xsM != (int64_t)(ps.A * P * ps.B) || ps.zsM != (int64_t)(ps.A * Q * ps.B))) return fastKronKernelNotFound;
  if (((uintptr_t)cx.src | (uintptr_t)cx.dst | (uintptr_t)cx.Y) & 15) return fastKronKernelNotFound;
  if (cx.fsQ == 1 && (((uintptr_t)cx.F[0]) & 15)) return fastKronKernelNotFound;
  const bool xt = ps.B == 1;
  if (cx.tf32 && cx.dt == DType::F32) {
    const fastKronError e = launchGemmTf32(ps, cx);
    if (e != fastKronKernelNotFound) return e;          // shapes it does not take run in fp32 below
  }
  if (cx.dt == DType::F32) {
    constexpr int TJ = 128;
    const int mode = xt ? 2 : (ps.B % TJ == 0 ? 0 : 1);
    if (P == 64 && Q == 64) {
      if (xt) return launchGemmOne<float, 64, 64, TJ, 32, 3, 8, 8, true, 8, 3, true>(ps, cx, mode);
      return launchGemmOne<float, 64, 64, TJ, 32, 3, 8, 8, false, 16, 3>(ps, cx, mode);
    }
    if (P == 128 && Q == 128) {
      if (xt) return launchGemmOne<float, 128, 128, TJ, 32, 2, 8, 8, true, 8, 1, true>(ps, cx, mode);
      constexpr int TW = 256;                       // wide tile where the trailing extent allows it
      if (ps.B % TW == 0 || TW % ps.B == 0)
        return launchGemmOne<float, 128, 128, TW, 32, 3, 8, 16, false, 8, 1, true>(ps, cx, ps.B % TW == 0 ? 0 : 1);
      return launchGemmOne<float, 128, 128, TJ, 16, 3, 16, 8, false, 8, 2>(ps, cx, mode);
    }
  } else {
    constexpr int TJ = 128;
    const int mode = xt ? 2 : (ps.B % TJ == 0 ? 0 : 1);
    if (P == 64 && Q == 64) {
      if (xt) return launchGemmOne<double, 64, 64, TJ, 32, 2, 8, 4, true, 8, 1>(ps, cx, mode);
      return launchGemmOne<double, 64, 64, TJ, 32, 3, 8, 4, false, 8, 1>(ps, cx, mode);
    }
  }
  return fastKronKernelNotFound;
}

int gemmTmaTimeouts() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, gGemmTmaTimeouts, sizeof(int)) != cudaSuccess) { cudaGetLastError(); return -1; }
  return v;
}

}  // namespace fkb

// Non-zero if a bounded wait on a TMA stage barrier ever gave up in this process (tests).
extern "C" int fkbGemmTmaTimeouts() { return fkb::gemmTmaTimeouts(); }

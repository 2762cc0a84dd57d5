// Offline tuner for the large-factor kernel (kernel_gemm.cuh): times a list of tile-shape
// variants on synthetic passes and prints a table; the shapes compiled into kernel_gemm.cu
// are the winners of this sweep on B200.  Also prints the two FFMA ceilings the kernel is
// judged against: a register-only 8x8 outer-product stream and the same stream fed by
// 128-bit shared-memory loads.
//
//   make -C fastkron_b200/csrc tune && fastkron_b200/csrc/build/tune_gemm
//
// (The role of the reference's run-time autotuner, src/autotuner/autotuner.cpp:24-328, for
// this kernel family: measurement happens once, offline.)
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "kernel_gemm.cuh"
using namespace fkb;

template <typename T, int P, int Q, int TJ, int PC, int STAGES, int MQ, int MJ, bool XT, int UNR, int MINB, bool PACK>
static void runVariant(const char* name, const T* X, T* Z, const T* F, unsigned long long chunks, unsigned long long B) {
  using C = GemmCfg<T, P, Q, TJ, PC, STAGES, MQ, MJ, XT>;
  if (const char* flt = getenv("FKB_TUNE_FILTER")) if (!strstr(name, flt)) return;
  GemmArgs<T> a{};
  a.X = X; a.Z = Z; a.Y = nullptr; a.F = F; a.fsP = Q; a.fsQ = 1; a.numChunks = chunks; a.B = B;
  a.alpha = 1; a.beta = 0; a.epilogue = 0;
  if (XT) { a.mode = 2; a.numTiles = (chunks + TJ - 1) / TJ; a.tilesPerChunk = 1; }
  else if (B % TJ == 0) { a.mode = 0; a.tilesPerChunk = B / TJ; a.numTiles = chunks * a.tilesPerChunk; }
  else { a.mode = 1; a.tilesPerChunk = 1; a.numTiles = (chunks + TJ / B - 1) / (TJ / B); }
  auto kern = gemmPassKernel<T, P, Q, TJ, PC, STAGES, MQ, MJ, XT, UNR, MINB, PACK>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM) != cudaSuccess) {
    printf("%-46s needs %zu bytes of shared memory: skipped\n", name, C::SMEM);
    cudaGetLastError();
    return;
  }
  int occ = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, C::THREADS, C::SMEM);
  if (occ < 1) { printf("%-46s does not fit an SM\n", name); return; }
  cudaFuncAttributes fa;
  cudaFuncGetAttributes(&fa, kern);
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
  unsigned long long grid = (unsigned long long)sms * occ;
  if (grid > a.numTiles) grid = a.numTiles;
  CUtensorMap dummyMap;
  memset(&dummyMap, 0, sizeof(dummyMap));     // this tool measures the cp.async staging
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0); cudaEventCreate(&e1);
  float best = 1e9f;
  for (int it = 0; it < 6; it++) {
    cudaEventRecord(e0);
    kern<<<(unsigned)grid, C::THREADS, C::SMEM>>>(a, dummyMap);
    cudaEventRecord(e1); cudaEventSynchronize(e1);
    float ms; cudaEventElapsedTime(&ms, e0, e1);
    if (it >= 2 && ms < best) best = ms;
  }
  const cudaError_t err = cudaGetLastError();
  const double flops = 2.0 * chunks * B * P * Q;
  printf("%-62s thr=%4d CTAs/SM=%d regs=%3d spill=%4zu smem=%6zu  %8.3f ms  %7.2f TFLOP/s  %s\n", name, C::THREADS, occ,
         fa.numRegs, (size_t)fa.localSizeBytes, C::SMEM, best, flops / best / 1e9, err == cudaSuccess ? "" : cudaGetErrorString(err));
  cudaEventDestroy(e0); cudaEventDestroy(e1);
}

// ---- FFMA ceilings ---------------------------------------------------------------------
template <int MQ, int MJ, bool LDS, int THREADS, int MINB>
__global__ void __launch_bounds__(THREADS, MINB) outerProbe(float* out, int iters, const float* init) {
  __shared__ __align__(16) float sf[1024];
  __shared__ __align__(16) float sx[1024];
  for (int i = threadIdx.x; i < 1024; i += THREADS) { sf[i] = init[i]; sx[i] = init[1024 + i]; }
  __syncthreads();
  float acc[MQ][MJ];
#pragma unroll
  for (int i = 0; i < MQ; i++)
#pragma unroll
    for (int j = 0; j < MJ; j++) acc[i][j] = 0.f;
  float f[MQ], x[MJ];
#pragma unroll
  for (int i = 0; i < MQ; i++) f[i] = sf[(threadIdx.x + i) & 1023];
#pragma unroll
  for (int j = 0; j < MJ; j++) x[j] = sx[(threadIdx.x + j) & 1023];
  const int lane = threadIdx.x & 31;
  for (int it = 0; it < iters; it++) {
#pragma unroll 8
    for (int p = 0; p < 32; p++) {
      if (LDS) {
#pragma unroll
        for (int g = 0; g < MQ / 4; g++) {
          const float4 v = *reinterpret_cast<const float4*>(sf + ((p * 32 + g * 16 + (lane & 3) * 4) & 1023));
          f[g * 4] = v.x; f[g * 4 + 1] = v.y; f[g * 4 + 2] = v.z; f[g * 4 + 3] = v.w;
        }
#pragma unroll
        for (int g = 0; g < MJ / 4; g++) {
          const float4 v = *reinterpret_cast<const float4*>(sx + ((p * 32 + g * 128 + (lane >> 2) * 4) & 1023));
          x[g * 4] = v.x; x[g * 4 + 1] = v.y; x[g * 4 + 2] = v.z; x[g * 4 + 3] = v.w;
        }
      }
#pragma unroll
      for (int i = 0; i < MQ; i++)
#pragma unroll
        for (int j = 0; j < MJ; j++) acc[i][j] = fmaf(f[i], x[j], acc[i][j]);
    }
  }
  float s = 0;
#pragma unroll
  for (int i = 0; i < MQ; i++)
#pragma unroll
    for (int j = 0; j < MJ; j++) s += acc[i][j];
  out[blockIdx.x * THREADS + threadIdx.x] = s;
}

template <int MQ, int MJ, bool LDS, int THREADS, int MINB>
static void runProbe(const char* name, float* out, const float* init) {
  auto k = outerProbe<MQ, MJ, LDS, THREADS, MINB>;
  int occ = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k, THREADS, 0);
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
  const int iters = 2000, grid = sms * occ;
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0); cudaEventCreate(&e1);
  float best = 1e9f;
  for (int r = 0; r < 5; r++) {
    cudaEventRecord(e0); k<<<grid, THREADS>>>(out, iters, init); cudaEventRecord(e1); cudaEventSynchronize(e1);
    float ms; cudaEventElapsedTime(&ms, e0, e1);
    if (r >= 1 && ms < best) best = ms;
  }
  const double fl = 2.0 * grid * THREADS * (double)iters * 32 * MQ * MJ;
  printf("%-62s thr=%4d CTAs/SM=%d  %8.3f ms  %7.2f TFLOP/s\n", name, THREADS, occ, best, fl / best / 1e9);
}


// Same stream on the packed instruction (fma.rn.f32x2 of sm_100: two independent IEEE fp32
// FMAs per lane and instruction, so half the issue slots for the same arithmetic).  The
// accumulators pair neighbouring j; the factor operand must hold the same value in both
// halves: DUP = 0 duplicates in registers inside the loop, DUP = 1 reads (f, f) pairs that
// were stored duplicated in shared memory.
template <int MQ, int MJ, bool LDS, int DUP, int THREADS, int MINB>
__global__ void __launch_bounds__(THREADS, MINB) outerProbe2(float* out, int iters, const float* init) {
  __shared__ __align__(16) float sf[2048];
  __shared__ __align__(16) float sx[1024];
  for (int i = threadIdx.x; i < 1024; i += THREADS) { sf[2 * i] = sf[2 * i + 1] = init[i]; sx[i] = init[1024 + i]; }
  __syncthreads();
  float2 acc[MQ][MJ / 2];
#pragma unroll
  for (int i = 0; i < MQ; i++)
#pragma unroll
    for (int j = 0; j < MJ / 2; j++) acc[i][j] = make_float2(0.f, 0.f);
  float2 f[MQ], x[MJ / 2];
#pragma unroll
  for (int i = 0; i < MQ; i++) { const float v = sf[(threadIdx.x + i) & 1023]; f[i] = make_float2(v, v); }
#pragma unroll
  for (int j = 0; j < MJ / 2; j++) x[j] = make_float2(sx[(threadIdx.x + 2 * j) & 1023], sx[(threadIdx.x + 2 * j + 1) & 1023]);
  const int lane = threadIdx.x & 31;
  for (int it = 0; it < iters; it++) {
#pragma unroll 8
    for (int p = 0; p < 32; p++) {
      if (LDS) {
        if (DUP) {
#pragma unroll
          for (int g = 0; g < MQ / 2; g++) {
            const float4 v = *reinterpret_cast<const float4*>(sf + ((p * 64 + g * 16 + (lane & 3) * 4) & 2047));
            f[g * 2] = make_float2(v.x, v.y); f[g * 2 + 1] = make_float2(v.z, v.w);
          }
        } else {
#pragma unroll
          for (int g = 0; g < MQ / 4; g++) {
            const float4 v = *reinterpret_cast<const float4*>(sf + ((p * 32 + g * 16 + (lane & 3) * 4) & 1023));
            f[g * 4] = make_float2(v.x, v.x); f[g * 4 + 1] = make_float2(v.y, v.y);
            f[g * 4 + 2] = make_float2(v.z, v.z); f[g * 4 + 3] = make_float2(v.w, v.w);
          }
        }
#pragma unroll
        for (int g = 0; g < MJ / 4; g++) {
          const float4 v = *reinterpret_cast<const float4*>(sx + ((p * 32 + g * 128 + (lane >> 2) * 4) & 1023));
          x[g * 2] = make_float2(v.x, v.y); x[g * 2 + 1] = make_float2(v.z, v.w);
        }
      }
#pragma unroll
      for (int i = 0; i < MQ; i++)
#pragma unroll
        for (int j = 0; j < MJ / 2; j++) acc[i][j] = __ffma2_rn(f[i], x[j], acc[i][j]);
    }
  }
  float s = 0;
#pragma unroll
  for (int i = 0; i < MQ; i++)
#pragma unroll
    for (int j = 0; j < MJ / 2; j++) s += acc[i][j].x + acc[i][j].y;
  out[blockIdx.x * THREADS + threadIdx.x] = s;
}

template <int MQ, int MJ, bool LDS, int DUP, int THREADS, int MINB>
static void runProbe2(const char* name, float* out, const float* init) {
  auto k = outerProbe2<MQ, MJ, LDS, DUP, THREADS, MINB>;
  int occ = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k, THREADS, 0);
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
  const int iters = 2000, grid = sms * occ;
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0); cudaEventCreate(&e1);
  float best = 1e9f;
  for (int r = 0; r < 5; r++) {
    cudaEventRecord(e0); k<<<grid, THREADS>>>(out, iters, init); cudaEventRecord(e1); cudaEventSynchronize(e1);
    float ms; cudaEventElapsedTime(&ms, e0, e1);
    if (r >= 1 && ms < best) best = ms;
  }
  const double fl = 2.0 * grid * THREADS * (double)iters * 32 * MQ * MJ;
  printf("%-62s thr=%4d CTAs/SM=%d  %8.3f ms  %7.2f TFLOP/s\n", name, THREADS, occ, best, fl / best / 1e9);
}

int main() {
  const unsigned long long ch = 1024, Bb = 4096;          // 1024 x 64 x 4096 floats = 1 GiB per buffer
  float *X, *Z, *F, *init;
  const size_t n = ch * 128 * Bb / 2;
  if (cudaMalloc(&X, n * 4) != cudaSuccess || cudaMalloc(&Z, n * 4) != cudaSuccess ||
      cudaMalloc(&F, 128 * 128 * 4) != cudaSuccess || cudaMalloc(&init, 2048 * 4) != cudaSuccess) {
    printf("allocation failed\n");
    return 1;
  }
  cudaMemset(X, 0, n * 4); cudaMemset(F, 0, 128 * 128 * 4); cudaMemset(init, 0, 2048 * 4);
#define RUN1(P, Q, TJ, PC, ST, MQ, MJ, XT, UNR, MINB, CH, BB, PK) \
  runVariant<float, P, Q, TJ, PC, ST, MQ, MJ, XT, UNR, MINB, PK>(#P "x" #Q " TJ" #TJ " PC" #PC " S" #ST " " #MQ "x" #MJ " xt=" #XT " unroll" #UNR " minb" #MINB " packed=" #PK, X, Z, F, CH, BB)
#define RUN(P, Q, TJ, PC, ST, MQ, MJ, XT, UNR, MINB, CH, BB) \
  RUN1(P, Q, TJ, PC, ST, MQ, MJ, XT, UNR, MINB, CH, BB, false); RUN1(P, Q, TJ, PC, ST, MQ, MJ, XT, UNR, MINB, CH, BB, true)
  printf("== FFMA ceilings (no global traffic)\n");
  runProbe<8, 8, false, 128, 4>("8x8 outer product, registers only", Z, init);
  runProbe<8, 8, true, 128, 4>("8x8 outer product, operands from shared memory", Z, init);
  runProbe<16, 8, true, 128, 2>("16x8 outer product, operands from shared memory", Z, init);
  printf("== the same on packed FFMA2 (fma.rn.f32x2)\n");
  runProbe2<8, 8, false, 0, 128, 4>("8x8 packed, registers only", Z, init);
  runProbe2<8, 8, true, 0, 128, 4>("8x8 packed, smem operands, factor duplicated in registers", Z, init);
  runProbe2<8, 8, true, 1, 128, 4>("8x8 packed, smem operands, factor stored duplicated", Z, init);
  runProbe2<16, 8, true, 1, 128, 2>("16x8 packed, smem operands, factor stored duplicated", Z, init);
  runProbe2<8, 16, true, 1, 128, 2>("8x16 packed, smem operands, factor stored duplicated", Z, init);
  if (getenv("FKB_TUNE_PROBES_ONLY")) return 0;
  printf("== 64x64, trailing extent 4096 (tile mode 0)\n");
  RUN(64, 64, 128, 32, 3, 8, 8, false, 16, 3, ch, Bb);
  RUN(64, 64, 128, 32, 3, 8, 8, false, 8, 3, ch, Bb);
  RUN(64, 64, 128, 32, 3, 8, 8, false, 4, 3, ch, Bb);
  RUN(64, 64, 128, 32, 4, 8, 8, false, 8, 3, ch, Bb);
  RUN(64, 64, 128, 32, 2, 8, 8, false, 16, 4, ch, Bb);
  RUN(64, 64, 128, 16, 3, 8, 8, false, 16, 4, ch, Bb);
  RUN(64, 64, 128, 16, 4, 8, 8, false, 16, 4, ch, Bb);
  RUN(64, 64, 128, 32, 3, 8, 8, false, 32, 3, ch, Bb);
  RUN(64, 64, 128, 16, 4, 8, 8, false, 16, 3, ch, Bb);
  RUN(64, 64, 128, 64, 2, 8, 8, false, 8, 3, ch, Bb);
  RUN(64, 64, 256, 32, 3, 8, 8, false, 8, 2, ch, Bb);
  RUN(64, 64, 256, 32, 3, 8, 8, false, 32, 2, ch, Bb);
  RUN(64, 64, 256, 32, 3, 8, 8, false, 8, 1, ch, Bb);
  RUN(64, 64, 256, 32, 3, 8, 4, false, 8, 2, ch, Bb);
  RUN(64, 64, 256, 32, 3, 16, 8, false, 8, 1, ch, Bb);
  RUN(64, 64, 256, 32, 3, 8, 16, false, 8, 1, ch, Bb);
  printf("== 64x64, contiguous contraction index (tile mode 2)\n");
  RUN(64, 64, 128, 32, 3, 8, 8, true, 8, 3, ch * Bb, 1);
  RUN(64, 64, 256, 32, 2, 8, 8, true, 8, 2, ch * Bb, 1);
  RUN(64, 64, 256, 32, 2, 16, 8, true, 8, 1, ch * Bb, 1);
  RUN(128, 128, 128, 32, 2, 8, 8, true, 8, 1, ch / 2 * Bb, 1);
  printf("== 128x128, trailing extent 4096\n");
  RUN(128, 128, 128, 16, 3, 16, 8, false, 8, 2, ch / 2, Bb);
  RUN(128, 128, 128, 32, 3, 8, 8, false, 8, 1, ch / 2, Bb);
  RUN(128, 128, 256, 32, 3, 8, 8, false, 8, 1, ch / 2, Bb);
  RUN(128, 128, 256, 32, 3, 16, 8, false, 8, 1, ch / 2, Bb);
  RUN(128, 128, 256, 32, 3, 8, 16, false, 8, 1, ch / 2, Bb);
  return 0;
}

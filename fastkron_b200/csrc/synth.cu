// Seeded synthetic inputs for tests and benchmarks, generated directly in HBM.
// Element i of the stream with seed s is u(s, i) = SplitMix64(s*C + i) mapped to a
// uniform value in [-1, 1) through its top 53 bits.  fastkron_b200/synth.py holds
// the bit-identical numpy version.  Built as its own small library
// (libfkb_synth.so) so that the product library contains only the FastKron ABI.
#include <cuda_runtime.h>
#include <stdint.h>

__host__ __device__ inline uint64_t fkbSplitMix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__host__ __device__ inline double fkbUniformPm1(uint64_t seed, uint64_t i) {
  const uint64_t h = fkbSplitMix64(seed * 0xD1342543DE82EF95ull + i);
  return (double)(h >> 11) * (2.0 / 9007199254740992.0) - 1.0;
}

template <typename T>
__global__ void fillUniformKernel(T* dst, uint64_t n, uint64_t seed, uint64_t offset) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    dst[i] = (T)fkbUniformPm1(seed, offset + i);
}

extern "C" {
int fkbFillUniformF32(float* dst, uint64_t n, uint64_t seed, uint64_t offset, void* stream) {
  fillUniformKernel<float><<<148 * 8, 256, 0, (cudaStream_t)stream>>>(dst, n, seed, offset);
  return (int)cudaGetLastError();
}
int fkbFillUniformF64(double* dst, uint64_t n, uint64_t seed, uint64_t offset, void* stream) {
  fillUniformKernel<double><<<148 * 8, 256, 0, (cudaStream_t)stream>>>(dst, n, seed, offset);
  return (int)cudaGetLastError();
}
}

// The same streams on the host (multi-threaded), for operands that start in host memory.
extern "C" {
void fkbFillUniformHostF32(float* dst, uint64_t n, uint64_t seed, uint64_t offset) {
#pragma omp parallel for schedule(static)
  for (long long i = 0; i < (long long)n; i++) dst[i] = (float)fkbUniformPm1(seed, offset + (uint64_t)i);
}
void fkbFillUniformHostF64(double* dst, uint64_t n, uint64_t seed, uint64_t offset) {
#pragma omp parallel for schedule(static)
  for (long long i = 0; i < (long long)n; i++) dst[i] = fkbUniformPm1(seed, offset + (uint64_t)i);
}
// FP32 / FP64 FMA peak of a device from its properties, in TFLOP/s:
// SMs x lanes x 2 x maximum SM clock, with 128 FP32 and 64 FP64 lanes per SM on compute
// capability 10.x.  Returns 0 when the device cannot be queried.
double fkbSimtPeakFromProps(int device, int isDouble) {
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { cudaGetLastError(); return 0.0; }
  int khz = 0;
  if (cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, device) != cudaSuccess) { cudaGetLastError(); return 0.0; }
  const double lanes = isDouble ? 64.0 : 128.0;
  return (double)prop.multiProcessorCount * lanes * 2.0 * (double)khz * 1e3 / 1e12;
}
}

// ---- arithmetic peak probes (used by bench.py for the FP32 / FP64 rooflines) --------
// Each thread runs 16 independent FMA chains; the result is stored so the work is kept.
template <typename T>
__global__ void __launch_bounds__(256) fmaPeakKernel(T* out, int iters, T a, T b) {
  T acc[16];
#pragma unroll
  for (int i = 0; i < 16; i++) acc[i] = (T)(threadIdx.x + i);
  for (int it = 0; it < iters; it++) {
#pragma unroll
    for (int i = 0; i < 16; i++) acc[i] = fma(acc[i], a, b);
  }
  T s = 0;
#pragma unroll
  for (int i = 0; i < 16; i++) s += acc[i];
  out[(size_t)blockIdx.x * blockDim.x + threadIdx.x] = s;
}

extern "C" {
// Runs the probe once on `stream`; returns the number of FMAs executed (0 on failure).
// `out` must hold blocks*256 elements.
unsigned long long fkbFmaPeakF32(float* out, int blocks, int iters, void* stream) {
  fmaPeakKernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>(out, iters, 0.999f, 0.001f);
  if (cudaGetLastError() != cudaSuccess) return 0;
  return (unsigned long long)blocks * 256ull * 16ull * (unsigned long long)iters;
}
unsigned long long fkbFmaPeakF64(double* out, int blocks, int iters, void* stream) {
  fmaPeakKernel<double><<<blocks, 256, 0, (cudaStream_t)stream>>>(out, iters, 0.999, 0.001);
  if (cudaGetLastError() != cudaSuccess) return 0;
  return (unsigned long long)blocks * 256ull * 16ull * (unsigned long long)iters;
}
}

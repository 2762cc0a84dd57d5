// Shared-memory tile kernel for small square power-of-two factors.
//
// One pass contracts NF consecutive tensor modes of size P in place:
//   [chunks][G = P^NF][B]  ->  same shape,   chunks = M*A.
// A CTA stages a super-tile of R sub-tiles in shared memory, applies the NF
// factors one after the other without leaving the SM, and streams the result
// out with 128-bit stores.  A sub-tile is one [G] block (narrow, B == 1) or a
// [G][W] slab with W = 128 bytes of trailing elements (wide, B > 1).
//
// Inside a step every thread owns whole fibres (the P inputs and P outputs of
// one contraction), so a step is read-all / compute / write-all per thread and
// needs no barrier except between steps; the tile is updated in place.
//
// Shared-memory addressing.  Logical tile index i lives at phys(i): the 16-byte
// chunk index inside each 128-byte line is XOR-ed with a 3-bit fold of the line
// number.  phys is linear over XOR, and because P, W and the strides are powers
// of two the index of (fibre, p) is fibreBase | p*S, hence
//   phys(fibreBase + p*S) = phys(fibreBase) ^ phys(p*S)
// with the second term a compile-time constant in the unrolled p loop.  The fold
// makes both the contiguous-fibre step (stride 1) and the strided steps free of
// bank conflicts for 128-bit accesses.
//
// The arithmetic of each contraction is the reference's: for every output the
// products are accumulated over p ascending (src/kernels/cuda/mma.cuh:1-15),
// factors applied from the last of the group to the first
// (src/kmm/kmmalgo.cpp:172-214).
#pragma once

#include "kernels.h"

#include <cmath>

namespace fkb {

template <typename T>
struct TileArgs {
  const T* X; T* Z; const T* Y;
  const T* F[kMaxGroup];
  long long fsP, fsQ;
  unsigned long long B;              // trailing extent in elements
  unsigned long long tilesPerChunk;  // B / W (1 for narrow)
  unsigned long long numSub;         // chunks * tilesPerChunk
  int R;                             // sub-tiles per super-tile
  T alpha, beta;
  int epilogue;
  // strided batch: super-tile index = entry * supersPerEntry + super-tile within the entry
  unsigned batch;
  unsigned long long supersPerEntry, bsX, bsZ, bsY;
  unsigned long long bsF[kMaxGroup];
  int batchedF;                      // some factor differs between entries: reload on entry change
  int bulkOut;                       // TMA kernels: drain with bulk tensor stores (no epilogue arithmetic)
};

constexpr int kTileThreads = 128;
constexpr int kTileMinBlocks = 3;     // two tile buffers of ~32 KB per CTA: three CTAs per SM
constexpr int kStepUnroll = 4;        // p iterations unrolled in a contraction step
constexpr int kTileMaxR = 64;

__host__ __device__ constexpr int ipow(int b, int e) { return e == 0 ? 1 : b * ipow(b, e - 1); }

template <typename T, bool SWZ = true>
__host__ __device__ constexpr unsigned physIdx(unsigned idx) {
  if (!SWZ) return idx;                          // linear tile (filled by TMA; wide layouts only)
  constexpr int LB = (sizeof(T) == 4) ? 5 : 4;   // log2(elements per 128-byte line)
  constexpr int VB = (sizeof(T) == 4) ? 2 : 1;   // log2(elements per 16-byte chunk)
  const unsigned line = idx >> LB;
  const unsigned h = (line ^ (line >> 3) ^ (line >> 6) ^ (line >> 9)) & 7u;
  return idx ^ (h << VB);
}

template <typename T>
struct alignas(16) Vec16 {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};

// W consecutive elements, W * sizeof(T) <= 16 bytes, naturally aligned.
template <typename T, int W>
struct alignas(W * sizeof(T)) VecW {
  T v[W];
};

// Accumulator budget of one thread in a contraction step: 64 registers' worth of
// outputs (64 floats / 32 doubles), i.e. kAcc/P whole fibres.
template <typename T>
struct StepShape {
  static constexpr int kAcc = 256 / (int)sizeof(T);
};
template <typename T, int P>
__host__ __device__ constexpr int stepFibres() { return StepShape<T>::kAcc / P > 0 ? StepShape<T>::kAcc / P : 1; }

__device__ __forceinline__ void cpAsync16(void* smemDst, const void* gmemSrc) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smemDst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmemSrc) : "memory");
}
__device__ __forceinline__ void cpAsync16Zfill(void* smemDst, const void* gmemSrc, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smemDst);
  const int n = valid ? 16 : 0;     // src-size 0: nothing is read, the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmemSrc), "r"(n) : "memory");
}
__device__ __forceinline__ void cpAsyncWaitAll() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
}

// Compiler-only ordering point: keeps the fully unrolled loops from hoisting every
// shared-memory load of a step to its top (which costs hundreds of registers).
__host__ __device__ __forceinline__ void schedFence() {
#ifdef __CUDA_ARCH__
  asm volatile("" ::: "memory");
#endif
}

// ---- one contraction step over a tile of E elements, mode stride S ----------

// fp32 steps use the packed FMA of sm_100 (fma.rn.f32x2: two independent IEEE fp32 FMAs per
// lane and instruction, bit-identical to two scalar FMAs) on the device; the host build of
// these templates (the CPU emulation of the tile kernels) keeps the scalar form.
#if defined(__CUDA_ARCH__)
constexpr bool kPackedFma = true;
#else
constexpr bool kPackedFma = false;
#endif

// Accumulators of a strided step: U groups of W neighbouring fibres, P outputs each.
// axpy(u, q0, f, x): acc[u][k][q0 + i] += f[i] * x[k] for the W fibres of group u and one
// piece f[0..FV) of a factor row.  MODE 0: scalar FMAs.  MODE 1: pairs of neighbouring
// fibres (the x pair is natural, f is duplicated into both halves: FV moves per piece).
// MODE 2: pairs of neighbouring q (the f pair is natural, x is duplicated: W moves per
// piece); the cheaper of the two is chosen from the shape.
template <typename T, int U, int W, int P, int FV, int MODE>
struct FibreAcc {
  T v[U][W][P];
  __host__ __device__ __forceinline__ void clear() {
#pragma unroll
    for (int u = 0; u < U; u++)
#pragma unroll
      for (int k = 0; k < W; k++)
#pragma unroll
        for (int q = 0; q < P; q++) v[u][k][q] = T(0);
  }
  __host__ __device__ __forceinline__ void axpy(int u, int q0, const T (&f)[FV], const T (&x)[W]) {
#pragma unroll
    for (int k = 0; k < W; k++)
#pragma unroll
      for (int i = 0; i < FV; i++) v[u][k][q0 + i] = fma(x[k], f[i], v[u][k][q0 + i]);
  }
  __host__ __device__ __forceinline__ T at(int u, int k, int q) const { return v[u][k][q]; }
};
#if defined(__CUDA_ARCH__)
template <int U, int W, int P, int FV>
struct FibreAcc<float, U, W, P, FV, 1> {
  float2 v[U][W / 2][P];
  __device__ __forceinline__ void clear() {
#pragma unroll
    for (int u = 0; u < U; u++)
#pragma unroll
      for (int k = 0; k < W / 2; k++)
#pragma unroll
        for (int q = 0; q < P; q++) v[u][k][q] = make_float2(0.f, 0.f);
  }
  __device__ __forceinline__ void axpy(int u, int q0, const float (&f)[FV], const float (&x)[W]) {
#pragma unroll
    for (int i = 0; i < FV; i++) {
      const float2 ff = make_float2(f[i], f[i]);
#pragma unroll
      for (int k = 0; k < W / 2; k++)
        v[u][k][q0 + i] = __ffma2_rn(make_float2(x[2 * k], x[2 * k + 1]), ff, v[u][k][q0 + i]);
    }
  }
  __device__ __forceinline__ float at(int u, int k, int q) const { return (k & 1) ? v[u][k >> 1][q].y : v[u][k >> 1][q].x; }
};
template <int U, int W, int P, int FV>
struct FibreAcc<float, U, W, P, FV, 2> {
  float2 v[U][W][P / 2];
  __device__ __forceinline__ void clear() {
#pragma unroll
    for (int u = 0; u < U; u++)
#pragma unroll
      for (int k = 0; k < W; k++)
#pragma unroll
        for (int q = 0; q < P / 2; q++) v[u][k][q] = make_float2(0.f, 0.f);
  }
  __device__ __forceinline__ void axpy(int u, int q0, const float (&f)[FV], const float (&x)[W]) {
#pragma unroll
    for (int k = 0; k < W; k++) {
      const float2 xx = make_float2(x[k], x[k]);
#pragma unroll
      for (int i = 0; i < FV / 2; i++)
        v[u][k][q0 / 2 + i] = __ffma2_rn(xx, make_float2(f[2 * i], f[2 * i + 1]), v[u][k][q0 / 2 + i]);
    }
  }
  __device__ __forceinline__ float at(int u, int k, int q) const { return (q & 1) ? v[u][k][q >> 1].y : v[u][k][q >> 1].x; }
};
#endif

// Strided fibres, S >= W: a thread owns NFIB = kAcc/P fibres, as U groups of W
// neighbouring ones (W * sizeof(T) <= 16 bytes); every access is one W-wide
// shared-memory transaction, consecutive lanes take consecutive groups.
template <typename T, int P, int S, int THREADS, bool SWZ = true>
__host__ __device__ __forceinline__ void stepStrided(T* __restrict__ tile, const T* __restrict__ Fs, int E, int tid) {
  constexpr int VEC = Vec16<T>::N;
  constexpr int NFIB = stepFibres<T, P>();
  constexpr int W = NFIB < VEC ? NFIB : VEC;
  constexpr int U = NFIB / W;
  constexpr int FV = P < VEC ? P : VEC;
  using V = VecW<T, W>;
  using FVv = Vec16<T>;
  const int nvg = E / (P * W);
  for (int vg0 = tid; vg0 < nvg; vg0 += THREADS * U) {
    unsigned pb[U];
    bool ok[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      int vg = vg0 + u * THREADS;
      ok[u] = vg < nvg;
      if (!ok[u]) vg = vg0;
      const unsigned lo = (unsigned)vg % (S / W);
      const unsigned hi = (unsigned)vg / (S / W);
      pb[u] = physIdx<T, SWZ>(hi * (unsigned)(S * P) + lo * W);
    }
    constexpr int ACC_MODE = !(kPackedFma && sizeof(T) == 4) ? 0
                             : (FV % 2 == 0 && U * W < P)    ? 2
                             : (W % 2 == 0)                  ? 1 : 0;
    FibreAcc<T, U, W, P, FV, ACC_MODE> acc;
    acc.clear();

    // Partially unrolled on purpose: a fully unrolled step of P = 16 or 32 is several
    // thousand instructions and the fused kernels then miss in the instruction cache.
#pragma unroll(P < kStepUnroll ? P : kStepUnroll)
    for (int p = 0; p < P; p++) {
      V xv[U];
#pragma unroll
      for (int u = 0; u < U; u++)
        xv[u] = *reinterpret_cast<const V*>(tile + (pb[u] ^ physIdx<T, SWZ>((unsigned)(p * S))));
#pragma unroll
      for (int q0 = 0; q0 < P; q0 += FV) {
        T f[FV];
        if (FV == VEC) {
          const FVv fv = *reinterpret_cast<const FVv*>(Fs + p * P + q0);
#pragma unroll
          for (int i = 0; i < FV; i++) f[i] = fv.v[i];
        } else {
#pragma unroll
          for (int i = 0; i < FV; i++) f[i] = Fs[p * P + q0 + i];
        }
#pragma unroll
        for (int u = 0; u < U; u++) acc.axpy(u, q0, f, xv[u].v);
      }
      schedFence();
    }
#pragma unroll
    for (int q = 0; q < P; q++) {
#pragma unroll
      for (int u = 0; u < U; u++) {
        V ov;
#pragma unroll
        for (int k = 0; k < W; k++) ov.v[k] = acc.at(u, k, q);
        if (ok[u]) *reinterpret_cast<V*>(tile + (pb[u] ^ physIdx<T, SWZ>((unsigned)(q * S)))) = ov;
      }
    }
  }
}

// Accumulators of a contiguous step: NFIB whole fibres of P outputs.
// axpy(k, q0, x, f): acc[k][q0 + i] += x * f[i] for one 16-byte piece f of a factor row.
template <typename T, int NFIB, int P, bool PACK>
struct RowAcc {
  static constexpr int VEC = Vec16<T>::N;
  T v[NFIB][P];
  __host__ __device__ __forceinline__ void clear() {
#pragma unroll
    for (int k = 0; k < NFIB; k++)
#pragma unroll
      for (int q = 0; q < P; q++) v[k][q] = T(0);
  }
  __host__ __device__ __forceinline__ void axpy(int k, int q0, T x, const T (&f)[VEC]) {
#pragma unroll
    for (int i = 0; i < VEC; i++) v[k][q0 + i] = fma(x, f[i], v[k][q0 + i]);
  }
  __host__ __device__ __forceinline__ T at(int k, int q) const { return v[k][q]; }
};
#if defined(__CUDA_ARCH__)
template <int NFIB, int P>
struct RowAcc<float, NFIB, P, true> {
  float2 v[NFIB][P / 2];
  __device__ __forceinline__ void clear() {
#pragma unroll
    for (int k = 0; k < NFIB; k++)
#pragma unroll
      for (int q = 0; q < P / 2; q++) v[k][q] = make_float2(0.f, 0.f);
  }
  __device__ __forceinline__ void axpy(int k, int q0, float x, const float (&f)[4]) {
    const float2 xx = make_float2(x, x);
    v[k][q0 / 2] = __ffma2_rn(xx, make_float2(f[0], f[1]), v[k][q0 / 2]);
    v[k][q0 / 2 + 1] = __ffma2_rn(xx, make_float2(f[2], f[3]), v[k][q0 / 2 + 1]);
  }
  __device__ __forceinline__ float at(int k, int q) const { return (q & 1) ? v[k][q >> 1].y : v[k][q >> 1].x; }
};
#endif

// Contiguous fibres (S == 1, P >= VEC): a thread owns NFIB whole fibres, reads
// and writes them as 128-bit pieces along p / q.
template <typename T, int P, int THREADS, bool SWZ = true>
__host__ __device__ __forceinline__ void stepContig(T* __restrict__ tile, const T* __restrict__ Fs, int E, int tid) {
  constexpr int VEC = Vec16<T>::N;
  constexpr int NFIB = stepFibres<T, P>();
  using V = Vec16<T>;
  const int nfib = E / P;
  for (int f0 = tid; f0 < nfib; f0 += THREADS * NFIB) {
    unsigned pb[NFIB];
    bool ok[NFIB];
#pragma unroll
    for (int k = 0; k < NFIB; k++) {
      int f = f0 + k * THREADS;
      ok[k] = f < nfib;
      if (!ok[k]) f = f0;
      pb[k] = physIdx<T, SWZ>((unsigned)f * P);
    }
    RowAcc<T, NFIB, P, kPackedFma> acc;
    acc.clear();

#pragma unroll((P / VEC) < (kStepUnroll / VEC) ? (P / VEC) : (kStepUnroll / VEC > 0 ? kStepUnroll / VEC : 1))
    for (int p0 = 0; p0 < P; p0 += VEC) {
      V xv[NFIB];
#pragma unroll
      for (int k = 0; k < NFIB; k++)
        xv[k] = *reinterpret_cast<const V*>(tile + (pb[k] ^ physIdx<T, SWZ>((unsigned)p0)));
#pragma unroll
      for (int pp = 0; pp < VEC; pp++) {
#pragma unroll
        for (int q0 = 0; q0 < P; q0 += VEC) {
          const V fv = *reinterpret_cast<const V*>(Fs + (p0 + pp) * P + q0);
#pragma unroll
          for (int k = 0; k < NFIB; k++) acc.axpy(k, q0, xv[k].v[pp], fv.v);
        }
        schedFence();
      }
    }
#pragma unroll
    for (int q0 = 0; q0 < P; q0 += VEC) {
#pragma unroll
      for (int k = 0; k < NFIB; k++) {
        V ov;
#pragma unroll
        for (int i = 0; i < VEC; i++) ov.v[i] = acc.at(k, q0 + i);
        if (ok[k]) *reinterpret_cast<V*>(tile + (pb[k] ^ physIdx<T, SWZ>((unsigned)q0))) = ov;
      }
    }
  }
}

// Any stride, any P: one fibre per thread with scalar accesses.  Only reached
// for the few shapes the vector steps cannot express (P or S below one 16-byte
// chunk).
template <typename T, int P, int S, int THREADS, bool SWZ = true>
__host__ __device__ __forceinline__ void stepScalar(T* __restrict__ tile, const T* __restrict__ Fs, int E, int tid) {
  const int nfib = E / P;
  for (int f = tid; f < nfib; f += THREADS) {
    const unsigned lo = (unsigned)f % S;
    const unsigned hi = (unsigned)f / S;
    const unsigned base = hi * (unsigned)(S * P) + lo;
    T x[P], o[P];
#pragma unroll
    for (int p = 0; p < P; p++) x[p] = tile[physIdx<T, SWZ>(base + (unsigned)(p * S))];
#pragma unroll
    for (int q = 0; q < P; q++) {
      T acc = T(0);
#pragma unroll
      for (int p = 0; p < P; p++) acc = fma(x[p], Fs[p * P + q], acc);
      o[q] = acc;
    }
#pragma unroll
    for (int q = 0; q < P; q++) tile[physIdx<T, SWZ>(base + (unsigned)(q * S))] = o[q];
  }
}

// fp64, P = 8 on the DMMA tensor path (mma.sync.m8n8k4.f64): a warp takes 8 neighbouring
// fibres at a time, A = the fibres (8 x 8 inputs, two k-steps of 4), B = the factor (held in
// two registers per lane for the whole step), C = the 8 x 8 outputs.  Per 64 outputs a lane
// issues 2 loads, 2 MMAs and 2 stores instead of 16 DFMAs plus operand loads; the FP64 tensor
// rate of B200 equals its DFMA rate (37 TFLOP/s measured for both), so the gain is in issue
// slots and shared-memory instructions, which is what bounds the SIMT form of this step.
// A group's inputs are read and its outputs written by the lanes of one warp, and mma.sync
// orders them, so the in-place update needs no barrier, as in the SIMT steps.
#if defined(__CUDA_ARCH__)
__device__ __forceinline__ void dmma884(double& c0, double& c1, double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};\n"
               : "+d"(c0), "+d"(c1) : "d"(a), "d"(b));
}
template <int S, int THREADS>
__device__ __forceinline__ void stepDmma8(double* __restrict__ tile, const double* __restrict__ Fs, int E, int tid) {
  constexpr int P = 8;
  const int lane = tid & 31, warp = tid >> 5, r = lane >> 2, t = lane & 3;
  const double b0 = Fs[t * P + r], b1 = Fs[(t + 4) * P + r];
  const int nfib = E / P;
  const int ngroups = (nfib + 7) / 8;              // the last group may be partial (tiny tiles)
  for (int gid = warp; gid < ngroups; gid += THREADS / 32) {
    const unsigned phi = (unsigned)gid * 8 + r;
    const bool live = (int)phi < nfib;
    const unsigned base = (S == 1) ? phi * P : (phi / S) * (unsigned)(S * P) + phi % S;
    const unsigned pb = physIdx<double>(base);
    const double a0 = live ? tile[pb ^ physIdx<double>((unsigned)(t * S))] : 0.0;
    const double a1 = live ? tile[pb ^ physIdx<double>((unsigned)((t + 4) * S))] : 0.0;
    double c0 = 0.0, c1 = 0.0;
    dmma884(c0, c1, a0, b0);
    dmma884(c0, c1, a1, b1);
    if (!live) continue;
    if (S == 1) {
      Vec16<double> o;
      o.v[0] = c0; o.v[1] = c1;
      *reinterpret_cast<Vec16<double>*>(tile + (pb ^ physIdx<double>((unsigned)(2 * t)))) = o;
    } else {
      tile[pb ^ physIdx<double>((unsigned)(2 * t * S))] = c0;
      tile[pb ^ physIdx<double>((unsigned)((2 * t + 1) * S))] = c1;
    }
  }
}
// Two neighbouring modes in one go, the intermediate never leaving registers.  A warp takes
// an 8 x 8 block X[a][b] (a: the slower mode, stride 8*Sb; b: the faster one, stride Sb).
//   first  C1t[qb][a]  = sum_b Fb[b][qb] * X[a][b]      A = Fb^T (constant), B = X^T
//   then   C2t[qb][qa] = sum_a C1t[qb][a] * Fa[a][qa]   A = C1t,            B = Fa (constant)
// The m8n8k4 C fragment gives lane (r, t) the entries [qb = r][a = 2t, 2t+1]; taking a = 2t
// as the contraction index of the first k-step and a = 2t+1 of the second (with Fa's rows
// permuted the same way) makes that fragment directly the A operand: no shuffles.  Shared
// memory is read and written once per two factors instead of once per factor.
template <int Sb, int THREADS>
__device__ __forceinline__ void stepDmma8Pair(double* __restrict__ tile, const double* __restrict__ Fb,
                                              const double* __restrict__ Fa, int E, int tid) {
  constexpr int P = 8;
  constexpr int Sa = Sb * P;
  const int lane = tid & 31, warp = tid >> 5, r = lane >> 2, t = lane & 3;
  if constexpr (Sb == 1) {
    // The two modes are the innermost ones: a warp takes one 8 x 8 block (64 contiguous doubles).
    // first product: A[m = qb = r][k = b = t + 4k'] = Fb[b][qb]
    const double fb0 = Fb[t * P + r], fb1 = Fb[(t + 4) * P + r];
    // second product: B[k][n = qa = r], k-step 0 <-> a = 2t, k-step 1 <-> a = 2t + 1
    const double fa0 = Fa[(2 * t) * P + r], fa1 = Fa[(2 * t + 1) * P + r];
    const int nblocks = E / (P * P);
    for (int blk = warp; blk < nblocks; blk += THREADS / 32) {
      const unsigned pb = physIdx<double>((unsigned)blk * (unsigned)(Sa * P));
      // B[k = b][n = a = r] = X[a = r][b = t + 4k']
      const double x0 = tile[pb ^ physIdx<double>((unsigned)(r * Sa + t))];
      const double x1 = tile[pb ^ physIdx<double>((unsigned)(r * Sa + (t + 4)))];
      double c0 = 0.0, c1 = 0.0;            // C1t[qb = r][a = 2t], [a = 2t + 1]
      dmma884(c0, c1, fb0, x0);
      dmma884(c0, c1, fb1, x1);
      double d0 = 0.0, d1 = 0.0;            // C2t[qb = r][qa = 2t], [qa = 2t + 1]
      dmma884(d0, d1, c0, fa0);
      dmma884(d0, d1, c1, fa1);
      // lanes with odd t store their two outputs in the other order: each store instruction then
      // touches both halves of the 128-byte lines (2 wavefronts instead of 4)
      const unsigned o0 = (unsigned)(t & 1), o1 = o0 ^ 1u;
      tile[pb ^ physIdx<double>((unsigned)((2 * t + o0) * Sa + r))] = o0 ? d1 : d0;
      tile[pb ^ physIdx<double>((unsigned)((2 * t + o1) * Sa + r))] = o1 ? d1 : d0;
    }
  } else {
    // Outer modes (Sb even): a warp takes two neighbouring blocks (lo, lo + 1) at once so that
    // its 8-byte accesses cover both halves of the 16-byte shared-memory chunks and its stores
    // are 16-byte vectors; with the first product's k-steps taking b in {0,1,4,5} and {2,3,6,7}
    // every load is 2 and every store 4 wavefronts, the minimum.
    //   first product, one per half h of the a index:  C_h[qb][(a', lo)] = sum_b Fb[b][qb] X[4h + a'][b][lo]
    //     A[m = qb = r][k] = Fb[b(k)][qb];  B[k][n = r] with n = 2a' + lo
    //   its C fragment (n = 2t, 2t+1 <-> a' = t, lo = 0, 1) is the A operand (k = t <-> a = 4h + t) of
    //   second product, one per lo:  D_lo[qb][qa] = sum_a C[qb][a][lo] Fa[a][qa],  B[k = t][n = qa = r] = Fa[4h + t][qa]
    static_assert(Sb % 2 == 0, "block pairs");
    const int b0 = (t & 1) | ((t & 2) << 1), b1 = b0 + 2;
    const double fb0 = Fb[b0 * P + r], fb1 = Fb[b1 * P + r];
    const double fa0 = Fa[t * P + r], fa1 = Fa[(4 + t) * P + r];
    const unsigned ap = (unsigned)r >> 1, lob = (unsigned)r & 1u;
    const int npairs = E / (2 * P * P);
    for (int pr = warp; pr < npairs; pr += THREADS / 32) {
      const unsigned blk = 2u * (unsigned)pr;
      const unsigned lo = blk % Sb, hi = blk / Sb;
      const unsigned pb = physIdx<double>(hi * (unsigned)(Sa * P) + lo);
      const double x00 = tile[pb ^ physIdx<double>(ap * Sa + (unsigned)b0 * Sb + lob)];
      const double x01 = tile[pb ^ physIdx<double>(ap * Sa + (unsigned)b1 * Sb + lob)];
      const double x10 = tile[pb ^ physIdx<double>((4u + ap) * Sa + (unsigned)b0 * Sb + lob)];
      const double x11 = tile[pb ^ physIdx<double>((4u + ap) * Sa + (unsigned)b1 * Sb + lob)];
      double c00 = 0.0, c01 = 0.0, c10 = 0.0, c11 = 0.0;      // c[h][lo] = C[qb = r][a = 4h + t][lo]
      dmma884(c00, c01, fb0, x00);
      dmma884(c00, c01, fb1, x01);
      dmma884(c10, c11, fb0, x10);
      dmma884(c10, c11, fb1, x11);
      double d00 = 0.0, d01 = 0.0, d10 = 0.0, d11 = 0.0;      // d[lo][o] = D[qb = r][qa = 2t + o][lo]
      dmma884(d00, d01, c00, fa0);
      dmma884(d00, d01, c10, fa1);
      dmma884(d10, d11, c01, fa0);
      dmma884(d10, d11, c11, fa1);
      *reinterpret_cast<double2*>(tile + (pb ^ physIdx<double>((unsigned)((2 * t) * Sa + r * Sb)))) = make_double2(d00, d10);
      *reinterpret_cast<double2*>(tile + (pb ^ physIdx<double>((unsigned)((2 * t + 1) * Sa + r * Sb)))) = make_double2(d01, d11);
    }
  }
}
#endif

template <typename T, int P, int S, int THREADS, bool SWZ = true>
__host__ __device__ __forceinline__ void stepDispatch(T* tile, const T* Fs, int E, int tid) {
#if defined(__CUDA_ARCH__)
  if constexpr (SWZ && sizeof(T) == 8 && P == 8 && (S == 1 || S % 8 == 0)) {
    stepDmma8<S, THREADS>(tile, Fs, E, tid);
    return;
  }
#endif
  constexpr int VEC = Vec16<T>::N;
  constexpr int NFIB = stepFibres<T, P>();
  constexpr int W = NFIB < VEC ? NFIB : VEC;
  if constexpr (S >= W && S % W == 0) {
    stepStrided<T, P, S, THREADS, SWZ>(tile, Fs, E, tid);
  } else if constexpr (S == 1 && P >= VEC) {
    stepContig<T, P, THREADS, SWZ>(tile, Fs, E, tid);
  } else {
    stepScalar<T, P, S, THREADS, SWZ>(tile, Fs, E, tid);
  }
}

// Apply factors J, J-1, ..., 0 of the group (J = NF-1 first).
template <typename T, int P, int NF, int BT, int THREADS, int J, bool SWZ = true>
struct StepChain {
  static __device__ __forceinline__ void run(T* tile, const T* Fs, int E) {
    constexpr int S = ipow(P, NF - 1 - J) * BT;
#if defined(__CUDA_ARCH__)
    if constexpr (SWZ && sizeof(T) == 8 && P == 8 && J >= 1 && (S == 1 || S % 8 == 0)) {
      // factors J and J-1 together, intermediate in registers
      stepDmma8Pair<S, THREADS>(tile, Fs + J * P * P, Fs + (J - 1) * P * P, E, (int)threadIdx.x);
      __syncthreads();
      StepChain<T, P, NF, BT, THREADS, J - 2, SWZ>::run(tile, Fs, E);
      return;
    }
#endif
    stepDispatch<T, P, S, THREADS, SWZ>(tile, Fs + J * P * P, E, (int)threadIdx.x);
    __syncthreads();
    StepChain<T, P, NF, BT, THREADS, J - 1, SWZ>::run(tile, Fs, E);
  }
};
template <typename T, int P, int NF, int BT, int THREADS, bool SWZ>
struct StepChain<T, P, NF, BT, THREADS, -1, SWZ> {
  static __device__ __forceinline__ void run(T*, const T*, int) {}
};
template <typename T, int P, int NF, int BT, int THREADS, bool SWZ>
struct StepChain<T, P, NF, BT, THREADS, -2, SWZ> {
  static __device__ __forceinline__ void run(T*, const T*, int) {}
};

// Global element offset of tile index idx.  Narrow super-tiles are one contiguous run
// starting at `contigBase`; wide ones look up the base of their sub-tile.
template <bool WIDE, int SUB, int BT>
__host__ __device__ __forceinline__ unsigned long long tileGlobalOffset(const unsigned long long* bases,
                                                                        unsigned long long contigBase,
                                                                        unsigned idx, unsigned long long B) {
  if constexpr (!WIDE) {
    return contigBase + idx;
  } else {
    const unsigned r = idx / SUB, w = idx % SUB;
    return bases[r] + (unsigned long long)(w / BT) * B + (w % BT);
  }
}

// Visit every 16-byte vector of a super-tile of nsub sub-tiles once: f(tileIndex, globalOffset).
// A thread keeps its position inside the sub-tile and walks sub-tiles, so the per-vector
// address work is an add (narrow: the super-tile is one contiguous run).
template <typename T, bool WIDE, int SUB, int BT, int THREADS, typename F>
__device__ __forceinline__ void forEachTileVector(const unsigned long long* bases, unsigned long long contigBase,
                                                  int nsub, unsigned long long B, F&& f) {
  constexpr int VEC = Vec16<T>::N;
  constexpr int VPS = SUB / VEC;                     // vectors per sub-tile
  if constexpr (!WIDE) {
    const int nvec = nsub * VPS;
    for (int v = threadIdx.x; v < nvec; v += THREADS) f((unsigned)v * VEC, contigBase + (unsigned long long)v * VEC);
  } else if constexpr (VPS >= THREADS) {
    for (int r = 0; r < nsub; r++) {
      const unsigned long long base = bases[r];
#pragma unroll 4
      for (int j = threadIdx.x; j < VPS; j += THREADS) {
        const unsigned w = (unsigned)j * VEC;
        f((unsigned)r * SUB + w, base + (unsigned long long)(w / BT) * B + (w % BT));
      }
    }
  } else {
    constexpr int SPT = THREADS / VPS;                // sub-tiles per sweep of the CTA
    const unsigned w = (threadIdx.x % VPS) * VEC;
    const unsigned long long gw = (unsigned long long)(w / BT) * B + (w % BT);
    for (int r = threadIdx.x / VPS; r < nsub; r += SPT) f((unsigned)r * SUB + w, bases[r] + gw);
  }
}

// The same enumeration by counter: the i-th vector of this thread (i < tileVectorCount),
// for loops that want several vectors in flight at once.
template <typename T, bool WIDE, int SUB, int THREADS>
__device__ __forceinline__ int tileVectorCount(int nsub) {
  constexpr int VPS = SUB / Vec16<T>::N;
  if constexpr (!WIDE) {
    const int nvec = nsub * VPS;
    return nvec > (int)threadIdx.x ? (nvec - (int)threadIdx.x + THREADS - 1) / THREADS : 0;
  } else if constexpr (VPS >= THREADS) {
    return nsub * (VPS / THREADS);
  } else {
    constexpr int SPT = THREADS / VPS;
    const int r0 = threadIdx.x / VPS;
    return nsub > r0 ? (nsub - r0 + SPT - 1) / SPT : 0;
  }
}
template <typename T, bool WIDE, int SUB, int BT, int THREADS>
__device__ __forceinline__ void tileVectorAt(const unsigned long long* bases, unsigned long long contigBase,
                                             unsigned long long B, int i, unsigned& idx, unsigned long long& goff) {
  constexpr int VEC = Vec16<T>::N;
  constexpr int VPS = SUB / VEC;
  if constexpr (!WIDE) {
    const unsigned v = threadIdx.x + (unsigned)i * THREADS;
    idx = v * VEC; goff = contigBase + (unsigned long long)v * VEC;
  } else if constexpr (VPS >= THREADS) {
    constexpr int PER = VPS / THREADS;
    const unsigned r = (unsigned)i / PER, j = threadIdx.x + ((unsigned)i % PER) * THREADS;
    const unsigned w = j * VEC;
    idx = r * SUB + w; goff = bases[r] + (unsigned long long)(w / BT) * B + (w % BT);
  } else {
    constexpr int SPT = THREADS / VPS;
    const unsigned r = threadIdx.x / VPS + (unsigned)i * SPT;
    const unsigned w = (threadIdx.x % VPS) * VEC;
    idx = r * SUB + w; goff = bases[r] + (unsigned long long)(w / BT) * B + (w % BT);
  }
}

// mbarrier / TMA primitives for the tile ring (one CTA, no multicast).
// Set when a bounded wait on a tile barrier gave up.  One copy per translation unit; only the
// unit that instantiates TMA-staged kernels (fp32 wide) ever writes it.
static __device__ int gTileTmaTimeouts = 0;
__device__ __forceinline__ void tileMbarInit(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"((unsigned)__cvta_generic_to_shared(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void tileMbarExpectTx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"((unsigned)__cvta_generic_to_shared(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool tileMbarTryWait(unsigned long long* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok) : "r"((unsigned)__cvta_generic_to_shared(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Gives up after about two seconds, records that and reports failure.
__device__ __forceinline__ bool tileMbarWaitBounded(unsigned long long* bar, unsigned parity) {
  if (tileMbarTryWait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!tileMbarTryWait(bar, parity)) {
    if (clock64() - t0 > 4000000000ll) { atomicExch(&gTileTmaTimeouts, 1); return false; }
  }
  return true;
}
// One box {BT, rows, 1, 1} of the [entries][chunks][G][B] view at (x = b0, y = g0, z = chunk, w = entry).
__device__ __forceinline__ void tileTmaLoad(void* smemDst, const void* tmap, int x, int y, int z, int w, unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n"
      ::"r"((unsigned)__cvta_generic_to_shared(smemDst)), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(w),
        "r"((unsigned)__cvta_generic_to_shared(bar)) : "memory");
}

// The same box from shared memory to global memory (bulk-group completion).
__device__ __forceinline__ void tileTmaStore(const void* tmap, int x, int y, int z, int w, const void* smemSrc) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%1, %2, %3, %4}], [%5];\n"
      ::"l"(tmap), "r"(x), "r"(y), "r"(z), "r"(w), "r"((unsigned)__cvta_generic_to_shared(smemSrc)) : "memory");
}

struct alignas(64) TileTmaMap { unsigned char bytes[128]; };   // a CUtensorMap, kept opaque here

// The pass kernel.  Persistent CTAs walk super-tiles with a ring of two tile buffers: while the
// contraction steps and the stores of super-tile t run, super-tile t+1 is already on its way
// into the other buffer, so a CTA never sits idle waiting for memory once the ring is primed.
// Staging:
//   TMA == false  16-byte cp.async from every thread into the XOR-swizzled layout (any layout;
//                 the narrow steps and the DMMA steps need the swizzle)
//   TMA == true   wide fp32 tiles: lanes of a warp always run along the trailing index there, so
//                 a linear [G][W] sub-tile is already free of bank conflicts and one elected
//                 thread can stage it with cp.async.bulk.tensor (boxes of up to 256 rows of 128
//                 bytes, completion on an mbarrier with a bounded wait); a pass without alpha /
//                 beta*Y also drains its tiles with bulk tensor stores from shared memory
//                 (a.bulkOut), so neither direction spends registers or issue slots on addresses
template <typename T, int P, int NF, bool WIDE, bool TMA, int MINB = kTileMinBlocks, int NBUF = 2>
__global__ void __launch_bounds__(kTileThreads, MINB)
tilePassKernel(const TileArgs<T> a, const __grid_constant__ TileTmaMap tmap, const __grid_constant__ TileTmaMap tmapOut) {
  constexpr int THREADS = kTileThreads;
  constexpr int VEC = Vec16<T>::N;
  constexpr int BT = WIDE ? (int)(128 / sizeof(T)) : 1;
  constexpr int G = ipow(P, NF);
  constexpr int SUB = G * BT;
  constexpr bool SWZ = !TMA;
  constexpr int BOXR = G < 256 ? G : 256;             // rows of one TMA box
  static_assert(!TMA || (WIDE && sizeof(T) == 4), "TMA staging: wide fp32 tiles");
  using V = Vec16<T>;

  extern __shared__ __align__(1024) unsigned char smemRaw[];
  const size_t tileElems = (size_t)a.R * SUB;
  static_assert(NBUF == 1 || NBUF == 2, "one tile buffer (load, compute, store in turn) or a ring of two");
  T* tiles = reinterpret_cast<T*>(smemRaw);           // NBUF buffers of tileElems
  T* Fs = tiles + NBUF * tileElems;
  unsigned long long* basesAll = reinterpret_cast<unsigned long long*>(Fs + NF * P * P);   // [2][kTileMaxR]
  __shared__ __align__(8) unsigned long long fullBar[2];

  if (TMA && threadIdx.x == 0) {
    tileMbarInit(&fullBar[0], 1);
    tileMbarInit(&fullBar[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  // factors -> shared memory as [k][p][q]
  for (int i = threadIdx.x; i < NF * P * P; i += THREADS) {
    const int k = i / (P * P), p = (i / P) % P, q = i % P;
    Fs[i] = a.F[k][(long long)p * a.fsP + (long long)q * a.fsQ];
  }

  const unsigned long long R = (unsigned long long)a.R;
  const unsigned long long totalSupers = a.supersPerEntry * a.batch;

  // Super-tile u of the whole (batched) launch: entry and first sub-tile within the entry.
  auto locate = [&](unsigned long long u, unsigned long long& bt, unsigned long long& st0) {
    bt = a.batch > 1 ? u / a.supersPerEntry : 0;
    st0 = (u - bt * a.supersPerEntry) * R;
  };

  // Bases of the sub-tiles of super-tile u, and its loads into buffer b.
  auto stage = [&](unsigned long long u, int b) {
    unsigned long long bt, st0;
    locate(u, bt, st0);
    const T* X = a.X + bt * a.bsX;
    const unsigned long long left = a.numSub - st0;
    const int nsub = left < R ? (int)left : (int)R;
    unsigned long long* bases = basesAll + b * kTileMaxR;
    T* tile = tiles + (size_t)b * tileElems;
    if constexpr (TMA) {
      if (threadIdx.x == 0) {
        // the bulk stores that drained this buffer's previous tile must have read it
        if (a.bulkOut) asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
        tileMbarExpectTx(&fullBar[b], (unsigned)(nsub * SUB * sizeof(T)));
        for (int r = 0; r < nsub; r++) {
          const unsigned long long st = st0 + r;
          const unsigned long long chunk = st / a.tilesPerChunk, bt2 = st % a.tilesPerChunk;
          bases[r] = chunk * (unsigned long long)G * a.B + bt2 * (unsigned long long)BT;
#pragma unroll
          for (int g0 = 0; g0 < G; g0 += BOXR)
            tileTmaLoad(tile + (size_t)r * SUB + (size_t)g0 * BT, &tmap, (int)(bt2 * BT), g0, (int)chunk, (int)bt, &fullBar[b]);
        }
      }
    } else {
      if constexpr (WIDE) {
        // every thread derives the base of the sub-tiles it copies itself (sharing them through
        // shared memory would need a barrier in the middle of the other buffer's arithmetic)
        constexpr int VPS = SUB / VEC;
        auto subBase = [&](unsigned long long st) -> unsigned long long {
          if (a.numSub <= 0xFFFFFFFFull) {
            const unsigned s32 = (unsigned)st, t32 = (unsigned)a.tilesPerChunk;
            const unsigned c = s32 / t32, bt2 = s32 - c * t32;
            return (unsigned long long)c * (unsigned long long)G * a.B + (unsigned long long)bt2 * BT;
          }
          return (st / a.tilesPerChunk) * (unsigned long long)G * a.B + (st % a.tilesPerChunk) * (unsigned long long)BT;
        };
        if constexpr (VPS >= THREADS) {
          for (int r = 0; r < nsub; r++) {
            const unsigned long long base = subBase(st0 + r);
            if (threadIdx.x == 0) bases[r] = base;
#pragma unroll 4
            for (int j = threadIdx.x; j < VPS; j += THREADS) {
              const unsigned w = (unsigned)j * VEC;
              cpAsync16(tile + physIdx<T, SWZ>((unsigned)r * SUB + w), X + base + (unsigned long long)(w / BT) * a.B + (w % BT));
            }
          }
        } else {
          constexpr int SPT = THREADS / VPS;
          const unsigned w = (threadIdx.x % VPS) * VEC;
          const unsigned long long gw = (unsigned long long)(w / BT) * a.B + (w % BT);
          for (int r = threadIdx.x / VPS; r < nsub; r += SPT) {
            const unsigned long long base = subBase(st0 + r);
            if (w == 0) bases[r] = base;
            cpAsync16(tile + physIdx<T, SWZ>((unsigned)r * SUB + w), X + base + gw);
          }
        }
      } else {
        forEachTileVector<T, WIDE, SUB, BT, THREADS>(bases, st0 * G, nsub, a.B, [&](unsigned idx, unsigned long long goff) {
          cpAsync16(tile + physIdx<T, SWZ>(idx), X + goff);
        });
      }
    }
  };

  unsigned long long u = blockIdx.x;
  if (NBUF == 2) {
    if (u < totalSupers) stage(u, 0);
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  }
  unsigned phases = 0;
  unsigned long long curEntry = 0;          // entry whose factors are in shared memory
  for (int it = 0; u < totalSupers; u += gridDim.x, it++) {
    const int b = NBUF == 2 ? (it & 1) : 0;
    unsigned long long bt, st0;
    locate(u, bt, st0);
    const unsigned long long left = a.numSub - st0;
    const int nsub = left < R ? (int)left : (int)R;
    if (NBUF == 2) {
      // the other buffer's previous contents were stored before the barrier that ended the last
      // iteration: refill it now, then wait for this iteration's tile only
      if (u + gridDim.x < totalSupers) stage(u + gridDim.x, b ^ 1);
    } else {
      stage(u, 0);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    if (a.batchedF && bt != curEntry) {
      // this entry has factors of its own (the last iteration's barrier ordered their last use)
      for (int i = threadIdx.x; i < NF * P * P; i += THREADS) {
        const int k = i / (P * P), p = (i / P) % P, q = i % P;
        Fs[i] = a.F[k][bt * a.bsF[k] + (long long)p * a.fsP + (long long)q * a.fsQ];
      }
      curEntry = bt;
    }
    if constexpr (TMA) {
      if (!tileMbarWaitBounded(&fullBar[b], (phases >> b) & 1u)) return;
      phases ^= 1u << b;
    } else if (NBUF == 2) {
      asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();

    T* tile = tiles + (size_t)b * tileElems;
    const unsigned long long* bases = basesAll + b * kTileMaxR;
    const int E = nsub * SUB;
    StepChain<T, P, NF, BT, THREADS, NF - 1, SWZ>::run(tile, Fs, E);

    T* Z = a.Z + bt * a.bsZ;
    const T* Y = a.Y ? a.Y + bt * a.bsY : nullptr;
    const bool epi = a.epilogue != 0;
    const bool useY = epi && a.beta != T(0) && Y != nullptr;
    if (TMA && a.bulkOut) {
      // generic-proxy writes of the last step -> visible to the async proxy, then one thread
      // issues the boxes (same coordinates as the loads, on the output's tensor map)
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      __syncthreads();
      if (threadIdx.x == 0) {
        for (int r = 0; r < nsub; r++) {
          const unsigned long long st = st0 + r;
          const unsigned long long chunk = st / a.tilesPerChunk, bt2 = st % a.tilesPerChunk;
#pragma unroll
          for (int g0 = 0; g0 < G; g0 += BOXR)
            tileTmaStore(&tmapOut, (int)(bt2 * BT), g0, (int)chunk, (int)bt, tile + (size_t)r * SUB + (size_t)g0 * BT);
        }
        asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
      }
      continue;            // the next iteration's barrier orders the buffer's reuse by the steps
    }
    if (useY) {
      // Y may be Z itself, so the compiler has to keep every read of Y ahead of the next
      // store and one vector would be in flight per thread; reading a batch of Y first keeps
      // EB loads in flight (element i of Y is only ever needed for element i of Z).
      constexpr int EB = 4;      // more would spill registers in the contraction steps
      const int cnt = tileVectorCount<T, WIDE, SUB, THREADS>(nsub);
      for (int i0 = 0; i0 < cnt; i0 += EB) {
        V y[EB];
#pragma unroll
        for (int e = 0; e < EB; e++) {
          if (i0 + e < cnt) {
            unsigned idx; unsigned long long go;
            tileVectorAt<T, WIDE, SUB, BT, THREADS>(bases, st0 * G, a.B, i0 + e, idx, go);
            y[e] = *reinterpret_cast<const V*>(Y + go);
          }
        }
#pragma unroll
        for (int e = 0; e < EB; e++) {
          if (i0 + e < cnt) {
            unsigned idx; unsigned long long go;         // recomputed: cheaper than keeping EB offsets live
            tileVectorAt<T, WIDE, SUB, BT, THREADS>(bases, st0 * G, a.B, i0 + e, idx, go);
            V o = *reinterpret_cast<const V*>(tile + physIdx<T, SWZ>(idx));
#pragma unroll
            for (int i = 0; i < VEC; i++) o.v[i] = fma(a.beta, y[e].v[i], a.alpha * o.v[i]);
            *reinterpret_cast<V*>(Z + go) = o;
          }
        }
      }
    } else
    forEachTileVector<T, WIDE, SUB, BT, THREADS>(bases, st0 * G, nsub, a.B, [&](unsigned idx, unsigned long long goff) {
      V o = *reinterpret_cast<const V*>(tile + physIdx<T, SWZ>(idx));
      if (epi) {
#pragma unroll
        for (int i = 0; i < VEC; i++) o.v[i] = a.alpha * o.v[i];
      }
      *reinterpret_cast<V*>(Z + goff) = o;
    });
    __syncthreads();
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
  // shared memory must stay alive until the last bulk stores have read it
  if (TMA && a.bulkOut && threadIdx.x == 0) asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
}

// ---- transposing variant ---------------------------------------------------------
// First pass of a problem whose input and output disagree on which index is
// contiguous (KMM with opX = T: row-major in, m-contiguous out; MKM with opX = T:
// the reverse).  The group is the trailing one (B == 1).  A super-tile is
// [aT chunks][mT rows][G]; the row-major side moves whole [G] runs with 128-bit
// accesses, the m-contiguous side moves mT consecutive m per access: a thread takes
// one 16-byte piece of a fibre from shared memory and issues VEC scalar global
// accesses, each of which is contiguous across the lanes of the warp.
template <typename T>
struct TileTrArgs {
  const T* X; T* Z; const T* Y;
  const T* F[kMaxGroup];
  long long fsP, fsQ;
  unsigned long long M, A;           // rows and leading chunks per row
  int mT, aT;                        // rows / chunks per super-tile (mT a power of two)
  unsigned long long mBlocks, numSuper;
  T alpha, beta;
  int epilogue;
  int vecM;                          // the m-contiguous side may move 16-byte vectors (M and mT multiples of VEC, aligned)
};

constexpr unsigned long long kNoBase = ~0ull;

// TR == 1: row-major input, m-contiguous output.  TR == 2: the reverse.
template <typename T, int P, int NF, int TR>
__global__ void __launch_bounds__(kTileThreads, kTileMinBlocks) tileTransposeKernel(const TileTrArgs<T> a) {
  constexpr int THREADS = kTileThreads;
  constexpr int VEC = Vec16<T>::N;
  constexpr int G = ipow(P, NF);
  using V = Vec16<T>;

  extern __shared__ __align__(1024) unsigned char smemRaw[];
  const int R = a.mT * a.aT;
  T* tile = reinterpret_cast<T*>(smemRaw);
  T* Fs = tile + (size_t)R * G;
  unsigned long long* baseRow = reinterpret_cast<unsigned long long*>(Fs + NF * P * P);
  unsigned long long* baseCol = baseRow + kTileMaxR;

  for (int i = threadIdx.x; i < NF * P * P; i += THREADS) {
    const int k = i / (P * P), p = (i / P) % P, q = i % P;
    Fs[i] = a.F[k][(long long)p * a.fsP + (long long)q * a.fsQ];
  }

  for (unsigned long long sup = blockIdx.x; sup < a.numSuper; sup += gridDim.x) {
    const unsigned long long m0 = (sup % a.mBlocks) * a.mT, a0 = (sup / a.mBlocks) * a.aT;
    if ((int)threadIdx.x < R) {
      const unsigned long long m = m0 + threadIdx.x % a.mT, ac = a0 + threadIdx.x / a.mT;
      const bool ok = m < a.M && ac < a.A;
      baseRow[threadIdx.x] = ok ? (m * a.A + ac) * (unsigned long long)G : kNoBase;
      baseCol[threadIdx.x] = ac * (unsigned long long)G * a.M + m;
    }
    __syncthreads();

    const int E = R * G;
    const int nvec = E / VEC;
    if (TR == 1) {
      for (int v = threadIdx.x; v < nvec; v += THREADS) {
        const unsigned idx = (unsigned)v * VEC;
        const unsigned r = idx / G, w = idx % G;
        const bool ok = baseRow[r] != kNoBase;
        cpAsync16Zfill(tile + physIdx<T>(idx), ok ? a.X + baseRow[r] + w : a.X, ok);
      }
      cpAsyncWaitAll();
    } else if (a.vecM) {
      // m-contiguous input, 16 bytes along m per access: a thread takes VEC consecutive rows at
      // one g and scatters them into the VEC fibres (the transposition happens here)
      const unsigned mq = (unsigned)a.mT / VEC;
      const int items = (R / VEC) * G;
      for (int it = threadIdx.x; it < items; it += THREADS) {
        const unsigned q = (unsigned)it % mq, rest = (unsigned)it / mq;
        const unsigned g = rest % G, r0 = (rest / G) * a.mT + q * VEC;
        const bool ok = baseRow[r0] != kNoBase;
        V x;
        if (ok) x = *reinterpret_cast<const V*>(a.X + baseCol[r0] + (unsigned long long)g * a.M);
#pragma unroll
        for (int e = 0; e < VEC; e++) tile[physIdx<T>((r0 + e) * G + g)] = ok ? x.v[e] : T(0);
      }
    } else {
      for (int v = threadIdx.x; v < nvec; v += THREADS) {
        const unsigned mi = (unsigned)v % a.mT, rest = (unsigned)v / a.mT;
        const unsigned gv = rest % (G / VEC), r = (rest / (G / VEC)) * a.mT + mi;
        V x;
        const bool ok = baseRow[r] != kNoBase;
#pragma unroll
        for (int e = 0; e < VEC; e++)
          x.v[e] = ok ? a.X[baseCol[r] + (unsigned long long)(gv * VEC + e) * a.M] : T(0);
        *reinterpret_cast<V*>(tile + physIdx<T>(r * G + gv * VEC)) = x;
      }
    }
    __syncthreads();

    StepChain<T, P, NF, 1, THREADS, NF - 1>::run(tile, Fs, E);

    const bool useY = a.epilogue && a.beta != T(0) && a.Y != nullptr;
    if (TR == 1 && a.vecM) {
      // m-contiguous output, 16 bytes along m per access: a thread gathers one g of VEC
      // consecutive rows from shared memory (the XOR swizzle keeps rows that are whole fibres
      // apart in different banks) and issues one vector store; the lanes of a warp run along m
      // first, so a warp writes whole 128-byte lines.  Y is read in batches ahead of the stores
      // for the reason given in the pass kernel.
      const unsigned mq = (unsigned)a.mT / VEC;
      const int items = (R / VEC) * G;
      constexpr int EB = 4;
      for (int it0 = threadIdx.x; it0 < items; it0 += THREADS * EB) {
        V y[EB];
        unsigned long long off[EB];
        unsigned src[EB];
        bool ok[EB];
#pragma unroll
        for (int e = 0; e < EB; e++) {
          const int it = it0 + e * THREADS;
          ok[e] = it < items;
          const unsigned q = (unsigned)(ok[e] ? it : it0) % mq, rest = (unsigned)(ok[e] ? it : it0) / mq;
          const unsigned g = rest % G, r0 = (rest / G) * a.mT + q * VEC;
          ok[e] = ok[e] && baseRow[r0] != kNoBase;
          off[e] = baseCol[r0] + (unsigned long long)g * a.M;
          src[e] = r0 * G + g;
          if (ok[e] && useY) y[e] = *reinterpret_cast<const V*>(a.Y + off[e]);
        }
#pragma unroll
        for (int e = 0; e < EB; e++) {
          if (!ok[e]) continue;
          V o;
#pragma unroll
          for (int i = 0; i < VEC; i++) {
            T val = tile[physIdx<T>(src[e] + (unsigned)i * G)];
            if (a.epilogue) val = a.alpha * val;
            if (useY) val = fma(a.beta, y[e].v[i], val);
            o.v[i] = val;
          }
          *reinterpret_cast<V*>(a.Z + off[e]) = o;
        }
      }
    } else if (TR == 1) {
      for (int v = threadIdx.x; v < nvec; v += THREADS) {
        const unsigned mi = (unsigned)v % a.mT, rest = (unsigned)v / a.mT;
        const unsigned gv = rest % (G / VEC), r = (rest / (G / VEC)) * a.mT + mi;
        if (baseRow[r] == kNoBase) continue;
        const V o = *reinterpret_cast<const V*>(tile + physIdx<T>(r * G + gv * VEC));
#pragma unroll
        for (int e = 0; e < VEC; e++) {
          const unsigned long long off = baseCol[r] + (unsigned long long)(gv * VEC + e) * a.M;
          T val = o.v[e];
          if (a.epilogue) val = a.alpha * val;
          if (useY) val = fma(a.beta, a.Y[off], val);
          a.Z[off] = val;
        }
      }
    } else {
      for (int v = threadIdx.x; v < nvec; v += THREADS) {
        const unsigned idx = (unsigned)v * VEC;
        const unsigned r = idx / G, w = idx % G;
        if (baseRow[r] == kNoBase) continue;
        const unsigned long long goff = baseRow[r] + w;
        V o = *reinterpret_cast<const V*>(tile + physIdx<T>(idx));
        if (a.epilogue) {
#pragma unroll
          for (int i = 0; i < VEC; i++) o.v[i] = a.alpha * o.v[i];
          if (useY) {
            const V y = *reinterpret_cast<const V*>(a.Y + goff);
#pragma unroll
            for (int i = 0; i < VEC; i++) o.v[i] = fma(a.beta, y.v[i], o.v[i]);
          }
        }
        *reinterpret_cast<V*>(a.Z + goff) = o;
      }
    }
    __syncthreads();
  }
}


}  // namespace fkb

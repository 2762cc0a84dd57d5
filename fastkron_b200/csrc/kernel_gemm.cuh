// Large-factor kernel: one tensor mode of size P contracted with a P x Q factor,
//   [chunks][P][B] -> [chunks][Q][B],
// written as a register-blocked FFMA/DFMA GEMM  C[q, j] = sum_p F[p, q] * X[p, j]
// where j runs over TJ trailing positions (or, when B is small, over several whole
// chunks).  The factor stays resident in shared memory for the life of the
// (persistent) CTA; X streams through a ring of cp.async stages, PC rows of p at a
// time, so the global loads of tile t+1 overlap the arithmetic of tile t.  Every
// thread owns an MQ x MJ block of outputs whose rows/columns are spread in 16-byte
// groups so that both the shared-memory operand reads and the global stores are
// 128-bit and conflict free: a warp is 4 (q) x 8 (j) lanes, so a factor read touches
// 64 contiguous bytes (broadcast to the other lanes) and an X read 128.
//
// Two shared-memory layouts of the X stage:
//   XT == false  [p][j]     (B >= 4): global runs along the trailing index
//   XT == true   [j][p+pad] (B == 1): the contracted index itself is contiguous
//
// Arithmetic matches one step of the reference's sliced multiply
// (src/kernels/cuda/kernel.cuh:53-224): products accumulated over p ascending,
// alpha/beta applied by the pass that consumes factor 0.
#pragma once

#include "kernels.h"
#include "kernel_tile.cuh"   // Vec16, cpAsync16

namespace fkb {

template <typename T>
struct GemmArgs {
  const T* X; T* Z; const T* Y; const T* F;
  long long fsP, fsQ;
  unsigned long long numChunks;      // M*A
  unsigned long long B;              // trailing extent
  unsigned long long numTiles;
  unsigned long long tilesPerChunk;  // mode 0: B / TJ
  int mode;                          // 0: B >= TJ, 1: 4 <= B < TJ, 2: B == 1 (XT)
  T alpha, beta;
  int epilogue;
};

__device__ __forceinline__ void cpAsync16Zfill(void* smemDst, const void* gmemSrc, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smemDst);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmemSrc), "r"(n) : "memory");
}
__device__ __forceinline__ void cpAsyncCommit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cpAsyncWait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

template <typename T, int P, int Q, int TJ, int PC, int STAGES, int MQ, int MJ, bool XT>
struct GemmCfg {
  static constexpr int VEC = 16 / (int)sizeof(T);
  static constexpr int NGQ = MQ / VEC, NGJ = MJ / VEC;
  static constexpr int THREADS = (Q / MQ) * (TJ / MJ);
  static constexpr int NWQ = (Q / MQ) / 4;              // warps along q (4 q-lanes per warp)
  static constexpr int PAD = VEC;
  static constexpr int STAGE_ELEMS = XT ? TJ * (PC + PAD) : PC * TJ;
  static constexpr int NCH = P / PC;
  static constexpr size_t SMEM = ((size_t)P * Q + (size_t)STAGES * STAGE_ELEMS) * sizeof(T);
  static_assert(P % PC == 0 && Q % (4 * MQ) == 0 && TJ % (8 * MJ) == 0, "tile shape");
  static_assert(MQ % VEC == 0 && MJ % VEC == 0 && PC % VEC == 0, "vector shape");
};

template <typename T, int P, int Q, int TJ, int PC, int STAGES, int MQ, int MJ, bool XT>
__global__ void __launch_bounds__((Q / MQ) * (TJ / MJ), ((Q / MQ) * (TJ / MJ) <= 256 ? 2 : 1))
gemmPassKernel(const GemmArgs<T> a) {
  using C = GemmCfg<T, P, Q, TJ, PC, STAGES, MQ, MJ, XT>;
  using V = Vec16<T>;
  constexpr int VEC = C::VEC, THREADS = C::THREADS, NGQ = C::NGQ, NGJ = C::NGJ;
  constexpr int QS = Q / NGQ;          // stride between a thread's q groups
  constexpr int JS = TJ / NGJ;         // stride between a thread's j groups (non-XT)
  constexpr int JT = TJ / MJ;          // stride between a thread's j's (XT)

  extern __shared__ __align__(16) unsigned char smemRaw[];
  T* Fs = reinterpret_cast<T*>(smemRaw);
  T* stages = Fs + P * Q;

  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int tq = (warp % C::NWQ) * 4 + (lane & 3);
  const int tj = (warp / C::NWQ) * 8 + (lane >> 2);

  // factor -> shared memory [p][q]
  if (a.fsQ == 1) {
    for (int v = tid; v < P * Q / VEC; v += THREADS) {
      const int p = (v * VEC) / Q, q = (v * VEC) % Q;
      *reinterpret_cast<V*>(Fs + p * Q + q) = *reinterpret_cast<const V*>(a.F + (long long)p * a.fsP + q);
    }
  } else {
    for (int i = tid; i < P * Q; i += THREADS) {
      const int q = i / P, p = i % P;               // walk the stored (q-major) order
      Fs[p * Q + q] = a.F[(long long)p * a.fsP + (long long)q * a.fsQ];
    }
  }

  const unsigned long long first = blockIdx.x, step = gridDim.x;
  const unsigned long long myTiles = first < a.numTiles ? (a.numTiles - first + step - 1) / step : 0;
  const unsigned long long total = myTiles * C::NCH;
  const unsigned long long PB = (unsigned long long)P * a.B, QB = (unsigned long long)Q * a.B;

  auto issue = [&](unsigned long long s) {
    const unsigned long long t = first + (s / C::NCH) * step;
    const int c = (int)(s % C::NCH);
    T* st = stages + (size_t)(s % STAGES) * C::STAGE_ELEMS;
    if constexpr (!XT) {
      unsigned long long base = 0, n0 = 0;
      if (a.mode == 0) base = (t / a.tilesPerChunk) * PB + (t % a.tilesPerChunk) * (unsigned long long)TJ;
      else n0 = t * ((unsigned long long)TJ / a.B);
      constexpr int VPR = TJ / VEC;                 // vectors per p row
#pragma unroll 4
      for (int v = tid; v < PC * VPR; v += THREADS) {
        const int pl = v / VPR, j = (v % VPR) * VEC;
        const unsigned long long prow = (unsigned long long)(c * PC + pl) * a.B;
        if (a.mode == 0) {
          cpAsync16(st + pl * TJ + j, a.X + base + prow + j);
        } else {
          const unsigned long long n = n0 + (unsigned long long)j / a.B;
          const bool ok = n < a.numChunks;
          cpAsync16Zfill(st + pl * TJ + j, ok ? a.X + n * PB + prow + (unsigned long long)j % a.B : a.X, ok);
        }
      }
    } else {
      const unsigned long long n0 = t * (unsigned long long)TJ;
      constexpr int VPR = PC / VEC;                 // vectors per j row
#pragma unroll 4
      for (int v = tid; v < TJ * VPR; v += THREADS) {
        const int j = v / VPR, pv = (v % VPR) * VEC;
        const unsigned long long n = n0 + j;
        const bool ok = n < a.numChunks;
        cpAsync16Zfill(st + j * (PC + C::PAD) + pv, ok ? a.X + n * P + c * PC + pv : a.X, ok);
      }
    }
  };

  T acc[MQ][MJ];
#pragma unroll
  for (int i = 0; i < MQ; i++)
#pragma unroll
    for (int j = 0; j < MJ; j++) acc[i][j] = T(0);

#pragma unroll
  for (int s = 0; s < STAGES - 1; s++) {
    if ((unsigned long long)s < total) issue(s);
    cpAsyncCommit();
  }
  __syncthreads();   // factor visible

  for (unsigned long long s = 0; s < total; s++) {
    cpAsyncWait<STAGES - 2>();
    __syncthreads();
    if (s + STAGES - 1 < total) issue(s + STAGES - 1);
    cpAsyncCommit();

    const int c = (int)(s % C::NCH);
    const T* st = stages + (size_t)(s % STAGES) * C::STAGE_ELEMS;
    const T* fr = Fs + (size_t)c * PC * Q + tq * VEC;
    if constexpr (!XT) {
      const T* xr = st + tj * VEC;
#pragma unroll 8
      for (int pl = 0; pl < PC; pl++) {
        V xv[NGJ], fv[NGQ];
#pragma unroll
        for (int g = 0; g < NGJ; g++) xv[g] = *reinterpret_cast<const V*>(xr + pl * TJ + g * JS);
#pragma unroll
        for (int g = 0; g < NGQ; g++) fv[g] = *reinterpret_cast<const V*>(fr + pl * Q + g * QS);
#pragma unroll
        for (int qi = 0; qi < MQ; qi++)
#pragma unroll
          for (int ji = 0; ji < MJ; ji++)
            acc[qi][ji] = fma(fv[qi / VEC].v[qi % VEC], xv[ji / VEC].v[ji % VEC], acc[qi][ji]);
      }
    } else {
      const T* xr = st + tj * (PC + C::PAD);
#pragma unroll 2
      for (int p0 = 0; p0 < PC; p0 += VEC) {
        V xv[MJ];
#pragma unroll
        for (int ji = 0; ji < MJ; ji++) xv[ji] = *reinterpret_cast<const V*>(xr + ji * JT * (PC + C::PAD) + p0);
#pragma unroll
        for (int pp = 0; pp < VEC; pp++) {
          V fv[NGQ];
#pragma unroll
          for (int g = 0; g < NGQ; g++) fv[g] = *reinterpret_cast<const V*>(fr + (p0 + pp) * Q + g * QS);
#pragma unroll
          for (int qi = 0; qi < MQ; qi++)
#pragma unroll
            for (int ji = 0; ji < MJ; ji++)
              acc[qi][ji] = fma(fv[qi / VEC].v[qi % VEC], xv[ji].v[pp], acc[qi][ji]);
        }
      }
    }

    if (c == C::NCH - 1) {
      // tile finished: stream the MQ x MJ block out and clear it
      const unsigned long long t = first + (s / C::NCH) * step;
      const bool epi = a.epilogue != 0;
      const bool useY = epi && a.beta != T(0) && a.Y != nullptr;
      if constexpr (!XT) {
        unsigned long long base = 0, n0 = 0;
        if (a.mode == 0) base = (t / a.tilesPerChunk) * QB + (t % a.tilesPerChunk) * (unsigned long long)TJ;
        else n0 = t * ((unsigned long long)TJ / a.B);
#pragma unroll
        for (int qi = 0; qi < MQ; qi++) {
          const int q = (qi / VEC) * QS + tq * VEC + (qi % VEC);
#pragma unroll
          for (int g = 0; g < NGJ; g++) {
            const int j = g * JS + tj * VEC;
            unsigned long long off;
            bool ok = true;
            if (a.mode == 0) {
              off = base + (unsigned long long)q * a.B + j;
            } else {
              const unsigned long long n = n0 + (unsigned long long)j / a.B;
              ok = n < a.numChunks;
              off = n * QB + (unsigned long long)q * a.B + (unsigned long long)j % a.B;
            }
            if (ok) {
              V o;
#pragma unroll
              for (int e = 0; e < VEC; e++) o.v[e] = epi ? a.alpha * acc[qi][g * VEC + e] : acc[qi][g * VEC + e];
              if (useY) {
                const V y = *reinterpret_cast<const V*>(a.Y + off);
#pragma unroll
                for (int e = 0; e < VEC; e++) o.v[e] = fma(a.beta, y.v[e], o.v[e]);
              }
              *reinterpret_cast<V*>(a.Z + off) = o;
            }
          }
        }
      } else {
        const unsigned long long n0 = t * (unsigned long long)TJ;
#pragma unroll
        for (int ji = 0; ji < MJ; ji++) {
          const unsigned long long n = n0 + tj + ji * JT;
          if (n < a.numChunks) {
#pragma unroll
            for (int g = 0; g < NGQ; g++) {
              const unsigned long long off = n * Q + g * QS + tq * VEC;
              V o;
#pragma unroll
              for (int e = 0; e < VEC; e++) o.v[e] = epi ? a.alpha * acc[g * VEC + e][ji] : acc[g * VEC + e][ji];
              if (useY) {
                const V y = *reinterpret_cast<const V*>(a.Y + off);
#pragma unroll
                for (int e = 0; e < VEC; e++) o.v[e] = fma(a.beta, y.v[e], o.v[e]);
              }
              *reinterpret_cast<V*>(a.Z + off) = o;
            }
          }
        }
      }
#pragma unroll
      for (int i = 0; i < MQ; i++)
#pragma unroll
        for (int j = 0; j < MJ; j++) acc[i][j] = T(0);
    }
  }
  cpAsyncWait<0>();
}

}  // namespace fkb

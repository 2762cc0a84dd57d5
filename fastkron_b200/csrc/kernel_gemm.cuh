// Large-factor kernel: one tensor mode of size P contracted with a P x Q factor,
//   [chunks][P][B] -> [chunks][Q][B],
// written as a register-blocked FFMA/DFMA GEMM  C[q, j] = sum_p F[p, q] * X[p, j]
// where j runs over TJ trailing positions (or, when B is small, over several whole
// chunks).  The factor stays resident in shared memory for the life of the
// (persistent) CTA; X streams through a ring of stages, PC rows of p at a time, so the
// global loads of tile t+1 overlap the arithmetic of tile t.  A stage is filled by one
// TMA instruction (cp.async.bulk.tensor.3d, completion on an mbarrier) in the main tile
// mode and by 16-byte cp.async from every thread in the others.  Every
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

#include <cuda.h>            // CUtensorMap (type only; the encoder is fetched at run time)

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
  Scatter sc;                        // parts > 0: rows go to other GPUs' buffers
  // Split contraction index on the input side (mode 0 only): row p of chunk n lives at
  // n*nStride + (p / pSplit)*pOuter + (p % pSplit)*B.  pSplit == 0: plain [n][P][B].
  // (Input of the multi-GPU phase 2, received as [sender][M][P/G][B].)
  unsigned pSplit = 0;
  unsigned long long pOuter = 0, nStride = 0;
  // mode 0 without split input: stages are filled by TMA (cp.async.bulk.tensor, one
  // instruction per stage issued by one thread, completion on an mbarrier) instead of
  // 16-byte cp.async from every thread.
  int useTma = 0;
};

// ---- mbarrier / TMA primitives (sm_90+ PTX; no multicast, one CTA) ---------------------
__device__ int gGemmTmaTimeouts = 0;     // set when a bounded wait on a stage barrier gave up

__device__ __forceinline__ void mbarInit(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"((unsigned)__cvta_generic_to_shared(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarInitFence() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
__device__ __forceinline__ void mbarExpectTx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"((unsigned)__cvta_generic_to_shared(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbarTryWait(unsigned long long* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok) : "r"((unsigned)__cvta_generic_to_shared(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Wait for a stage; gives up after about two seconds, records that and reports failure.
__device__ __forceinline__ bool mbarWaitBounded(unsigned long long* bar, unsigned parity) {
  if (mbarTryWait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbarTryWait(bar, parity)) {
    if (clock64() - t0 > 4000000000ll) { atomicExch(&gGemmTmaTimeouts, 1); return false; }
  }
  return true;
}
__device__ __forceinline__ void tmaLoad3D(void* smemDst, const CUtensorMap* tmap, int x, int y, int z,
                                          unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
      ::"r"((unsigned)__cvta_generic_to_shared(smemDst)), "l"(tmap), "r"(x), "r"(y), "r"(z),
        "r"((unsigned)__cvta_generic_to_shared(bar)) : "memory");
}

// Pointer to output row (chunk n, row q), trailing position 0.
template <typename T, int Q>
__device__ __forceinline__ T* gemmOutRow(const GemmArgs<T>& a, unsigned long long n, int q) {
  if (a.sc.parts > 0) {
    const unsigned d = (unsigned)q / (unsigned)a.sc.qPer, ql = (unsigned)q - d * (unsigned)a.sc.qPer;
    const unsigned long long m = n / a.sc.aLoc, ac = n - m * a.sc.aLoc;
    return reinterpret_cast<T*>(a.sc.base[d]) + (long long)m * a.sc.sM + (long long)ac * a.sc.sA +
           (long long)ql * a.sc.sQ + a.sc.zOff;
  }
  return a.Z + n * ((unsigned long long)Q * a.B) + (unsigned long long)q * a.B;
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

// The MQ x MJ accumulators of one thread.  With PACK, fp32 blocks are held as pairs and updated with the
// packed instruction of sm_100 (fma.rn.f32x2: two independent IEEE fp32 FMAs per lane, hence
// bit-identical to two scalar FMAs, for one issue slot); the scalar FFMA stream of this loop
// needs every issue slot of the SM for the arithmetic alone, so each shared-memory load,
// address update or barrier costs FMA throughput, and the packed form frees half of the
// slots.  Pairs run along j (the operand pair comes straight out of the 128-bit X load and
// the factor value is duplicated into both halves), or along q in the layout whose X values
// arrive one p-vector per j (the factor pair is natural there and x is duplicated).
template <typename T, int MQ, int MJ, bool PAIRQ, bool PACK>
struct AccBlock {
  T v[MQ][MJ];
  __device__ __forceinline__ T& at(int q, int j) { return v[q][j]; }
  __device__ __forceinline__ void clear() {
#pragma unroll
    for (int i = 0; i < MQ; i++)
#pragma unroll
      for (int j = 0; j < MJ; j++) v[i][j] = T(0);
  }
  // v[q][j] += f[q] * x[j] for the whole block
  __device__ __forceinline__ void rank1(const T (&f)[MQ], const T (&x)[MJ]) {
#pragma unroll
    for (int i = 0; i < MQ; i++)
#pragma unroll
      for (int j = 0; j < MJ; j++) v[i][j] = fma(f[i], x[j], v[i][j]);
  }
};

template <int MQ, int MJ>
struct AccBlock<float, MQ, MJ, false, true> {
  static_assert(MJ % 2 == 0, "pairs along j");
  float2 v[MQ][MJ / 2];
  __device__ __forceinline__ float& at(int q, int j) { return (j & 1) ? v[q][j >> 1].y : v[q][j >> 1].x; }
  __device__ __forceinline__ void clear() {
#pragma unroll
    for (int i = 0; i < MQ; i++)
#pragma unroll
      for (int j = 0; j < MJ / 2; j++) v[i][j] = make_float2(0.f, 0.f);
  }
  __device__ __forceinline__ void rank1(const float (&f)[MQ], const float (&x)[MJ]) {
#pragma unroll
    for (int i = 0; i < MQ; i++) {
      const float2 ff = make_float2(f[i], f[i]);
#pragma unroll
      for (int j = 0; j < MJ / 2; j++) v[i][j] = __ffma2_rn(ff, make_float2(x[2 * j], x[2 * j + 1]), v[i][j]);
    }
  }
};
template <int MQ, int MJ>
struct AccBlock<float, MQ, MJ, true, true> {
  static_assert(MQ % 2 == 0, "pairs along q");
  float2 v[MQ / 2][MJ];
  __device__ __forceinline__ float& at(int q, int j) { return (q & 1) ? v[q >> 1][j].y : v[q >> 1][j].x; }
  __device__ __forceinline__ void clear() {
#pragma unroll
    for (int i = 0; i < MQ / 2; i++)
#pragma unroll
      for (int j = 0; j < MJ; j++) v[i][j] = make_float2(0.f, 0.f);
  }
  __device__ __forceinline__ void rank1(const float (&f)[MQ], const float (&x)[MJ]) {
#pragma unroll
    for (int j = 0; j < MJ; j++) {
      const float2 xx = make_float2(x[j], x[j]);
#pragma unroll
      for (int i = 0; i < MQ / 2; i++) v[i][j] = __ffma2_rn(make_float2(f[2 * i], f[2 * i + 1]), xx, v[i][j]);
    }
  }
};

// ABL (the tuning tool only; always 0 in the library): timing ablations that produce wrong
// results on purpose -- bit 0 drops the global stores, bit 1 the stage loads after the first
// ring fill, bit 2 the CTA barrier of the stage loop.
template <typename T, int P, int Q, int TJ, int PC, int STAGES, int MQ, int MJ, bool XT, int UNR = 8, int MINB = 0, bool PACK = false, int ABL = 0>
__global__ void __launch_bounds__((Q / MQ) * (TJ / MJ), (MINB > 0 ? MINB : ((Q / MQ) * (TJ / MJ) <= 256 ? 2 : 1)))
gemmPassKernel(const GemmArgs<T> a, const __grid_constant__ CUtensorMap tmap) {
  using C = GemmCfg<T, P, Q, TJ, PC, STAGES, MQ, MJ, XT>;
  using V = Vec16<T>;
  constexpr int VEC = C::VEC, THREADS = C::THREADS, NGQ = C::NGQ, NGJ = C::NGJ;
  constexpr int QS = Q / NGQ;          // stride between a thread's q groups
  constexpr int JS = TJ / NGJ;         // stride between a thread's j groups (non-XT)
  constexpr int JT = TJ / MJ;          // stride between a thread's j's (XT)

  extern __shared__ __align__(1024) unsigned char smemRaw[];
  T* Fs = reinterpret_cast<T*>(smemRaw);
  T* stages = Fs + P * Q;
  __shared__ __align__(8) unsigned long long fullBar[STAGES];

  const int tid = threadIdx.x;
  const bool tma = !XT && a.useTma != 0;
  if (tma && tid == 0) {
#pragma unroll
    for (int i = 0; i < STAGES; i++) mbarInit(&fullBar[i], 1);
    mbarInitFence();
  }
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

  const unsigned first = blockIdx.x, step = gridDim.x;
  const unsigned numTiles = (unsigned)a.numTiles;        // the launcher keeps this below 2^31
  const unsigned myTiles = first < numTiles ? (numTiles - first + step - 1) / step : 0;
  const unsigned total = myTiles * C::NCH;
  const unsigned long long PB = (unsigned long long)P * a.B, QB = (unsigned long long)Q * a.B;
  const unsigned tpc = (unsigned)a.tilesPerChunk;        // mode 0
  const unsigned cpt = a.mode == 1 ? (unsigned)(TJ / a.B) : (unsigned)TJ;   // chunks per tile, modes 1/2

  // Per-thread constants of the stage loads.  A stage is filled by THREADS threads
  // taking 16-byte vectors in order, so a thread keeps one column position and walks
  // rows: all divisions happen here, once.
  constexpr int VPR = XT ? PC / VEC : TJ / VEC;          // vectors per stage row
  constexpr int RPP = THREADS / VPR;                     // rows covered per sweep of the CTA
  constexpr int NLD = (XT ? TJ : PC) / RPP;              // loads per thread per stage
  static_assert(THREADS % VPR == 0 && (XT ? TJ : PC) % RPP == 0, "stage load shape");
  const int ldCol = (tid % VPR) * VEC;                   // j (non-XT) or p offset (XT)
  const int ldRow = tid / VPR;                           // first p row (non-XT) or first j (XT)
  unsigned long long ldOff = 0;                          // global offset of (ldRow, ldCol) in a tile
  unsigned ldChunk = 0;                                  // chunk of the tile the column lies in (mode 1)
  if constexpr (!XT) {
    if (a.mode == 0) ldOff = (unsigned long long)ldRow * a.B + ldCol;
    else { ldChunk = (unsigned)(ldCol / a.B); ldOff = ldChunk * PB + (unsigned long long)ldRow * a.B + ldCol % a.B; }
  } else {
    ldOff = (unsigned long long)ldRow * P + ldCol;
  }
  const unsigned long long ldStep = XT ? (unsigned long long)RPP * P : (unsigned long long)RPP * a.B;
  T* const ldSmem = stages + (XT ? ldRow * (PC + C::PAD) + ldCol : ldRow * TJ + ldCol);
  constexpr int ldSmemStep = XT ? RPP * (PC + C::PAD) : RPP * TJ;

  // issue state: walks (tile, chunk) pairs in order
  unsigned isTile = first;
  int isC = 0;
  unsigned isSlot = 0;
  auto issue = [&]() {
    T* dst = ldSmem + (size_t)isSlot * C::STAGE_ELEMS;
    if constexpr (!XT) {
      if (a.mode == 0) {
        const unsigned n = isTile / tpc, bt = isTile - n * tpc;
        if (tma) {
          if (tid == 0) {
            mbarExpectTx(&fullBar[isSlot], (unsigned)(C::STAGE_ELEMS * sizeof(T)));
            tmaLoad3D(stages + (size_t)isSlot * C::STAGE_ELEMS, &tmap, (int)(bt * TJ), isC * PC, (int)n, &fullBar[isSlot]);
          }
        } else if (a.pSplit == 0) {
          const T* src = a.X + n * PB + (unsigned long long)bt * TJ + (unsigned long long)isC * PC * a.B + ldOff;
#pragma unroll
          for (int i = 0; i < NLD; i++) { cpAsync16(dst, src); dst += ldSmemStep; src += ldStep; }
        } else {
          const T* base = a.X + n * a.nStride + (unsigned long long)bt * TJ + ldCol;
#pragma unroll
          for (int i = 0; i < NLD; i++) {
            const unsigned p = (unsigned)(isC * PC + ldRow + i * RPP);
            const unsigned po = p / a.pSplit, pi = p - po * a.pSplit;
            cpAsync16(dst, base + po * a.pOuter + (unsigned long long)pi * a.B);
            dst += ldSmemStep;
          }
        }
      } else {
        const unsigned long long n0 = (unsigned long long)isTile * cpt;
        const bool ok = n0 + ldChunk < a.numChunks;
        const T* src = ok ? a.X + n0 * PB + (unsigned long long)isC * PC * a.B + ldOff : a.X;
#pragma unroll
        for (int i = 0; i < NLD; i++) { cpAsync16Zfill(dst, src, ok); dst += ldSmemStep; if (ok) src += ldStep; }
      }
    } else {
      const unsigned long long n0 = (unsigned long long)isTile * TJ;
      const T* src = a.X + n0 * P + isC * PC + ldOff;
#pragma unroll
      for (int i = 0; i < NLD; i++) {
        const bool ok = n0 + ldRow + i * RPP < a.numChunks;
        cpAsync16Zfill(dst, ok ? src : a.X, ok);
        dst += ldSmemStep; src += ldStep;
      }
    }
    if (++isC == C::NCH) { isC = 0; isTile += step; }
    if (++isSlot == STAGES) isSlot = 0;
  };

  AccBlock<T, MQ, MJ, XT, PACK && sizeof(T) == 4> acc;
  acc.clear();

#pragma unroll
  for (int s = 0; s < STAGES - 1; s++) {
    if ((unsigned)s < total) issue();
    cpAsyncCommit();
  }
  __syncthreads();   // factor visible

  unsigned curTile = first;
  int c = 0;
  unsigned slot = 0;
  unsigned phases = 0;                 // bit i: parity of the next completion of fullBar[i]
  for (unsigned s = 0; s < total; s++) {
    if (tma && !(ABL & 2)) {
      if (!mbarWaitBounded(&fullBar[slot], (phases >> slot) & 1u)) return;
      phases ^= 1u << slot;
    } else {
      cpAsyncWait<STAGES - 2>();
    }
    if (!(ABL & 4)) __syncthreads();
    if (s + STAGES - 1 < total && !(ABL & 2)) issue();
    cpAsyncCommit();

    const T* st = stages + (size_t)slot * C::STAGE_ELEMS;
    const T* fr = Fs + (size_t)c * PC * Q + tq * VEC;
    if constexpr (!XT) {
      const T* xr = st + tj * VEC;
#pragma unroll UNR
      for (int pl = 0; pl < PC; pl++) {
        V xv[NGJ], fv[NGQ];
#pragma unroll
        for (int g = 0; g < NGJ; g++) xv[g] = *reinterpret_cast<const V*>(xr + pl * TJ + g * JS);
#pragma unroll
        for (int g = 0; g < NGQ; g++) fv[g] = *reinterpret_cast<const V*>(fr + pl * Q + g * QS);
        T fq[MQ], xj[MJ];
#pragma unroll
        for (int qi = 0; qi < MQ; qi++) fq[qi] = fv[qi / VEC].v[qi % VEC];
#pragma unroll
        for (int ji = 0; ji < MJ; ji++) xj[ji] = xv[ji / VEC].v[ji % VEC];
        acc.rank1(fq, xj);
      }
    } else {
      const T* xr = st + tj * (PC + C::PAD);
#pragma unroll (UNR / VEC > 0 ? UNR / VEC : 1)
      for (int p0 = 0; p0 < PC; p0 += VEC) {
        V xv[MJ];
#pragma unroll
        for (int ji = 0; ji < MJ; ji++) xv[ji] = *reinterpret_cast<const V*>(xr + ji * JT * (PC + C::PAD) + p0);
#pragma unroll
        for (int pp = 0; pp < VEC; pp++) {
          V fv[NGQ];
#pragma unroll
          for (int g = 0; g < NGQ; g++) fv[g] = *reinterpret_cast<const V*>(fr + (p0 + pp) * Q + g * QS);
          T fq[MQ], xj[MJ];
#pragma unroll
          for (int qi = 0; qi < MQ; qi++) fq[qi] = fv[qi / VEC].v[qi % VEC];
#pragma unroll
          for (int ji = 0; ji < MJ; ji++) xj[ji] = xv[ji].v[pp];
          acc.rank1(fq, xj);
        }
      }
    }

    if (c == C::NCH - 1) {
      // tile finished: stream the MQ x MJ block out and clear it
      const unsigned t = curTile;
      const bool epi = a.epilogue != 0;
      const bool useY = epi && a.beta != T(0) && a.Y != nullptr;
      // Common case first and kept short (the steady-state loop has to stay small enough
      // for the instruction cache): plain pass, no epilogue, no redistribution.
      if ((ABL & 8) && !XT) {
        // ablation: the tile goes to a shared-memory staging area instead of global memory (what an
        // epilogue drained by bulk tensor stores would cost the compute warps)
        T* outS = stages + (size_t)STAGES * C::STAGE_ELEMS;
#pragma unroll
        for (int qi = 0; qi < MQ; qi++) {
          T* pq = outS + ((qi / VEC) * QS + tq * VEC + (qi % VEC)) * TJ + tj * VEC;
#pragma unroll
          for (int g = 0; g < NGJ; g++) {
            V o;
#pragma unroll
            for (int e = 0; e < VEC; e++) o.v[e] = acc.at(qi, g * VEC + e);
            *reinterpret_cast<V*>(pq + g * JS) = o;
          }
        }
      } else if ((ABL & 1) && a.numTiles != 0xFFFFFFFFull) {
        // ablation: keep the accumulators alive without storing them
        T sum = T(0);
#pragma unroll
        for (int qi = 0; qi < MQ; qi++)
#pragma unroll
          for (int ji = 0; ji < MJ; ji++) sum += XT ? acc.at(qi, ji) : acc.at(qi, ji);
        if (sum == T(12345.678)) a.Z[0] = sum;
      } else if (!epi && a.sc.parts == 0 && (XT || a.mode == 0)) {
        if constexpr (!XT) {
          const unsigned nn = t / tpc, bt = t - nn * tpc;
          T* p0 = a.Z + nn * QB + (unsigned long long)bt * TJ + tj * VEC + (unsigned long long)(tq * VEC) * a.B;
#pragma unroll
          for (int qi = 0; qi < MQ; qi++) {
            T* pq = p0 + (unsigned long long)((qi / VEC) * QS + (qi % VEC)) * a.B;
#pragma unroll
            for (int g = 0; g < NGJ; g++) {
              V o;
#pragma unroll
              for (int e = 0; e < VEC; e++) o.v[e] = acc.at(qi, g * VEC + e);
              *reinterpret_cast<V*>(pq + g * JS) = o;
            }
          }
        } else {
          const unsigned long long n0 = (unsigned long long)t * TJ + tj;
          T* p0 = a.Z + n0 * Q + tq * VEC;
#pragma unroll
          for (int ji = 0; ji < MJ; ji++) {
            if (n0 + ji * JT < a.numChunks) {
#pragma unroll
              for (int g = 0; g < NGQ; g++) {
                V o;
#pragma unroll
                for (int e = 0; e < VEC; e++) o.v[e] = acc.at(g * VEC + e, ji);
                *reinterpret_cast<V*>(p0 + (size_t)ji * JT * Q + g * QS) = o;
              }
            }
          }
        }
      } else if constexpr (!XT) {
#pragma unroll
        for (int g = 0; g < NGJ; g++) {
          const int j = g * JS + tj * VEC;
          unsigned long long n, col;
          bool ok = true;
          if (a.mode == 0) {
            const unsigned nn = t / tpc, bt = t - nn * tpc;
            n = nn; col = (unsigned long long)bt * TJ + j;
          } else {
            n = (unsigned long long)t * cpt + (unsigned)(j / a.B);
            ok = n < a.numChunks;
            col = j % a.B;
          }
          if (ok) {
            // everything of the output address that does not depend on q, once per group
            const bool sc = a.sc.parts > 0;
            unsigned long long rowBase;
            if (sc) {
              const unsigned long long m = n / a.sc.aLoc, ac = n - m * a.sc.aLoc;
              rowBase = (unsigned long long)((long long)m * a.sc.sM + (long long)ac * a.sc.sA + a.sc.zOff) + col;
            } else {
              rowBase = n * QB + col;
            }
            const unsigned qPer = (unsigned)a.sc.qPer;
#pragma unroll
            for (int qi = 0; qi < MQ; qi++) {
              const int q = (qi / VEC) * QS + tq * VEC + (qi % VEC);
              T* dst;
              if (sc) {
                const unsigned d = (unsigned)q / qPer, ql = (unsigned)q - d * qPer;
                dst = reinterpret_cast<T*>(a.sc.base[d]) + rowBase + (unsigned long long)ql * (unsigned long long)a.sc.sQ;
              } else {
                dst = a.Z + rowBase + (unsigned long long)q * a.B;
              }
              V o;
#pragma unroll
              for (int e = 0; e < VEC; e++) o.v[e] = epi ? a.alpha * acc.at(qi, g * VEC + e) : acc.at(qi, g * VEC + e);
              if (useY) {
                const V y = *reinterpret_cast<const V*>(a.Y + (dst - a.Z));
#pragma unroll
                for (int e = 0; e < VEC; e++) o.v[e] = fma(a.beta, y.v[e], o.v[e]);
              }
              *reinterpret_cast<V*>(dst) = o;
            }
          }
        }
      } else {
        const unsigned long long n0 = (unsigned long long)t * TJ;
#pragma unroll
        for (int ji = 0; ji < MJ; ji++) {
          const unsigned long long n = n0 + tj + ji * JT;
          if (n < a.numChunks) {
#pragma unroll
            for (int g = 0; g < NGQ; g++) {
              if (a.sc.parts > 0) {
                // redistributed rows are not contiguous in q: one element at a time
#pragma unroll
                for (int e = 0; e < VEC; e++)
                  *gemmOutRow<T, Q>(a, n, g * QS + tq * VEC + e) = epi ? a.alpha * acc.at(g * VEC + e, ji) : acc.at(g * VEC + e, ji);
                continue;
              }
              const unsigned long long off = n * Q + g * QS + tq * VEC;
              V o;
#pragma unroll
              for (int e = 0; e < VEC; e++) o.v[e] = epi ? a.alpha * acc.at(g * VEC + e, ji) : acc.at(g * VEC + e, ji);
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
      acc.clear();
      curTile += step;
    }
    if (++c == C::NCH) c = 0;
    if (++slot == STAGES) slot = 0;
  }
  cpAsyncWait<0>();
}

}  // namespace fkb

// Large-factor kernel for ANY factor shape: one tensor mode of size P contracted with a P x Q
// factor, [chunks][P][B] -> [chunks][Q][B], for every P, Q, B, stride pattern and alignment
// that the two fixed-shape kernels (kernel_gemm.cuh: 64x64, 128x128) do not take: non-square
// factors (31x63, 297x127), sizes that are not powers of two (12, 24, 50, 127, 129, 255, 297),
// P > 128, fp64 128x128, operands that are not 16-byte aligned, transposed first passes.
// (The reference covers these with one template that loops over tiles of P and masks partial
// tiles, src/kernels/cuda/kernel.cuh:174, falling back through four optimisation levels,
// src/kernel_db/kernel_db.cpp:317-366.)
//
// Same formulation as the fixed-shape kernels -- a register-blocked contraction
//   C[q, j] = sum_p F[p, q] * X[p, j],    8 x 8 (fp32) or 8 x 4 (fp64) outputs per thread,
// j running over the trailing positions of all chunks (so a tile may span chunks when B is
// small) -- with everything that was a compile-time constant there a run-time value here:
//   * the contraction runs over chunks of PC rows of p; per chunk a [PC][TQ] piece of the
//     factor and a [PC][TJ] piece of X are staged in shared memory (two buffers, cp.async), rows
//     and columns beyond P, Q or the last position zero-filled, so partial tiles need no special
//     arithmetic;
//   * three tile shapes, chosen by Q: 64 (q) x 128 (j) with PC = 32 for Q > 32, and 32 x 256 or
//     16 x 256 with PC = 16 for narrower factors (a 12x12 or 16x16 factor would fill a 64-wide
//     tile and a 32-row chunk to a few per cent; these passes are bound by HBM once the tile
//     fits the factor);
//   * the products of an output are accumulated over p ascending across the chunks, i.e. in the
//     reference's order (src/kernels/cuda/mma.cuh:1-15);
//   * global accesses are 16-byte vectors when strides and alignment allow, single elements
//     otherwise (4- or 8-byte cp.async, scalar stores), always with consecutive lanes on
//     consecutive addresses of the contiguous index where there is one;
//   * stores are masked.
// Two shared-memory layouts of the X piece as in the fixed-shape kernels: [p][j] when the
// trailing index is the contiguous one, [j][p + pad] when the contracted index itself is
// (trailing extent 1, dense input).
#include "kernels.h"
#include "gemm_table.h"
#include "kernel_tile.cuh"   // Vec16, cpAsync16

namespace fkb {

template <typename T>
struct AnyArgs {
  const T* X; T* Z; const T* Y; const T* F;
  long long fsP, fsQ;
  unsigned P, Q;
  unsigned long long A, B, M;            // chunk n = m*A + a, trailing extent B
  long long xsM, xsA, xsG, xsB;          // input  (m, a, p, b) at m*xsM + a*xsA + p*xsG + b*xsB
  long long zsM, zsA, zsG, zsB;          // output (m, a, q, b) likewise
  unsigned long long Jtotal;             // M*A*B trailing positions in all
  unsigned qTiles;
  unsigned long long numTiles;           // qTiles * ceil(Jtotal / TJ), q-tile fastest
  T alpha, beta;
  int epilogue;
  int vecX, vecZ, vecF;                  // 16-byte accesses allowed on X / on Z and Y / on F rows
  int vecZJ;                             // [j][p] staging only: the output is contiguous along the chunk index
                                         // (zsA == 1, the rotating layout of the forward variants): 16-byte
                                         // stores along j after a transposition through shared memory
  // strided batch: tile index = entry * tilesPerEntry + tile within the entry (a tile never spans entries)
  unsigned batch;
  unsigned long long tilesPerEntry, bsX, bsZ, bsY, bsF;
};

template <int BYTES>
__device__ __forceinline__ void cpAsyncZfill(void* smemDst, const void* gmemSrc, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smemDst);
  const int n = valid ? BYTES : 0;
  if (BYTES == 16)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmemSrc), "r"(n) : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;\n" ::"r"(s), "l"(gmemSrc), "n"(BYTES), "r"(n) : "memory");
}

template <typename T, int TQ_>
struct AnyCfg {
  static_assert(TQ_ == 64 || TQ_ == 32 || TQ_ == 16, "tile heights that exist");
  static constexpr int VEC = 16 / (int)sizeof(T);
  static constexpr int TQ = TQ_, MQ = (TQ_ == 16 ? 4 : 8), MJ = 2 * VEC, THREADS = 128;
  static constexpr int WQ = TQ / MQ / 4;                         // warps along q (4 q-lanes per warp)
  static constexpr int TJ = (THREADS / (TQ / MQ)) * MJ;          // TQ 64: 128 (fp32), 64 (fp64); else 256, 128
  static constexpr int PC = (TQ_ == 64 ? 32 : 16), PAD = VEC;
  static constexpr int NGQ = MQ / VEC, NGJ = MJ / VEC, QS = TQ / NGQ, JS = TJ / NGJ, JT = TJ / MJ;
  static constexpr int XELEMS_N = PC * TJ, XELEMS_T = TJ * (PC + PAD);
  static constexpr int XELEMS = XELEMS_T > XELEMS_N ? XELEMS_T : XELEMS_N;
  static constexpr int FELEMS = PC * TQ;
  static constexpr size_t SMEM = 2 * (size_t)(XELEMS + FELEMS) * sizeof(T);
  // the [j][p] variant may park a finished [TQ][TJ + VEC] tile in the two X buffers
  static_assert(TQ * (TJ + VEC) <= 2 * XELEMS, "output tile fits the X buffers");
};

// Address pieces of trailing position J: chunk (m, a) and b.
template <typename T>
__device__ __forceinline__ void splitJ(const AnyArgs<T>& a, unsigned long long J, unsigned long long& m,
                                       unsigned long long& ac, unsigned long long& b) {
  const unsigned long long n = J / a.B;
  b = J - n * a.B;
  m = n / a.A;
  ac = n - m * a.A;
}

template <typename T, bool XT, int TQ_>
__global__ void __launch_bounds__(128, 3) gemmAnyKernel(const AnyArgs<T> a0) {
  using C = AnyCfg<T, TQ_>;
  using V = Vec16<T>;
  constexpr int VEC = C::VEC, TQ = C::TQ, TJ = C::TJ, PC = C::PC, MQ = C::MQ, MJ = C::MJ, THREADS = C::THREADS;
  constexpr int NGQ = C::NGQ, NGJ = C::NGJ, QS = C::QS, JS = C::JS, JT = C::JT, PAD = C::PAD;

  extern __shared__ __align__(1024) unsigned char smemRaw[];
  T* Xs = reinterpret_cast<T*>(smemRaw);                  // [2][XELEMS]
  T* Fs = Xs + 2 * C::XELEMS;                             // [2][FELEMS]

  // [j][p] staging: input offset of row j of the tile (-1 beyond the last position), once per tile
  __shared__ long long rowBase[XT ? TJ : 1];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tq = (warp % C::WQ) * 4 + (lane & 3);         // TQ / MQ q positions
  const int tj = (warp / C::WQ) * 8 + (lane >> 2);        // THREADS / (TQ / MQ) j positions

  const unsigned nch = (a0.P + PC - 1) / PC;
  for (unsigned long long gtile = blockIdx.x; gtile < a0.numTiles; gtile += gridDim.x) {
    // the entry's operands (a copy of the arguments with shifted pointers keeps the body unchanged)
    AnyArgs<T> a = a0;
    unsigned long long tile = gtile;
    if (a0.batch > 1) {
      const unsigned long long bt = gtile / a0.tilesPerEntry;
      tile = gtile - bt * a0.tilesPerEntry;
      a.X = a0.X + bt * a0.bsX; a.Z = a0.Z + bt * a0.bsZ; a.F = a0.F + bt * a0.bsF;
      a.Y = a0.Y ? a0.Y + bt * a0.bsY : nullptr;
    }
    const unsigned qt = (unsigned)(tile % a.qTiles);
    const unsigned long long J0 = (tile / a.qTiles) * (unsigned long long)TJ;
    const unsigned q0 = qt * TQ;
    if constexpr (XT) {
      // (the barrier that ended the previous tile's last chunk ordered the last reads of the table)
      for (int r = tid; r < TJ; r += THREADS) {
        const unsigned long long J = J0 + r;
        long long base = -1;
        if (J < a.Jtotal) {
          unsigned long long m, ac, b;
          splitJ(a, J, m, ac, b);
          base = (long long)m * a.xsM + (long long)ac * a.xsA;
        }
        rowBase[r] = base;
      }
      __syncthreads();
    }

    // ---- stage loader: chunk c of the contraction into buffer c & 1 --------------------------
    auto issue = [&](unsigned c) {
      T* xs = Xs + (size_t)(c & 1) * C::XELEMS;
      T* fs = Fs + (size_t)(c & 1) * C::FELEMS;
      const unsigned p0 = c * PC;
      // factor piece [PC][TQ]
      if (a.vecF) {
        for (int v = tid; v < PC * TQ / VEC; v += THREADS) {
          const unsigned pl = (unsigned)(v * VEC) / TQ, q = (unsigned)(v * VEC) % TQ;
          const bool ok = p0 + pl < a.P && q0 + q < a.Q;     // Q % VEC == 0: whole vectors
          cpAsyncZfill<16>(fs + pl * TQ + q, ok ? a.F + (long long)(p0 + pl) * a.fsP + (q0 + q) : a.F, ok);
        }
      } else if (a.fsQ == 1 || a.fsP != 1) {
        for (int i = tid; i < PC * TQ; i += THREADS) {
          const unsigned pl = (unsigned)i / TQ, q = (unsigned)i % TQ;
          const bool ok = p0 + pl < a.P && q0 + q < a.Q;
          cpAsyncZfill<(int)sizeof(T)>(fs + pl * TQ + q, ok ? a.F + (long long)(p0 + pl) * a.fsP + (long long)(q0 + q) * a.fsQ : a.F, ok);
        }
      } else {
        for (int i = tid; i < PC * TQ; i += THREADS) {          // stored q-major: walk p fastest
          const unsigned q = (unsigned)i / PC, pl = (unsigned)i % PC;
          const bool ok = p0 + pl < a.P && q0 + q < a.Q;
          cpAsyncZfill<(int)sizeof(T)>(fs + pl * TQ + q, ok ? a.F + (long long)(p0 + pl) + (long long)(q0 + q) * a.fsQ : a.F, ok);
        }
      }
      // X piece
      if constexpr (!XT) {
        if (a.vecX) {
          // a vector never straddles a chunk: B % VEC == 0 and J0 % VEC == 0
          constexpr int VPR = TJ / VEC, RPP = THREADS / VPR;
          const unsigned j = (unsigned)(tid % VPR) * VEC;
          const unsigned long long J = J0 + j;
          const bool okJ = J < a.Jtotal;
          unsigned long long m = 0, ac = 0, b = 0;
          if (okJ) splitJ(a, J, m, ac, b);
          const T* col = a.X + (long long)m * a.xsM + (long long)ac * a.xsA + (long long)b;
#pragma unroll
          for (int pl = tid / VPR; pl < PC; pl += RPP) {
            const bool ok = okJ && p0 + pl < a.P;
            cpAsyncZfill<16>(xs + pl * TJ + j, ok ? col + (long long)(p0 + pl) * a.xsG : a.X, ok);
          }
        } else {
          constexpr int CPT = THREADS / TJ > 0 ? THREADS / TJ : 1;   // threads per column (or columns per thread)
          for (unsigned j = (unsigned)tid % TJ; j < (unsigned)TJ; j += THREADS) {
            const unsigned long long J = J0 + j;
            const bool okJ = J < a.Jtotal;
            unsigned long long m = 0, ac = 0, b = 0;
            if (okJ) splitJ(a, J, m, ac, b);
            const T* col = a.X + (long long)m * a.xsM + (long long)ac * a.xsA + (long long)b * a.xsB;
            for (int pl = tid / TJ; pl < PC; pl += CPT) {
              const bool ok = okJ && p0 + pl < a.P;
              cpAsyncZfill<(int)sizeof(T)>(xs + pl * TJ + j, ok ? col + (long long)(p0 + pl) * a.xsG : a.X, ok);
            }
          }
        }
      } else {
        // trailing extent 1, p contiguous: position J is chunk n = J, row of P values
        if (a.vecX) {
          constexpr int VPR = PC / VEC, RPP = THREADS / VPR;
          const unsigned pl = (unsigned)(tid % VPR) * VEC;
#pragma unroll 4
          for (int j = tid / VPR; j < TJ; j += RPP) {
            const long long base = rowBase[j];
            const bool ok = base >= 0 && p0 + pl < a.P;         // P % VEC == 0: whole vectors
            cpAsyncZfill<16>(xs + j * (PC + PAD) + pl, ok ? a.X + base + (p0 + pl) : a.X, ok);
          }
        } else {
          constexpr int RPP = THREADS / PC;
          const unsigned pl = (unsigned)tid % PC;
#pragma unroll 4
          for (int j = tid / PC; j < TJ; j += RPP) {
            const long long base = rowBase[j];
            const bool ok = base >= 0 && p0 + pl < a.P;
            cpAsyncZfill<(int)sizeof(T)>(xs + j * (PC + PAD) + pl, ok ? a.X + base + (p0 + pl) : a.X, ok);
          }
        }
      }
      asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    T acc[MQ][MJ];
#pragma unroll
    for (int i = 0; i < MQ; i++)
#pragma unroll
      for (int j = 0; j < MJ; j++) acc[i][j] = T(0);

    issue(0);
    for (unsigned c = 0; c < nch; c++) {
      if (c + 1 < nch) {
        issue(c + 1);
        asm volatile("cp.async.wait_group 1;\n" ::: "memory");
      } else {
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
      }
      __syncthreads();
      const T* xs = Xs + (size_t)(c & 1) * C::XELEMS;
      const T* fr = Fs + (size_t)(c & 1) * C::FELEMS + tq * VEC;
      if constexpr (!XT) {
        const T* xr = xs + tj * VEC;
#pragma unroll 8
        for (int pl = 0; pl < PC; pl++) {
          V xv[NGJ], fv[NGQ];
#pragma unroll
          for (int g = 0; g < NGJ; g++) xv[g] = *reinterpret_cast<const V*>(xr + pl * TJ + g * JS);
#pragma unroll
          for (int g = 0; g < NGQ; g++) fv[g] = *reinterpret_cast<const V*>(fr + pl * TQ + g * QS);
#pragma unroll
          for (int qi = 0; qi < MQ; qi++)
#pragma unroll
            for (int ji = 0; ji < MJ; ji++)
              acc[qi][ji] = fma(fv[qi / VEC].v[qi % VEC], xv[ji / VEC].v[ji % VEC], acc[qi][ji]);
        }
      } else {
        const T* xr = xs + tj * (PC + PAD);
#pragma unroll 2
        for (int pv = 0; pv < PC; pv += VEC) {
          V xv[MJ];
#pragma unroll
          for (int ji = 0; ji < MJ; ji++) xv[ji] = *reinterpret_cast<const V*>(xr + ji * JT * (PC + PAD) + pv);
#pragma unroll
          for (int pp = 0; pp < VEC; pp++) {
            V fv[NGQ];
#pragma unroll
            for (int g = 0; g < NGQ; g++) fv[g] = *reinterpret_cast<const V*>(fr + (pv + pp) * TQ + g * QS);
#pragma unroll
            for (int qi = 0; qi < MQ; qi++)
#pragma unroll
              for (int ji = 0; ji < MJ; ji++)
                acc[qi][ji] = fma(fv[qi / VEC].v[qi % VEC], xv[ji].v[pp], acc[qi][ji]);
          }
        }
      }
      __syncthreads();           // the buffer just read is refilled two chunks from now
    }

    // ---- masked stores (alpha / beta*Y on the epilogue pass) ---------------------------------
    const bool epi = a.epilogue != 0;
    const bool useY = epi && a.beta != T(0) && a.Y != nullptr;
    if constexpr (!XT) {
#pragma unroll
      for (int g = 0; g < NGJ; g++) {
        const unsigned long long J = J0 + (unsigned)(g * JS + tj * VEC);
        if (J >= a.Jtotal) continue;
        unsigned long long m, ac, b;
        splitJ(a, J, m, ac, b);
        if (a.vecZ) {
          const long long rowBase = (long long)m * a.zsM + (long long)ac * a.zsA + (long long)b;
#pragma unroll
          for (int qi = 0; qi < MQ; qi++) {
            const unsigned q = q0 + (unsigned)((qi / VEC) * QS + tq * VEC + (qi % VEC));
            if (q >= a.Q) continue;
            const long long off = rowBase + (long long)q * a.zsG;
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
        } else {
#pragma unroll
          for (int e = 0; e < VEC; e++) {
            if (J + e >= a.Jtotal) break;
            if (e > 0 && ++b == a.B) { b = 0; if (++ac == a.A) { ac = 0; m++; } }
            const long long rowBase = (long long)m * a.zsM + (long long)ac * a.zsA + (long long)b * a.zsB;
#pragma unroll
            for (int qi = 0; qi < MQ; qi++) {
              const unsigned q = q0 + (unsigned)((qi / VEC) * QS + tq * VEC + (qi % VEC));
              if (q >= a.Q) continue;
              const long long off = rowBase + (long long)q * a.zsG;
              T val = epi ? a.alpha * acc[qi][g * VEC + e] : acc[qi][g * VEC + e];
              if (useY) val = fma(a.beta, a.Y[off], val);
              a.Z[off] = val;
            }
          }
        }
      }
    } else if (a.vecZJ) {
      // the loop's last barrier is behind every thread: the X buffers are free; park the tile
      // there as [q][j] and write rows of it with 16-byte stores along j
      constexpr int LDO = TJ + VEC;
      T* ot = Xs;
#pragma unroll
      for (int qi = 0; qi < MQ; qi++) {
        const int ql = (qi / VEC) * QS + tq * VEC + (qi % VEC);
#pragma unroll
        for (int ji = 0; ji < MJ; ji++) ot[ql * LDO + tj + ji * JT] = acc[qi][ji];
      }
      __syncthreads();
      constexpr int VPR = TJ / VEC;
      for (int idx = tid; idx < TQ * VPR; idx += THREADS) {
        const int ql = idx / VPR, jv = (idx % VPR) * VEC;
        const unsigned long long J = J0 + (unsigned)jv;
        const unsigned q = q0 + (unsigned)ql;
        if (J >= a.Jtotal || q >= a.Q) continue;            // A % VEC == 0: vectors are whole and stay in one row
        unsigned long long m, ac, b;
        splitJ(a, J, m, ac, b);
        const long long off = (long long)m * a.zsM + (long long)ac + (long long)q * a.zsG;
        V o = *reinterpret_cast<const V*>(ot + ql * LDO + jv);
        if (epi) {
#pragma unroll
          for (int e = 0; e < VEC; e++) o.v[e] = a.alpha * o.v[e];
          if (useY) {
            const V y = *reinterpret_cast<const V*>(a.Y + off);
#pragma unroll
            for (int e = 0; e < VEC; e++) o.v[e] = fma(a.beta, y.v[e], o.v[e]);
          }
        }
        *reinterpret_cast<V*>(a.Z + off) = o;
      }
      // (the next tile's table fill ends in a barrier before any thread refills the X buffers)
    } else {
#pragma unroll
      for (int ji = 0; ji < MJ; ji++) {
        const unsigned long long J = J0 + (unsigned)(tj + ji * JT);
        if (J >= a.Jtotal) continue;
        unsigned long long m, ac, b;
        splitJ(a, J, m, ac, b);
        const long long rowBase = (long long)m * a.zsM + (long long)ac * a.zsA;
#pragma unroll
        for (int g = 0; g < NGQ; g++) {
          const unsigned q = q0 + (unsigned)(g * QS + tq * VEC);
          if (q >= a.Q) continue;
          if (a.vecZ) {                                    // zsG == 1, Q % VEC == 0: whole vectors
            const long long off = rowBase + (long long)q;
            V o;
#pragma unroll
            for (int e = 0; e < VEC; e++) o.v[e] = epi ? a.alpha * acc[g * VEC + e][ji] : acc[g * VEC + e][ji];
            if (useY) {
              const V y = *reinterpret_cast<const V*>(a.Y + off);
#pragma unroll
              for (int e = 0; e < VEC; e++) o.v[e] = fma(a.beta, y.v[e], o.v[e]);
            }
            *reinterpret_cast<V*>(a.Z + off) = o;
          } else {
#pragma unroll
            for (int e = 0; e < VEC; e++) {
              if (q + e >= a.Q) break;
              const long long off = rowBase + (long long)(q + e) * a.zsG;
              T val = epi ? a.alpha * acc[g * VEC + e][ji] : acc[g * VEC + e][ji];
              if (useY) val = fma(a.beta, a.Y[off], val);
              a.Z[off] = val;
            }
          }
        }
      }
    }
  }
}

// One launcher per kernel instantiation: the shared-memory opt-in and the occupancy are
// properties of (kernel, device).
template <typename T, bool XT, int TQ_>
static fastKronError launchAnyKernel(const AnyArgs<T>& a, const LaunchCtx& cx) {
  using C = AnyCfg<T, TQ_>;
  auto kern = gemmAnyKernel<T, XT, TQ_>;
  static bool attrDev[kMaxDevices] = {false};
  static int occDev[kMaxDevices] = {0};
  const int dev = currentDeviceSlot();
  if (!attrDev[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM);
    if (e != cudaSuccess) return cudaToFk(e);
    int n = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, C::THREADS, C::SMEM);
    if (e != cudaSuccess || n < 1) return e != cudaSuccess ? cudaToFk(e) : fastKronKernelNotFound;
    occDev[dev] = n;
    attrDev[dev] = true;
  }
  unsigned long long grid = (unsigned long long)cx.smCount * occDev[dev];
  if (grid > a.numTiles) grid = a.numTiles;
  kern<<<(unsigned)grid, C::THREADS, C::SMEM, cx.stream>>>(a);
  return cudaToFk(cudaGetLastError());
}

template <typename T, int TQ_>
static fastKronError launchGemmAnyT(const Pass& ps, const LaunchCtx& cx) {
  using C = AnyCfg<T, TQ_>;
  constexpr int VEC = C::VEC;
  AnyArgs<T> a;
  a.X = (const T*)cx.src; a.Z = (T*)cx.dst; a.Y = (const T*)cx.Y; a.F = (const T*)cx.F[0];
  a.fsP = cx.fsP; a.fsQ = cx.fsQ;
  a.P = ps.P[0]; a.Q = ps.Q[0];
  a.A = ps.A; a.B = ps.B; a.M = ps.M;
  a.xsM = ps.xsM; a.xsA = ps.xsA; a.xsG = ps.xsG; a.xsB = ps.xsB;
  a.zsM = ps.zsM; a.zsA = ps.zsA; a.zsG = ps.zsG; a.zsB = ps.zsB;
  a.Jtotal = ps.M * ps.A * ps.B;
  a.alpha = (T)cx.alpha; a.beta = (T)cx.beta; a.epilogue = ps.epilogue ? 1 : 0;
  a.vecZJ = 0;
  if (a.Jtotal == 0) return fastKronSuccess;
  a.qTiles = (a.Q + C::TQ - 1) / C::TQ;
  a.tilesPerEntry = (unsigned long long)a.qTiles * ((a.Jtotal + C::TJ - 1) / C::TJ);
  a.batch = cx.batch; a.bsX = cx.bsX; a.bsZ = cx.bsZ; a.bsY = cx.bsY; a.bsF = cx.bsF[0];
  a.numTiles = a.tilesPerEntry * a.batch;

  auto mult = [](long long v, long long m) { return v % m == 0; };
  auto al16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  // the contracted index itself contiguous and nothing behind it: [j][p] staging
  const bool xt = ps.B == 1 && ps.xsG == 1;
  if (!xt) {
    a.vecX = ps.xsB == 1 && mult((long long)ps.B, VEC) && mult(ps.xsM, VEC) && mult(ps.xsA, VEC) && mult(ps.xsG, VEC) && al16(a.X);
    a.vecZ = ps.zsB == 1 && mult((long long)ps.B, VEC) && mult(ps.zsM, VEC) && mult(ps.zsA, VEC) && mult(ps.zsG, VEC) && al16(a.Z) &&
             (a.Y == nullptr || al16(a.Y));
  } else {
    a.vecX = mult((long long)a.P, VEC) && mult(ps.xsM, VEC) && mult(ps.xsA, VEC) && al16(a.X);
    a.vecZ = ps.zsG == 1 && mult((long long)a.Q, VEC) && mult(ps.zsM, VEC) && mult(ps.zsA, VEC) && al16(a.Z) &&
             (a.Y == nullptr || al16(a.Y));
    // (fp32 only: measured on B200, 16x16^4 forward 0.90 -> 0.72 ms, 8x8^6 5.0 -> 3.4 ms; fp64 scalar stores
    // already make 64-byte runs per quarter warp and showed no gain from the shared-memory round trip)
    a.vecZJ = sizeof(T) == 4 && !a.vecZ && ps.zsA == 1 && mult((long long)ps.A, VEC) && mult(ps.zsM, VEC) && mult(ps.zsG, VEC) && al16(a.Z) &&
              (a.Y == nullptr || al16(a.Y));
  }
  a.vecF = cx.fsQ == 1 && mult((long long)a.Q, VEC) && mult(cx.fsP, VEC) && al16(a.F);
  if (a.batch > 1) {
    a.vecX = a.vecX && mult((long long)a.bsX, VEC);
    a.vecZ = a.vecZ && mult((long long)a.bsZ, VEC) && mult((long long)a.bsY, VEC);
    a.vecZJ = a.vecZJ && mult((long long)a.bsZ, VEC) && mult((long long)a.bsY, VEC);
    a.vecF = a.vecF && mult((long long)a.bsF, VEC);
  }

  return xt ? launchAnyKernel<T, true, TQ_>(a, cx) : launchAnyKernel<T, false, TQ_>(a, cx);
}

// Tile height by factor width: the narrowest tile that holds all of Q (up to 64).
template <typename T>
static fastKronError launchGemmAnyQ(const Pass& ps, const LaunchCtx& cx) {
  const uint32_t Q = ps.Q[0];
  if (Q <= 16) return launchGemmAnyT<T, 16>(ps, cx);
  if (Q <= 32) return launchGemmAnyT<T, 32>(ps, cx);
  return launchGemmAnyT<T, 64>(ps, cx);
}

// Any single-factor pass the eligibility rule (gemm_table.h) admits whose operands are plain strided tensors (no
// redistribution over GPUs, no split input).
fastKronError launchGemmAny(const Pass& ps, const LaunchCtx& cx) {
  if (ps.nf != 1 || cx.scatter.parts > 0 || cx.pSplit != 0) return fastKronKernelNotFound;
  if (!gemmAnyEligible(ps.P[0], ps.Q[0])) return fastKronKernelNotFound;
  if (cx.dt == DType::F32) return launchGemmAnyQ<float>(ps, cx);
  return launchGemmAnyQ<double>(ps, cx);
}

}  // namespace fkb

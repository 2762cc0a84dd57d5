// Opt-in TF32 tensor-core variant of the large-factor pass (fp32 operands, P = Q in {64, 128}).
//
// Not the default path: fp32 results of the default kernels match an fp32 CPU computation to
// rounding, this one reads the fp32 operands as TF32 (10-bit mantissa) on the 5th-generation
// tensor cores and accumulates in fp32.  It is used only when the handle carries
// fastKronOptionsTF32 or the environment has FASTKRON_TF32=1, and its tolerance is its own:
// a few 1e-3 of the row maximum after four chained factors (tests/test_tf32_gpu.py).
//
// One pass is  Z[n][q][j] = sum_p F[p][q] * X[n][p][j]  over the dense view [chunks][P][B].
// A CTA tile is 128 rows of the (n, j) index space times all Q outputs:
//   D[128 x Q] (TMEM, fp32) = A[128 x P] * B[P x Q],  issued as P/8 tcgen05.mma.kind::tf32.
//   B >= 32:  A = X tile with j contiguous ("MN-major"): four TMA boxes write it as [4 atoms][P][32
//             floats] with the 128-byte swizzle of 32-byte atoms (the one TF32 operands of that
//             orientation need); an atom is 32 consecutive j of one chunk.  B % 128 == 0:
//             the four atoms are 128 consecutive j; B = 64 / 32: two / four chunks per tile.
//   B == 1 :  A = 128 chunks with p contiguous ("K-major"): TMA writes [P/32 slabs][128][32 floats].
//   The factor is written once per CTA as [Q/32][P][32 floats] with that swizzle (MN-major B).
// Warp roles (192 threads): warp 0 lane 0 issues TMA loads into a ring of stages; warp 1 owns
// the TMEM allocation and lane 0 issues the MMAs (completion via tcgen05.commit on mbarriers);
// warps 2-5 read the accumulator with tcgen05.ld (one TMEM lane quarter each) and store it.
// Two accumulators alternate so that the epilogue of a tile overlaps the loads and MMAs of
// the next.  Every barrier wait is time-bounded; a wait that gives up raises an abort flag
// that ends all role loops, TMEM is released on every path, and the host sees
// fkbGemmTcTimeouts() != 0.  No cluster launch, no multicast.
//
// SPLIT variant (fastKronOptionsTF32x3 / FASTKRON_TF32=3; 64x64 factors): every fp32 operand is
// split into two TF32 numbers, hi = rna_tf32(v) and lo = rna_tf32(v - hi), and a product is
// formed as lo*hi + hi*lo + hi*hi on the tensor cores with fp32 accumulation (the dropped lo*lo
// term and the rounding of lo are of relative size 2^-21): results agree with the fp32 kernels to
// about 1e-6 of the row maximum, i.e. well inside the fp32 tolerance of the default path, at
// three times the tensor-core work, which still leaves the pass bound by HBM.  The factor is
// split once per CTA into two shared-memory copies; four more warps ("converters", 320 threads
// in all) split each X stage in place (hi) and into a second buffer of the stage (lo) between
// its arrival and its MMAs, and hand it over through one more mbarrier per stage.
#include <cuda.h>
#include <string.h>
#include <stdlib.h>

#include "kernels.h"
#include "gemm_table.h"

namespace fkb {

__device__ int gGemmTcTimeouts = 0;

namespace tc {

constexpr int kThreads = 192;
constexpr int kConvThreads = 128;                  // SPLIT: four converter warps after the six role warps
constexpr int kRows = 128;                         // MMA M: rows of (n, j) per tile

// v as a TF32 number (round to nearest, ties away; the low 13 mantissa bits come back zero)
__device__ __forceinline__ float tf32Round(float v) {
  unsigned u;
  asm("cvt.rna.tf32.f32 %0, %1;\n" : "=r"(u) : "f"(v));
  return __uint_as_float(u);
}

struct Args {
  float* Z; const float* Y; const float* F;
  long long fsP, fsQ;
  unsigned long long numChunks, B;
  unsigned numTiles;
  unsigned tilesPerChunk;                          // B >= 128: B / 128
  unsigned chunksPerTile;                          // B < 128: 128 / B;  B == 1: 128
  float alpha, beta;
  int epilogue;
};

__device__ __forceinline__ unsigned smemAddr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbarInit(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smemAddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarExpectTx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smemAddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbarArrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smemAddr(bar)) : "memory");
}
__device__ __forceinline__ bool mbarTryWait(unsigned long long* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok) : "r"(smemAddr(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// About two seconds at most; also gives up as soon as another role has raised the abort flag.
__device__ __forceinline__ bool waitBounded(unsigned long long* bar, unsigned parity, volatile int* abortFlag) {
  if (mbarTryWait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbarTryWait(bar, parity)) {
    if (*abortFlag) return false;
    if (clock64() - t0 > 4000000000ll) { *abortFlag = 1; atomicExch(&gGemmTcTimeouts, 1); return false; }
  }
  return true;
}

__device__ __forceinline__ void tmaLoad3D(void* dst, const CUtensorMap* tm, int c0, int c1, int c2,
                                          unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
      ::"r"(smemAddr(dst)), "l"(tm), "r"(c0), "r"(c1), "r"(c2), "r"(smemAddr(bar)) : "memory");
}
__device__ __forceinline__ void tmaLoad2D(void* dst, const CUtensorMap* tm, int c0, int c1, unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
      ::"r"(smemAddr(dst)), "l"(tm), "r"(c0), "r"(c1), "r"(smemAddr(bar)) : "memory");
}

// Shared-memory matrix descriptor of tcgen05.mma: start address, leading and stride byte
// offsets (all in 16-byte units), descriptor version 1, swizzle mode.
//   kSwz128: rows of 128 bytes, 16-byte units XOR (row % 8); used for K-major operands
//            (8 rows per atom; SBO = distance between 8-row groups).
//   kSwz128Atom32: rows of 128 bytes, 32-byte units XOR (row % 4); the only swizzle TF32
//            operands may have when their M / N index is the contiguous one.  A row is one k,
//            an atom is 4 rows: SBO = distance between atoms along k (512 bytes for packed
//            rows), LBO = distance between atoms of 32 elements along M / N.
constexpr unsigned long long kSwz128 = 2, kSwz128Atom32 = 1;
__device__ __forceinline__ unsigned long long smemDesc(unsigned addr, unsigned lboBytes, unsigned sboBytes,
                                                       unsigned long long swizzle) {
  return (unsigned long long)((addr & 0x3FFFFu) >> 4) | ((unsigned long long)(lboBytes >> 4) << 16) |
         ((unsigned long long)(sboBytes >> 4) << 32) | (1ull << 46) | (swizzle << 61);
}
// Instruction descriptor: D = fp32, A = B = TF32, M = 128, N = n; aMN / bMN: operand has its
// M / N index contiguous in shared memory.
__host__ __device__ constexpr unsigned instrDesc(int n, bool aMN, bool bMN) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((aMN ? 1u : 0u) << 15) | ((bMN ? 1u : 0u) << 16) |
         ((unsigned)(n >> 3) << 17) | ((unsigned)(kRows >> 4) << 24);
}
__device__ __forceinline__ void mmaTf32(unsigned tmemD, unsigned long long aDesc, unsigned long long bDesc,
                                        unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmemD), "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mmaCommit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smemAddr(bar)) : "memory");
}
__device__ __forceinline__ void tmemLoad32(unsigned taddr, unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmemLoadWait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void fenceBeforeSync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fenceAfterSync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// Stages of the X ring.  SPLIT stages are twice as large (hi and lo copies).
__host__ __device__ constexpr int stagesOf(int P, bool XT, bool SPLIT) {
  return SPLIT ? (XT ? 2 : 3) : (P == 64 ? 4 : 2);
}

// P = Q.  XT: trailing extent 1 (contraction index contiguous in X).  SPLIT: three TF32 products
// per fp32 product (see the head of the file).
template <int P, bool XT, bool SPLIT>
__global__ void __launch_bounds__(SPLIT ? kThreads + kConvThreads : kThreads, 1)
gemmTf32Kernel(const Args a, const __grid_constant__ CUtensorMap tmX) {
  static_assert(!SPLIT || P == 64, "the split variant exists for 64x64 factors");
  constexpr int Q = P;
  constexpr int NS = stagesOf(P, XT, SPLIT);                // stages of the X ring
  constexpr unsigned kStageBytes = (unsigned)P * kRows * 4u;
  constexpr unsigned kStageStride = SPLIT ? 2u * kStageBytes : kStageBytes;   // SPLIT: [hi][lo]
  constexpr unsigned kFactorBytes = (unsigned)P * Q * 4u;
  constexpr unsigned kAtomBytes = (unsigned)P * 128u;        // one [P][32 floats] atom column of an MN-major operand
  constexpr int kCols = 2 * Q;                              // TMEM columns: two accumulators

  extern __shared__ unsigned char smemRaw[];
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smemRaw + 1023) & ~(uintptr_t)1023);
  unsigned char* Fs = base;                                 // [Q/32][P][32] floats, swizzled (SPLIT: hi, then lo)
  unsigned char* stages = base + (size_t)kFactorBytes * (SPLIT ? 2 : 1);
  __shared__ __align__(8) unsigned long long fullBar[NS], emptyBar[NS], convBar[NS], accFull[2], accEmpty[2];
  __shared__ unsigned tmemBaseSlot;
  __shared__ int abortFlag;
  // XT epilogue: a thread holds 32 consecutive q of one chunk, but a coalesced store wants 32
  // consecutive q across the lanes of a warp; each epilogue warp transposes through its own
  // 32 x 33 scratch.
  __shared__ float xpose[XT ? 4 : 1][XT ? 32 * 33 : 1];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int i = 0; i < NS; i++) { mbarInit(&fullBar[i], 1); mbarInit(&emptyBar[i], 1); mbarInit(&convBar[i], kConvThreads / 32); }
    for (int i = 0; i < 2; i++) { mbarInit(&accFull[i], 1); mbarInit(&accEmpty[i], 4); }
    abortFlag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smemAddr(&tmemBaseSlot)), "r"(kCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  // factor -> shared memory: element (p, q) of atom column q / 32 sits in row p, 32-byte unit
  // ((q % 32) / 8) ^ (p % 4): the 128-byte swizzle with 32-byte atoms.
  for (int i = tid; i < P * Q; i += (int)blockDim.x) {
    int p, q;
    if (a.fsQ == 1) { p = i / Q; q = i % Q; } else { q = i / P; p = i % P; }     // walk the stored order
    const float v = a.F[(long long)p * a.fsP + (long long)q * a.fsQ];
    const unsigned off = (unsigned)(q >> 5) * kAtomBytes + (unsigned)p * 128u + ((((unsigned)(q & 31) >> 3) ^ ((unsigned)p & 3u)) << 5) +
                         ((unsigned)q & 7u) * 4u;
    if constexpr (SPLIT) {
      const float hi = tf32Round(v);
      *reinterpret_cast<float*>(Fs + off) = hi;
      *reinterpret_cast<float*>(Fs + kFactorBytes + off) = tf32Round(v - hi);
    } else {
      *reinterpret_cast<float*>(Fs + off) = v;
    }
  }
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");      // generic-proxy writes -> tensor-core reads
  fenceBeforeSync();
  __syncthreads();
  fenceAfterSync();
  const unsigned tmemBase = *(volatile unsigned*)&tmemBaseSlot;
  volatile int* abortP = &abortFlag;

  const unsigned first = blockIdx.x, step = gridDim.x;
  const unsigned myTiles = first < a.numTiles ? (a.numTiles - first + step - 1) / step : 0;

  if (warp == 0) {
    // ---- producer ------------------------------------------------------------------
    if (lane == 0) {
      unsigned t = first;
      for (unsigned it = 0; it < myTiles && !*abortP; it++, t += step) {
        const unsigned s = it % NS, ph = (it / NS) & 1u;
        if (!waitBounded(&emptyBar[s], ph ^ 1u, abortP)) break;
        mbarExpectTx(&fullBar[s], kStageBytes);
        unsigned char* dst = stages + (size_t)s * kStageStride;
        if constexpr (!XT) {
          // four atoms of [P][32 j]; one whose chunk lies past the end is zero-filled by the TMA
          unsigned n0, j0, atomsPerChunk;
          if (a.B >= 128) { n0 = t / a.tilesPerChunk; j0 = (t - n0 * a.tilesPerChunk) * 128u; atomsPerChunk = 4; }
          else { n0 = t * a.chunksPerTile; j0 = 0; atomsPerChunk = 4u / a.chunksPerTile; }
#pragma unroll
          for (unsigned at = 0; at < 4; at++)
            tmaLoad3D(dst + (size_t)at * kAtomBytes, &tmX, (int)(j0 + (at % atomsPerChunk) * 32u), 0,
                      (int)(n0 + at / atomsPerChunk), &fullBar[s]);
        } else {
#pragma unroll
          for (int sl = 0; sl < P / 32; sl++)
            tmaLoad2D(dst + (size_t)sl * (kRows * 128), &tmX, sl * 32, (int)(t * (unsigned)kRows), &fullBar[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issue -------------------------------------------------------------------
    if (lane == 0) {
      constexpr unsigned idesc = instrDesc(Q, !XT, true);
      for (unsigned it = 0; it < myTiles && !*abortP; it++) {
        const unsigned s = it % NS, ph = (it / NS) & 1u;
        const unsigned acc = it & 1u, aph = (it >> 1) & 1u;
        // SPLIT: the converters hand the stage over (they waited for its arrival themselves)
        if (!waitBounded(SPLIT ? &convBar[s] : &fullBar[s], ph, abortP)) break;
        if (!waitBounded(&accEmpty[acc], aph ^ 1u, abortP)) break;
        fenceAfterSync();
        const unsigned stageAddr = smemAddr(stages + (size_t)s * kStageStride);
        const unsigned fAddr = smemAddr(Fs);
        const unsigned tmemD = tmemBase + acc * (unsigned)Q;
        // one sweep over the contraction index: A operand at xAddr, factor copy at fBase
        auto sweep = [&](unsigned xAddr, unsigned fBase, bool fresh) {
#pragma unroll
          for (int ks = 0; ks < P / 8; ks++) {
            unsigned long long ad, bd;
            if constexpr (!XT) ad = smemDesc(xAddr + (unsigned)ks * 1024u, kAtomBytes, 512u, kSwz128Atom32);
            else ad = smemDesc(xAddr + (unsigned)(ks / 4) * (kRows * 128u) + (unsigned)(ks % 4) * 32u, 16u, 1024u, kSwz128);
            bd = smemDesc(fBase + (unsigned)ks * 1024u, kAtomBytes, 512u, kSwz128Atom32);
            mmaTf32(tmemD, ad, bd, idesc, (ks > 0 || !fresh) ? 1u : 0u);
          }
        };
        if constexpr (SPLIT) {
          sweep(stageAddr + kStageBytes, fAddr, true);              // lo * hi   (small terms first)
          sweep(stageAddr, fAddr + kFactorBytes, false);            // hi * lo
          sweep(stageAddr, fAddr, false);                           // hi * hi
        } else {
          sweep(stageAddr, fAddr, true);
        }
        mmaCommit(&emptyBar[s]);        // stage reusable once these MMAs have read it
        mmaCommit(&accFull[acc]);       // accumulator complete
      }
    }
  } else if (SPLIT && warp >= kThreads / 32) {
    // ---- converters (SPLIT): stage -> hi in place, lo behind it -------------------------------
    const int ct = tid - kThreads;
    for (unsigned it = 0; it < myTiles; it++) {
      const unsigned s = it % NS, ph = (it / NS) & 1u;
      bool ok = !*abortP && waitBounded(&fullBar[s], ph, abortP);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      float4* hiP = reinterpret_cast<float4*>(stages + (size_t)s * kStageStride);
      float4* loP = reinterpret_cast<float4*>(stages + (size_t)s * kStageStride + kStageBytes);
#pragma unroll 4
      for (int i = ct; i < (int)(kStageBytes / 16); i += kConvThreads) {
        const float4 v = hiP[i];
        float4 h, l;
        h.x = tf32Round(v.x); h.y = tf32Round(v.y); h.z = tf32Round(v.z); h.w = tf32Round(v.w);
        l.x = tf32Round(v.x - h.x); l.y = tf32Round(v.y - h.y); l.z = tf32Round(v.z - h.z); l.w = tf32Round(v.w - h.w);
        hiP[i] = h;
        loP[i] = l;
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // these writes -> tensor-core reads
      __syncwarp();
      if (lane == 0) mbarArrive(&convBar[s]);
    }
  } else {
    // ---- epilogue: warp w reads TMEM lanes [32*(w%4), +32) ---------------------------------
    const unsigned quarter = (unsigned)warp & 3u;
    const unsigned row = quarter * 32u + (unsigned)lane;             // row of the tile this thread owns
    const bool epi = a.epilogue != 0;
    const bool useY = epi && a.beta != 0.f && a.Y != nullptr;
    unsigned t = first;
    for (unsigned it = 0; it < myTiles; it++, t += step) {
      const unsigned acc = it & 1u, aph = (it >> 1) & 1u;
      bool ok = !*abortP && waitBounded(&accFull[acc], aph, abortP);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      fenceAfterSync();
      // where this thread's row goes
      unsigned long long n, zoff;
      bool live = true;
      if constexpr (!XT) {
        unsigned long long col;
        if (a.B >= 128) { const unsigned nn = t / a.tilesPerChunk, bt = t - nn * a.tilesPerChunk; n = nn; col = (unsigned long long)bt * 128u + row; }
        else { n = (unsigned long long)t * a.chunksPerTile + row / (unsigned)a.B; col = row % (unsigned)a.B; live = n < a.numChunks; }
        zoff = n * (unsigned long long)Q * a.B + col;                // + q * B
      } else {
        n = (unsigned long long)t * kRows + row; live = n < a.numChunks;
        zoff = n * (unsigned long long)Q;                            // + q
      }
#pragma unroll 1
      for (int c0 = 0; c0 < Q; c0 += 32) {
        unsigned r[32];
        tmemLoad32(tmemBase + ((quarter * 32u) << 16) + acc * (unsigned)Q + (unsigned)c0, r);
        tmemLoadWait();
        if (c0 + 32 == Q) {                                         // accumulator fully read: hand it back
          fenceBeforeSync();
          __syncwarp();
          if (lane == 0) mbarArrive(&accEmpty[acc]);
        }
        if (live) {
          if constexpr (!XT) {
#pragma unroll
            for (int i = 0; i < 32; i++) {
              const unsigned long long o = zoff + (unsigned long long)(c0 + i) * a.B;
              float v = __uint_as_float(r[i]);
              if (epi) { v = a.alpha * v; if (useY) v = fmaf(a.beta, a.Y[o], v); }
              a.Z[o] = v;
            }
          }
        }
        if constexpr (XT) {
          // rows of this warp: chunks n0 .. n0+31, columns c0 .. c0+31
          float* sc = xpose[quarter];
#pragma unroll
          for (int i = 0; i < 32; i++) sc[lane * 33 + i] = __uint_as_float(r[i]);
          __syncwarp();
          const unsigned long long nBase = (unsigned long long)t * kRows + quarter * 32u;
#pragma unroll 8
          for (int rr = 0; rr < 32; rr++) {
            const unsigned long long nn = nBase + (unsigned)rr;
            if (nn < a.numChunks) {
              const unsigned long long o = nn * (unsigned long long)Q + (unsigned)(c0 + lane);
              float v = sc[rr * 33 + lane];
              if (epi) { v = a.alpha * v; if (useY) v = fmaf(a.beta, a.Y[o], v); }
              a.Z[o] = v;
            }
          }
          __syncwarp();
        }
      }
    }
  }

  // ---- teardown: every role gets here (all waits are bounded); release TMEM ----------------
  fenceBeforeSync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    fenceAfterSync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmemBase), "r"(kCols) : "memory");
  }
}

// launches of the plain / split kernels by this process (tests check that the opt-in took effect)
static unsigned long long gLaunches[2] = {0, 0};

// cuTensorMapEncodeTiled from the driver, without linking libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encoder() {
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

template <int P, bool XT, bool SPLIT>
static fastKronError launchOne(const Pass& ps, const LaunchCtx& cx) {
  constexpr int NS = stagesOf(P, XT, SPLIT);
  const unsigned long long chunks = ps.M * ps.A, B = ps.B;
  EncodeTiledFn enc = encoder();
  if (!enc || chunks == 0 || chunks > 0x7FFFFFFFull || B > 0x7FFFFFFFull) return fastKronKernelNotFound;

  Args a;
  a.Z = (float*)cx.dst; a.Y = (const float*)cx.Y; a.F = (const float*)cx.F[0];
  a.fsP = cx.fsP; a.fsQ = cx.fsQ;
  a.numChunks = chunks; a.B = B;
  a.alpha = (float)cx.alpha; a.beta = (float)cx.beta; a.epilogue = ps.epilogue ? 1 : 0;
  a.tilesPerChunk = 1; a.chunksPerTile = 1;
  unsigned long long tiles;
  CUtensorMap tm;
  memset(&tm, 0, sizeof(tm));
  const cuuint32_t one4[4] = {1, 1, 1, 1};
  if (!XT) {
    const unsigned ch = B >= 128 ? 1u : (unsigned)(128 / B);          // chunks per tile
    if (B >= 128) { a.tilesPerChunk = (unsigned)(B / 128); tiles = chunks * a.tilesPerChunk; }
    else { a.chunksPerTile = ch; tiles = (chunks + ch - 1) / ch; }
    // view [chunks][P][B]; one box = one atom: P rows of 32 consecutive j of one chunk.  (Trailing
    // extents below 32 would need several chunks side by side in one 128-byte row; a TMA box whose
    // inner extent is below the swizzle span is not packed that way in shared memory, so those
    // passes stay on the fp32 kernel.)
    const cuuint64_t dims[3] = {B, (cuuint64_t)P, chunks};
    const cuuint64_t strides[2] = {B * 4, (cuuint64_t)P * B * 4};
    const cuuint32_t box[3] = {32, (cuuint32_t)P, 1};
    if (enc(&tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(cx.src), dims, strides, box, one4,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return fastKronKernelNotFound;
  } else {
    a.chunksPerTile = kRows;
    tiles = (chunks + kRows - 1) / kRows;
    const cuuint64_t dims[2] = {(cuuint64_t)P, chunks};
    const cuuint64_t strides[1] = {(cuuint64_t)P * 4};
    const cuuint32_t box[2] = {32, (cuuint32_t)kRows};
    if (enc(&tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(cx.src), dims, strides, box, one4,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return fastKronKernelNotFound;
  }
  if (tiles >= (1ull << 31)) return fastKronKernelNotFound;
  a.numTiles = (unsigned)tiles;

  const size_t smem = ((size_t)P * P * 4 + (size_t)NS * P * kRows * 4) * (SPLIT ? 2 : 1) + 1024;
  auto kern = gemmTf32Kernel<P, XT, SPLIT>;
  static bool attrDev[kMaxDevices] = {false};
  bool& attr = attrDev[currentDeviceSlot()];
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { cudaGetLastError(); return fastKronKernelNotFound; }
    attr = true;
  }
  unsigned grid = (unsigned)cx.smCount;
  if (grid > a.numTiles) grid = a.numTiles;
  kern<<<grid, SPLIT ? kThreads + kConvThreads : kThreads, smem, cx.stream>>>(a, tm);
  gLaunches[SPLIT ? 1 : 0]++;
  return cudaToFk(cudaGetLastError());
}

}  // namespace tc

// Eligible: fp32, P = Q in {64, 128}, dense operands aligned to 16 bytes, no redistribution,
// trailing extent 1, 32, 64 or a multiple of 128.  Anything else: fastKronKernelNotFound, and
// the caller runs the default fp32 kernel.
fastKronError launchGemmTf32(const Pass& ps, const LaunchCtx& cx) {
  if (cx.dt != DType::F32 || ps.nf != 1 || ps.xsB != 1 || ps.zsB != 1) return fastKronKernelNotFound;
  if (cx.scatter.parts > 0 || cx.pSplit != 0) return fastKronKernelNotFound;
  const uint32_t P = ps.P[0], Q = ps.Q[0];
  if (P != Q || (P != 64 && P != 128)) return fastKronKernelNotFound;
  if (((uintptr_t)cx.src | (uintptr_t)cx.dst | (uintptr_t)cx.Y) & 15) return fastKronKernelNotFound;
  const uint64_t B = ps.B;
  const bool xt = B == 1;
  if (!xt && !(B == 32 || B == 64 || B % 128 == 0)) return fastKronKernelNotFound;
  if (cx.tf32 == 3) {
    // fp32-level results from three TF32 products: 64x64 factors only (128x128 stays on the fp32 kernel)
    if (P != 64) return fastKronKernelNotFound;
    return xt ? tc::launchOne<64, true, true>(ps, cx) : tc::launchOne<64, false, true>(ps, cx);
  }
  if (P == 64) return xt ? tc::launchOne<64, true, false>(ps, cx) : tc::launchOne<64, false, false>(ps, cx);
  return xt ? tc::launchOne<128, true, false>(ps, cx) : tc::launchOne<128, false, false>(ps, cx);
}

unsigned long long gemmTcLaunches(int split) { return tc::gLaunches[split ? 1 : 0]; }

int gemmTcTimeouts() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, gGemmTcTimeouts, sizeof(int)) != cudaSuccess) { cudaGetLastError(); return -1; }
  return v;
}

}  // namespace fkb

// Non-zero if a bounded barrier wait of the TF32 kernel ever gave up in this process (tests).
extern "C" int fkbGemmTcTimeouts() { return fkb::gemmTcTimeouts(); }
// Launches of the TF32 (split = 0) or split-TF32 (split = 1) kernel by this process so far.
extern "C" unsigned long long fkbGemmTcLaunches(int split) { return fkb::gemmTcLaunches(split); }

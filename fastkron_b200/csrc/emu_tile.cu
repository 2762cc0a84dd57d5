// Host emulation of the shared-memory tile kernel.
//
// The contraction steps of kernel_tile.cuh are __host__ __device__ functions of
// (tile, factors, element count, thread id).  This program runs them on the CPU,
// thread id by thread id and step by step (a step boundary is where the kernel
// has its barrier), with the same super-tile bookkeeping as the kernel, and
// compares the result with a direct mode-by-mode contraction.  It validates the
// swizzled shared-memory indexing, the fibre ownership and the global offsets of
// every instantiated (type, P, NF, layout) without needing a GPU.
//
// usage: emu_tile            (exit code 0 = every configuration matches)
#include <cstdio>
#include <cstdlib>
#include <cmath>
#include <vector>

#include "kernel_tile.cuh"
#include "tile_table.h"

using namespace fkb;

template <typename T, int P, int NF, int BT, int J, bool SWZ>
struct HostChain {
  static void run(T* tile, const T* Fs, int E) {
    constexpr int S = ipow(P, NF - 1 - J) * BT;
    for (int tid = 0; tid < kTileThreads; tid++)
      stepDispatch<T, P, S, kTileThreads, SWZ>(tile, Fs + J * P * P, E, tid);
    HostChain<T, P, NF, BT, J - 1, SWZ>::run(tile, Fs, E);
  }
};
template <typename T, int P, int NF, int BT, bool SWZ>
struct HostChain<T, P, NF, BT, -1, SWZ> {
  static void run(T*, const T*, int) {}
};

static double urand(unsigned long long& s) {
  s = s * 6364136223846793005ull + 1442695040888963407ull;
  return (double)((s >> 11) & ((1ull << 53) - 1)) / 9007199254740992.0 * 2.0 - 1.0;
}

// SWZ = false: the linear tile layout of the TMA-staged kernels (wide fp32 only).
template <typename T, int P, int NF, bool WIDE, bool SWZ = true>
static int runOne(int R, unsigned long long chunks, unsigned long long Bmul) {
  constexpr int VEC = Vec16<T>::N;
  constexpr int BT = WIDE ? (int)(128 / sizeof(T)) : 1;
  constexpr int G = ipow(P, NF);
  constexpr int SUB = G * BT;
  const unsigned long long B = WIDE ? (unsigned long long)BT * Bmul : 1;
  const unsigned long long total = chunks * G * B;
  unsigned long long seed = 12345 + P * 131 + NF * 17 + (WIDE ? 7 : 0);
  std::vector<T> X(total), Z(total, T(0)), Fs((size_t)NF * P * P);
  for (auto& v : X) v = (T)urand(seed);
  for (auto& v : Fs) v = (T)urand(seed);

  // ---- emulated kernel ----
  const unsigned long long tilesPerChunk = WIDE ? B / BT : 1;
  const unsigned long long numSub = chunks * tilesPerChunk;
  std::vector<T> tile((size_t)R * SUB);
  std::vector<unsigned long long> bases(R);
  for (unsigned long long st0 = 0; st0 < numSub; st0 += R) {
    const int nsub = (numSub - st0 < (unsigned long long)R) ? (int)(numSub - st0) : R;
    for (int r = 0; r < nsub; r++) {
      const unsigned long long st = st0 + r;
      bases[r] = (st / tilesPerChunk) * (unsigned long long)G * B + (st % tilesPerChunk) * BT;
    }
    const int E = nsub * SUB, nvec = E / VEC;
    std::vector<int> written(E, 0);
    for (int v = 0; v < nvec; v++) {
      const unsigned idx = (unsigned)v * VEC;
      const unsigned long long goff = tileGlobalOffset<WIDE, SUB, BT>(bases.data(), st0 * G, idx, B);
      const unsigned ph = physIdx<T, SWZ>(idx);
      for (int i = 0; i < VEC; i++) { tile[ph + i] = X[goff + i]; written[ph + i]++; }
    }
    for (int i = 0; i < E; i++) if (written[i] != 1) { printf("swizzle is not a permutation\n"); return 1; }
    HostChain<T, P, NF, BT, NF - 1, SWZ>::run(tile.data(), Fs.data(), E);
    for (int v = 0; v < nvec; v++) {
      const unsigned idx = (unsigned)v * VEC;
      const unsigned long long goff = tileGlobalOffset<WIDE, SUB, BT>(bases.data(), st0 * G, idx, B);
      const unsigned ph = physIdx<T, SWZ>(idx);
      for (int i = 0; i < VEC; i++) Z[goff + i] = tile[ph + i];
    }
  }

  // ---- direct contraction: modes NF-1 .. 0 of [chunks][P..P][B] ----
  std::vector<double> cur(X.begin(), X.end()), nxt(total);
  for (int j = NF - 1; j >= 0; j--) {
    const unsigned long long S = (unsigned long long)ipow(P, NF - 1 - j) * B;   // stride of mode j
    const unsigned long long outer = total / (S * P);
    for (unsigned long long o = 0; o < outer; o++)
      for (unsigned long long s = 0; s < S; s++)
        for (int q = 0; q < P; q++) {
          double acc = 0;
          for (int p = 0; p < P; p++) acc += cur[o * S * P + p * S + s] * (double)Fs[(size_t)j * P * P + p * P + q];
          nxt[o * S * P + q * S + s] = acc;
        }
    cur.swap(nxt);
  }
  double maxErr = 0, maxRef = 0;
  for (unsigned long long i = 0; i < total; i++) {
    maxErr = fmax(maxErr, fabs((double)Z[i] - cur[i]));
    maxRef = fmax(maxRef, fabs(cur[i]));
  }
  const double tol = (sizeof(T) == 4 ? 2e-5 : 1e-13) * (maxRef > 1 ? maxRef : 1);
  const bool ok = maxErr <= tol;
  printf("%s P=%-2d NF=%d %s%s R=%-2d chunks=%llu B=%llu  maxErr=%.3g (ref %.3g)  %s\n",
         sizeof(T) == 4 ? "f32" : "f64", P, NF, WIDE ? "wide  " : "narrow", SWZ ? "" : " linear", R, chunks, B, maxErr, maxRef,
         ok ? "ok" : "MISMATCH");
  return ok ? 0 : 1;
}

template <typename T>
static int runAll() {
  int bad = 0;
  // R = 3 exercises several sub-tiles per super-tile and a ragged last super-tile.
#define EMU_N(p, n) if ((size_t)ipow(p, n) * sizeof(T) >= 16) { bad += runOne<T, p, n, false>(3, 7, 1); bad += runOne<T, p, n, false>(1, 2, 1); }
#define EMU_W(p, n) bad += runOne<T, p, n, true>(3, 2, 2); bad += runOne<T, p, n, true>(1, 1, 1); \
  if (sizeof(T) == 4) bad += runOne<T, p, n, true, false>(3, 2, 2);
  FKB_TILE_NARROW(EMU_N)
  FKB_TILE_WIDE(EMU_W)
#undef EMU_N
#undef EMU_W
  return bad;
}

int main() {
  int bad = runAll<float>() + runAll<double>();
  printf("%s (%d mismatching configurations)\n", bad ? "FAILED" : "PASSED", bad);
  return bad ? 1 : 0;
}

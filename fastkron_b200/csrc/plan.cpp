// Host planner: turns a GeMKM/GeKMM problem into a list of kernel passes.
//
// Mathematics.  With X viewed as a tensor [M][P1][P2]...[PN] (row-major over the
// columns), the product X (F1 (x) ... (x) FN) contracts mode i with factor Fi.
// The reference applies the factors from the last to the first and rotates the
// contracted mode to the front after every step (src/kmm/kmmalgo.cpp:172-214,
// src/kernels/cuda/global-store.cuh:248-256); after N steps the rotation is the
// identity.  This planner keeps the same factor order (so every partial sum is
// the same number) but, outside the forward variants, leaves each contracted
// mode in place: a pass maps [M][A][P...][B] to [M][A][Q...][B].  Loads and
// stores of a pass then have identical, contiguous access patterns and a block
// of columns owned by one GPU stays a block.  The forward variants must expose
// the reference's intermediate matrices, so they use the rotating layout.
//
// Buffers follow the reference's observable rules (src/kmm/kmmalgo.cpp:72-115):
// X and the factors are never written, the last pass writes Z, earlier passes
// alternate temp1/temp2, and without temp2 the result buffer doubles as scratch.

#include "fk_common.h"
#include "tile_table.h"
#include "gemm_table.h"
#include "tile_db.h"

#include <sstream>
#include <stdlib.h>

namespace fkb {

static bool isPow2(uint32_t v) { return v && !(v & (v - 1)); }

// Layout of a matrix with `cols` columns: element (m, c) at m*ms + c*cs.
struct Layout { int64_t ms, cs; };

static Layout inputLayout(const Problem& pr) {
  const int64_t K = (int64_t)pr.K();
  bool rowMajor = (pr.mm == MMType::MKM) ? (pr.opX == fastKronOp_N) : (pr.opX == fastKronOp_T);
  return rowMajor ? Layout{K, 1} : Layout{1, (int64_t)pr.M};
}
static Layout matLayout(const Problem& pr, uint64_t cols) {
  // Intermediates and the result share the result's orientation.
  return (pr.mm == MMType::MKM) ? Layout{(int64_t)cols, 1} : Layout{1, (int64_t)pr.M};
}

struct TileChoice { int nf; int tileB; int tileR; };

// Tuner hook (fastkron_b200/tune.py): cap on the fusion depth of every plan made by this
// process; 0 = none.
static int gMaxFuseOverride = 0;
void setMaxFuseOverride(int cap) { gMaxFuseOverride = cap > 0 ? cap : 0; }
// Measurement hook: plans made while it is set use the one-thread-per-output kernel for every
// pass (the correctness floor that the tiled kernels are compared with).
static bool gForceGeneric = false;
void setForceGenericOverride(bool on) { gForceGeneric = on; }

// How many equal factors to fuse for the shared-memory tile kernel.  `avail` equal factors are
// available; B is the (folded) trailing extent.  The choice is limited to the kernels that
// exist (tile_table.h) and whose tile fits: narrow tiles fuse while one [P^nf] block stays
// within 32 KB, wide tiles while [P^nf][128 bytes] stays within 64 KB.  Among the depths that
// fit, the swept table (tile_db.h: fusion depth per element type, P, layout and number of
// factors left) decides; shapes the sweep did not visit spread the factors evenly over the
// passes they need anyway (a pass's time grows with its depth, its memory traffic does not).
// Returns nf == 0 when no kernel fits.
static TileChoice chooseTile(DType dt, uint32_t P, int avail, uint64_t B, bool fusion, int maxFuse) {
  const size_t es = dtypeSize(dt);
  TileChoice c{0, 1, 0};
  const bool wide = B > 1;
  if (!fusion) avail = 1;
  if (avail > kMaxGroup) avail = kMaxGroup;
  const int left = avail;                       // factors of the run still to be applied
  if (maxFuse > 0 && maxFuse < avail) avail = maxFuse;
  if (gMaxFuseOverride > 0 && gMaxFuseOverride < avail) avail = gMaxFuseOverride;
  if (wide) {
    const uint64_t W = 128 / es;
    if (B % W != 0) return c;
    c.tileB = (int)W;
  }
  auto fits = [&](int nf) {
    if (!tileInTable(P, nf, wide)) return false;
    uint64_t g = 1; for (int k = 0; k < nf; k++) g *= P;
    return wide ? g * 128 <= 64 * 1024 : (g * es <= 32 * 1024 && (g * es) % 16 == 0);
  };
  int deepest = 0;
  for (int nf = avail; nf >= 1; nf--) if (fits(nf)) { deepest = nf; break; }
  if (deepest == 0) return c;
  c.nf = deepest;
  const int swept = tileFuseDepth(dt, P, wide, left);
  if (swept >= 1 && swept <= deepest && fits(swept)) { c.nf = swept; return c; }
  if (c.nf < left) {
    const int passes = (left + c.nf - 1) / c.nf;
    int even = (left + passes - 1) / passes;
    while (even >= 1 && !fits(even)) even--;
    if (even >= 1 && even < c.nf) c.nf = even;
  }
  return c;
}

fastKronError makePlan(const Problem& pr, const PlanOptions& optIn, Plan* out) {
  PlanOptions opt = optIn;
  if (gForceGeneric) opt.forceGeneric = true;
  if (!out || pr.N == 0 || pr.N > (uint32_t)kMaxFactors || pr.M == 0)
    return fastKronInvalidArgument;
  for (uint32_t i = 0; i < pr.N; i++)
    if (pr.P[i] == 0 || pr.Q[i] == 0) return fastKronInvalidArgument;

  out->passes.clear();
  // current mode sizes (P before contraction, Q after)
  uint64_t d[kMaxFactors];
  for (uint32_t i = 0; i < pr.N; i++) d[i] = pr.P[i];

  // factor element strides: (p,q) -> p*fsP + q*fsQ is resolved at launch time
  // from opF and the mm type; nothing to do here.

  Layout cur = inputLayout(pr);
  uint64_t curCols = pr.K();

  int i = (int)pr.N - 1;
  while (i >= 0) {
    Pass ps;
    const uint32_t P = pr.P[i], Q = pr.Q[i];
    uint64_t A = 1, B = 1;
    for (int j = 0; j < i; j++) A *= d[j];
    for (uint32_t j = i + 1; j < pr.N; j++) B *= d[j];

    int nf = 1;
    ps.kind = KernelKind::Generic;

    if (pr.forward) {
      // rotating layout: input [S][P], output [Q][S], S = cols/P
      const uint64_t S = curCols / P;
      const uint64_t outCols = S * Q;
      Layout nxt = matLayout(pr, outCols);
      ps.f0 = i; ps.nf = 1; ps.M = pr.M; ps.A = S; ps.B = 1;
      ps.P[0] = P; ps.Q[0] = Q;
      ps.xsM = cur.ms; ps.xsA = (int64_t)P * cur.cs; ps.xsG = cur.cs; ps.xsB = cur.cs;
      ps.zsM = nxt.ms; ps.zsA = nxt.cs; ps.zsG = (int64_t)S * nxt.cs; ps.zsB = nxt.cs;
      // the any-shape large-factor kernel takes arbitrary strides, so the rotating layout too
      if (!opt.forceGeneric && gemmAnyEligible(P, Q)) { ps.kind = KernelKind::Gemm; ps.variant = 3; }
      cur = nxt; curCols = outCols;
    } else {
      // how many factors could share a pass with factor i
      int same = 1;
      while (i - same >= 0 && pr.P[i - same] == P && pr.Q[i - same] == Q &&
             !(opt.isolateFirst && i - same == 0)) same++;

      uint64_t outColsOne = curCols / P * Q;
      Layout nxtOne = matLayout(pr, outColsOne);
      bool inRow  = (cur.cs == 1);
      bool outRow = (nxtOne.cs == 1);

      bool tileOk = !opt.forceGeneric && P == Q && isPow2(P) && P >= 2 && P <= 32 &&
                    inRow == outRow && opt.align >= 16;
      uint64_t Bf = B;
      if (tileOk && !inRow) Bf = B * pr.M;     // m is the fastest index: fold it into B
      if (tileOk) {
        TileChoice tc = chooseTile(pr.dt, P, same, Bf, opt.fusion, opt.maxFuse);
        if (tc.nf >= 1) {
          nf = tc.nf;
          ps.kind = KernelKind::Tile;
          ps.tileB = tc.tileB; ps.tileR = tc.tileR;
        }
      }
      // First pass of a problem whose input and result disagree on the contiguous index
      // (opX = T for MKM, opX = T for KMM): the transposing tile kernel moves [rows][G]
      // tiles; keep G*es <= 4 KB so that at least 16 rows fit a 64 KB tile.
      if (ps.kind == KernelKind::Generic && !opt.forceGeneric && inRow != outRow && B == 1 && P == Q &&
          isPow2(P) && P >= 2 && P <= 32 && opt.align >= 16) {
        const size_t es = dtypeSize(pr.dt);
        int avail = opt.fusion ? same : 1;
        if (avail > kMaxGroup) avail = kMaxGroup;
        if (opt.maxFuse > 0 && opt.maxFuse < avail) avail = opt.maxFuse;
        if (gMaxFuseOverride > 0 && gMaxFuseOverride < avail) avail = gMaxFuseOverride;
        for (int n = avail; n >= 1; n--) {
          if (!tileInTable(P, n, false)) continue;
          uint64_t g = 1; for (int k = 0; k < n; k++) g *= P;
          if (g * es <= 4096 && (g * es) % 16 == 0) {
            nf = n; ps.kind = KernelKind::Tile; ps.variant = inRow ? 1 : 2; ps.tileB = 1;
            break;
          }
        }
      }

      if (ps.kind == KernelKind::Generic && !opt.forceGeneric && inRow == outRow && opt.align >= 16) {
        // large factors: register-blocked contraction, one factor per pass
        const uint64_t Bg = inRow ? B : B * pr.M;
        if (gemmEligible(pr.dt, P, Q, Bg)) ps.kind = KernelKind::Gemm;
      }
      if (ps.kind == KernelKind::Generic && !opt.forceGeneric && gemmAnyEligible(P, Q)) {
        // every other shape the eligibility rule admits (64 elements or more, or at least 5x5): the any-shape kernel (variant 3),
        // whatever the strides, the alignment or the orientations of input and result
        ps.kind = KernelKind::Gemm;
        ps.variant = 3;
      }

      const int f0 = i - nf + 1;
      uint64_t Pg = 1, Qg = 1;
      for (int k = 0; k < nf; k++) { ps.P[k] = pr.P[f0 + k]; ps.Q[k] = pr.Q[f0 + k]; Pg *= ps.P[k]; Qg *= ps.Q[k]; }
      A = 1; for (int j = 0; j < f0; j++) A *= d[j];
      const uint64_t outCols = curCols / Pg * Qg;
      Layout nxt = matLayout(pr, outCols);
      ps.f0 = f0; ps.nf = nf; ps.M = pr.M; ps.A = A; ps.B = B;
      ps.xsM = cur.ms; ps.xsB = cur.cs; ps.xsG = (int64_t)B * cur.cs; ps.xsA = (int64_t)(Pg * B) * cur.cs;
      ps.zsM = nxt.ms; ps.zsB = nxt.cs; ps.zsG = (int64_t)B * nxt.cs; ps.zsA = (int64_t)(Qg * B) * nxt.cs;
      if (ps.kind != KernelKind::Generic && (ps.variant == 0 || ps.variant == 3) && !inRow && !outRow) {
        // folded view: [1][A][G][B*M], unit stride along the folded index
        ps.M = 1; ps.B = B * pr.M;
        ps.xsM = 0; ps.zsM = 0;
        ps.xsB = 1; ps.zsB = 1;
        ps.xsG = (int64_t)ps.B; ps.zsG = (int64_t)ps.B;
        ps.xsA = (int64_t)(Pg * ps.B); ps.zsA = (int64_t)(Qg * ps.B);
      }
      for (int k = 0; k < nf; k++) d[f0 + k] = pr.Q[f0 + k];
      cur = nxt; curCols = outCols;
    }
    out->passes.push_back(ps);
    i -= ps.nf;
  }

  // ---- buffer assignment -------------------------------------------------
  const size_t n = out->passes.size();
  out->usesT2 = false;
  for (size_t k = 0; k < n; k++) {
    Pass& ps = out->passes[k];
    const bool last = (k + 1 == n);
    ps.epilogue = last;
    if (pr.forward) {
      ps.src = (k == 0) ? Buf::X : out->passes[k - 1].dst;
      // the pass consuming factor f writes Intermediates[f-1]; the last writes Z
      ps.dst = last ? Buf::Z : (Buf)((int)Buf::I0 + (ps.f0 - 1));
      continue;
    }
    Buf seq[2];
    if (opt.haveT2) { seq[0] = Buf::T1; seq[1] = Buf::T2; }
    else if (n % 2 == 1) { seq[0] = Buf::Z; seq[1] = Buf::T1; }
    else { seq[0] = Buf::T1; seq[1] = Buf::Z; }
    ps.src = (k == 0) ? Buf::X : out->passes[k - 1].dst;
    ps.dst = last ? Buf::Z : seq[k & 1];
    if (!last && (ps.dst == Buf::T2 || ps.dst == Buf::Z)) out->usesT2 = true;
  }
  return fastKronSuccess;
}

std::string Plan::describe() const {
  std::ostringstream os;
  static const char* kn[] = {"generic", "tile", "gemm"};
  auto bn = [](Buf b) -> std::string {
    switch (b) { case Buf::X: return "X"; case Buf::T1: return "T1"; case Buf::T2: return "T2";
                 case Buf::Z: return "Z"; default: return "I" + std::to_string((int)b - (int)Buf::I0); }
  };
  for (size_t k = 0; k < passes.size(); k++) {
    const Pass& p = passes[k];
    os << "pass" << k << " " << kn[(int)p.kind] << " f[" << p.f0 << ".." << (p.f0 + p.nf - 1) << "]"
       << " P=" << p.P[0] << " Q=" << p.Q[0] << " M=" << p.M << " A=" << p.A << " B=" << p.B
       << " x(" << p.xsM << "," << p.xsA << "," << p.xsG << "," << p.xsB << ")"
       << " z(" << p.zsM << "," << p.zsA << "," << p.zsG << "," << p.zsB << ")"
       << " tileB=" << p.tileB << " tileR=" << p.tileR << " var=" << p.variant
       << " " << bn(p.src) << "->" << bn(p.dst) << (p.epilogue ? " epi" : "") << "\n";
  }
  return os.str();
}

}  // namespace fkb

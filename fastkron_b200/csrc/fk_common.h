// Shared host-side types of the engine: problem description, pass description,
// error plumbing.  No CUDA types appear here so that the planner can be compiled
// and unit-tested without a device.
#pragma once

#include <stdint.h>
#include <stddef.h>
#include <vector>
#include <string>

#include "fastkron.h"

namespace fkb {

constexpr int kMaxFactors = 64;      // the reference's limit (src/kmm/kmmalgo.h:336)
constexpr int kMaxGroup   = 8;       // most factors one kernel launch applies

enum class DType : int { F32 = 0, F64 = 1 };
enum class MMType : int { MKM = 0, KMM = 1 };

inline size_t dtypeSize(DType t) { return t == DType::F32 ? 4 : 8; }

// Which device kernel family executes a pass.
enum class KernelKind : int {
  Generic = 0,   // one thread per output element, arbitrary strides, any P/Q
  Tile    = 1,   // small power-of-two square factors fused in shared memory
  Gemm    = 2    // large factors, register-blocked FFMA/DFMA contraction
};

// Logical buffer ids a pass reads from / writes to.
enum class Buf : int { X = 0, T1 = 1, T2 = 2, Z = 3, I0 = 4 /* I0+k: forward intermediate k */ };

// The complete user-visible problem (one entry of a batch).
struct Problem {
  MMType   mm   = MMType::MKM;
  DType    dt   = DType::F32;
  uint32_t M    = 0;
  uint32_t N    = 0;
  uint32_t P[kMaxFactors] = {0};
  uint32_t Q[kMaxFactors] = {0};
  fastKronOp opX = fastKronOp_N;
  fastKronOp opF = fastKronOp_N;
  uint32_t batch = 1;
  bool     forward = false;     // keep all intermediates in the reference's layout

  uint64_t K() const { uint64_t k = 1; for (uint32_t i = 0; i < N; i++) k *= P[i]; return k; }
  uint64_t L() const { uint64_t l = 1; for (uint32_t i = 0; i < N; i++) l *= Q[i]; return l; }
  // columns of the matrix obtained after factors N-1 .. i have been applied
  uint64_t colsAfter(uint32_t i) const {
    uint64_t c = 1;
    for (uint32_t j = 0; j < i; j++) c *= P[j];
    for (uint32_t j = i; j < N; j++) c *= Q[j];
    return c;
  }
  uint64_t maxIntermediateCols() const {
    uint64_t best = 0;
    for (uint32_t i = 0; i < N; i++) { uint64_t c = colsAfter(i); if (c > best) best = c; }
    return best;
  }
};

// One kernel launch.  The input is viewed as a tensor [M][A][G...][B] and the
// output as [M][A][H...][B], where G... are the `nf` modes being contracted
// (sizes P of factors f0 .. f0+nf-1, f0 slowest) and H... their Q sizes.
// Offsets are in elements:
//   in (m,a,g,b)  = m*xsM + a*xsA + g*xsG + b*xsB      g = mixed radix over P's
//   out(m,a,h,b)  = m*zsM + a*zsA + h*zsG + b*zsB      h = mixed radix over Q's
// Factor i element (p,q) = F_i[p*fsP + q*fsQ].
struct Pass {
  KernelKind kind = KernelKind::Generic;
  int      f0 = 0, nf = 1;
  uint64_t M = 0, A = 1, B = 1;
  uint32_t P[kMaxGroup] = {0}, Q[kMaxGroup] = {0};
  int64_t  xsM = 0, xsA = 0, xsG = 0, xsB = 0;
  int64_t  zsM = 0, zsA = 0, zsG = 0, zsB = 0;
  Buf      src = Buf::X, dst = Buf::Z;
  bool     epilogue = false;    // apply alpha / beta*Y (Y laid out like the output)
  // tuning knobs chosen by the planner for Tile / Gemm kernels
  int      tileB = 1;           // trailing-dimension elements per tile
  int      tileR = 0;           // Tile kernels: super-tile size in KB (0 = the launcher's default)
  int      variant = 0;         // kernel-specific variant id
  uint64_t Pg() const { uint64_t g = 1; for (int i = 0; i < nf; i++) g *= P[i]; return g; }
  uint64_t Qg() const { uint64_t g = 1; for (int i = 0; i < nf; i++) g *= Q[i]; return g; }
};

struct Plan {
  std::vector<Pass> passes;
  bool usesT2 = false;          // plan touches the second temporary (or Z as scratch)
  std::string describe() const;
};

struct PlanOptions {
  bool fusion = true;           // fastKronOptionsUseFusion
  bool haveT2 = true;           // caller supplied temp2
  bool forceGeneric = false;    // debugging / parity cross-check
  bool isolateFirst = false;    // factor 0 gets a pass of its own (multi-GPU: that pass redistributes)
  int  maxFuse = 0;             // cap on the factors one tile pass fuses (0 = none); fastKronOptionsTune sweeps it
  size_t smemBudget = 200 * 1024;
  // pointer alignment of X / Z / temps in bytes (vector kernels need 16)
  int  align = 16;
};

// Build the list of passes for a problem.  Pure host code.
fastKronError makePlan(const Problem& pr, const PlanOptions& opt, Plan* out);
// Process-wide cap on the fusion depth (the offline tuner's hook; 0 = none).
void setMaxFuseOverride(int cap);
// Process-wide "every pass on the one-thread-per-output kernel" (measurement / cross-check hook).
void setForceGenericOverride(bool on);

}  // namespace fkb

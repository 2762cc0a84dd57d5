// Which large-factor (GEMM-style) kernels exist; shared by the planner and the
// launcher.  One entry per (element type, P, Q); TJ is the tile width along the
// trailing index.
#pragma once

#include <stdint.h>
#include "fk_common.h"

namespace fkb {

inline int gemmTileJ(DType) { return 128; }

inline bool gemmShapeInTable(DType dt, uint32_t P, uint32_t Q) {
  if (dt == DType::F32) return (P == 64 && Q == 64) || (P == 128 && Q == 128);
  return P == 64 && Q == 64;
}

// B is the trailing extent of the dense row-major view [chunks][P][B].
inline bool gemmEligible(DType dt, uint32_t P, uint32_t Q, uint64_t B) {
  if (!gemmShapeInTable(dt, P, Q)) return false;
  const uint64_t vec = 16 / dtypeSize(dt), TJ = (uint64_t)gemmTileJ(dt);
  if (B == 1) return true;
  if (B % vec != 0) return false;
  return (B % TJ == 0) || (TJ % B == 0);
}

// The any-shape large-factor kernel (kernel_gemm_any.cu) takes every single-factor pass whose
// factor has at least 64 elements, and smaller factors from 5x5 on (measured on B200 against the
// one-thread-per-output kernel: 6x6 and 7x7 passes 1.8-1.9 times faster, 5x5 1.2 times, 3x3
// slower); what is left stays with the tile kernels or, for the few shapes those do not cover,
// with the one-thread-per-output kernel.  The measurement hook fkbSetAnyMinElems replaces the
// rule by "P*Q >= n" (process-wide; 0 restores the rule).
inline int gAnyMinElems = 0;
inline bool gemmAnyEligible(uint32_t P, uint32_t Q) {
  if (gAnyMinElems > 0) return (uint64_t)P * Q >= (uint64_t)gAnyMinElems;
  return (uint64_t)P * Q >= 64 || (P >= 5 && Q >= 5);
}

}  // namespace fkb

// The set of shared-memory tile kernels that exist, shared by the planner (which
// may only choose from it) and by the kernel file (which instantiates it).
//
// A tile kernel is identified by (element type, P, NF, wide):
//   P    factor size (square, power of two, 2..32)
//   NF   number of equal factors fused in one pass
//   wide false: the trailing extent B is 1 and a sub-tile is one contiguous block
//               of P^NF elements; true: B > 1 and a sub-tile is [P^NF][W] with
//               W = 128 bytes of elements along the trailing index.
#pragma once

#include <stdint.h>
#include <stddef.h>

namespace fkb {

// X(P, NF) lists per layout; the same lists serve float and double.
#define FKB_TILE_NARROW(X) \
  X(2, 1) X(2, 2) X(2, 4) X(2, 8) \
  X(4, 1) X(4, 2) X(4, 3) X(4, 4) X(4, 6) \
  X(8, 1) X(8, 2) X(8, 3) X(8, 4) \
  X(16, 1) X(16, 2) X(16, 3) \
  X(32, 1) X(32, 2)

#define FKB_TILE_WIDE(X) \
  X(2, 1) X(2, 2) X(2, 4) X(2, 8) \
  X(4, 1) X(4, 2) X(4, 3) X(4, 4) \
  X(8, 1) X(8, 2) X(8, 3) \
  X(16, 1) X(16, 2) \
  X(32, 1)

inline bool tileInTable(uint32_t P, int nf, bool wide) {
#define FKB_CHK(p, n) if (P == p && nf == n) return true;
  if (wide) { FKB_TILE_WIDE(FKB_CHK) } else { FKB_TILE_NARROW(FKB_CHK) }
#undef FKB_CHK
  return false;
}

// Largest table entry with at most `avail` factors.
inline int tileBestNf(uint32_t P, int avail, bool wide) {
  for (int nf = avail; nf >= 1; nf--)
    if (tileInTable(P, nf, wide)) return nf;
  return 0;
}

}  // namespace fkb

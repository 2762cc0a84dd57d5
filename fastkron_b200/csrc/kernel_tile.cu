// Dispatcher of the shared-memory tile kernels (instantiated in
// kernel_tile_{f32,f64}_{narrow,wide}.cu).
#include "kernels.h"
#include "tile_table.h"
#include "tile_db.h"

namespace fkb {

template <typename T, bool WIDE>
fastKronError launchTileTW(const Pass& ps, const LaunchCtx& cx);
extern template fastKronError launchTileTW<float, false>(const Pass&, const LaunchCtx&);
extern template fastKronError launchTileTW<float, true>(const Pass&, const LaunchCtx&);
extern template fastKronError launchTileTW<double, false>(const Pass&, const LaunchCtx&);
extern template fastKronError launchTileTW<double, true>(const Pass&, const LaunchCtx&);

template <typename T, int TR>
fastKronError launchTileTr(const Pass& ps, const LaunchCtx& cx);
extern template fastKronError launchTileTr<float, 1>(const Pass&, const LaunchCtx&);
extern template fastKronError launchTileTr<float, 2>(const Pass&, const LaunchCtx&);
extern template fastKronError launchTileTr<double, 1>(const Pass&, const LaunchCtx&);
extern template fastKronError launchTileTr<double, 2>(const Pass&, const LaunchCtx&);

int tileTmaTimeouts();     // kernel_tile_f32_wide.cu, the only unit with TMA-staged tile kernels

bool tileSupported(DType dt, uint32_t P, int nf, int tileB) {
  (void)dt;
  return tileInTable(P, nf, tileB > 1);
}

fastKronError launchTile(const Pass& ps, const LaunchCtx& cx) {
  // The kernel assumes dense row-major [chunks][G][B] on both sides, unit
  // trailing stride, equal square factors and 16-byte aligned operands.
  const size_t es = dtypeSize(cx.dt);
  const bool wide = ps.B > 1;
  for (int k = 0; k < ps.nf; k++)
    if (ps.P[k] != ps.P[0] || ps.Q[k] != ps.P[0]) return fastKronKernelNotFound;
  if (ps.variant == 1 || ps.variant == 2) {
    // transposing first pass: only the row-major side needs 16-byte alignment
    if (wide) return fastKronKernelNotFound;
    const void* rowSide = ps.variant == 1 ? cx.src : cx.dst;
    if (((uintptr_t)rowSide & 15) || (ps.variant == 2 && ((uintptr_t)cx.Y & 15))) return fastKronKernelNotFound;
    if (cx.dt == DType::F32)
      return ps.variant == 1 ? launchTileTr<float, 1>(ps, cx) : launchTileTr<float, 2>(ps, cx);
    return ps.variant == 1 ? launchTileTr<double, 1>(ps, cx) : launchTileTr<double, 2>(ps, cx);
  }
  if (ps.xsB != 1 || ps.zsB != 1) return fastKronKernelNotFound;
  const uint64_t W = 128 / es;
  if (wide && ps.B % W != 0) return fastKronKernelNotFound;
  if (((uintptr_t)cx.src | (uintptr_t)cx.dst | (uintptr_t)cx.Y) & 15) return fastKronKernelNotFound;
  if (cx.dt == DType::F32)
    return wide ? launchTileTW<float, true>(ps, cx) : launchTileTW<float, false>(ps, cx);
  return wide ? launchTileTW<double, true>(ps, cx) : launchTileTW<double, false>(ps, cx);
}

}  // namespace fkb

// Tuner hook (fastkron_b200/tune.py): force one (tile KB, ring depth, CTAs per SM, TMA) choice on
// every tile kernel launched by this process; kb = 0 returns to the swept table.
extern "C" void fkbSetTileTuning(int kb, int nbuf, int minb, int tma) {
  fkb::TileTune& o = fkb::tileTuneOverride();
  o.kb = kb; o.nbuf = nbuf == 1 ? 1 : 2; o.minb = minb; o.tma = tma;
}

// Non-zero if a bounded wait on a tile barrier of the TMA-staged tile kernels ever gave up
// in this process on the current device (tests).
extern "C" int fkbTileTmaTimeouts() { return fkb::tileTmaTimeouts(); }

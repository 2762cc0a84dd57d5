// Generic sliced-multiply pass: one thread per output element, arbitrary
// element strides on every index, any factor shape.  It is the correctness
// floor of the engine: every pass the specialised kernels do not cover (odd
// factor sizes, rotating layouts of the forward variants, transposing first
// passes) runs here.  All offsets are 64-bit.
//
// Semantics of one pass (same arithmetic as one step of the reference's
// sliced multiply, src/kernels/cuda/kernel.cuh:53-224 with the output index of
// src/kernels/cuda/global-store.cuh:248-256, expressed with explicit strides):
//   out[m,a,q,b] = sum_p in[m,a,p,b] * F[p,q]            (p ascending)
//   out = alpha*out + beta*Y  on the pass that consumes factor 0.

#include "kernels.h"

namespace fkb {

struct GenericDims {
  // the four enumerated indices, fastest first; the q index has xs == 0
  unsigned long long size[4];
  long long xs[4];
  long long zs[4];
  int qDim;                 // which of the four is q
  int dimId[4];             // 0 = m, 1 = a, 2 = q, 3 = b for each enumerated index
  unsigned long long chunkA; // extent of the a index (chunk n = m*chunkA + a)
};

template <typename T>
struct GenericArgs {
  const T* X; const T* F; T* Z; const T* Y;
  GenericDims d;
  unsigned int P;
  long long xsP;            // input stride of the contracted index
  long long fsP, fsQ;
  T alpha, beta;
  int epilogue;
  unsigned long long total;
  Scatter sc;
  unsigned batch;                          // entries of a strided batch, one per blockIdx.y step
  unsigned long long bsX, bsZ, bsY, bsF;
};

template <typename T>
__global__ void __launch_bounds__(256) genericPassKernel(const GenericArgs<T> a) {
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  for (unsigned bt = blockIdx.y; bt < a.batch; bt += gridDim.y)
  for (unsigned long long idx = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
       idx < a.total; idx += stride) {
    unsigned long long rem = idx;
    long long xoff = 0, zoff = 0;
    unsigned long long q = 0;
    unsigned long long coord[4] = {0, 0, 0, 0};
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const unsigned long long c = rem % a.d.size[k];
      rem /= a.d.size[k];
      xoff += (long long)c * a.d.xs[k];
      zoff += (long long)c * a.d.zs[k];
      if (k == a.d.qDim) q = c;
      coord[a.d.dimId[k]] = c;
    }
    const T* xp = a.X + (unsigned long long)bt * a.bsX + xoff;
    const T* fp = a.F + (unsigned long long)bt * a.bsF + (long long)q * a.fsQ;
    const T* yp = a.Y ? a.Y + (unsigned long long)bt * a.bsY : nullptr;
    T* zp = a.Z + (unsigned long long)bt * a.bsZ;
    T acc = T(0);
    for (unsigned int p = 0; p < a.P; p++)
      acc = fma(__ldg(xp + (long long)p * a.xsP), __ldg(fp + (long long)p * a.fsP), acc);
    if (a.epilogue) {
      acc = a.alpha * acc;
      if (a.beta != T(0) && yp != nullptr) acc = fma(a.beta, yp[zoff], acc);
    }
    if (a.sc.parts > 0) {
      // chunk index n = m*A + a of the pass; split it the way the scatter wants it
      T* base = (T*)a.sc.base[q / a.sc.qPer];
      const unsigned long long n = coord[0] * a.d.chunkA + coord[1];
      const long long off = (long long)(n / a.sc.aLoc) * a.sc.sM + (long long)(n % a.sc.aLoc) * a.sc.sA +
                            (long long)(q % a.sc.qPer) * a.sc.sQ + a.sc.zOff + (long long)coord[3];
      base[off] = acc;
    } else {
      zp[zoff] = acc;
    }
  }
}

template <typename T>
static fastKronError launchGenericT(const Pass& ps, const LaunchCtx& cx) {
  if (ps.nf != 1) return fastKronKernelNotFound;
  GenericArgs<T> a;
  a.X = (const T*)cx.src; a.F = (const T*)cx.F[0]; a.Z = (T*)cx.dst; a.Y = (const T*)cx.Y;
  a.P = ps.P[0]; a.xsP = ps.xsG; a.fsP = cx.fsP; a.fsQ = cx.fsQ;
  a.alpha = (T)cx.alpha; a.beta = (T)cx.beta; a.epilogue = ps.epilogue ? 1 : 0;

  // enumerate the output indices in order of ascending output stride so that
  // neighbouring threads write neighbouring addresses
  struct D { unsigned long long n; long long xs, zs; int isQ; int id; };
  D ds[4] = { {ps.M, ps.xsM, ps.zsM, 0, 0}, {ps.A, ps.xsA, ps.zsA, 0, 1},
              {ps.Q[0], 0, ps.zsG, 1, 2},   {ps.B, ps.xsB, ps.zsB, 0, 3} };
  a.sc = cx.scatter;
  a.d.chunkA = ps.A;
  for (int i = 0; i < 4; i++)
    for (int j = i + 1; j < 4; j++) {
      auto key = [](const D& d) { return d.n == 1 ? (long long)(1ll << 62) : (d.zs < 0 ? -d.zs : d.zs); };
      if (key(ds[j]) < key(ds[i])) { D t = ds[i]; ds[i] = ds[j]; ds[j] = t; }
    }
  a.d.qDim = 0;
  a.total = 1;
  for (int i = 0; i < 4; i++) {
    a.d.size[i] = ds[i].n; a.d.xs[i] = ds[i].xs; a.d.zs[i] = ds[i].zs;
    if (ds[i].isQ) a.d.qDim = i;
    a.d.dimId[i] = ds[i].id;
    a.total *= ds[i].n;
  }
  if (a.total == 0) return fastKronSuccess;
  a.batch = cx.batch; a.bsX = cx.bsX; a.bsZ = cx.bsZ; a.bsY = cx.bsY; a.bsF = cx.bsF[0];
  if (a.sc.parts > 0 && a.batch > 1) return fastKronKernelNotFound;
  unsigned long long blocks = (a.total + 255) / 256;
  const unsigned long long cap = (unsigned long long)cx.smCount * 64;
  if (blocks > cap) blocks = cap;
  const dim3 grid((unsigned)blocks, a.batch < 65535u ? a.batch : 65535u);
  genericPassKernel<T><<<grid, 256, 0, cx.stream>>>(a);
  return cudaToFk(cudaGetLastError());
}

fastKronError launchGeneric(const Pass& ps, const LaunchCtx& cx) {
  return cx.dt == DType::F32 ? launchGenericT<float>(ps, cx) : launchGenericT<double>(ps, cx);
}

}  // namespace fkb

// Multi-GPU GeMKM: the entry points of include/fastkronMg.h and, for hosts that run one
// process per GPU, the same schedule per rank (fkbMgPipe*).
//
// Distribution (same as the reference, src/handle/distrib_handle.cu:52-414 and
// src/handle/handle.cpp:411-416): GPU (r, c) of a gpusInM x gpusInK grid owns rows
// [r*M/GM, ...) and columns [c*K/GK, ...) of X and of the result; factors are replicated.
// Rows need no communication.  Columns do: with X as the tensor [M][P1][P2]...[PN], a
// column block is a range of the leading index p1.
//
//   phase 1  every GPU contracts modes N..2 of its block [M][P1/GK][P2..PN] locally.  The
//            pass that applies factor 2 hands its output over: row (m, p1, q2) belongs to
//            GPU q2 / (Q2/GK), which thereby receives [M][P1][Q2/GK][Q3..QN] -- all of p1,
//            a slice of q2.  (The all-to-all of the reference: ncclSend/ncclRecv plus pack and
//            unpack kernels, distrib_handle.cu:276-347, or its P2P store variant,
//            src/kernels/cuda/global-store.cuh:1-25.)
//   phase 2  every GPU contracts mode 1 of what it received; row (m, q1) belongs to GPU
//            q1 / (Q1/GK) at its canonical place [M][Q1/GK][Q2][Q3..QN].
//
// Two exchanges are the minimum for a column-sharded input and output.  Two transports:
//   fused   the producing kernel stores every output row straight into the owner's buffer
//           (128-bit peer stores).  Any factor shape.
//   staged  the producing kernel fills per-destination blocks in local memory and the copy
//           engines ship them (cudaMemcpyAsync / cudaMemcpy2DAsync on side streams), so the
//           NVLink traffic needs no SM.  Needs the large-factor kernel for phase 2.
// The rows are cut into `parts` independent slices that run out of phase: while one slice's
// blocks travel, another slice computes (rows never communicate, so a slice is a complete
// small problem).  Enqueue order on the one compute stream of a GPU:
//   P1(0), P1(1), P2(0), P1(2), P2(1), ..., P2(parts-1).
//
// Ordering between GPUs never happens inside a kernel.  One process driving all GPUs
// (fastKronMgSGEMM) uses CUDA events across devices.  One process per GPU cannot (an event
// wait captures whatever record the waiting process has seen, and processes do not see each
// other's calls), so there every rank owns a small array of 32-bit sequence flags in device
// memory that its peers map through CUDA IPC: a sender's stream writes the call's sequence
// number into the receiver's flag after its copies (cuStreamWriteValue32), the receiver's
// stream waits for it (cuStreamWaitValue32) -- stream-ordered memory operations executed by
// the GPU's front end, no SM, no kernel, no collective library.  No TMA multicast anywhere.
//
// Requirements: N >= 2 when GK > 1, and GK divides P1, Q1 and Q2 (the reference has the
// analogous divisibility rules, src/kmm/kmmalgo.cpp:51-70).  fp32, row-major, opX = opF = N
// only, like the reference (distrib_handle.cu:247-250).

#include "engine.h"
#include "gemm_table.h"
#include "fastkronMg.h"

#include <cuda.h>

#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <memory>
#include <vector>

namespace fkb {

// ---- one rank's view of the problem -------------------------------------------------------

struct MgRank {
  int g = 0, gk = 1;                      // column rank, column-group size
  uint32_t M = 0, N = 0;                  // local rows, number of factors
  const uint32_t* Ps = nullptr;           // global factor shapes
  const uint32_t* Qs = nullptr;
  cudaStream_t stream = nullptr;
  int smCount = 148;
};

static fastKronError mgCheck(const MgRank& r) {
  if (r.gk < 1 || r.gk > kMaxParts || r.g < 0 || r.g >= r.gk || r.N == 0 || r.N > (uint32_t)kMaxFactors || r.M == 0)
    return fastKronInvalidArgument;
  if (r.gk > 1) {
    if (r.N < 2) return fastKronInvalidKMMProblem;
    if (r.Ps[0] % r.gk || r.Qs[0] % r.gk || r.Qs[1] % r.gk) return fastKronInvalidKMMProblem;
  }
  return fastKronSuccess;
}

static uint64_t prodQ(const MgRank& r, uint32_t from) {
  uint64_t b = 1;
  for (uint32_t i = from; i < r.N; i++) b *= r.Qs[i];
  return b;
}

// Scatter descriptors (pure arithmetic; also exported for the host-side tests).
static void mgScatter1(const MgRank& r, Scatter* sc) {
  const uint64_t p1loc = r.Ps[0] / r.gk, q2loc = r.Qs[1] / r.gk, B = prodQ(r, 2);
  sc->parts = r.gk; sc->qPer = q2loc; sc->aLoc = p1loc;
  sc->sM = (long long)(r.Ps[0] * q2loc * B); sc->sA = (long long)(q2loc * B); sc->sQ = (long long)B;
  sc->zOff = (long long)(r.g * p1loc * q2loc * B);
}
static void mgScatter2(const MgRank& r, Scatter* sc) {
  const uint64_t q1loc = r.Qs[0] / r.gk, q2loc = r.Qs[1] / r.gk, B = prodQ(r, 2);
  sc->parts = r.gk; sc->qPer = q1loc; sc->aLoc = 1;
  sc->sM = (long long)(q1loc * r.Qs[1] * B); sc->sA = 0; sc->sQ = (long long)(r.Qs[1] * B);
  sc->zOff = (long long)(r.g * q2loc * B);
}

// Phase 1: modes N..2 of the local block; the last pass hands its rows to bases[d].
// packed == false: bases[d] is rank d's receive area laid out [M][P1][Q2/G][B] (fused
// transport).  packed == true: bases[d] is a block that holds only this rank's rows,
// [M][P1/G][Q2/G][B] (staged transport).
static fastKronError mgPhase1(Engine* e, const MgRank& r, const float* x, const float* const* Fs, float* t1,
                              float* t2, void* const bases[], bool packed) {
  fastKronError err = mgCheck(r);
  if (err != fastKronSuccess) return err;
  const uint32_t p1loc = r.Ps[0] / r.gk;
  Problem lp;
  lp.mm = MMType::MKM; lp.dt = DType::F32; lp.N = r.N - 1;
  const uint64_t rows = (uint64_t)r.M * p1loc;
  if (rows >= (1ull << 32)) return fastKronInvalidKMMProblem;
  lp.M = (uint32_t)rows;
  for (uint32_t i = 1; i < r.N; i++) { lp.P[i - 1] = r.Ps[i]; lp.Q[i - 1] = r.Qs[i]; }
  PlanOptions po;
  po.isolateFirst = true; po.haveT2 = true; po.align = 16;
  Plan plan;
  err = makePlan(lp, po, &plan);
  if (err != fastKronSuccess) return err;
  for (size_t k = 0; k < plan.passes.size(); k++) {
    Pass ps = plan.passes[k];
    const bool last = (k + 1 == plan.passes.size());
    LaunchCtx cx;
    cx.stream = r.stream; cx.dt = DType::F32; cx.smCount = r.smCount;
    auto buf = [&](Buf b) -> void* {
      switch (b) { case Buf::X: return const_cast<float*>(x); case Buf::T1: return t1; case Buf::T2: return t2;
                   default: return bases[r.g]; }
    };
    cx.src = buf(ps.src);
    cx.dst = buf(ps.dst);
    for (int f = 0; f < ps.nf; f++) cx.F[f] = Fs[1 + ps.f0 + f];
    factorStrides(MMType::MKM, fastKronOp_N, ps.P[0], ps.Q[0], &cx.fsP, &cx.fsQ);
    ps.epilogue = false;
    if (last) {
      if (ps.nf != 1 || ps.f0 != 0) return fastKronOtherError;
      if (ps.kind == KernelKind::Tile) ps.kind = KernelKind::Generic;   // only Generic/Gemm redistribute
      mgScatter1(r, &cx.scatter);
      if (packed) {
        cx.scatter.sM = (long long)(cx.scatter.aLoc * cx.scatter.qPer) * cx.scatter.sQ;   // P1/G rows per m
        cx.scatter.zOff = 0;
      }
      for (int d = 0; d < r.gk; d++) cx.scatter.base[d] = bases[d];
    }
    err = e->launchPass(ps, cx);
    if (err != fastKronSuccess) return err;
  }
  return fastKronSuccess;
}

// Phase 2, fused transport: mode 1 of the received tensor [M][P1][Q2/GK * Q3..QN]; rows go
// to resultPeers[d].
static fastKronError mgPhase2(Engine* e, const MgRank& r, const float* recv, const float* F0,
                              void* const resultPeers[]) {
  fastKronError err = mgCheck(r);
  if (err != fastKronSuccess) return err;
  const uint64_t B2 = (r.Qs[1] / r.gk) * prodQ(r, 2);
  Pass ps;
  ps.f0 = 0; ps.nf = 1; ps.M = r.M; ps.A = 1; ps.B = B2;
  ps.P[0] = r.Ps[0]; ps.Q[0] = r.Qs[0];
  ps.xsM = (int64_t)(r.Ps[0] * B2); ps.xsA = ps.xsM; ps.xsG = (int64_t)B2; ps.xsB = 1;
  ps.zsM = (int64_t)(r.Qs[0] * B2); ps.zsA = ps.zsM; ps.zsG = (int64_t)B2; ps.zsB = 1;
  ps.kind = gemmEligible(DType::F32, r.Ps[0], r.Qs[0], B2) ? KernelKind::Gemm : KernelKind::Generic;
  LaunchCtx cx;
  cx.stream = r.stream; cx.dt = DType::F32; cx.smCount = r.smCount;
  cx.src = recv; cx.dst = resultPeers[r.g];
  cx.F[0] = F0;
  factorStrides(MMType::MKM, fastKronOp_N, ps.P[0], ps.Q[0], &cx.fsP, &cx.fsQ);
  mgScatter2(r, &cx.scatter);
  for (int d = 0; d < r.gk; d++) cx.scatter.base[d] = resultPeers[d];
  return e->launchPass(ps, cx);
}

// True when the staged transport can run the problem: phase 2 reads its input as received,
// [sender][M][P1/G][B2], which only the large-factor kernel's split-input mode does.
static bool mgStagedEligible(const MgRank& r) {
  if (r.gk < 2 || r.N < 2) return false;
  const uint64_t B2 = (r.Qs[1] / r.gk) * prodQ(r, 2);
  return gemmEligible(DType::F32, r.Ps[0], r.Qs[0], B2) && B2 % (uint64_t)gemmTileJ(DType::F32) == 0;
}

// Phase 2, staged transport: output block d = [M][Q1/G][B2] for rank d at stage2 + d*blk2.
static fastKronError mgPhase2Staged(Engine* e, const MgRank& r, const float* recv, const float* F0, float* stage2) {
  if (!mgStagedEligible(r)) return fastKronKernelNotFound;
  const uint64_t p1loc = r.Ps[0] / r.gk, q1loc = r.Qs[0] / r.gk;
  const uint64_t B2 = (r.Qs[1] / r.gk) * prodQ(r, 2);
  Pass ps;
  ps.f0 = 0; ps.nf = 1; ps.M = r.M; ps.A = 1; ps.B = B2;
  ps.P[0] = r.Ps[0]; ps.Q[0] = r.Qs[0];
  ps.xsM = (int64_t)(r.Ps[0] * B2); ps.xsA = ps.xsM; ps.xsG = (int64_t)B2; ps.xsB = 1;
  ps.zsM = (int64_t)(r.Qs[0] * B2); ps.zsA = ps.zsM; ps.zsG = (int64_t)B2; ps.zsB = 1;
  ps.kind = KernelKind::Gemm;
  LaunchCtx cx;
  cx.stream = r.stream; cx.dt = DType::F32; cx.smCount = r.smCount;
  cx.src = recv; cx.dst = stage2;
  cx.F[0] = F0;
  factorStrides(MMType::MKM, fastKronOp_N, ps.P[0], ps.Q[0], &cx.fsP, &cx.fsQ);
  cx.pSplit = (unsigned)p1loc; cx.pOuter = (unsigned long long)r.M * p1loc * B2; cx.nStride = p1loc * B2;
  cx.scatter.parts = r.gk; cx.scatter.qPer = q1loc; cx.scatter.aLoc = 1;
  cx.scatter.sM = (long long)(q1loc * B2); cx.scatter.sA = 0; cx.scatter.sQ = (long long)B2; cx.scatter.zOff = 0;
  const uint64_t blk = (uint64_t)r.M * q1loc * B2;
  for (int d = 0; d < r.gk; d++) cx.scatter.base[d] = stage2 + (size_t)d * blk;
  return e->launchPass(ps, cx);
}

// ---- stream memory operations (driver API, fetched at run time) ---------------------------

typedef CUresult (*StreamValue32Fn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
struct StreamMemOps {
  StreamValue32Fn write = nullptr, wait = nullptr;
  bool ok() const { return write && wait; }
};
static const StreamMemOps& streamMemOps() {
  static StreamMemOps ops = [] {
    StreamMemOps o;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuStreamWriteValue32", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      o.write = reinterpret_cast<StreamValue32Fn>(p);
    else
      cudaGetLastError();
    p = nullptr;
    if (cudaGetDriverEntryPoint("cuStreamWaitValue32", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      o.wait = reinterpret_cast<StreamValue32Fn>(p);
    else
      cudaGetLastError();
    return o;
  }();
  return ops;
}

// ---- staged blocks moved by a kernel ------------------------------------------------------------
// One launch per exchange: for each of n destinations a dense [rows][width] block of the local
// staging area goes to rows of pitch dpitch in that destination's memory (peer stores; 16-byte
// vectors).  A thread carries one vector per destination at a time, so the traffic of an
// exchange is spread over all peers all the time.  No waiting inside: ordering stays with the
// stream (events or sequence flags written after the launch).
struct MgCopyArgs {
  const float* src[kMaxParts];
  float* dst[kMaxParts];
  int n = 0;
  unsigned long long rows = 0, width = 0, dpitch = 0;      // elements
};

__global__ void __launch_bounds__(256) mgCopyKernel(const MgCopyArgs a) {
  const unsigned long long w4 = a.width / 4, p4 = a.dpitch / 4, total = a.rows * w4;
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    unsigned long long o = i;
    if (a.rows > 1) { const unsigned long long r = i / w4; o = r * p4 + (i - r * w4); }
    float4 v[kMaxParts];
#pragma unroll
    for (int d = 0; d < kMaxParts; d++)
      if (d < a.n) v[d] = __ldcs(reinterpret_cast<const float4*>(a.src[d]) + i);
#pragma unroll
    for (int d = 0; d < kMaxParts; d++)
      if (d < a.n) reinterpret_cast<float4*>(a.dst[d])[o] = v[d];
  }
}

static bool mgCopyKernelOk(const MgCopyArgs& a) {
  if (a.n < 1 || a.n > kMaxParts || a.rows == 0 || a.width == 0 || a.width % 4 || a.dpitch % 4) return false;
  for (int d = 0; d < a.n; d++)
    if ((((uintptr_t)a.src[d]) | ((uintptr_t)a.dst[d])) & 15) return false;
  return true;
}
static fastKronError mgCopyLaunch(const MgCopyArgs& a, int ctas, cudaStream_t s) {
  mgCopyKernel<<<ctas, 256, 0, s>>>(a);
  return cudaToFk(cudaGetLastError());
}

// ---- the pipelined schedule of one rank ---------------------------------------------------

// Number of row slices: FASTKRON_MG_PARTS when set (a supported knob), else by the size of the
// rank's block -- slices below a few tens of MB only add launches and copies; measured on C5 with
// 4 GPUs: 17.1 ms with 4 slices, 14.7 ms with 8.  (Slices only pay with the staged transport: the
// fused one runs them one after the other on the compute stream, so it gets one.)
static int mgDefaultParts(uint64_t rows, uint64_t blockElems) {
  int want;
  if (const char* e = getenv("FASTKRON_MG_PARTS")) want = atoi(e);
  else want = blockElems >= (1ull << 27) ? 8 : (blockElems >= (1ull << 24) ? 2 : 1);
  if (want < 1) want = 1;
  if (want > 16) want = 16;
  while (want > 1 && rows % (uint64_t)want != 0) want--;
  return want;
}

struct MgPipe {
  Engine* eng = nullptr;
  int device = 0;
  MgRank rank;                            // rank.M = rows of ONE slice
  std::vector<uint32_t> Ps, Qs;
  int parts = 1;
  bool staged = false;
  bool useFlags = false;                  // one process per GPU: order by sequence flags
  uint64_t Kloc = 0, Lloc = 0, blk1 = 0, blk2 = 0, B2 = 0;
  uint64_t tmpSlice = 0, recvSlice = 0;   // elements per slice
  // local buffers (owned when `owned`, else the caller's)
  bool owned = false;
  float *t1 = nullptr, *t2 = nullptr, *stage1 = nullptr, *recv = nullptr, *result = nullptr, *xdev = nullptr;
  uint32_t* flags = nullptr;              // [2][parts][gk], only with useFlags
  // peers' buffers as this process can address them (index = column rank)
  void* recvPeer[kMaxParts] = {nullptr};
  void* resultPeer[kMaxParts] = {nullptr};
  uint32_t* flagPeer[kMaxParts] = {nullptr};
  bool peersSet = false;
  cudaStream_t compute = nullptr;
  // side streams of the transport: a slice's copies are spread over them by destination, so
  // several copy engines (and NVLink paths to different peers) work at once
  static constexpr int NC = 8;            // at most; `nc` of them exist
  int nc = 4;
  cudaStream_t copy[NC] = {nullptr};
  // who moves the staged blocks: the copy engines (cudaMemcpyAsync per destination) or one
  // kernel per exchange that reads the staging area and stores to every peer (smCtas > 0)
  int smCtas = 0;
  cudaStream_t h2d = nullptr, d2h = nullptr;
  // fused transport with several row slices: the slices alternate between `lanes` streams, each
  // launching on 1/lanes of the CTA slots, so that the passes of one slice that store to the
  // peers (bound by NVLink) run beside the local passes of the next (bound by arithmetic)
  int lanes = 1;
  cudaStream_t lane[2] = {nullptr, nullptr};
  cudaEvent_t evFork = nullptr, evStagger = nullptr;
  // per slice: passes done (evC2, evC3), host block arrived (evIn); per slice and side stream:
  // this rank's outgoing copies of exchange 1 / 2 done (evX1, evX2)
  std::vector<cudaEvent_t> evC2, evC3, evX1, evX2, evIn;
  uint32_t seq = 0;
  // optional timing of the exchanges (fkbMgPipeTrace): per (phase, slice) an event when the copies
  // may start and one per side stream when its copies of that exchange are done
  bool trace = false;
  std::vector<cudaEvent_t> trBegin, trEnd;     // [2][parts], [2][parts][NC]
  MgPipe* const* group = nullptr;         // one process: the pipes of this row group, by column rank

  size_t flagIndex(int phase, int slice, int src) const { return ((size_t)phase * parts + slice) * rank.gk + src; }
};

static void mgPipeDestroy(MgPipe* p) {
  if (!p) return;
  int cur = 0;
  cudaGetDevice(&cur);
  cudaSetDevice(p->device);
  for (auto* v : {&p->evC2, &p->evC3, &p->evX1, &p->evX2, &p->evIn, &p->trBegin, &p->trEnd})
    for (cudaEvent_t e : *v) cudaEventDestroy(e);
  for (cudaStream_t s : p->copy)
    if (s) cudaStreamDestroy(s);
  for (cudaStream_t s : {p->h2d, p->d2h, p->lane[0], p->lane[1]})
    if (s) cudaStreamDestroy(s);
  for (cudaEvent_t e : {p->evFork, p->evStagger})
    if (e) cudaEventDestroy(e);
  if (p->owned) {
    for (float* b : {p->t1, p->t2, p->stage1, p->recv, p->result, p->xdev})
      if (b) cudaFree(b);
  }
  if (p->flags) cudaFree(p->flags);
  cudaSetDevice(cur);
  delete p;
}

// Streams and events of a pipe; the device must be current.
static fastKronError mgPipeInitStreams(MgPipe* p) {
  int lo = 0, hi = 0;
  cudaDeviceGetStreamPriorityRange(&lo, &hi);
  // FASTKRON_MG_COPY_STREAMS = 1..8 side streams (default 4); FASTKRON_MG_COPY=sm[:ctas] moves the
  // staged blocks with a kernel instead of the copy engines (supported knobs)
  if (const char* e = getenv("FASTKRON_MG_COPY_STREAMS")) {
    const int v = atoi(e);
    if (v >= 1 && v <= MgPipe::NC) p->nc = v;
  }
  if (const char* e = getenv("FASTKRON_MG_COPY")) {
    if (!strncmp(e, "sm", 2)) {
      p->smCtas = 48;
      if (e[2] == ':' && atoi(e + 3) > 0) p->smCtas = atoi(e + 3);
      if (p->smCtas > 1024) p->smCtas = 1024;
    }
  }
  for (int i = 0; i < p->nc; i++)
    if (cudaStreamCreateWithPriority(&p->copy[i], cudaStreamNonBlocking, hi) != cudaSuccess) return fastKronOtherError;
  if (p->lanes > 1) {
    for (int i = 0; i < p->lanes; i++)
      if (cudaStreamCreateWithPriority(&p->lane[i], cudaStreamNonBlocking, lo) != cudaSuccess) return fastKronOtherError;
    if (cudaEventCreateWithFlags(&p->evFork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&p->evStagger, cudaEventDisableTiming) != cudaSuccess)
      return fastKronOtherError;
  }
  if (cudaStreamCreateWithPriority(&p->h2d, cudaStreamNonBlocking, hi) != cudaSuccess) return fastKronOtherError;
  if (cudaStreamCreateWithPriority(&p->d2h, cudaStreamNonBlocking, hi) != cudaSuccess) return fastKronOtherError;
  for (auto* v : {&p->evC2, &p->evC3, &p->evX1, &p->evX2, &p->evIn}) {
    const int n = (v == &p->evX1 || v == &p->evX2) ? p->parts * MgPipe::NC : p->parts;
    for (int s = 0; s < n; s++) {
      cudaEvent_t ev;
      if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) return fastKronOtherError;
      v->push_back(ev);
    }
  }
  return fastKronSuccess;
}

// Geometry of a pipe from (rows per rank, factor shapes, group size, slices).
static fastKronError mgPipeGeometry(MgPipe* p, int g, int gk, uint32_t rows, uint32_t N, const uint32_t* Ps,
                                    const uint32_t* Qs, int parts, int wantStaged, bool autoParts = false) {
  p->Ps.assign(Ps, Ps + N);
  p->Qs.assign(Qs, Qs + N);
  p->rank.g = g; p->rank.gk = gk; p->rank.N = N; p->rank.Ps = p->Ps.data(); p->rank.Qs = p->Qs.data();
  p->rank.M = rows;
  fastKronError err = mgCheck(p->rank);
  if (err != fastKronSuccess) return err;
  if (gk < 2) return fastKronInvalidArgument;
  uint64_t K = 1, L = 1;
  for (uint32_t i = 0; i < N; i++) { K *= Ps[i]; L *= Qs[i]; }
  p->Kloc = K / gk; p->Lloc = L / gk;
  if (parts < 1 || rows % (uint32_t)parts != 0) return fastKronInvalidArgument;
  p->parts = parts;
  p->rank.M = rows / parts;
  const bool can = mgStagedEligible(p->rank);
  // FASTKRON_MG_MODE=fused|staged overrides the automatic choice (a supported knob)
  if (wantStaged < 0) {
    const char* m = getenv("FASTKRON_MG_MODE");
    if (m && !strcmp(m, "fused")) wantStaged = 0;
    else if (m && !strcmp(m, "staged") && can) wantStaged = 1;
  }
  if (wantStaged == 1 && !can) return fastKronKernelNotFound;
  // Automatic choice, from measurements on 8 B200 behind NVSwitch (C5): with two GPUs half of
  // every block stays local and storing straight from the kernels wins (25.5 ms against 28.5 ms);
  // with four, the copy engines win (14.6 against 16.4 ms) because the kernels then run at full
  // speed while the NVLink traffic of another row slice is in flight; with eight, seven
  // concurrent copies per exchange only reach about 380 GB/s per GPU and the exchanges outlast
  // the arithmetic (10.1 ms), so the kernels' own stores win again (9.6 ms).
  if (wantStaged < 0) wantStaged = (can && gk >= 3 && gk < 8) ? 1 : 0;
  p->staged = wantStaged == 1;
  // Fused transport: one slice on the compute stream, except for eight and more GPUs, where most
  // of a pass's output crosses NVLink and two lanes (FASTKRON_MG_LANES=1|2 overrides) let the
  // slices' NVLink-bound passes run beside the next slices' local ones (C5, 8 GPUs: 8.9 ms
  // against 9.5 ms).
  int wantLanes = 1;
  if (!p->staged) {
    const char* e = getenv("FASTKRON_MG_LANES");
    wantLanes = e ? (atoi(e) == 2 ? 2 : 1) : (gk >= 8 ? 2 : 1);
    if (wantLanes == 1 && autoParts && !getenv("FASTKRON_MG_PARTS")) {
      p->parts = 1;
      p->rank.M = rows;
    }
  }
  p->lanes = (wantLanes == 2 && p->parts >= 2) ? 2 : 1;
  const uint64_t B = prodQ(p->rank, 2);
  const uint64_t p1loc = Ps[0] / gk, q1loc = Qs[0] / gk, q2loc = Qs[1] / gk;
  p->B2 = q2loc * B;
  p->blk1 = (uint64_t)p->rank.M * p1loc * q2loc * B;
  p->blk2 = (uint64_t)p->rank.M * q1loc * p->B2;
  // widest local intermediate per slice = the global one divided by the group size
  Problem full;
  full.N = N;
  for (uint32_t i = 0; i < N; i++) { full.P[i] = Ps[i]; full.Q[i] = Qs[i]; }
  const uint64_t cols = N == 1 ? (K > L ? K : L) : full.maxIntermediateCols();
  p->tmpSlice = (uint64_t)p->rank.M * (cols / gk);
  p->recvSlice = (uint64_t)p->rank.M * Ps[0] * p->B2;
  return fastKronSuccess;
}

// The stream that runs the kernels of slice s, and the SM count its launches size their grids for.
static cudaStream_t mgLaneOf(const MgPipe* p, int s) { return p->lanes > 1 ? p->lane[s % p->lanes] : p->compute; }
static int mgLaneSms(const MgPipe* p) { return p->lanes > 1 ? (p->rank.smCount + p->lanes - 1) / p->lanes : p->rank.smCount; }
// Start of a call: the lanes continue where the caller's stream stands.
static fastKronError mgFork(MgPipe* p) {
  if (p->lanes <= 1) return fastKronSuccess;
  if (cudaEventRecord(p->evFork, p->compute) != cudaSuccess) return fastKronOtherError;
  for (int i = 0; i < p->lanes; i++)
    if (cudaStreamWaitEvent(p->lane[i], p->evFork, 0) != cudaSuccess) return fastKronOtherError;
  return fastKronSuccess;
}

// ---- ordering primitives --------------------------------------------------------------------
// A slice's outgoing copies of one exchange run on the NC side streams (fused transport: there
// are none, the kernel itself stored the rows and "side stream" means the compute stream).
// mgSignal records, per side stream, that this rank's copies of (phase, slice) on it are done;
// with flags, the message towards rank d is written right after the copy to d instead.
static fastKronError mgSignal(MgPipe* p, int phase, int slice) {
  std::vector<cudaEvent_t>& ev = phase == 0 ? p->evX1 : p->evX2;
  for (int c = 0; c < p->nc; c++) {
    cudaStream_t s = p->staged ? p->copy[c] : mgLaneOf(p, slice);
    if (cudaEventRecord(ev[(size_t)slice * MgPipe::NC + c], s) != cudaSuccess) return fastKronOtherError;
    if (!p->staged) break;                 // one stream only: event 0 stands for the slice
  }
  return fastKronSuccess;
}
static fastKronError mgWaitEvents(MgPipe* q, int phase, int slice, cudaStream_t s) {
  const std::vector<cudaEvent_t>& ev = phase == 0 ? q->evX1 : q->evX2;
  for (int c = 0; c < (q->staged ? q->nc : 1); c++)
    if (cudaStreamWaitEvent(s, ev[(size_t)slice * MgPipe::NC + c], 0) != cudaSuccess) return fastKronOtherError;
  return fastKronSuccess;
}
static fastKronError mgFlagTo(MgPipe* p, int phase, int slice, int d, cudaStream_t s) {
  if (!p->useFlags) return fastKronSuccess;
  const StreamMemOps& ops = streamMemOps();
  uint32_t* addr = p->flagPeer[d] + p->flagIndex(phase, slice, p->rank.g);
  if (ops.write((CUstream)s, (CUdeviceptr)(uintptr_t)addr, p->seq, 0) != CUDA_SUCCESS) return fastKronOtherError;
  return fastKronSuccess;
}
// `s` waits until every OTHER rank's blocks of (phase, slice) have landed here.
static fastKronError mgWaitAll(MgPipe* p, int phase, int slice, cudaStream_t s) {
  const int G = p->rank.gk, g = p->rank.g;
  if (p->useFlags) {
    const StreamMemOps& ops = streamMemOps();
    for (int d = 0; d < G; d++) {
      if (d == g) continue;
      uint32_t* addr = p->flags + p->flagIndex(phase, slice, d);
      if (ops.wait((CUstream)s, (CUdeviceptr)(uintptr_t)addr, p->seq, 0 /* >= */) != CUDA_SUCCESS) return fastKronOtherError;
    }
    return fastKronSuccess;
  }
  for (int d = 0; d < G; d++) {
    if (d == g) continue;
    fastKronError err = mgWaitEvents(p->group[d], phase, slice, s);
    if (err != fastKronSuccess) return err;
  }
  return fastKronSuccess;
}

// ---- the two halves of a slice --------------------------------------------------------------

static fastKronError mgEnqueueP1(MgPipe* p, int s, const float* x, const float* const* Fs) {
  const int G = p->rank.gk, g = p->rank.g;
  MgRank r = p->rank;
  cudaStream_t ks = mgLaneOf(p, s);
  r.stream = ks;
  r.smCount = mgLaneSms(p);
  // the second lane starts half a slice late, so that its NVLink-bound passes fall beside the
  // first lane's local ones
  if (p->lanes > 1 && s == 1 && cudaStreamWaitEvent(ks, p->evStagger, 0) != cudaSuccess) return fastKronOtherError;
  float* t1 = p->t1 + (size_t)s * p->tmpSlice;
  float* t2 = p->t2 + (size_t)s * p->tmpSlice;
  float* recvS = (float*)p->recvPeer[g] + (size_t)s * p->recvSlice;
  const float* xs = x + (size_t)s * r.M * p->Kloc;
  void* bases[kMaxParts];
  if (p->staged) {
    float* st = p->stage1 + (size_t)s * p->tmpSlice;
    for (int d = 0; d < G; d++) bases[d] = st + (size_t)d * p->blk1;
    bases[g] = recvS + (size_t)g * p->blk1;          // this rank's own block needs no transport
  } else {
    for (int d = 0; d < G; d++) bases[d] = (float*)p->recvPeer[d] + (size_t)s * p->recvSlice;
  }
  fastKronError err = mgPhase1(p->eng, r, xs, Fs, t1, t2, bases, p->staged);
  if (err != fastKronSuccess) return err;
  if (cudaEventRecord(p->evC2[s], ks) != cudaSuccess) return fastKronOtherError;
  if (p->lanes > 1 && s == 0 && cudaEventRecord(p->evStagger, ks) != cudaSuccess) return fastKronOtherError;
  if (p->staged) {
    if (p->trace) cudaEventRecord(p->trBegin[s], ks);
    for (int c = 0; c < p->nc; c++)
      if (cudaStreamWaitEvent(p->copy[c], p->evC2[s], 0) != cudaSuccess) return fastKronOtherError;
    MgCopyArgs ca;
    for (int k = 1; k < G; k++) {
      const int d = (g + k) % G;
      ca.src[k - 1] = (const float*)bases[d];
      ca.dst[k - 1] = (float*)p->recvPeer[d] + (size_t)s * p->recvSlice + (size_t)g * p->blk1;
    }
    ca.n = G - 1; ca.rows = 1; ca.width = p->blk1; ca.dpitch = p->blk1;
    if (p->smCtas > 0 && mgCopyKernelOk(ca)) {
      // one kernel for all destinations, exchanges of successive slices on alternating streams
      cudaStream_t cs = p->copy[s % p->nc];
      if ((err = mgCopyLaunch(ca, p->smCtas, cs)) != fastKronSuccess) return err;
      for (int k = 1; k < G; k++)
        if ((err = mgFlagTo(p, 0, s, (g + k) % G, cs)) != fastKronSuccess) return err;
    } else {
      for (int k = 1; k < G; k++) {
        const int d = (g + k) % G;
        cudaStream_t cs = p->copy[(k + s) % p->nc];
        if (cudaMemcpyAsync(ca.dst[k - 1], ca.src[k - 1], p->blk1 * sizeof(float), cudaMemcpyDeviceToDevice, cs) != cudaSuccess)
          return fastKronOtherError;
        if ((err = mgFlagTo(p, 0, s, d, cs)) != fastKronSuccess) return err;
      }
    }
  } else {
    for (int k = 1; k < G; k++)
      if ((err = mgFlagTo(p, 0, s, (g + k) % G, ks)) != fastKronSuccess) return err;
  }
  if (p->trace && p->staged)
    for (int c = 0; c < p->nc; c++) cudaEventRecord(p->trEnd[(size_t)s * MgPipe::NC + c], p->copy[c]);
  return mgSignal(p, 0, s);
}

static fastKronError mgEnqueueP2(MgPipe* p, int s, const float* F0) {
  const int G = p->rank.gk, g = p->rank.g;
  MgRank r = p->rank;
  cudaStream_t ks = mgLaneOf(p, s);
  r.stream = ks;
  r.smCount = mgLaneSms(p);
  fastKronError err = mgWaitAll(p, 0, s, ks);
  if (err != fastKronSuccess) return err;
  const float* recvS = (const float*)p->recvPeer[g] + (size_t)s * p->recvSlice;
  const uint64_t q1loc = p->Qs[0] / G;
  const size_t resSlice = (size_t)s * r.M * p->Lloc;            // rows of this slice in a result block
  if (p->staged) {
    float* st2 = p->t1 + (size_t)s * p->tmpSlice;               // free again: every local pass of the slice is done
    err = mgPhase2Staged(p->eng, r, recvS, F0, st2);
    if (err != fastKronSuccess) return err;
    if (cudaEventRecord(p->evC3[s], ks) != cudaSuccess) return fastKronOtherError;
    if (p->trace) cudaEventRecord(p->trBegin[(size_t)p->parts + s], ks);
    for (int c = 0; c < p->nc; c++)
      if (cudaStreamWaitEvent(p->copy[c], p->evC3[s], 0) != cudaSuccess) return fastKronOtherError;
    const size_t rows = (size_t)r.M * q1loc, width = p->B2 * sizeof(float), dpitch = (size_t)G * width;
    MgCopyArgs ca;
    for (int k = 0; k < G; k++) {
      const int d = (g + k) % G;
      ca.src[k] = st2 + (size_t)d * p->blk2;
      ca.dst[k] = (float*)p->resultPeer[d] + resSlice + (size_t)g * p->B2;
    }
    ca.n = G; ca.rows = rows; ca.width = p->B2; ca.dpitch = (size_t)G * p->B2;
    if (p->smCtas > 0 && mgCopyKernelOk(ca)) {
      cudaStream_t cs = p->copy[(s + 1) % p->nc];
      if ((err = mgCopyLaunch(ca, p->smCtas, cs)) != fastKronSuccess) return err;
      for (int k = 1; k < G; k++)
        if ((err = mgFlagTo(p, 1, s, (g + k) % G, cs)) != fastKronSuccess) return err;
    } else {
      for (int k = 0; k < G; k++) {
        const int d = (g + k) % G;
        cudaStream_t cs = p->copy[(k + s) % p->nc];
        if (cudaMemcpy2DAsync(ca.dst[k], dpitch, ca.src[k], width, width, rows, cudaMemcpyDeviceToDevice, cs) != cudaSuccess)
          return fastKronOtherError;
        if (d != g && (err = mgFlagTo(p, 1, s, d, cs)) != fastKronSuccess) return err;
      }
    }
  } else {
    void* res[kMaxParts];
    for (int d = 0; d < G; d++) res[d] = (float*)p->resultPeer[d] + resSlice;
    err = mgPhase2(p->eng, r, recvS, F0, res);
    if (err != fastKronSuccess) return err;
    for (int k = 1; k < G; k++)
      if ((err = mgFlagTo(p, 1, s, (g + k) % G, ks)) != fastKronSuccess) return err;
  }
  if (p->trace && p->staged)
    for (int c = 0; c < p->nc; c++)
      cudaEventRecord(p->trEnd[((size_t)p->parts + s) * MgPipe::NC + c], p->copy[c]);
  return mgSignal(p, 1, s);
}

// `stream` waits until slice s of this rank's result block is complete: its own outgoing
// copies are done and every peer's rows have arrived.
static fastKronError mgWaitResult(MgPipe* p, int s, cudaStream_t stream) {
  fastKronError err = mgWaitEvents(p, 1, s, stream);
  if (err != fastKronSuccess) return err;
  return mgWaitAll(p, 1, s, stream);
}

// The enqueue order of a call as (half, slice) pairs: P1(0), then P1(i), P2(i-1), ..., P2(last).
static void mgOrder(int parts, std::vector<std::pair<int, int>>* order) {
  order->clear();
  order->push_back({1, 0});
  for (int i = 1; i < parts; i++) { order->push_back({1, i}); order->push_back({2, i - 1}); }
  order->push_back({2, parts - 1});
}

// ---- multi-GPU state of a handle (one process driving all GPUs) ----------------------------

struct MgState {
  int gpus = 1, gm = 1, gk = 1;
  bool oneDevice = false;                 // all logical GPUs live on the current device (emulation)
  std::vector<int> device;                // physical device of logical GPU g
  std::vector<cudaStream_t> stream;
  std::vector<int> smCount;
  std::vector<cudaEvent_t> ev1, ev2;
  // pipes of the last problem (index = logical GPU), rebuilt when the problem changes
  std::vector<MgPipe*> pipes;
  std::string pipeKey;
};

void mgAdjustSizes(const MgState* mg, const Problem& pr, size_t* yElems, size_t* tmpElems) {
  // per-device counts; the temporary is doubled: the second halves are the receive area of the
  // first exchange and the staging area of the transport (the reference doubles it for its
  // NCCL staging, src/handle/handle.cpp:327-338)
  const uint64_t rows = pr.M / mg->gm;
  const uint64_t cols = (pr.N == 1) ? (pr.K() > pr.L() ? pr.K() : pr.L()) : pr.maxIntermediateCols();
  *yElems = (size_t)(rows * (pr.L() / mg->gk));
  *tmpElems = (size_t)(rows * (cols / mg->gk)) * (mg->gk > 1 ? 2 : 1);
}

static void mgDropPipes(MgState* mg) {
  for (MgPipe* p : mg->pipes) mgPipeDestroy(p);
  mg->pipes.clear();
  mg->pipeKey.clear();
}

void mgDestroy(MgState* mg) {
  if (!mg) return;
  mgDropPipes(mg);
  for (cudaEvent_t e : mg->ev1) cudaEventDestroy(e);
  for (cudaEvent_t e : mg->ev2) cudaEventDestroy(e);
  delete mg;
}

}  // namespace fkb

using namespace fkb;

static inline Engine* E(fastKronHandle h) { return reinterpret_cast<Engine*>(h); }

extern "C" {

// reference: src/fastkron.cpp:109-111, src/kernel_db/cuda_kernel_db.cu:62-186.  Defaults as
// there (gpusInK -1 -> 2, gpusInM -1 -> 1); a grid that does not multiply to `gpus` is an
// error code here instead of abort().  With the environment variable
// FASTKRON_MG_ONE_DEVICE=1 all logical GPUs are placed on the current device (used to test
// the distributed schedule on a single GPU).
fastKronError fastKronMgInitCUDA(fastKronHandle handle, void* streams, int gpus, int gpusInM, int gpusInK,
                                 int gpuLocalKrons) {
  (void)gpuLocalKrons;   // the schedule always uses the minimum of two exchanges
  if (!handle || gpus < 1 || gpus > 64) return fastKronInvalidArgument;
  Engine* e = E(handle);
  if (!e->hasBackend(fastKronBackend_CUDA)) return fastKronBackendNotAvailable;
  int gk = gpusInK >= 1 ? gpusInK : (gpus == 1 ? 1 : 2);
  int gm = gpusInM >= 1 ? gpusInM : 1;
  if (gk * gm != gpus || gk > kMaxParts) return fastKronInvalidArgument;
  const char* one = getenv("FASTKRON_MG_ONE_DEVICE");
  const bool oneDevice = one && one[0] == '1';
  int ndev = 0, cur = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || cudaGetDevice(&cur) != cudaSuccess) {
    cudaGetLastError();
    return fastKronBackendNotAvailable;
  }
  if (!oneDevice && ndev < gpus) return fastKronInvalidArgument;

  MgState* mg = new MgState;
  mg->gpus = gpus; mg->gm = gm; mg->gk = gk; mg->oneDevice = oneDevice;
  cudaStream_t* st = reinterpret_cast<cudaStream_t*>(streams);
  for (int g = 0; g < gpus; g++) {
    const int dev = oneDevice ? cur : g;
    mg->device.push_back(dev);
    mg->stream.push_back(st ? st[g] : nullptr);
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess || prop.major != 10) {
      cudaGetLastError(); delete mg; return fastKronBackendNotAvailable;
    }
    mg->smCount.push_back(prop.multiProcessorCount);
  }
  // peer access for the direct stores and copies (reference: cuda_kernel_db.cu:83-93)
  if (!oneDevice) {
    for (int a = 0; a < gpus; a++) {
      cudaSetDevice(a);
      for (int b = 0; b < gpus; b++) {
        if (a == b) continue;
        int can = 0;
        cudaDeviceCanAccessPeer(&can, a, b);
        if (!can) { cudaSetDevice(cur); delete mg; return fastKronBackendNotAvailable; }
        cudaError_t pe = cudaDeviceEnablePeerAccess(b, 0);
        if (pe != cudaSuccess && pe != cudaErrorPeerAccessAlreadyEnabled) { cudaSetDevice(cur); delete mg; return fastKronOtherError; }
        cudaGetLastError();
      }
    }
  }
  for (int g = 0; g < gpus; g++) {
    cudaSetDevice(mg->device[g]);
    cudaEvent_t a, b;
    if (cudaEventCreateWithFlags(&a, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&b, cudaEventDisableTiming) != cudaSuccess) {
      cudaSetDevice(cur); mgDestroy(mg); return fastKronOtherError;
    }
    mg->ev1.push_back(a); mg->ev2.push_back(b);
  }
  cudaSetDevice(cur);
  if (e->mg) mgDestroy(e->mg);
  e->mg = mg;
  // the handle itself is usable for single-device calls on the current device as well
  if (!e->cudaReady()) e->initCUDA(st ? &st[0] : nullptr);
  return fastKronSuccess;
}

// reference: src/fastkron.cpp:389-394 -> src/handle/distrib_handle.cu:504-521.  Blocking.
fastKronError fastKronMgSGEMM(fastKronHandle handle, const uint32_t NumKronMats, void* x[], void* kronMats[],
                              void* result[], uint32_t M, uint32_t N, uint32_t K, uint32_t KronMatCols[],
                              uint32_t KronMatRows[], void* temp1[], void* temp2[], void* streams) {
  (void)N;
  if (!handle || !x || !kronMats || !result || !temp1 || !temp2 || !KronMatCols || !KronMatRows)
    return fastKronInvalidArgument;
  Engine* e = E(handle);
  MgState* mg = e->mg;
  if (!mg) return fastKronOtherError;
  const uint32_t n = NumKronMats;
  if (n == 0 || n > (uint32_t)kMaxFactors) return fastKronInvalidArgument;
  uint64_t kk = 1;
  for (uint32_t i = 0; i < n; i++) kk *= KronMatRows[i];
  if (kk != K || M % mg->gm || K % mg->gk) return fastKronInvalidKMMProblem;
  cudaStream_t* st = reinterpret_cast<cudaStream_t*>(streams);
  int cur = 0;
  cudaGetDevice(&cur);

  Problem full;
  full.mm = MMType::MKM; full.dt = DType::F32; full.M = M; full.N = n;
  for (uint32_t i = 0; i < n; i++) { full.P[i] = KronMatRows[i]; full.Q[i] = KronMatCols[i]; }
  size_t yElems = 0, tmpElems = 0;
  e->sizes(full, &yElems, &tmpElems);
  mgAdjustSizes(mg, full, &yElems, &tmpElems);
  const size_t half = tmpElems / 2;
  const uint32_t rows = M / mg->gm;

  fastKronError err = fastKronSuccess;
  auto streamOf = [&](int g) { return st ? st[g] : mg->stream[g]; };

  if (mg->gk == 1) {
    // rows only: every GPU runs the ordinary single-device plan on its rows
    for (int g = 0; g < mg->gpus && err == fastKronSuccess; g++) {
      cudaSetDevice(mg->device[g]);
      Problem lp = full; lp.M = rows;
      PlanOptions po; po.haveT2 = true;
      Plan plan;
      err = makePlan(lp, po, &plan);
      if (err != fastKronSuccess) break;
      CallOperands ops;
      ops.X = x[g]; ops.Fs = reinterpret_cast<const void* const*>(&kronMats[(size_t)g * n]);
      ops.Z = result[g]; ops.temp1 = temp1[g]; ops.temp2 = temp2[g];
      err = e->execute(lp, plan, ops, streamOf(g), mg->smCount[g]);
    }
  } else {
    // One pipe per GPU, kept while the problem stays the same.  Buffers are the caller's:
    //   temp1[g] = [ t1 | receive area ],  temp2[g] = [ t2 | staging area of exchange 1 ]
    std::string key = std::to_string(M) + ":" + std::to_string(n);
    for (uint32_t i = 0; i < n; i++) key += ":" + std::to_string(KronMatRows[i]) + "x" + std::to_string(KronMatCols[i]);
    if (mg->pipeKey != key) {
      mgDropPipes(mg);
      MgRank probe;
      probe.g = 0; probe.gk = mg->gk; probe.M = rows; probe.N = n; probe.Ps = KronMatRows; probe.Qs = KronMatCols;
      err = mgCheck(probe);
      const int parts = err == fastKronSuccess ? mgDefaultParts(rows, (uint64_t)rows * (K / mg->gk)) : 1;
      for (int g = 0; g < mg->gpus && err == fastKronSuccess; g++) {
        cudaSetDevice(mg->device[g]);
        MgPipe* p = new MgPipe;
        mg->pipes.push_back(p);
        p->eng = e; p->device = mg->device[g];
        err = mgPipeGeometry(p, g % mg->gk, mg->gk, rows, n, KronMatRows, KronMatCols, parts, -1, true);
        if (err == fastKronSuccess) err = mgPipeInitStreams(p);
        p->rank.smCount = mg->smCount[g];
      }
      if (err == fastKronSuccess) mg->pipeKey = key; else mgDropPipes(mg);
    }
    if (err == fastKronSuccess) {
      for (int g = 0; g < mg->gpus; g++) {
        MgPipe* p = mg->pipes[g];
        const int row = g / mg->gk;
        p->compute = streamOf(g);
        p->t1 = (float*)temp1[g]; p->t2 = (float*)temp2[g];
        p->stage1 = (float*)temp2[g] + half;
        p->group = &mg->pipes[(size_t)row * mg->gk];
        for (int d = 0; d < mg->gk; d++) {
          p->recvPeer[d] = (float*)temp1[row * mg->gk + d] + half;
          p->resultPeer[d] = result[row * mg->gk + d];
        }
        cudaSetDevice(mg->device[g]);
        if (err == fastKronSuccess) err = mgFork(p);
      }
      std::vector<std::pair<int, int>> order;
      mgOrder(mg->pipes[0]->parts, &order);
      // stage-major, GPU-minor: every GPU's signal of a (phase, slice) is enqueued before any
      // GPU's wait for it
      for (size_t o = 0; o < order.size() && err == fastKronSuccess; o++) {
        for (int g = 0; g < mg->gpus && err == fastKronSuccess; g++) {
          cudaSetDevice(mg->device[g]);
          MgPipe* p = mg->pipes[g];
          const float* const* Fs = reinterpret_cast<const float* const*>(&kronMats[(size_t)g * n]);
          err = order[o].first == 1 ? mgEnqueueP1(p, order[o].second, (const float*)x[g], Fs)
                                    : mgEnqueueP2(p, order[o].second, Fs[0]);
        }
      }
      for (int g = 0; g < mg->gpus && err == fastKronSuccess; g++) {
        cudaSetDevice(mg->device[g]);
        MgPipe* p = mg->pipes[g];
        for (int s = 0; s < p->parts && err == fastKronSuccess; s++) err = mgWaitResult(p, s, p->compute);
      }
    }
  }
  // the call is blocking, like the reference's (it joins its per-GPU threads)
  for (int g = 0; g < mg->gpus; g++) {
    cudaSetDevice(mg->device[g]);
    if (cudaStreamSynchronize(streamOf(g)) != cudaSuccess && err == fastKronSuccess) err = cudaToFk(cudaGetLastError());
    if (g < (int)mg->pipes.size())
      for (cudaStream_t cs : mg->pipes[g]->copy)
        if (cs && cudaStreamSynchronize(cs) != cudaSuccess && err == fastKronSuccess) err = cudaToFk(cudaGetLastError());
  }
  cudaSetDevice(cur);
  return err;
}

// reference: src/handle/distrib_handle.cu:428-464
fastKronError fastKronMgAllocX(fastKronHandle handle, void* dX[], void* hX, uint32_t M, uint32_t K) {
  if (!handle || !dX || !hX) return fastKronInvalidArgument;
  MgState* mg = E(handle)->mg;
  if (!mg) return fastKronOtherError;
  if (M % mg->gm || K % mg->gk) return fastKronInvalidKMMProblem;
  const size_t gM = M / mg->gm, gK = K / mg->gk;
  int cur = 0;
  cudaGetDevice(&cur);
  fastKronError err = fastKronSuccess;
  for (int g = 0; g < mg->gpus && err == fastKronSuccess; g++) {
    cudaSetDevice(mg->device[g]);
    const int row = g / mg->gk, col = g % mg->gk;
    if (cudaMalloc(&dX[g], gM * gK * sizeof(float)) != cudaSuccess) { cudaGetLastError(); err = fastKronOtherError; break; }
    if (cudaMemcpy2D(dX[g], gK * sizeof(float), (const float*)hX + (size_t)row * gM * K + (size_t)col * gK,
                     (size_t)K * sizeof(float), gK * sizeof(float), gM, cudaMemcpyHostToDevice) != cudaSuccess) {
      cudaGetLastError(); err = fastKronOtherError;
    }
  }
  cudaSetDevice(cur);
  return err;
}

// reference: src/handle/distrib_handle.cu:466-502
fastKronError fastKronMgGatherY(fastKronHandle handle, void* dY[], void* hY, uint32_t M, uint32_t K,
                                uint32_t NumKronMats, uint32_t KronMatCols[], uint32_t KronMatRows[]) {
  (void)K; (void)KronMatRows;
  if (!handle || !dY || !hY || !KronMatCols) return fastKronInvalidArgument;
  MgState* mg = E(handle)->mg;
  if (!mg) return fastKronOtherError;
  uint64_t L = 1;
  for (uint32_t i = 0; i < NumKronMats; i++) L *= KronMatCols[i];
  if (M % mg->gm || L % mg->gk) return fastKronInvalidKMMProblem;
  const size_t gM = M / mg->gm, gL = L / mg->gk;
  int cur = 0;
  cudaGetDevice(&cur);
  fastKronError err = fastKronSuccess;
  for (int g = 0; g < mg->gpus && err == fastKronSuccess; g++) {
    cudaSetDevice(mg->device[g]);
    const int row = g / mg->gk, col = g % mg->gk;
    if (cudaMemcpy2D((float*)hY + (size_t)row * gM * L + (size_t)col * gL, (size_t)L * sizeof(float), dY[g],
                     gL * sizeof(float), gL * sizeof(float), gM, cudaMemcpyDeviceToHost) != cudaSuccess) {
      cudaGetLastError(); err = fastKronOtherError;
    }
  }
  cudaSetDevice(cur);
  return err;
}

// ---- the same schedule for one-process-per-GPU hosts (not part of the reference ABI) ------
// A torchrun-style host owns the ranks.  Every rank creates a pipe on its own device (the pipe
// allocates its buffers with cudaMalloc so that they can be shared), publishes CUDA IPC handles
// of its receive area, result block and flag array (fkbMgPipeLocalBuffers + fkbIpcExport),
// maps its peers' (fkbIpcOpen) and hands the mapped pointers back (fkbMgPipeSetPeers).  After
// that fkbMgPipeRun enqueues a complete product on the handle's stream: when the stream reaches
// the end of the call this rank's result block [M][L/G] is complete.  Calls may follow one
// another without host synchronisation; the sequence flags order them.
//   parts   row slices (0 = choose from the block size / FASTKRON_MG_PARTS)
//   staged  1 = copy-engine transport, 0 = peer stores from the kernels, -1 = staged when the
//           shapes allow it
fastKronError fkbMgPipeCreate(fastKronHandle handle, int rank, int world, uint32_t M, uint32_t N,
                              const uint32_t Ps[], const uint32_t Qs[], int parts, int staged, void** pipeOut) {
  if (!handle || !Ps || !Qs || !pipeOut || world < 2 || world > kMaxParts || rank < 0 || rank >= world)
    return fastKronInvalidArgument;
  Engine* e = E(handle);
  if (!e->cudaReady()) return fastKronBackendNotAvailable;
  if (!streamMemOps().ok()) return fastKronBackendNotAvailable;
  uint64_t K = 1;
  for (uint32_t i = 0; i < N; i++) K *= Ps[i];
  const bool autoParts = parts <= 0;
  if (autoParts) parts = mgDefaultParts(M, (uint64_t)M * (K / world));
  std::unique_ptr<MgPipe, void (*)(MgPipe*)> p(new MgPipe, mgPipeDestroy);
  p->eng = e;
  cudaGetDevice(&p->device);
  p->useFlags = true;
  fastKronError err = mgPipeGeometry(p.get(), rank, world, M, N, Ps, Qs, parts, staged, autoParts);
  if (err != fastKronSuccess) return err;
  p->rank.smCount = e->smCount();
  if ((err = mgPipeInitStreams(p.get())) != fastKronSuccess) return err;
  p->owned = true;
  const size_t tmpBytes = (size_t)p->parts * p->tmpSlice * sizeof(float);
  const size_t recvBytes = (size_t)p->parts * p->recvSlice * sizeof(float);
  const size_t flagBytes = (size_t)2 * p->parts * world * sizeof(uint32_t);
  bool ok = cudaMalloc(&p->t1, tmpBytes) == cudaSuccess && cudaMalloc(&p->t2, tmpBytes) == cudaSuccess &&
            cudaMalloc(&p->recv, recvBytes) == cudaSuccess &&
            cudaMalloc(&p->result, (size_t)M * p->Lloc * sizeof(float)) == cudaSuccess &&
            cudaMalloc(&p->flags, flagBytes) == cudaSuccess;
  if (ok && p->staged) ok = cudaMalloc(&p->stage1, tmpBytes) == cudaSuccess;
  if (!ok) { cudaGetLastError(); return fastKronOtherError; }
  if (cudaMemset(p->flags, 0, flagBytes) != cudaSuccess) return fastKronOtherError;
  cudaDeviceSynchronize();
  *pipeOut = p.release();
  return fastKronSuccess;
}

// Compute lanes of a pipe (1, or 2 for the fused transport on eight and more GPUs).
int fkbMgPipeLanes(void* pipe) { return pipe ? reinterpret_cast<MgPipe*>(pipe)->lanes : 0; }

fastKronError fkbMgPipeLocalBuffers(void* pipe, void** recv, size_t* recvBytes, void** result, size_t* resultBytes,
                                    void** flags, size_t* flagBytes, int* parts, int* staged) {
  MgPipe* p = reinterpret_cast<MgPipe*>(pipe);
  if (!p) return fastKronInvalidArgument;
  if (recv) *recv = p->recv;
  if (recvBytes) *recvBytes = (size_t)p->parts * p->recvSlice * sizeof(float);
  if (result) *result = p->result;
  if (resultBytes) *resultBytes = (size_t)p->parts * p->rank.M * p->Lloc * sizeof(float);
  if (flags) *flags = p->flags;
  if (flagBytes) *flagBytes = (size_t)2 * p->parts * p->rank.gk * sizeof(uint32_t);
  if (parts) *parts = p->parts;
  if (staged) *staged = p->staged ? 1 : 0;
  return fastKronSuccess;
}

// Pointers through which this process reaches every rank's receive area, result block and
// flag array (entry `rank` = the local buffers themselves).
fastKronError fkbMgPipeSetPeers(void* pipe, void* const recvPeers[], void* const resultPeers[],
                                void* const flagPeers[]) {
  MgPipe* p = reinterpret_cast<MgPipe*>(pipe);
  if (!p || !recvPeers || !resultPeers || !flagPeers) return fastKronInvalidArgument;
  for (int d = 0; d < p->rank.gk; d++) {
    if (!recvPeers[d] || !resultPeers[d] || !flagPeers[d]) return fastKronInvalidArgument;
    p->recvPeer[d] = recvPeers[d];
    p->resultPeer[d] = resultPeers[d];
    p->flagPeer[d] = reinterpret_cast<uint32_t*>(flagPeers[d]);
  }
  if (p->recvPeer[p->rank.g] != p->recv || p->resultPeer[p->rank.g] != p->result) return fastKronInvalidArgument;
  p->peersSet = true;
  return fastKronSuccess;
}

// x: this rank's [M][K/G] block on the device; Fs: host array of N device pointers.  With
// hostX / hostZ (pinned host memory, [M][K/G] and [M][L/G], contiguous) the call also moves
// the operands: every slice is copied in before its first pass and copied out as soon as it
// is complete, on side streams, so the copies of one slice overlap the passes of the others.
static fastKronError mgPipeRun(MgPipe* p, const float* x, const float* const Fs[], const float* hostX, float* hostZ) {
  if (!p || !Fs || !p->peersSet || (!x && !hostX)) return fastKronInvalidArgument;
  Engine* e = p->eng;
  p->compute = e->stream();
  p->seq++;
  const uint32_t Mi = p->rank.M;
  fastKronError err = fastKronSuccess;
  if (hostX) {
    if (!p->xdev && cudaMalloc(&p->xdev, (size_t)p->parts * Mi * p->Kloc * sizeof(float)) != cudaSuccess) {
      cudaGetLastError();
      return fastKronOtherError;
    }
    x = p->xdev;
    // the device copy of X may only be overwritten once the previous call has finished with it
    cudaEvent_t tail = p->evIn[0];
    if (cudaEventRecord(tail, p->compute) != cudaSuccess || cudaStreamWaitEvent(p->h2d, tail, 0) != cudaSuccess)
      return fastKronOtherError;
    for (int s = 0; s < p->parts; s++) {
      const size_t off = (size_t)s * Mi * p->Kloc;
      if (cudaMemcpyAsync(p->xdev + off, hostX + off, (size_t)Mi * p->Kloc * sizeof(float), cudaMemcpyHostToDevice,
                          p->h2d) != cudaSuccess ||
          cudaEventRecord(p->evIn[s], p->h2d) != cudaSuccess)
        return fastKronOtherError;
    }
  }
  if ((err = mgFork(p)) != fastKronSuccess) return err;
  std::vector<std::pair<int, int>> order;
  mgOrder(p->parts, &order);
  for (size_t o = 0; o < order.size() && err == fastKronSuccess; o++) {
    const int s = order[o].second;
    if (order[o].first == 1) {
      if (hostX && cudaStreamWaitEvent(mgLaneOf(p, s), p->evIn[s], 0) != cudaSuccess) return fastKronOtherError;
      err = mgEnqueueP1(p, s, x, Fs);
    } else {
      err = mgEnqueueP2(p, s, Fs[0]);
      if (err == fastKronSuccess && hostZ) {
        // slice s of the result leaves as soon as every rank's rows of it have landed
        err = mgWaitResult(p, s, p->d2h);
        const size_t off = (size_t)s * Mi * p->Lloc;
        if (err == fastKronSuccess &&
            cudaMemcpyAsync(hostZ + off, p->result + off, (size_t)Mi * p->Lloc * sizeof(float), cudaMemcpyDeviceToHost,
                            p->d2h) != cudaSuccess)
          err = fastKronOtherError;
      }
    }
  }
  for (int s = 0; s < p->parts && err == fastKronSuccess; s++) err = mgWaitResult(p, s, p->compute);
  if (err == fastKronSuccess && hostZ) {
    cudaEvent_t done = p->evC3[0];       // free again: every use of it in this call is enqueued
    if (cudaEventRecord(done, p->d2h) != cudaSuccess || cudaStreamWaitEvent(p->compute, done, 0) != cudaSuccess)
      err = fastKronOtherError;
  }
  return err;
}

fastKronError fkbMgPipeRun(void* pipe, const float* x, const float* const Fs[]) {
  return mgPipeRun(reinterpret_cast<MgPipe*>(pipe), x, Fs, nullptr, nullptr);
}
fastKronError fkbMgPipeRunHost(void* pipe, const float* hostX, const float* const Fs[], float* hostZ) {
  if (!hostX || !hostZ) return fastKronInvalidArgument;
  return mgPipeRun(reinterpret_cast<MgPipe*>(pipe), nullptr, Fs, hostX, hostZ);
}

void fkbMgPipeDestroy(void* pipe) { mgPipeDestroy(reinterpret_cast<MgPipe*>(pipe)); }

// Timing of the exchanges of the staged transport (measurement hook).  on != 0: the next calls
// record, per exchange (phase, slice), when its copies may start and when each side stream has
// finished them.  fkbMgPipeTraceGet synchronises the device and writes, for exchange e =
// phase*parts + slice, out[2e] = milliseconds from "may start" to the last copy's end and
// out[2e+1] = bytes this rank sent in it; returns the number of exchanges written.
fastKronError fkbMgPipeTrace(void* pipe, int on) {
  MgPipe* p = reinterpret_cast<MgPipe*>(pipe);
  if (!p) return fastKronInvalidArgument;
  if (on && p->trBegin.empty()) {
    for (int i = 0; i < 2 * p->parts; i++) { cudaEvent_t e; if (cudaEventCreate(&e) != cudaSuccess) return fastKronOtherError; p->trBegin.push_back(e); }
    for (int i = 0; i < 2 * p->parts * MgPipe::NC; i++) { cudaEvent_t e; if (cudaEventCreate(&e) != cudaSuccess) return fastKronOtherError; p->trEnd.push_back(e); }
  }
  p->trace = on != 0;
  return fastKronSuccess;
}
int fkbMgPipeTraceGet(void* pipe, double* out, int maxExchanges) {
  MgPipe* p = reinterpret_cast<MgPipe*>(pipe);
  if (!p || !out || p->trBegin.empty() || !p->staged) return 0;
  cudaDeviceSynchronize();
  const int G = p->rank.gk;
  int n = 0;
  for (int e = 0; e < 2 * p->parts && n < maxExchanges; e++, n++) {
    float worst = 0.f;
    for (int c = 0; c < p->nc; c++) {
      float ms = 0.f;
      if (cudaEventElapsedTime(&ms, p->trBegin[e], p->trEnd[(size_t)e * MgPipe::NC + c]) != cudaSuccess) { cudaGetLastError(); ms = 0.f; }
      if (ms > worst) worst = ms;
    }
    out[2 * n] = worst;
    out[2 * n + 1] = (double)(G - 1) * (double)(e < p->parts ? p->blk1 : p->blk2) * sizeof(float);
  }
  return n;
}

// The two redistribution maps as plain numbers, for host-side (CPU) tests of the schedule:
// out[0..6] = parts, qPer, aLoc, sM, sA, sQ, zOff.
fastKronError fkbMgScatterDesc(int phase, int rank, int world, uint32_t N, const uint32_t Ps[],
                               const uint32_t Qs[], long long out[7]) {
  if (!Ps || !Qs || !out) return fastKronInvalidArgument;
  MgRank r;
  r.g = rank; r.gk = world; r.M = 1; r.N = N; r.Ps = Ps; r.Qs = Qs;
  fastKronError err = mgCheck(r);
  if (err != fastKronSuccess) return err;
  Scatter sc;
  if (phase == 1) mgScatter1(r, &sc); else mgScatter2(r, &sc);
  out[0] = sc.parts; out[1] = (long long)sc.qPer; out[2] = (long long)sc.aLoc;
  out[3] = sc.sM; out[4] = sc.sA; out[5] = sc.sQ; out[6] = sc.zOff;
  return fastKronSuccess;
}

// The enqueue order of a call with `parts` row slices as (half, slice) pairs, for the CPU
// tests of the schedule: out[2*i] = 1 (first half) or 2 (second half), out[2*i+1] = slice.
int fkbMgOrder(int parts, int out[], int maxPairs) {
  std::vector<std::pair<int, int>> order;
  mgOrder(parts < 1 ? 1 : parts, &order);
  int n = 0;
  for (; n < (int)order.size() && n < maxPairs; n++) { out[2 * n] = order[n].first; out[2 * n + 1] = order[n].second; }
  return (int)order.size();
}

// CUDA IPC helpers so that a Python host can exchange buffer handles between ranks.
int fkbIpcExport(void* ptr, unsigned char handleOut[64]) {
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e == cudaSuccess) memcpy(handleOut, &h, sizeof(h));
  return (int)e;
}
int fkbIpcOpen(const unsigned char handleIn[64], void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handleIn, sizeof(h));
  return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}
int fkbIpcClose(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }

}  // extern "C"

// Multi-GPU GeMKM: the entry points of include/fastkronMg.h plus a per-rank form of the
// same two phases for one-process-per-GPU hosts.
//
// Distribution (same as the reference, src/handle/distrib_handle.cu:52-414 and
// src/handle/handle.cpp:411-416): GPU (r, c) of a gpusInM x gpusInK grid owns rows
// [r*M/GM, ...) and columns [c*K/GK, ...) of X and of the result; factors are replicated.
// Rows need no communication.  Columns do: with X as the tensor [M][P1][P2]...[PN], a
// column block is a range of the leading index p1.
//
//   phase 1  every GPU contracts modes N..2 of its block [M][P1/GK][P2..PN] locally.  The
//            pass that applies factor 2 does not write locally: output row (m, p1, q2)
//            goes to GPU q2 / (Q2/GK), which thereby receives [M][P1][Q2/GK][Q3..QN] --
//            all of p1, a slice of q2.  This is the all-to-all of the reference
//            (ncclSend/ncclRecv + pack/unpack kernels, distrib_handle.cu:276-347, or its
//            P2P store variant, src/kernels/cuda/global-store.cuh:1-25) fused into the
//            producing kernel as plain 128-bit peer stores over NVLink.
//   barrier  all GPUs of the row group finished phase 1.
//   phase 2  every GPU contracts mode 1 of what it received; output row (m, q1) goes to
//            GPU q1 / (Q1/GK) at its canonical place [M][Q1/GK][Q2][Q3..QN], again by peer
//            stores from the producing kernel.
//   barrier  the result blocks are complete.
//
// Two exchanges are the minimum for a column-sharded input and output.  Nothing here waits
// inside a kernel: ordering is by stream events (one process) or by a collective the host
// enqueues between the phases (one process per GPU), so the code is safe to emulate with
// several logical GPUs on one device.  No TMA multicast, no device-side flags.
//
// Requirements: N >= 2 when GK > 1, and GK divides P1, Q1 and Q2 (the reference has the
// analogous divisibility rules, src/kmm/kmmalgo.cpp:51-70).  fp32, row-major, opX = opF = N
// only, like the reference (distrib_handle.cu:247-250).

#include "engine.h"
#include "gemm_table.h"
#include "fastkronMg.h"

#include <string.h>
#include <vector>

namespace fkb {

struct MgState {
  int gpus = 1, gm = 1, gk = 1;
  bool oneDevice = false;                 // all logical GPUs live on the current device (emulation)
  std::vector<int> device;                // physical device of logical GPU g
  std::vector<cudaStream_t> stream;
  std::vector<int> smCount;
  std::vector<cudaEvent_t> ev1, ev2;
};

void mgAdjustSizes(const MgState* mg, const Problem& pr, size_t* yElems, size_t* tmpElems) {
  // per-device counts; the temporary is doubled: its second half is the receive area of the
  // first exchange (the reference doubles it for its NCCL staging, src/handle/handle.cpp:327-338)
  const uint64_t rows = pr.M / mg->gm;
  const uint64_t cols = (pr.N == 1) ? (pr.K() > pr.L() ? pr.K() : pr.L()) : pr.maxIntermediateCols();
  *yElems = (size_t)(rows * (pr.L() / mg->gk));
  *tmpElems = (size_t)(rows * (cols / mg->gk)) * (mg->gk > 1 ? 2 : 1);
}

void mgDestroy(MgState* mg) {
  if (!mg) return;
  for (cudaEvent_t e : mg->ev1) cudaEventDestroy(e);
  for (cudaEvent_t e : mg->ev2) cudaEventDestroy(e);
  delete mg;
}

// ---- the two phases for one rank --------------------------------------------------------

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

// Phase 1: modes N..2 of the local block; the last pass redistributes into recvPeers[d].
// stage: 0 = all passes, 1 = only the local passes, 2 = only the redistributing pass.
// packed: destination blocks hold only this rank's rows, [M][P1/G][Q2/G][B] (staged form).
static fastKronError mgPhase1(Engine* e, const MgRank& r, const float* x, const float* const* Fs, float* t1,
                              float* t2, void* const recvPeers[], int stage = 0, bool packed = false) {
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
    if ((stage == 1 && last) || (stage == 2 && !last)) continue;
    LaunchCtx cx;
    cx.stream = r.stream; cx.dt = DType::F32; cx.smCount = r.smCount; cx.tilesPerCta = e->tilesPerCta();
    auto buf = [&](Buf b) -> void* {
      switch (b) { case Buf::X: return const_cast<float*>(x); case Buf::T1: return t1; case Buf::T2: return t2;
                   default: return recvPeers[r.g]; }
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
      for (int d = 0; d < r.gk; d++) cx.scatter.base[d] = recvPeers[d];
    }
    err = e->launchPass(ps, cx);
    if (err != fastKronSuccess) return err;
  }
  return fastKronSuccess;
}

// Phase 2: mode 1 of the received tensor [M][P1][Q2/GK * Q3..QN]; rows go to resultPeers[d].
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
  cx.stream = r.stream; cx.dt = DType::F32; cx.smCount = r.smCount; cx.tilesPerCta = e->tilesPerCta();
  cx.src = recv; cx.dst = resultPeers[r.g];
  cx.F[0] = F0;
  factorStrides(MMType::MKM, fastKronOp_N, ps.P[0], ps.Q[0], &cx.fsP, &cx.fsQ);
  mgScatter2(r, &cx.scatter);
  for (int d = 0; d < r.gk; d++) cx.scatter.base[d] = resultPeers[d];
  return e->launchPass(ps, cx);
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
  // peer access for the direct stores (reference: cuda_kernel_db.cu:83-93)
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

  fastKronError err = fastKronSuccess;
  auto streamOf = [&](int g) { return st ? st[g] : mg->stream[g]; };

  if (mg->gk == 1) {
    // rows only: every GPU runs the ordinary single-device plan on its rows
    for (int g = 0; g < mg->gpus && err == fastKronSuccess; g++) {
      cudaSetDevice(mg->device[g]);
      Problem lp = full; lp.M = M / mg->gm;
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
    // phase 1 on every GPU
    for (int g = 0; g < mg->gpus && err == fastKronSuccess; g++) {
      cudaSetDevice(mg->device[g]);
      const int row = g / mg->gk, col = g % mg->gk;
      MgRank r;
      r.g = col; r.gk = mg->gk; r.M = M / mg->gm; r.N = n; r.Ps = KronMatRows; r.Qs = KronMatCols;
      r.stream = streamOf(g); r.smCount = mg->smCount[g];
      void* recv[kMaxParts];
      for (int d = 0; d < mg->gk; d++) recv[d] = (float*)temp1[row * mg->gk + d] + half;
      err = mgPhase1(e, r, (const float*)x[g], reinterpret_cast<const float* const*>(&kronMats[(size_t)g * n]),
                     (float*)temp1[g], (float*)temp2[g], recv);
      if (err == fastKronSuccess && cudaEventRecord(mg->ev1[g], streamOf(g)) != cudaSuccess) err = fastKronOtherError;
    }
    // phase 2 once the whole row group delivered
    for (int g = 0; g < mg->gpus && err == fastKronSuccess; g++) {
      cudaSetDevice(mg->device[g]);
      const int row = g / mg->gk, col = g % mg->gk;
      for (int d = 0; d < mg->gk; d++) cudaStreamWaitEvent(streamOf(g), mg->ev1[row * mg->gk + d], 0);
      MgRank r;
      r.g = col; r.gk = mg->gk; r.M = M / mg->gm; r.N = n; r.Ps = KronMatRows; r.Qs = KronMatCols;
      r.stream = streamOf(g); r.smCount = mg->smCount[g];
      void* res[kMaxParts];
      for (int d = 0; d < mg->gk; d++) res[d] = result[row * mg->gk + d];
      err = mgPhase2(e, r, (const float*)temp1[g] + half, (const float*)kronMats[(size_t)g * n], res);
      if (err == fastKronSuccess && cudaEventRecord(mg->ev2[g], streamOf(g)) != cudaSuccess) err = fastKronOtherError;
    }
  }
  // the call is blocking, like the reference's (it joins its per-GPU threads)
  for (int g = 0; g < mg->gpus; g++) {
    cudaSetDevice(mg->device[g]);
    if (cudaStreamSynchronize(streamOf(g)) != cudaSuccess && err == fastKronSuccess) err = cudaToFk(cudaGetLastError());
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

// ---- per-rank form for one-process-per-GPU hosts (not part of the reference ABI) --------
// The host program owns the ranks (e.g. torch.distributed): it passes, for every rank of
// the column group, a pointer this process can store to (a CUDA IPC mapping), runs
// fkbMgRankPhase1 on every rank, enqueues a collective barrier on the same stream, runs
// fkbMgRankPhase2, and a second barrier.  `handle` must have been given its stream with
// fastKronInitCUDA.  M is the number of local rows.

fastKronError fkbMgRankPhase1(fastKronHandle handle, int rank, int world, uint32_t M, uint32_t N,
                              uint32_t Ps[], uint32_t Qs[], const float* x, const float* const Fs[],
                              float* temp1, float* temp2, void* const peerRecv[]) {
  if (!handle || !Ps || !Qs || !x || !Fs || !temp1 || !temp2 || !peerRecv) return fastKronInvalidArgument;
  Engine* e = E(handle);
  if (!e->cudaReady()) return fastKronBackendNotAvailable;
  MgRank r;
  r.g = rank; r.gk = world; r.M = M; r.N = N; r.Ps = Ps; r.Qs = Qs; r.stream = e->stream(); r.smCount = e->smCount();
  return mgPhase1(e, r, x, Fs, temp1, temp2, peerRecv);
}

// The same phase in two calls, so that a host can put an event between the local passes
// (stage 1) and the redistributing pass (stage 2).
fastKronError fkbMgRankPhase1Stage(fastKronHandle handle, int rank, int world, uint32_t M, uint32_t N,
                                   uint32_t Ps[], uint32_t Qs[], const float* x, const float* const Fs[],
                                   float* temp1, float* temp2, void* const peerRecv[], int stage) {
  if (!handle || !Ps || !Qs || !x || !Fs || !temp1 || !temp2 || !peerRecv || stage < 1 || stage > 2)
    return fastKronInvalidArgument;
  Engine* e = E(handle);
  if (!e->cudaReady()) return fastKronBackendNotAvailable;
  MgRank r;
  r.g = rank; r.gk = world; r.M = M; r.N = N; r.Ps = Ps; r.Qs = Qs; r.stream = e->stream(); r.smCount = e->smCount();
  return mgPhase1(e, r, x, Fs, temp1, temp2, peerRecv, stage);
}

fastKronError fkbMgRankPhase2(fastKronHandle handle, int rank, int world, uint32_t M, uint32_t N,
                              uint32_t Ps[], uint32_t Qs[], const float* recv, const float* F0,
                              void* const peerResult[]) {
  if (!handle || !Ps || !Qs || !recv || !F0 || !peerResult) return fastKronInvalidArgument;
  Engine* e = E(handle);
  if (!e->cudaReady()) return fastKronBackendNotAvailable;
  MgRank r;
  r.g = rank; r.gk = world; r.M = M; r.N = N; r.Ps = Ps; r.Qs = Qs; r.stream = e->stream(); r.smCount = e->smCount();
  return mgPhase2(e, r, recv, F0, peerResult);
}

// ---- staged form: the kernels write per-destination blocks into LOCAL staging buffers and
// the host moves the blocks with copy engines (cudaMemcpyAsync / cudaMemcpy2DAsync to
// IPC-mapped peer buffers), so NVLink traffic needs no SM and overlaps other rows' passes.
// Large-factor (64/128) shapes only: the phase-2 kernel reads its input as received,
// [sender][M][P1/G][B2].
//   stage1: G blocks of M*(P1/G)*(Q2/G)*B elements, block d = [M][P1/G][Q2/G][B] for rank d
//   recv  : G blocks of the same size, block s = what rank s staged for this rank
//   stage2: G blocks of M*(Q1/G)*B2 elements, block d = [M][Q1/G][B2] for rank d, to be placed
//           at columns [g*B2, (g+1)*B2) of rank d's [M*(Q1/G)][Q2*B] result.
fastKronError fkbMgRankPhase1Staged(fastKronHandle handle, int rank, int world, uint32_t M, uint32_t N,
                                    uint32_t Ps[], uint32_t Qs[], const float* x, const float* const Fs[],
                                    float* temp1, float* temp2, float* stage1, int stage) {
  if (!handle || !Ps || !Qs || !x || !Fs || !temp1 || !temp2 || !stage1 || stage < 0 || stage > 2)
    return fastKronInvalidArgument;
  Engine* e = E(handle);
  if (!e->cudaReady()) return fastKronBackendNotAvailable;
  MgRank r;
  r.g = rank; r.gk = world; r.M = M; r.N = N; r.Ps = Ps; r.Qs = Qs; r.stream = e->stream(); r.smCount = e->smCount();
  fastKronError err = mgCheck(r);
  if (err != fastKronSuccess) return err;
  const uint64_t p1loc = Ps[0] / world, q2loc = Qs[1] / world, B = prodQ(r, 2);
  const uint64_t blk = (uint64_t)M * p1loc * q2loc * B;
  void* bases[kMaxParts];
  for (int d = 0; d < world; d++) bases[d] = stage1 + (size_t)d * blk;
  // same kernels as the fused form; only the redistribution map differs (all bases local,
  // rows of a block packed as [M][P1/G][Q2/G][B])
  return mgPhase1(e, r, x, Fs, temp1, temp2, bases, stage, /*packed=*/true);
}

fastKronError fkbMgRankPhase2Staged(fastKronHandle handle, int rank, int world, uint32_t M, uint32_t N,
                                    uint32_t Ps[], uint32_t Qs[], const float* recv, const float* F0,
                                    float* stage2) {
  if (!handle || !Ps || !Qs || !recv || !F0 || !stage2) return fastKronInvalidArgument;
  Engine* e = E(handle);
  if (!e->cudaReady()) return fastKronBackendNotAvailable;
  MgRank r;
  r.g = rank; r.gk = world; r.M = M; r.N = N; r.Ps = Ps; r.Qs = Qs; r.stream = e->stream(); r.smCount = e->smCount();
  fastKronError err = mgCheck(r);
  if (err != fastKronSuccess) return err;
  const uint64_t p1loc = Ps[0] / world, q1loc = Qs[0] / world;
  const uint64_t B2 = (Qs[1] / world) * prodQ(r, 2);
  if (!gemmEligible(DType::F32, Ps[0], Qs[0], B2) || B2 % (uint64_t)gemmTileJ(DType::F32) != 0)
    return fastKronKernelNotFound;
  Pass ps;
  ps.f0 = 0; ps.nf = 1; ps.M = M; ps.A = 1; ps.B = B2;
  ps.P[0] = Ps[0]; ps.Q[0] = Qs[0];
  ps.xsM = (int64_t)(Ps[0] * B2); ps.xsA = ps.xsM; ps.xsG = (int64_t)B2; ps.xsB = 1;
  ps.zsM = (int64_t)(Qs[0] * B2); ps.zsA = ps.zsM; ps.zsG = (int64_t)B2; ps.zsB = 1;
  ps.kind = KernelKind::Gemm;
  LaunchCtx cx;
  cx.stream = r.stream; cx.dt = DType::F32; cx.smCount = r.smCount; cx.tilesPerCta = e->tilesPerCta();
  cx.src = recv; cx.dst = stage2;
  cx.F[0] = F0;
  factorStrides(MMType::MKM, fastKronOp_N, ps.P[0], ps.Q[0], &cx.fsP, &cx.fsQ);
  cx.pSplit = (unsigned)p1loc; cx.pOuter = (unsigned long long)M * p1loc * B2; cx.nStride = p1loc * B2;
  cx.scatter.parts = world; cx.scatter.qPer = q1loc; cx.scatter.aLoc = 1;
  cx.scatter.sM = (long long)(q1loc * B2); cx.scatter.sA = 0; cx.scatter.sQ = (long long)B2; cx.scatter.zOff = 0;
  const uint64_t blk = (uint64_t)M * q1loc * B2;
  for (int d = 0; d < world; d++) cx.scatter.base[d] = stage2 + (size_t)d * blk;
  // the launcher refuses the split input unless it runs the kernel: no generic fallback here
  fastKronError le = launchGemm(ps, cx);
  return le;
}

// Stream-ordered copies for the staged form (plain cudaMemcpyAsync / cudaMemcpy2DAsync,
// device to device; the destination may be an IPC mapping of a peer's buffer).
int fkbCopyAsync(void* dst, const void* src, size_t bytes, void* stream) {
  return (int)cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
}
int fkbCopy2DAsync(void* dst, size_t dpitch, const void* src, size_t spitch, size_t widthBytes, size_t height,
                   void* stream) {
  return (int)cudaMemcpy2DAsync(dst, dpitch, src, spitch, widthBytes, height, cudaMemcpyDeviceToDevice,
                                (cudaStream_t)stream);
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

// CUDA IPC helpers so that a Python host can exchange buffer handles between ranks.
int fkbIpcAlloc(void** ptr, size_t bytes) { return (int)cudaMalloc(ptr, bytes); }
int fkbIpcFree(void* ptr) { return (int)cudaFree(ptr); }
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

// Engine: validates a call the way the reference's handle does
// (src/handle/handle.cpp:114-199), plans it, and enqueues the passes.

#include "engine.h"

#include <sstream>
#include <stdio.h>
#include <string.h>

namespace fkb {

Engine::Engine(uint32_t backends) : backends_(backends) {}
Engine::~Engine() {
  if (mg) mgDestroy(mg);
  for (cudaEvent_t ev : evPool_) cudaEventDestroy(ev);
}

static unsigned long long gLaunches = 0;
unsigned long long Engine::launchCount() { return gLaunches; }

int Engine::passTimes(float* ms, int* kinds, int maxN) {
  const int n = (int)(evUsed_ / 2);
  int out = 0;
  for (int i = 0; i < n && out < maxN; i++, out++) {
    cudaEventSynchronize(evPool_[2 * i + 1]);
    float t = 0.f;
    cudaEventElapsedTime(&t, evPool_[2 * i], evPool_[2 * i + 1]);
    ms[out] = t;
    if (kinds) kinds[out] = evKinds_[i];
  }
  evUsed_ = 0;
  evKinds_.clear();
  return out;
}

fastKronError Engine::initCUDA(void* ptrToStream) {
  if (!hasBackend(fastKronBackend_CUDA)) return fastKronBackendNotAvailable;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return fastKronBackendNotAvailable; }
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) { cudaGetLastError(); return fastKronBackendNotAvailable; }
  // the kernels in this library are built for sm_100a only
  if (prop.major != 10) return fastKronBackendNotAvailable;
  device_ = dev;
  smCount_ = prop.multiProcessorCount;
  stream_ = ptrToStream ? *reinterpret_cast<cudaStream_t*>(ptrToStream) : nullptr;
  cudaReady_ = true;
  return fastKronSuccess;
}

fastKronError Engine::setStream(void* ptrToStream) {
  if (!ptrToStream) return fastKronInvalidArgument;
  if (!hasBackend(fastKronBackend_CUDA)) return fastKronBackendNotAvailable;
  stream_ = *reinterpret_cast<cudaStream_t*>(ptrToStream);
  return fastKronSuccess;
}

// Sizes follow the reference (src/handle/handle.cpp:305-342, 375-414): the
// result has M*L elements; a temporary must hold the widest matrix produced by
// any single-factor step (for one factor: the wider of X and Z).
fastKronError Engine::sizes(const Problem& pr, size_t* yElems, size_t* tmpElems) const {
  if (!yElems || !tmpElems) return fastKronInvalidArgument;
  if (pr.N == 0 || pr.N > (uint32_t)kMaxFactors) return fastKronInvalidArgument;
  const uint64_t L = pr.L(), K = pr.K();
  uint64_t cols = (pr.N == 1) ? (K > L ? K : L) : pr.maxIntermediateCols();
  *yElems = (size_t)pr.M * L;
  *tmpElems = (size_t)pr.M * cols;
  return fastKronSuccess;
}

fastKronError Engine::sizesForward(const Problem& pr, size_t* yElems, size_t* interElems) const {
  if (!yElems || !interElems) return fastKronInvalidArgument;
  if (pr.N == 0 || pr.N > (uint32_t)kMaxFactors) return fastKronInvalidArgument;
  for (uint32_t i = 1; i < pr.N; i++) interElems[i - 1] = (size_t)pr.M * pr.colsAfter(i);
  *yElems = (size_t)pr.M * pr.L();
  return fastKronSuccess;
}

static std::string planKey(const Problem& pr, const PlanOptions& o) {
  std::ostringstream os;
  os << (int)pr.mm << ':' << (int)pr.dt << ':' << pr.M << ':' << pr.N << ':' << (int)pr.opX << ':'
     << (int)pr.opF << ':' << pr.forward << ':' << o.fusion << o.haveT2 << o.forceGeneric << ':' << o.align;
  for (uint32_t i = 0; i < pr.N; i++) os << ':' << pr.P[i] << 'x' << pr.Q[i];
  return os.str();
}

// 0 = silent, 1 = INFO, 2 = DEBUG; read once from FASTKRON_LOG.
static int logLevel() {
  static const int lv = [] {
    const char* e = getenv("FASTKRON_LOG");
    if (!e) return 0;
    if (!strcmp(e, "INFO") || !strcmp(e, "info")) return 1;
    if (!strcmp(e, "DEBUG") || !strcmp(e, "debug")) return 2;
    return 0;
  }();
  return lv;
}

static int ptrAlign(const void* p) {
  const uintptr_t v = (uintptr_t)p;
  if (!p) return 16;
  return (v & 15) == 0 ? 16 : ((v & 7) == 0 ? 8 : 4);
}

fastKronError Engine::run(Problem pr, const CallOperands& ops) {
  if (!cudaReady_) return fastKronBackendNotAvailable;
  if (pr.N == 0 || pr.N > (uint32_t)kMaxFactors || pr.M == 0 || pr.batch == 0) return fastKronInvalidArgument;
  if (!ops.X || !ops.Fs || !ops.Z) return fastKronInvalidArgument;
  for (uint32_t i = 0; i < pr.N; i++) {
    if (pr.P[i] == 0 || pr.Q[i] == 0 || ops.Fs[i] == nullptr) return fastKronInvalidArgument;
  }
  if (pr.forward) {
    if (pr.N > 1 && !ops.intermediates) return fastKronInvalidArgument;
    for (uint32_t i = 0; i + 1 < pr.N; i++) if (!ops.intermediates[i]) return fastKronInvalidArgument;
  } else {
    if (!ops.temp1) return fastKronInvalidArgument;
    if ((const void*)ops.Z == ops.Y && !ops.temp2) return fastKronInvalidArgument;
    if (ops.beta != 0.0 && !ops.Y) return fastKronInvalidArgument;
  }

  // A KMM with a single column is an MKM with a single row whose factors are
  // read with the opposite op (reference: src/handle/handle.cpp:134-138).
  if (pr.mm == MMType::KMM && pr.M == 1) {
    pr.mm = MMType::MKM;
    pr.opX = fastKronOp_N;
    pr.opF = (pr.opF == fastKronOp_N) ? fastKronOp_T : fastKronOp_N;
  }

  const size_t es = dtypeSize(pr.dt);
  PlanOptions po;
  po.fusion = (options_ & fastKronOptionsUseFusion) != 0;
  po.haveT2 = ops.temp2 != nullptr;
  int al = 16;
  auto upd = [&](const void* p) { int a = ptrAlign(p); if (a < al) al = a; };
  upd(ops.X); upd(ops.Z); upd(ops.temp1); upd(ops.temp2);
  if (ops.beta != 0.0) upd(ops.Y);
  if (pr.forward) for (uint32_t i = 0; i + 1 < pr.N; i++) upd(ops.intermediates[i]);
  size_t yElems = 0, tmpElems = 0;
  sizes(pr, &yElems, &tmpElems);
  if (pr.batch > 1) {
    auto updS = [&](uint64_t s) { if ((s * es) % 16 != 0) al = 4; };
    updS(ops.strideX); updS(ops.strideZ); updS(tmpElems);
    if (ops.beta != 0.0) updS(ops.strideY);
    if (pr.forward && ops.strideI) for (uint32_t i = 0; i + 1 < pr.N; i++) updS(ops.strideI[i]);
  }
  po.align = al;

  // A batch of GeMKMs that shares its factors and whose X, Z (and Y) entries lie back to
  // back is one GeMKM with batch*M rows: rows are independent.  (The reference launches
  // its kernels with a batch grid dimension instead, src/kernels/gpu_kmmkernel.h:124-144.)
  if (pr.batch > 1 && pr.mm == MMType::MKM && pr.opX == fastKronOp_N && !pr.forward && ops.strideF &&
      (uint64_t)pr.M * pr.batch < (1ull << 32)) {
    bool shared = true;
    for (uint32_t i = 0; i < pr.N; i++) shared = shared && ops.strideF[i] == 0;
    const uint64_t K = pr.K(), L = pr.L();
    if (shared && ops.strideX == (uint64_t)pr.M * K && ops.strideZ == (uint64_t)pr.M * L &&
        (ops.beta == 0.0 || ops.strideY == (uint64_t)pr.M * L)) {
      Problem folded = pr;
      folded.M = pr.M * pr.batch;
      folded.batch = 1;
      return run(folded, ops);
    }
  }

  const std::string key = planKey(pr, po);
  auto it = planCache_.find(key);
  if (it == planCache_.end()) {
    Plan plan;
    fastKronError e = makePlan(pr, po, &plan);
    if (e != fastKronSuccess) return e;
    // fastKronOptionsTune: time candidate plans once on the caller's own buffers (X and the
    // factors are never written; Z and the temporaries are scratch until the real run) and keep
    // the fastest.  Candidates: the table's plan, the unfused plan, and every distinct plan that
    // a cap on the fusion depth produces (4+4, 3+3+2, 2+2+2+2, ...).  Skipped when Z aliases Y,
    // whose contents the trial runs would destroy.  (Role of the reference's Autotuner::tune,
    // src/autotuner/autotuner.cpp:24-328, with the candidates reduced to what differs here: the
    // kernels' own parameters are tuned offline, fastkron_b200/tune.py.)
    if ((options_ & fastKronOptionsTune) != 0 && pr.batch == 1 && (const void*)ops.Z != ops.Y) {
      std::vector<std::string> seen{plan.describe()};
      float best = timePlan(pr, plan, ops);
      for (int cap = 1; cap <= kMaxGroup && best > 0.f; cap++) {
        PlanOptions alt = po;
        alt.fusion = true;
        alt.maxFuse = cap;
        Plan other;
        if (makePlan(pr, alt, &other) != fastKronSuccess) continue;
        const std::string d = other.describe();
        bool dup = false;
        for (const std::string& s2 : seen) dup = dup || s2 == d;
        if (dup) continue;
        seen.push_back(d);
        const float t = timePlan(pr, other, ops);
        if (t > 0.f && t < best) { best = t; plan = other; }
      }
    }
    // FASTKRON_LOG=INFO (or DEBUG): one block per newly planned problem, as the reference prints
    // its chosen kernel series (src/env/env.cpp:57-65, src/handle/handle.cpp:160-170).
    if (logLevel() >= 1) fprintf(stderr, "[FastKron] plan %s\n%s", key.c_str(), plan.describe().c_str());
    it = planCache_.emplace(key, std::move(plan)).first;
  }
  const Plan& plan = it->second;

  if (pr.batch == 1) return execute(pr, plan, ops, stream_, smCount());

  // Strided batch in one launch per pass when every pass's kernel takes the batch as a grid
  // dimension (the reference batches in grid.z, src/kernels/gpu_kmmkernel.h:124-144) ...
  bool oneLaunch = true;
  for (const Pass& ps : plan.passes) oneLaunch = oneLaunch && passBatchCapable(ps);
  if (oneLaunch) return execute(pr, plan, ops, stream_, smCount(), pr.batch, tmpElems);

  // ... otherwise the same plan once per entry, on offset operands.
  std::vector<const void*> fs(pr.N);
  std::vector<void*> inter(pr.N > 1 ? pr.N - 1 : 0);
  for (uint32_t b = 0; b < pr.batch; b++) {
    CallOperands o = ops;
    o.X = (const char*)ops.X + (size_t)b * ops.strideX * es;
    o.Z = (char*)ops.Z + (size_t)b * ops.strideZ * es;
    if (ops.Y) o.Y = (const char*)ops.Y + (size_t)b * ops.strideY * es;
    if (ops.temp1) o.temp1 = (char*)ops.temp1 + (size_t)b * tmpElems * es;
    if (ops.temp2) o.temp2 = (char*)ops.temp2 + (size_t)b * tmpElems * es;
    for (uint32_t i = 0; i < pr.N; i++)
      fs[i] = (const char*)ops.Fs[i] + (size_t)b * (ops.strideF ? ops.strideF[i] : 0) * es;
    o.Fs = fs.data();
    if (pr.forward && pr.N > 1) {
      for (uint32_t i = 0; i + 1 < pr.N; i++) {
        const uint64_t s = ops.strideI ? ops.strideI[i] : (uint64_t)pr.M * pr.colsAfter(i + 1);
        inter[i] = (char*)ops.intermediates[i] + (size_t)b * s * es;
      }
      o.intermediates = inter.data();
    }
    fastKronError e = execute(pr, plan, o, stream_, smCount());
    if (e != fastKronSuccess) return e;
  }
  return fastKronSuccess;
}

// Average device time (ms) of a plan over three runs after one warm-up; negative on failure.
float Engine::timePlan(const Problem& pr, const Plan& plan, const CallOperands& ops) {
  cudaEvent_t a, b;
  if (cudaEventCreate(&a) != cudaSuccess) return -1.f;
  if (cudaEventCreate(&b) != cudaSuccess) { cudaEventDestroy(a); return -1.f; }
  float ms = -1.f;
  if (execute(pr, plan, ops, stream_, smCount()) == fastKronSuccess) {
    cudaEventRecord(a, stream_);
    bool ok = true;
    for (int i = 0; i < 3 && ok; i++) ok = execute(pr, plan, ops, stream_, smCount()) == fastKronSuccess;
    cudaEventRecord(b, stream_);
    if (ok && cudaEventSynchronize(b) == cudaSuccess && cudaEventElapsedTime(&ms, a, b) == cudaSuccess) ms /= 3.f;
    else ms = -1.f;
  }
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  return ms;
}

// One kernel launch: the pass's own kernel family, the generic kernel when that family
// declines a single-factor pass, optional event bracketing for the benchmark.
fastKronError Engine::launchPass(const Pass& ps, const LaunchCtx& cx) {
  cudaStream_t stream = cx.stream;
  cudaEvent_t evEnd = nullptr;
  if (profiling_) {
    while (evPool_.size() < evUsed_ + 2) {
      cudaEvent_t ev;
      if (cudaEventCreate(&ev) != cudaSuccess) return fastKronOtherError;
      evPool_.push_back(ev);
    }
    cudaEventRecord(evPool_[evUsed_], stream);
    evEnd = evPool_[evUsed_ + 1];
    evUsed_ += 2;
  }
  int ranKind = (int)ps.kind;
  fastKronError e = fastKronKernelNotFound;
  if (ps.kind == KernelKind::Tile) e = launchTile(ps, cx);
  else if (ps.kind == KernelKind::Gemm) e = launchGemm(ps, cx);
  if (e == fastKronKernelNotFound && ps.nf == 1) { e = launchGeneric(ps, cx); ranKind = (int)KernelKind::Generic; }
  if (evEnd) { cudaEventRecord(evEnd, stream); evKinds_.push_back(ranKind); }
  if (e != fastKronSuccess) return e;
  gLaunches++;
  return fastKronSuccess;
}

fastKronError Engine::execute(const Problem& pr, const Plan& plan, const CallOperands& ops,
                              cudaStream_t stream, int smCount, uint32_t batch, size_t tmpElems) {
  auto resolve = [&](Buf b) -> void* {
    switch (b) {
      case Buf::X:  return const_cast<void*>(ops.X);
      case Buf::T1: return ops.temp1;
      case Buf::T2: return ops.temp2;
      case Buf::Z:  return ops.Z;
      default:      return ops.intermediates ? ops.intermediates[(int)b - (int)Buf::I0] : nullptr;
    }
  };
  // alpha = 1 without a beta*Y term is no epilogue at all: the last pass then takes the kernels'
  // plain store path
  const bool trivialEpilogue = ops.alpha == 1.0 && (ops.beta == 0.0 || ops.Y == nullptr);
  for (const Pass& planned : plan.passes) {
    Pass ps = planned;
    if (trivialEpilogue) ps.epilogue = false;
    LaunchCtx cx;
    cx.stream = stream;
    cx.dt = pr.dt;
    cx.src = resolve(ps.src);
    cx.dst = resolve(ps.dst);
    if (!cx.src || !cx.dst || cx.dst == ops.X) return fastKronInvalidArgument;
    cx.Y = ps.epilogue ? ops.Y : nullptr;
    cx.alpha = ps.epilogue ? ops.alpha : 1.0;
    cx.beta = ps.epilogue ? ops.beta : 0.0;
    cx.smCount = smCount;
    cx.tf32 = tf32Mode();
    for (int k = 0; k < ps.nf; k++) cx.F[k] = ops.Fs[ps.f0 + k];
    factorStrides(pr.mm, pr.opF, ps.P[0], ps.Q[0], &cx.fsP, &cx.fsQ);
    if (batch > 1) {
      // element distance between the batch entries of a logical buffer
      auto strideOf = [&](Buf b) -> uint64_t {
        switch (b) {
          case Buf::X:  return ops.strideX;
          case Buf::T1: case Buf::T2: return tmpElems;
          case Buf::Z:  return ops.strideZ;
          default: {
            const int k = (int)b - (int)Buf::I0;
            return ops.strideI ? ops.strideI[k] : (uint64_t)pr.M * pr.colsAfter((uint32_t)k + 1);
          }
        }
      };
      cx.batch = batch;
      cx.bsX = strideOf(ps.src);
      cx.bsZ = strideOf(ps.dst);
      cx.bsY = ops.strideY;
      for (int k = 0; k < ps.nf; k++) cx.bsF[k] = ops.strideF ? ops.strideF[ps.f0 + k] : 0;
    }

    fastKronError e = launchPass(ps, cx);
    if (e != fastKronSuccess) return e;
  }
  return fastKronSuccess;
}

}  // namespace fkb

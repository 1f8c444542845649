// welder-multi: the chain on several GPUs of one machine, from ONE native process.
//
//   welder-multi --workload rows|batch|cols [--gpus N] [--steps K] [--warmup W]
//                [--batch b] [--m M] [--n N] [--k K] [--scale s]
//
// One host thread, one stream and one pair of events per GPU; NCCL communicators from
// ncclCommInitAll.  Work is shared the three ways the chain allows:
//   rows   every GPU runs its own M rows against a replicated B        (no collective)
//   batch  the batches are split over the GPUs                          (no collective)
//   cols   the columns are split on 256-column tile boundaries; every GPU leaves un-normalised
//          exp values and one (max, sum) pair per row, ONE ncclAllGather of the pairs
//          ([rows, 2] f32 per GPU over NVLink) lets each GPU normalise its own columns
//          (wtc_matmul_softmax_partial_launch / _finish_launch)
// A step is timed on every device between its own events after a common host barrier; the
// step time is the maximum over the devices.  Inputs are synthetic (xorshift values in
// [-1, 1) rounded to f16; the weights of `cols` scaled by 0.02).  After the timed loop a few
// rows are read back and their sums checked against 1 (over all GPUs' columns for `cols`).
// The reference is single-GPU (its profiler takes one context: solver/WelderProfiler.cpp:296-303);
// this tool is the multi-GPU process model of this build in native code.
#include "../../../include/wtc_launch.h"

#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <filesystem>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace {

struct Api {
  decltype(&wtc_matmul_softmax_launch) launch = nullptr;
  decltype(&wtc_matmul_softmax_partial_launch) partial = nullptr;
  decltype(&wtc_matmul_softmax_finish_launch) finish = nullptr;
  decltype(&wtc_matmul_softmax_workspace_bytes) wsBytes = nullptr;
  decltype(&wtc_check_device_status) status = nullptr;
  decltype(&wtc_last_error) lastError = nullptr;
};
struct Nccl {
  ncclResult_t (*commInitAll)(ncclComm_t *, int, const int *) = nullptr;
  ncclResult_t (*allGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*commDestroy)(ncclComm_t) = nullptr;
  const char *(*errorString)(ncclResult_t) = nullptr;
};

// reusable barrier for the worker threads
class Barrier {
public:
  explicit Barrier(int n) : n_(n) {}
  void wait() {
    std::unique_lock<std::mutex> lk(mu_);
    const int gen = gen_;
    if (++count_ == n_) { count_ = 0; ++gen_; cv_.notify_all(); }
    else cv_.wait(lk, [&] { return gen != gen_; });
  }
private:
  std::mutex mu_;
  std::condition_variable cv_;
  int n_, count_ = 0, gen_ = 0;
};

uint16_t f32_to_f16(float f) {   // round to nearest even; inputs here are small normals or zero
  uint32_t u; std::memcpy(&u, &f, 4);
  const uint32_t sign = (u >> 16) & 0x8000u;
  int32_t exp = static_cast<int32_t>((u >> 23) & 0xFF) - 127 + 15;
  uint32_t mant = u & 0x7FFFFFu;
  if (exp <= 0) {
    if (exp < -10) return static_cast<uint16_t>(sign);
    mant |= 0x800000u;
    const int shift = 14 - exp;
    uint32_t h = mant >> shift;
    const uint32_t rem = mant & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1))) ++h;
    return static_cast<uint16_t>(sign | h);
  }
  if (exp >= 31) return static_cast<uint16_t>(sign | 0x7C00u);
  uint32_t h = (static_cast<uint32_t>(exp) << 10) | (mant >> 13);
  const uint32_t rem = mant & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) ++h;
  return static_cast<uint16_t>(sign | h);
}
float f16_to_f32(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1F, mant = h & 0x3FFu;
  uint32_t u;
  if (exp == 0) {
    if (mant == 0) u = sign;
    else { int e = -1; uint32_t m = mant; do { ++e; m <<= 1; } while (!(m & 0x400u)); u = sign | ((127 - 15 - e) << 23) | ((m & 0x3FFu) << 13); }
  } else if (exp == 31) u = sign | 0x7F800000u | (mant << 13);
  else u = sign | ((exp - 15 + 127) << 23) | (mant << 13);
  float f; std::memcpy(&f, &u, 4);
  return f;
}
void fill_f16(std::vector<uint16_t> &v, uint32_t seed, float sigma) {
  uint32_t s = seed ? seed : 1;
  for (auto &x : v) {
    s ^= s << 13; s ^= s >> 17; s ^= s << 5;
    x = f32_to_f16((static_cast<float>(s) * (1.0f / 4294967296.0f) * 2.0f - 1.0f) * sigma);
  }
}

#define CKC(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { std::fprintf(stderr, "CUDA error in %s: %s\n", #call, cudaGetErrorString(e_)); failed = true; } } while (0)

} // namespace

int main(int argc, char **argv) {
  std::string workload = "rows";
  int gpus = 1, steps = 20, warmup = 5;
  long long batch = 0, M = 0, N = 0, K = 0;
  double scale = 0.0;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    auto val = [&]() -> std::string { return i + 1 < argc ? argv[++i] : ""; };
    if (a == "--workload") workload = val();
    else if (a == "--gpus") gpus = std::atoi(val().c_str());
    else if (a == "--steps") steps = std::atoi(val().c_str());
    else if (a == "--warmup") warmup = std::atoi(val().c_str());
    else if (a == "--batch") batch = std::atoll(val().c_str());
    else if (a == "--m") M = std::atoll(val().c_str());
    else if (a == "--n") N = std::atoll(val().c_str());
    else if (a == "--k") K = std::atoll(val().c_str());
    else if (a == "--scale") scale = std::atof(val().c_str());
    else { std::fprintf(stderr, "usage: welder-multi --workload rows|batch|cols [--gpus N] [--steps K] [--warmup W] [--batch b] [--m M] [--n N] [--k K] [--scale s]\n"); return 2; }
  }
  if (workload != "rows" && workload != "batch" && workload != "cols") { std::fprintf(stderr, "error: unknown workload %s\n", workload.c_str()); return 2; }
  if (gpus < 1 || gpus > 16 || steps < 1 || warmup < 0) { std::fprintf(stderr, "error: bad --gpus/--steps/--warmup\n"); return 2; }
  // defaults: the benchmark configurations the three ways of sharing were measured on
  float sigmaB = 1.0f;
  if (workload == "rows") { if (!batch) batch = 1; if (!M) M = 4096; if (!N) N = 1024; if (!K) K = 1024; if (scale == 0.0) scale = 1.0 / 32; }
  if (workload == "batch") { if (!batch) batch = 64; if (!M) M = 2048; if (!N) N = 2048; if (!K) K = 128; if (scale == 0.0) scale = 1.0 / std::sqrt(128.0); }
  if (workload == "cols") { if (!batch) batch = 1; if (!M) M = 8192; if (!N) N = 32000; if (!K) K = 4096; if (scale == 0.0) scale = 1.0; sigmaB = 0.02f; }
  if (workload == "cols" && batch != 1) { std::fprintf(stderr, "error: the column split takes batch 1\n"); return 2; }

  int have = 0;
  if (cudaGetDeviceCount(&have) != cudaSuccess || have < gpus) { std::fprintf(stderr, "error: %d GPUs asked for, %d visible\n", gpus, have); return 2; }

  // ---- the launch layer and NCCL, both loaded at run time
  std::string lib;
  if (const char *e = std::getenv("WTC_LAUNCH_LIB"); e && *e) lib = e;
  else {
    std::error_code ec;
    std::filesystem::path dir = std::filesystem::read_symlink("/proc/self/exe", ec).parent_path();
    for (int up = 0; up < 6 && lib.empty(); ++up, dir = dir.parent_path())
      if (std::filesystem::exists(dir / "libwtc_launch.so")) lib = (dir / "libwtc_launch.so").string();
  }
  void *h = lib.empty() ? nullptr : dlopen(lib.c_str(), RTLD_NOW | RTLD_LOCAL);
  if (!h) { std::fprintf(stderr, "error: cannot load libwtc_launch.so (%s)\n", lib.empty() ? "not found; set WTC_LAUNCH_LIB" : dlerror()); return 2; }
  Api api;
  api.launch = reinterpret_cast<decltype(api.launch)>(dlsym(h, "wtc_matmul_softmax_launch"));
  api.partial = reinterpret_cast<decltype(api.partial)>(dlsym(h, "wtc_matmul_softmax_partial_launch"));
  api.finish = reinterpret_cast<decltype(api.finish)>(dlsym(h, "wtc_matmul_softmax_finish_launch"));
  api.wsBytes = reinterpret_cast<decltype(api.wsBytes)>(dlsym(h, "wtc_matmul_softmax_workspace_bytes"));
  api.status = reinterpret_cast<decltype(api.status)>(dlsym(h, "wtc_check_device_status"));
  api.lastError = reinterpret_cast<decltype(api.lastError)>(dlsym(h, "wtc_last_error"));
  if (!api.launch || !api.partial || !api.finish || !api.wsBytes || !api.status || !api.lastError) { std::fprintf(stderr, "error: launch library lacks the expected entry points\n"); return 2; }
  Nccl nccl;
  std::vector<ncclComm_t> comms(gpus, nullptr);
  if (workload == "cols") {
    void *nh = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!nh) nh = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
    if (!nh) { std::fprintf(stderr, "error: cannot load libnccl.so.2: %s\n", dlerror()); return 2; }
    nccl.commInitAll = reinterpret_cast<decltype(nccl.commInitAll)>(dlsym(nh, "ncclCommInitAll"));
    nccl.allGather = reinterpret_cast<decltype(nccl.allGather)>(dlsym(nh, "ncclAllGather"));
    nccl.commDestroy = reinterpret_cast<decltype(nccl.commDestroy)>(dlsym(nh, "ncclCommDestroy"));
    nccl.errorString = reinterpret_cast<decltype(nccl.errorString)>(dlsym(nh, "ncclGetErrorString"));
    if (!nccl.commInitAll || !nccl.allGather || !nccl.commDestroy || !nccl.errorString) { std::fprintf(stderr, "error: libnccl lacks the expected entry points\n"); return 2; }
    std::vector<int> devs(gpus);
    for (int i = 0; i < gpus; ++i) devs[i] = i;
    const ncclResult_t r = nccl.commInitAll(comms.data(), gpus, devs.data());
    if (r != ncclSuccess) { std::fprintf(stderr, "error: ncclCommInitAll: %s\n", nccl.errorString(r)); return 2; }
  }

  // ---- shares
  const long long tiles = (N + 255) / 256;
  std::vector<long long> c0(gpus), c1(gpus), b0(gpus), b1(gpus);
  for (int r = 0, cs = 0, bs = 0; r < gpus; ++r) {
    const long long nt = tiles / gpus + (r < tiles % gpus ? 1 : 0), nb = batch / gpus + (r < batch % gpus ? 1 : 0);
    c0[r] = std::min<long long>(N, cs * 256LL); cs += static_cast<int>(nt); c1[r] = std::min<long long>(N, cs * 256LL);
    b0[r] = bs; bs += static_cast<int>(nb); b1[r] = bs;
  }

  // ---- host inputs (shared, read-only for the threads)
  const long long rowsAll = batch * M;
  std::vector<uint16_t> hostA(static_cast<size_t>(rowsAll) * K), hostB(static_cast<size_t>(workload == "batch" ? batch : 1) * K * N);
  fill_f16(hostA, 1, 1.0f);
  fill_f16(hostB, 2, sigmaB);

  std::vector<double> usPerStep(gpus, 0.0), sumsErr(gpus, 0.0);
  const int kSample = 4;
  std::vector<std::vector<double>> partialSums(gpus, std::vector<double>(kSample, 0.0));
  std::atomic<bool> anyFailed{false};
  Barrier barrier(gpus);

  auto worker = [&](int r) {
    bool failed = false;
    CKC(cudaSetDevice(r));
    cudaStream_t s = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    CKC(cudaStreamCreate(&s)); CKC(cudaEventCreate(&e0)); CKC(cudaEventCreate(&e1));
    // this rank's problem
    wtc_chain_desc d = {};
    d.struct_size = sizeof d;
    d.in_dtype = WTC_F16; d.out_dtype = WTC_F16; d.acc_dtype = WTC_F32;
    d.scale = static_cast<float>(scale);
    d.variant = WTC_VARIANT_FUSED;
    long long myBatch = batch, myN = N;
    const uint16_t *srcA = hostA.data();
    std::vector<uint16_t> sliceB;
    const uint16_t *srcB = hostB.data();
    if (workload == "batch") { myBatch = b1[r] - b0[r]; srcA = hostA.data() + static_cast<size_t>(b0[r]) * M * K; srcB = hostB.data() + static_cast<size_t>(b0[r]) * K * N; }
    if (workload == "cols") {
      myN = c1[r] - c0[r];
      sliceB.resize(static_cast<size_t>(K) * myN);
      for (long long k = 0; k < K; ++k) std::memcpy(&sliceB[static_cast<size_t>(k) * myN], &hostB[static_cast<size_t>(k) * N + c0[r]], static_cast<size_t>(myN) * 2);
      srcB = sliceB.data();
    }
    d.batch = static_cast<int32_t>(std::max<long long>(myBatch, 1));
    d.M = myBatch > 0 ? M : 0; d.N = myN; d.K = K;
    d.b_batch_stride = (workload == "batch" || d.batch == 1) ? 0 : -1;
    const size_t rows = static_cast<size_t>(d.batch) * d.M;
    const size_t aBytes = rows * K * 2, bBytes = static_cast<size_t>(workload == "batch" ? d.batch : 1) * K * myN * 2, oBytes = rows * myN * 2;
    void *dA = nullptr, *dB = nullptr, *dO = nullptr, *dW = nullptr, *dStats = nullptr, *dAll = nullptr;
    size_t ws = 0;
    if (api.wsBytes(&d, &ws) != 0) { std::fprintf(stderr, "rank %d: %s\n", r, api.lastError()); failed = true; }
    CKC(cudaMalloc(&dA, std::max<size_t>(aBytes, 16))); CKC(cudaMalloc(&dB, std::max<size_t>(bBytes, 16))); CKC(cudaMalloc(&dO, std::max<size_t>(oBytes, 16)));
    if (ws) CKC(cudaMalloc(&dW, ws));
    if (workload == "cols") { CKC(cudaMalloc(&dStats, rows * 8)); CKC(cudaMalloc(&dAll, rows * 8 * gpus)); }
    if (!failed) {
      CKC(cudaMemcpy(dA, srcA, aBytes, cudaMemcpyHostToDevice));
      CKC(cudaMemcpy(dB, srcB, bBytes, cudaMemcpyHostToDevice));
    }
    auto step = [&]() {
      if (failed || rows == 0 || myN == 0) return;
      if (workload == "cols") {
        if (api.partial(&d, dA, dB, dO, dW, ws, dStats, s, nullptr) != 0) { std::fprintf(stderr, "rank %d: %s\n", r, api.lastError()); failed = true; return; }
        const ncclResult_t nr = nccl.allGather(dStats, dAll, rows * 2, ncclFloat, comms[r], s);
        if (nr != ncclSuccess) { std::fprintf(stderr, "rank %d: ncclAllGather: %s\n", r, nccl.errorString(nr)); failed = true; return; }
        if (api.finish(&d, dO, dW, dAll, gpus, s) != 0) { std::fprintf(stderr, "rank %d: %s\n", r, api.lastError()); failed = true; }
      } else if (api.launch(&d, dA, dB, dO, dW, ws, s, nullptr) != 0) { std::fprintf(stderr, "rank %d: %s\n", r, api.lastError()); failed = true; }
    };
    // No rank starts a step that contains a collective unless every rank got this far: a rank
    // that failed in its set-up says so before the barrier, and then nobody launches.
    if (failed) anyFailed = true;
    barrier.wait();
    const bool go = !anyFailed;
    for (int i = 0; i < warmup && go; ++i) step();
    CKC(cudaStreamSynchronize(s));
    if (failed) anyFailed = true;
    barrier.wait();
    const bool go2 = !anyFailed;
    CKC(cudaEventRecord(e0, s));
    for (int i = 0; i < steps && go2; ++i) step();
    CKC(cudaEventRecord(e1, s));
    CKC(cudaEventSynchronize(e1));
    float ms = 0.f;
    if (!failed) CKC(cudaEventElapsedTime(&ms, e0, e1));
    usPerStep[r] = ms * 1e3 / steps;
    if (!failed && rows && api.status(nullptr, s) != 0) { std::fprintf(stderr, "rank %d: %s\n", r, api.lastError()); failed = true; }
    // row sums of a few rows of this rank's output
    if (!failed && rows && myN) {
      std::vector<uint16_t> row(static_cast<size_t>(myN));
      for (int t = 0; t < kSample; ++t) {
        const size_t ri = (rows - 1) * static_cast<size_t>(t) / (kSample - 1);
        CKC(cudaMemcpy(row.data(), static_cast<const char *>(dO) + ri * myN * 2, static_cast<size_t>(myN) * 2, cudaMemcpyDeviceToHost));
        double sum = 0.0;
        for (uint16_t v : row) sum += f16_to_f32(v);
        partialSums[r][t] = sum;
        if (workload != "cols") sumsErr[r] = std::max(sumsErr[r], std::fabs(sum - 1.0));
      }
    }
    barrier.wait();
    cudaFree(dA); cudaFree(dB); cudaFree(dO); if (dW) cudaFree(dW); if (dStats) cudaFree(dStats); if (dAll) cudaFree(dAll);
    cudaEventDestroy(e0); cudaEventDestroy(e1); cudaStreamDestroy(s);
    if (failed) anyFailed = true;
  };

  std::vector<std::thread> threads;
  for (int r = 0; r < gpus; ++r) threads.emplace_back(worker, r);
  for (auto &t : threads) t.join();
  if (workload == "cols") for (auto c : comms) if (c) nccl.commDestroy(c);
  if (anyFailed) { std::fprintf(stderr, "error: a rank failed\n"); return 1; }

  double worst = 0.0, sumErr = 0.0;
  for (double u : usPerStep) worst = std::max(worst, u);
  if (workload == "cols") {
    for (int t = 0; t < kSample; ++t) { double s = 0.0; for (int r = 0; r < gpus; ++r) s += partialSums[r][t]; sumErr = std::max(sumErr, std::fabs(s - 1.0)); }
  } else for (double e : sumsErr) sumErr = std::max(sumErr, e);
  const double flops = 2.0 * batch * M * N * K * (workload == "rows" ? gpus : 1);
  std::printf("{\"tool\": \"welder-multi\", \"workload\": \"%s\", \"gpus\": %d, \"steps\": %d, \"warmup\": %d, \"problem\": {\"batch\": %lld, \"M\": %lld, \"N\": %lld, \"K\": %lld}, "
              "\"scaling\": \"%s\", \"us_per_step\": %.3f, \"tflops\": %.2f, \"us_per_step_per_gpu\": [",
              workload.c_str(), gpus, steps, warmup, batch, M, N, K, workload == "rows" ? "weak" : "strong", worst, flops / (worst * 1e-6) / 1e12);
  for (int r = 0; r < gpus; ++r) std::printf("%s%.3f", r ? ", " : "", usPerStep[r]);
  std::printf("], \"row_sum_max_err\": %.3e, \"row_sums_ok\": %s}\n", sumErr, sumErr <= 1e-3 ? "true" : "false");
  return sumErr <= 1e-3 ? 0 : 1;
}

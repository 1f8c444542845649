// C-ABI launch layer (see include/wtc_launch.h for the contract).  Resolves a
// chain descriptor to one of the kernel families, encodes and caches the TMA
// tensor maps, and launches.  No CPU fallback: without a CUDA device every
// launch returns WTC_E_CUDA.
#include "../../include/wtc_launch.h"

#include "wtc_kernels.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <mutex>
#include <string>
#include <vector>

namespace {

thread_local std::string g_last_error;

int fail(int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

int cuda_fail(cudaError_t e, const char *what) {
  return fail(WTC_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

#ifdef WTC_BRINGUP
long long *g_timeline = nullptr;   // four regions of 148*48 stamps, used round-robin by consecutive launches
unsigned g_timeline_launch = 0;
#endif
// environment, read once
const int g_use_pdl = [] { const char *e = getenv("WTC_NO_PDL"); return (e && e[0] == '1') ? 0 : 1; }();

// registers / spills / stack of every instance of the tensor-core kernel template, from the
// `ptxas -v` report of this build (generated beside the objects)
struct KernelFacts { int bn, stages, cluster, epi, pair, out32, kd, tm, registers, spill_store, spill_load, stack; };
const KernelFacts kKernelFacts[] = {
#include "build/kernel_facts.inc"
};
const KernelFacts *facts_of(const wtc::TcVariant &v) {
  for (const KernelFacts &f : kKernelFacts)
    if (f.bn == v.bn && f.stages == v.stages && f.cluster == (v.cluster != 0) && f.epi == v.epi && f.pair == (v.pair != 0) && f.out32 == (v.out32 != 0) && f.kd == v.kd && f.tm == v.tm)
      return &f;
  return nullptr;
}

struct Resolved {
  wtc_chain_desc d;  // strides filled in
  wtc_plan_info plan;
  int bn;            // column tile of the tensor-core kernels: 256, or 128 when best.json asks for it
  int tm;            // rows of a tile: 128, or best.json's tileM when it is 64 and a kernel exists for it
  int kd;            // K depth of a pipeline stage: 64, or best.json's tileK when it is 32 or 128 and a kernel exists for it
  int num_rb, num_nb, num_kb;
  bool b_batched;
  bool tc_ok;
  // WTC_FLAG_MATMUL_F16: f32 operands are first rounded to dense f16 copies at the head of the
  // workspace, then `inner` (the same chain on f16 operands) runs on the copies
  bool trunc = false;
  size_t stage_a = 0, stage_b = 0;
  wtc_chain_desc inner;
};

size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

bool mult8(int64_t v) { return (v & 7) == 0; }

int resolve(const wtc_chain_desc *in, Resolved &r) {
  if (!in) return fail(WTC_E_ARG, "null descriptor");
  if (in->struct_size != static_cast<int32_t>(sizeof(wtc_chain_desc)))
    return fail(WTC_E_ARG, "descriptor struct_size %d does not match this library (%zu)", in->struct_size,
                sizeof(wtc_chain_desc));
  r.d = *in;
  wtc_chain_desc &d = r.d;
  if (d.batch < 1) return fail(WTC_E_ARG, "batch must be >= 1 (got %d)", d.batch);
  if (d.M < 0 || d.N < 0 || d.K < 0) return fail(WTC_E_ARG, "negative extent M=%lld N=%lld K=%lld", (long long)d.M, (long long)d.N, (long long)d.K);
  if (d.M > 0x7fffffff || d.N > 0x7fffffff || d.K > 0x7fffffff) return fail(WTC_E_ARG, "extent exceeds 2^31-1");
  if ((d.in_dtype != WTC_F32 && d.in_dtype != WTC_F16) || (d.out_dtype != WTC_F32 && d.out_dtype != WTC_F16) ||
      (d.acc_dtype != WTC_F32 && d.acc_dtype != WTC_F16))
    return fail(WTC_E_ARG, "unknown dtype (in=%d out=%d acc=%d)", d.in_dtype, d.out_dtype, d.acc_dtype);
  if (d.variant != WTC_VARIANT_FUSED && d.variant != WTC_VARIANT_BASELINE) return fail(WTC_E_ARG, "unknown variant %d", d.variant);
  if (d.tile_m < 0 || d.tile_n < 0 || d.tile_k < 0) return fail(WTC_E_ARG, "negative tile size");
  if (d.lda == 0) d.lda = d.K;
  if (d.ldb == 0) d.ldb = d.N;
  if (d.ldo == 0) d.ldo = d.N;
  if (d.lda < d.K || d.ldb < d.N || d.ldo < d.N) return fail(WTC_E_ARG, "row stride smaller than the row");
  r.b_batched = d.b_batch_stride >= 0;
  if (d.a_batch_stride == 0) d.a_batch_stride = d.M * d.lda;
  if (d.b_batch_stride == 0) d.b_batch_stride = d.K * d.ldb;
  if (d.o_batch_stride == 0) d.o_batch_stride = d.M * d.ldo;
  if (!r.b_batched) d.b_batch_stride = 0;

  r.trunc = false;
  if (d.flags & WTC_FLAG_MATMUL_F16) {
    if (d.in_dtype != WTC_F32) return fail(WTC_E_ARG, "WTC_FLAG_MATMUL_F16 needs f32 operands (in_dtype = WTC_F32)");
    wtc_chain_desc inner = d;
    inner.in_dtype = WTC_F16;
    inner.flags &= ~WTC_FLAG_MATMUL_F16;
    inner.lda = d.K; inner.a_batch_stride = d.M * d.K;
    inner.ldb = d.N; inner.b_batch_stride = r.b_batched ? d.K * d.N : -1;
    Resolved ri;
    int rc = resolve(&inner, ri);
    if (rc) return rc;
    const wtc_chain_desc outer = d;
    const bool bb = r.b_batched;
    r = ri;
    r.d = outer;
    r.b_batched = bb;
    r.inner = inner;
    r.trunc = true;
    r.tc_ok = false;          // the sharded and static-scratch entry points take f16 operands only
    r.stage_a = align256(static_cast<size_t>(d.batch) * d.M * d.K * 2);
    r.stage_b = align256(static_cast<size_t>(bb ? d.batch : 1) * d.K * d.N * 2);
    r.plan.workspace_bytes += r.stage_a + r.stage_b;
    r.plan.launches += 1;     // one launch rounds both operands
    return WTC_OK;
  }

  wtc_plan_info &p = r.plan;
  memset(&p, 0, sizeof(p));
  p.cluster_n = 1;
  r.tm = wtc::kTcBlockM;
  r.num_rb = static_cast<int>((d.M + wtc::kTcBlockM - 1) / wtc::kTcBlockM);
  // tileN = 128 is the second legal column tile; everything else resolves to 256.  Without a
  // tile hint the 128-column kernels are taken (a) for rows of at most 128 columns (half of a
  // 256-column tile would be padding: 6.4 vs 8.3 us on 8192x128x64) and (b) when 256-column
  // tiles would leave more than half of the SMs without a CTA while the 128-column clusters
  // still all fit the chip at once (measured: 4096x512x1024 12.6 vs 14.5 us, 1024x1024x512
  // 9.2 vs 11.1 us; but 2048x1024x1024 18.6 vs 14.5 us, where sixteen 8-CTA clusters need two rounds).
  r.bn = wtc::kTcBlockN;
  if (d.tile_n == 128) r.bn = 128;
  else if (d.tile_n == 0) {
    // clusters of n CTAs that are resident at once on a 148-SM part (8: measured 15; others: one short of 148 / n)
    static const int kResident[9] = {0, 148, 72, 47, 35, 27, 22, 18, 15};
    const int64_t units = static_cast<int64_t>(d.batch) * r.num_rb;
    const int64_t nb128 = (d.N + 127) / 128, nb256 = (d.N + 255) / 256;
    if (d.N <= 128) r.bn = 128;
    else if (!(d.flags & WTC_FLAG_FORCE_TILED) && nb128 <= 8 && units * nb256 <= 74 && units <= kResident[nb128]) r.bn = 128;
  }
  r.num_nb = static_cast<int>((d.N + r.bn - 1) / r.bn);
  // tileK is the K depth of one pipeline stage.  64 is the default; 32 and 128 have kernels in the
  // eight-warp epilogue family (f16 probabilities, no forced epilogue form or CTA pair; 128 deep with
  // 256-column tiles only in the tiled flavour, where no cluster statistics compete for the room).
  // tileM = 64 (tcgen05.mma with M = 64) has kernels in the same family, for stages 32 or 64 deep.
  r.kd = wtc::kTcBlockK;
  {
    const bool tiled_shape = r.num_nb > 8 || (d.flags & WTC_FLAG_FORCE_TILED);
    const int forced = WTC_FLAG_EPILOGUE_SPLIT | WTC_FLAG_EPILOGUE_RELAY | WTC_FLAG_PAIR;
    const bool family = d.variant == WTC_VARIANT_FUSED && !(d.flags & forced);
    const bool f32o = d.out_dtype == WTC_F32;
    if ((d.tile_k == 32 || d.tile_k == 128) && family && wtc::tc_stage_depth_legal(tiled_shape, r.bn, f32o, d.tile_k)) r.kd = d.tile_k;
    if (d.tile_m == 64 && family && wtc::tc_stage_depth_legal(tiled_shape, r.bn, f32o, r.kd, 64)) {
      r.tm = 64;
      r.num_rb = static_cast<int>((d.M + 63) / 64);
    }
  }
  r.num_kb = static_cast<int>((d.K + r.kd - 1) / r.kd);

  const bool tc_shape = d.in_dtype == WTC_F16 && d.M > 0 && d.N > 0 && d.K > 0 &&
                        mult8(d.K) && mult8(d.N) && mult8(d.lda) && mult8(d.ldb) && mult8(d.ldo) &&
                        mult8(d.a_batch_stride) && mult8(d.b_batch_stride) && mult8(d.o_batch_stride) &&
                        static_cast<int64_t>(d.batch) * r.num_rb * r.num_nb < 0x7fffffff;
  r.tc_ok = tc_shape && !(d.flags & WTC_FLAG_FORCE_SIMT) && d.variant == WTC_VARIANT_FUSED;

  if (d.variant == WTC_VARIANT_BASELINE) {
    // five kernels with C32[rows,N], E[rows,N], max[rows], sum[rows] in global memory.  For f16
    // chains the first is the same tcgen05 contraction the fused kernel runs (so that fused
    // against baseline measures the fusion, not the arithmetic unit); f32 chains take SIMT FMAs.
    p.launches = 5;
    const size_t rows = static_cast<size_t>(d.batch) * d.M;
    p.workspace_bytes = (2 * rows * d.N + 2 * rows) * sizeof(float);
    if (tc_shape && !(d.flags & WTC_FLAG_FORCE_SIMT)) {
      p.kernel = WTC_KERNEL_TC_UNFUSED;
      const wtc::TcVariant v = wtc::tc_choose_variant(true, r.bn, true, d.batch, r.num_rb, r.num_kb, 1, 0, 1, 148, 0);
      p.tile_m = wtc::kTcBlockM; p.tile_n = r.bn; p.tile_k = wtc::kTcBlockK;
      p.threads = wtc::tc_variant_threads(v); p.stages = v.stages; p.tmem_columns = 2 * r.bn; p.smem_bytes = wtc::tc_variant_smem_bytes(v);
      if (const KernelFacts *f = facts_of(v)) { p.registers = f->registers; p.spill_bytes = f->spill_store; p.stack_bytes = f->stack; }
    } else {
      p.kernel = WTC_KERNEL_SIMT_UNFUSED;
      p.threads = 256;
      p.tile_m = 8; p.tile_n = static_cast<int32_t>(d.N); p.tile_k = 64;
    }
  } else if (r.tc_ok) {
    p.tile_m = r.tm; p.tile_n = r.bn; p.tile_k = r.kd;
    p.tmem_columns = 2 * r.bn;
    // variant, threads, stages as the launchers choose them on a 148-SM part (the plan is made
    // without a device): clusters of n CTAs resident at once, measured (8: 15; others: one short of 148 / n)
    static const int kResidentClusters[9] = {0, 148, 72, 47, 35, 27, 22, 18, 15};
    const int pair_mode = (d.flags & WTC_FLAG_NO_PAIR) ? 1 : ((d.flags & WTC_FLAG_PAIR) ? 2 : 0);
    const int epi_mode = (d.flags & WTC_FLAG_EPILOGUE_SPLIT) ? wtc::kEpilogueSplit
                         : ((d.flags & WTC_FLAG_EPILOGUE_RELAY) ? wtc::kEpilogueRelay : wtc::kEpilogueAuto);
    const bool cluster = r.num_nb <= 8 && !(d.flags & WTC_FLAG_FORCE_TILED);
    const wtc::TcVariant v = wtc::tc_choose_variant(!cluster, r.bn, d.out_dtype == WTC_F32, d.batch, r.num_rb, r.num_kb,
                                                    cluster ? r.num_nb : 1, epi_mode, pair_mode, 148,
                                                    cluster ? kResidentClusters[r.num_nb] : 0, r.kd, r.tm);
    p.threads = wtc::tc_variant_threads(v);
    p.stages = v.stages;
    p.smem_bytes = wtc::tc_variant_smem_bytes(v);
    if (const KernelFacts *f = facts_of(v)) { p.registers = f->registers; p.spill_bytes = f->spill_store; p.stack_bytes = f->stack; }
    if (cluster) {
      p.kernel = WTC_KERNEL_TC_CLUSTER;
      p.launches = 1;
      p.cluster_n = r.num_nb;
    } else {
      p.kernel = WTC_KERNEL_TC_TILED;
      p.launches = 2;
      p.workspace_bytes = static_cast<size_t>(d.batch) * d.M * r.num_nb * sizeof(float2);
    }
  } else {
    p.kernel = WTC_KERNEL_SIMT_FUSED;
    p.launches = (d.M > 0 && d.N > 0) ? 1 : 0;
    p.threads = 256;
    p.tile_m = 16; p.tile_n = static_cast<int32_t>(d.N); p.tile_k = 64;
  }
  p.tile_substituted = ((d.tile_m && d.tile_m != p.tile_m) || (d.tile_n && d.tile_n != p.tile_n && d.tile_n < d.N) ||
                        (d.tile_k && d.tile_k != p.tile_k)) ? 1 : 0;
  return WTC_OK;
}

// ---- tensor maps -------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                              const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
std::mutex g_mu;
EncodeFn g_encode = nullptr;

int get_encoder() {
  if (g_encode) return WTC_OK;
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
    return fail(WTC_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  }
  g_encode = reinterpret_cast<EncodeFn>(fn);
  return WTC_OK;
}

struct MapKey {
  const void *ptr;
  uint64_t d0, d1, d2, s1, s2;
  uint32_t b0, b1;
  bool operator==(const MapKey &o) const {
    return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && s1 == o.s1 && s2 == o.s2 && b0 == o.b0 && b1 == o.b1;
  }
};
struct MapEntry { MapKey key; CUtensorMap map; bool used; };
// Encoded tensor maps, per host thread: a direct-mapped table looked up without a lock (a launch
// needs three maps; encoding one costs about a microsecond, a hit a few nanoseconds).
constexpr size_t kMapSlots = 512;
struct MapTable { MapEntry e[kMapSlots]; };
MapTable *map_table() {
  thread_local MapTable *t = nullptr;
  if (!t) t = new (std::nothrow) MapTable();
  return t;
}

// rank-3 tensor (d0 innermost, contiguous), or rank-4 when d3 > 0; f16 unless f32; 128-byte swizzle (64-byte on request), zero fill
int get_map(const void *ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1_bytes, uint64_t s2_bytes, uint32_t b0,
            uint32_t b1, CUtensorMap *out, bool f32 = false, uint64_t d3 = 0, uint64_t s3_bytes = 0, uint32_t b2 = 1, bool swizzle64 = false) {
  const MapKey key{ptr, d0, d1, d2 ^ (d3 << 32), s1_bytes, s2_bytes ^ (s3_bytes << 20), b0 | (f32 ? 0x80000000u : 0u) | (swizzle64 ? 0x40000000u : 0u), b1 | (b2 << 16)};
  MapTable *tab = map_table();
  uint64_t h = reinterpret_cast<uintptr_t>(ptr) * 0x9E3779B97F4A7C15ull;
  h ^= (d0 * 31 + d1) * 0xC2B2AE3D27D4EB4Full + key.d2 + s1_bytes + (static_cast<uint64_t>(key.b0) << 20) + key.b1;
  MapEntry *slot = tab ? &tab->e[(h >> 40) % kMapSlots] : nullptr;
  if (slot && slot->used && slot->key == key) { *out = slot->map; return WTC_OK; }
  {
    std::lock_guard<std::mutex> lk(g_mu);
    int rc = get_encoder();
    if (rc) return rc;
  }
  const cuuint32_t rank = d3 ? 4 : 3;
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {s1_bytes, s2_bytes, s3_bytes};
  cuuint32_t box[4] = {b0, b1, b2, 1};
  if (!d3) box[2] = 1;
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMap m;
  CUresult cr = g_encode(&m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, rank, const_cast<void *>(ptr), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS)
    return fail(WTC_E_CUDA, "cuTensorMapEncodeTiled failed (%d) for rank %u dims=(%llu,%llu,%llu,%llu) strides=(%llu,%llu,%llu) box=(%u,%u,%u)",
                (int)cr, rank, (unsigned long long)d0, (unsigned long long)d1, (unsigned long long)d2, (unsigned long long)d3,
                (unsigned long long)s1_bytes, (unsigned long long)s2_bytes, (unsigned long long)s3_bytes, b0, b1, b2);
  if (slot) { slot->key = key; slot->map = m; slot->used = true; }
  *out = m;
  return WTC_OK;
}

// The map of B [batch][K][N] (N contiguous).  When N is a multiple of 64 it is the rank-4 view
// [batch][N/64][K][64]: one copy then brings `blocks` 64-column blocks of a K block, each laid
// out as the tensor core wants it (one stage's k-rows x 128 bytes); otherwise one copy per 64 columns.
int get_map_b(const void *B, const Resolved &r, int blocks, CUtensorMap *out, int *b_blocks) {
  const wtc_chain_desc &d = r.d;
  const uint64_t nbatch = r.b_batched ? d.batch : 1;
  const uint64_t bstride = (r.b_batched ? d.b_batch_stride : d.K * d.ldb) * 2;
  if (d.N % 64 == 0) {
    *b_blocks = 1;
    return get_map(B, 64, d.K, d.N / 64, d.ldb * 2, 128, 64, r.kd, out, false, nbatch, bstride, blocks);
  }
  *b_blocks = 0;
  return get_map(B, d.N, d.K, nbatch, d.ldb * 2, bstride, 64, r.kd, out);
}

int num_sms() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached[dev] = n;
  }
  return cached[dev];
}

// Per-device status word used when the caller passes none: a word of the library's own device
// image (zero when the module loads), so reporting through it never allocates.  The symbol's
// name is a host-side handle; the address kernels can use is looked up once per device.
__device__ int g_default_status_word;
int *default_status() {
  static int *words[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!words[dev]) {
    int *ptr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_default_status_word) != cudaSuccess) return nullptr;
    words[dev] = ptr;
  }
  return words[dev];
}

// what a non-zero device status word means
int status_result(int v) {
  if (v == 0) return WTC_OK;
  static const char *names[] = {"ok", "a TMA stage never landed", "a pipeline stage was never released",
                                "an accumulator never completed", "an accumulator buffer was never drained",
                                "cluster peers never sent their row statistics",
                                "dynamic shared memory was not 1024-byte aligned"};
  return fail(WTC_E_DEVICE, "device status %d: %s", v, (v > 0 && v < 7) ? names[v] : "unknown");
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

wtc::SimtParams simt_params(const Resolved &r) {
  wtc::SimtParams s;
  s.batch = r.d.batch; s.M = (int)r.d.M; s.N = (int)r.d.N; s.K = (int)r.d.K;
  s.lda = r.d.lda; s.ldb = r.d.ldb; s.ldo = r.d.ldo;
  s.a_batch_stride = r.d.a_batch_stride; s.b_batch_stride = r.d.b_batch_stride; s.o_batch_stride = r.d.o_batch_stride;
  s.in_f16 = r.d.in_dtype == WTC_F16; s.out_f16 = r.d.out_dtype == WTC_F16;
  s.acc_mode = r.d.acc_dtype == WTC_F16 ? 1 : 0;
  s.scale = r.d.scale;
  return s;
}

// mode: 0 whole chain, 1 partial (leave un-normalised values + row stats)
int launch_resolved(Resolved &r, const void *A, const void *B, void *Out, void *ws, size_t ws_bytes, void *row_stats,
                    int mode, cudaStream_t s, int *status) {
  const wtc_chain_desc &d = r.d;
  if (d.M == 0 || d.N == 0) return WTC_OK;
  if (!Out || (d.K > 0 && (!A || !B))) return fail(WTC_E_ARG, "null operand pointer");

  if (r.trunc) {
    if (mode != 0) return fail(WTC_E_UNSUPPORTED, "the sharded form takes f16 operands");
    if (!ws || ws_bytes < r.plan.workspace_bytes)
      return fail(WTC_E_WORKSPACE, "rounding the f32 operands to f16 needs %zu workspace bytes, got %zu", r.plan.workspace_bytes, ws_bytes);
    if ((reinterpret_cast<uintptr_t>(ws) & 15) != 0) return fail(WTC_E_ARG, "workspace must be 16-byte aligned");
    unsigned char *base = static_cast<unsigned char *>(ws);
    const cudaError_t e = wtc::launch_round_to_f16(static_cast<const float *>(A), base, d.batch, d.M, d.K, d.lda, d.a_batch_stride,
                                                   static_cast<const float *>(B), base + r.stage_a, r.b_batched ? d.batch : 1, d.K, d.N, d.ldb,
                                                   r.b_batched ? d.b_batch_stride : 0, s);
    if (e != cudaSuccess) return cuda_fail(e, "operand rounding launch");
    Resolved ri;
    int rc = resolve(&r.inner, ri);
    if (rc) return rc;
    return launch_resolved(ri, base, base + r.stage_a, Out, base + r.stage_a + r.stage_b, ws_bytes - r.stage_a - r.stage_b, row_stats, 0, s, status);
  }

  if (r.plan.kernel == WTC_KERNEL_SIMT_UNFUSED || r.plan.kernel == WTC_KERNEL_TC_UNFUSED) {
    if (mode != 0) return fail(WTC_E_UNSUPPORTED, "the baseline variant has no sharded form");
    if (!ws || ws_bytes < r.plan.workspace_bytes)
      return fail(WTC_E_WORKSPACE, "baseline variant needs %zu workspace bytes, got %zu", r.plan.workspace_bytes, ws_bytes);
    const bool tc = r.plan.kernel == WTC_KERNEL_TC_UNFUSED && aligned16(A) && aligned16(B) && aligned16(ws) &&
                    (d.batch == 1 || d.o_batch_stride == d.M * d.ldo);
    if (!tc) {
      cudaError_t e = wtc::launch_simt_unfused(A, B, Out, ws, simt_params(r), s);
      return e == cudaSuccess ? WTC_OK : cuda_fail(e, "unfused pipeline launch");
    }
    const int sms = num_sms();
    if (sms <= 0) return fail(WTC_E_CUDA, "no usable CUDA device");
    const int64_t rows = static_cast<int64_t>(d.batch) * d.M;
    float *C32 = static_cast<float *>(ws);
    float *E = C32 + rows * d.N, *mx = E + rows * d.N, *sum = mx + rows;
    CUtensorMap tmA, tmB, tmC;
    int rc = get_map(A, d.K, d.M, d.batch, d.lda * 2, d.a_batch_stride * 2, wtc::kTcBlockK, wtc::kTcBlockM, &tmA);
    int b_blocks = 0;
    if (!rc) rc = get_map_b(B, r, r.bn / 64, &tmB, &b_blocks);
    if (!rc) rc = get_map(C32, d.N, d.M, d.batch, d.N * 4, d.M * d.N * 4, 32, 32, &tmC, true);
    if (rc) return rc;
    wtc::TcParams p;
    memset(&p, 0, sizeof(p));
    p.batch = d.batch; p.M = (int)d.M; p.N = (int)d.N; p.K = (int)d.K;
    p.num_rb = r.num_rb; p.num_nb = r.num_nb; p.num_kb = r.num_kb;
    p.b_batched = r.b_batched;
    p.b_blocks = b_blocks;
    p.group_rb = 16;
    p.round_logits_f16 = d.acc_dtype == WTC_F16;
    p.scale = d.scale;
    p.c2 = d.scale * 1.4426950408889634f;
    p.status = status ? status : default_status();
    p.use_pdl = g_use_pdl;
    p.out_f32 = 1;
    p.logits_only = 1;
    p.pair_mode = 1;
    p.num_items = d.batch * r.num_rb * r.num_nb;
    wtc::TcLaunchInfo info;
    cudaError_t e = wtc::launch_tiled_partial(tmA, tmB, tmC, p, r.bn, sms, s, &info);
    if (e == cudaSuccess)
      e = wtc::launch_softmax_passes(C32, E, mx, sum, Out, rows, d.M, (int)d.N, d.ldo, d.o_batch_stride, d.out_dtype == WTC_F16, s);
    return e == cudaSuccess ? WTC_OK : cuda_fail(e, "unfused tensor-core pipeline launch");
  }

  const bool ptr_ok = aligned16(A) && aligned16(B) && aligned16(Out);
  bool tiled = r.plan.kernel == WTC_KERNEL_TC_TILED || (mode == 1 && r.tc_ok);
  if ((r.plan.kernel == WTC_KERNEL_TC_CLUSTER || tiled) && ptr_ok) {
    const int sms = num_sms();
    if (sms <= 0) return fail(WTC_E_CUDA, "no usable CUDA device");
    CUtensorMap tmA, tmB, tmO;
    // A's box is one swizzle span wide at most: 64 columns (a 128-deep stage takes two), or 32 with the 64-byte swizzle
    int rc = get_map(A, d.K, d.M, d.batch, d.lda * 2, d.a_batch_stride * 2, r.kd < 64 ? r.kd : 64, r.tm, &tmA, false, 0, 0, 1, r.kd == 32);
    if (rc) return rc;
    // (a CTA pair loads half of the tile's columns per CTA: the variant decides the box)
    const int pm = (d.flags & WTC_FLAG_NO_PAIR) ? 1 : ((d.flags & WTC_FLAG_PAIR) ? 2 : 0);
    const wtc::TcVariant v = wtc::tc_choose_variant(tiled, r.bn, d.out_dtype == WTC_F32, d.batch, r.num_rb, r.num_kb, tiled ? 1 : r.num_nb, 0, pm, sms, 0, r.kd, r.tm);
    int b_blocks = 0;
    rc = get_map_b(B, r, v.pair ? r.bn / 128 : r.bn / 64, &tmB, &b_blocks);
    if (rc) return rc;
    const bool out32 = d.out_dtype == WTC_F32;
    rc = out32 ? get_map(Out, d.N, d.M, d.batch, d.ldo * 4, d.o_batch_stride * 4, 32, 32, &tmO, true)
               : get_map(Out, d.N, d.M, d.batch, d.ldo * 2, d.o_batch_stride * 2, 64, r.tm / 4, &tmO);   // a warp stores its quarter of the tile's rows
    if (rc) return rc;

    wtc::TcParams p;
    memset(&p, 0, sizeof(p));
    p.batch = d.batch; p.M = (int)d.M; p.N = (int)d.N; p.K = (int)d.K;
    p.num_rb = r.num_rb; p.num_nb = r.num_nb; p.num_kb = r.num_kb;
    p.b_batched = r.b_batched;
    p.b_blocks = b_blocks;
    p.group_rb = 16;
    p.round_logits_f16 = d.acc_dtype == WTC_F16;
    p.c2 = d.scale * 1.4426950408889634f;
    p.status = status ? status : default_status();
#ifdef WTC_BRINGUP
    p.timeline = g_timeline ? g_timeline + static_cast<size_t>(g_timeline_launch++ % 4) * 148 * 48 : nullptr;
#endif
    p.use_pdl = g_use_pdl;
    p.operands_ready = (d.flags & WTC_FLAG_OPERANDS_READY) ? 1 : 0;
    p.out_f32 = out32;
    p.stage_k = r.kd;
    p.tile_rows = r.tm;
    p.pair_mode = (d.flags & WTC_FLAG_NO_PAIR) ? 1 : ((d.flags & WTC_FLAG_PAIR) ? 2 : 0);
    p.epilogue_mode = (d.flags & WTC_FLAG_EPILOGUE_SPLIT) ? wtc::kEpilogueSplit
                      : ((d.flags & WTC_FLAG_EPILOGUE_RELAY) ? wtc::kEpilogueRelay : wtc::kEpilogueAuto);
    wtc::TcLaunchInfo info;
    cudaError_t e;
    if (!tiled) {
      p.num_items = d.batch * r.num_rb;
      e = wtc::launch_fused_cluster(tmA, tmB, tmO, p, r.bn, r.num_nb, sms, s, &info);
      if (e != cudaSuccess) return cuda_fail(e, "fused cluster kernel launch");
      return WTC_OK;
    }
    const size_t need = static_cast<size_t>(d.batch) * d.M * r.num_nb * sizeof(float2);
    if (!ws || ws_bytes < need) return fail(WTC_E_WORKSPACE, "tiled schedule needs %zu workspace bytes, got %zu", need, ws_bytes);
    p.num_items = d.batch * r.num_rb * r.num_nb;
    p.tile_stats = static_cast<float2 *>(ws);
    e = wtc::launch_tiled_partial(tmA, tmB, tmO, p, r.bn, sms, s, &info);
    if (e != cudaSuccess) return cuda_fail(e, "tiled kernel launch");
    const int64_t rows = static_cast<int64_t>(d.batch) * d.M;
    if (mode == 1) {
      if (!row_stats) return fail(WTC_E_ARG, "partial launch needs a row_stats buffer");
      if (d.o_batch_stride != d.M * d.ldo && d.batch > 1) return fail(WTC_E_UNSUPPORTED, "sharded form needs densely stacked batches");
      e = wtc::launch_row_stats(p.tile_stats, static_cast<float2 *>(row_stats), rows, r.num_nb, s);
      return e == cudaSuccess ? WTC_OK : cuda_fail(e, "row statistics launch");
    }
    if (d.o_batch_stride != d.M * d.ldo && d.batch > 1) return fail(WTC_E_UNSUPPORTED, "tiled schedule needs densely stacked output batches");
    e = wtc::launch_rescale_rows(Out, d.out_dtype == WTC_F32, rows, (int)d.N, d.ldo, r.bn, r.num_nb, p.tile_stats, nullptr, 0, s);
    return e == cudaSuccess ? WTC_OK : cuda_fail(e, "row rescale launch");
  }

  if (mode != 0) return fail(WTC_E_UNSUPPORTED, "the sharded form needs f16 operands/output with 16-byte aligned rows");
  cudaError_t e = wtc::launch_simt_fused(A, B, Out, simt_params(r), s);
  if (e == cudaErrorInvalidValue) return fail(WTC_E_UNSUPPORTED, "N=%lld: one row of logits does not fit shared memory on the SIMT path", (long long)d.N);
  return e == cudaSuccess ? WTC_OK : cuda_fail(e, "SIMT fused kernel launch");
}

} // namespace

extern "C" {

int wtc_abi_version(void) { return WTC_ABI_VERSION; }

const char *wtc_last_error(void) { return g_last_error.c_str(); }

int wtc_plan_query(const wtc_chain_desc *desc, wtc_plan_info *out) {
  if (!out) return fail(WTC_E_ARG, "null plan pointer");
  Resolved r;
  int rc = resolve(desc, r);
  if (rc) return rc;
  *out = r.plan;
  return WTC_OK;
}

int wtc_matmul_softmax_workspace_bytes(const wtc_chain_desc *desc, size_t *bytes) {
  if (!bytes) return fail(WTC_E_ARG, "null size pointer");
  Resolved r;
  int rc = resolve(desc, r);
  if (rc) return rc;
  size_t need = r.plan.workspace_bytes;
  // the sharded form always runs the tiled schedule
  if (r.tc_ok) {
    const size_t tiled = static_cast<size_t>(r.d.batch) * r.d.M * r.num_nb * sizeof(float2);
    if (tiled > need) need = tiled;
  }
  *bytes = need;
  return WTC_OK;
}

int wtc_matmul_softmax_launch(const wtc_chain_desc *desc, const void *A, const void *B, void *Out, void *workspace,
                              size_t workspace_bytes, void *stream, int *device_status) {
  Resolved r;
  int rc = resolve(desc, r);
  if (rc) return rc;
  return launch_resolved(r, A, B, Out, workspace, workspace_bytes, nullptr, 0, static_cast<cudaStream_t>(stream), device_status);
}

int wtc_matmul_softmax_partial_launch(const wtc_chain_desc *desc, const void *A, const void *B, void *Out, void *workspace,
                                      size_t workspace_bytes, void *row_stats, void *stream, int *device_status) {
  Resolved r;
  int rc = resolve(desc, r);
  if (rc) return rc;
  if (!r.tc_ok) return fail(WTC_E_UNSUPPORTED, "the sharded form needs f16 operands with 16-byte aligned rows");
  return launch_resolved(r, A, B, Out, workspace, workspace_bytes, row_stats, 1, static_cast<cudaStream_t>(stream), device_status);
}

int wtc_matmul_softmax_finish_launch(const wtc_chain_desc *desc, void *Out, const void *workspace, const void *all_stats,
                                     int32_t num_parts, void *stream) {
  Resolved r;
  int rc = resolve(desc, r);
  if (rc) return rc;
  if (!r.tc_ok) return fail(WTC_E_UNSUPPORTED, "the sharded form needs f16 operands/output with 16-byte aligned rows");
  if (r.d.M == 0 || r.d.N == 0) return WTC_OK;
  if (!Out || !workspace || !all_stats || num_parts < 1) return fail(WTC_E_ARG, "null pointer or num_parts < 1");
  const int64_t rows = static_cast<int64_t>(r.d.batch) * r.d.M;
  cudaError_t e = wtc::launch_rescale_rows(Out, r.d.out_dtype == WTC_F32, rows, (int)r.d.N, r.d.ldo, r.bn, r.num_nb,
                                           static_cast<const float2 *>(workspace), static_cast<const float2 *>(all_stats),
                                           num_parts, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? WTC_OK : cuda_fail(e, "row rescale launch");
}

int wtc_check_device_status(const int *device_status, void *stream) {
  cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
  int *own = device_status ? nullptr : default_status();
  const int *src = device_status ? device_status : own;
  if (!src) return fail(WTC_E_CUDA, "no status word");
  int v = 0;
  e = cudaMemcpy(&v, src, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return cuda_fail(e, "reading the device status word");
  // the library's own word is reported once, then cleared (a caller's word is the caller's to clear)
  if (v != 0 && own) cudaMemsetAsync(own, 0, sizeof(int), static_cast<cudaStream_t>(stream));
  return status_result(v);
}

int wtc_matmul_softmax_time(const wtc_chain_desc *desc, const void *A, const void *B, void *Out, void *workspace,
                            size_t workspace_bytes, void *stream, int warmup, int iters, float *avg_ms) {
  if (!avg_ms || iters < 1 || warmup < 0) return fail(WTC_E_ARG, "bad timing arguments");
  Resolved r;
  int rc = resolve(desc, r);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  for (int i = 0; i < warmup; ++i) {
    rc = launch_resolved(r, A, B, Out, workspace, workspace_bytes, nullptr, 0, s, nullptr);
    if (rc) return rc;
  }
  cudaEvent_t e0, e1;
  cudaError_t e = cudaEventCreate(&e0);
  if (e != cudaSuccess) return cuda_fail(e, "cudaEventCreate");
  e = cudaEventCreate(&e1);
  if (e != cudaSuccess) { cudaEventDestroy(e0); return cuda_fail(e, "cudaEventCreate"); }
  cudaEventRecord(e0, s);
  for (int i = 0; i < iters && rc == 0; ++i)
    rc = launch_resolved(r, A, B, Out, workspace, workspace_bytes, nullptr, 0, s, nullptr);
  cudaEventRecord(e1, s);
  e = cudaEventSynchronize(e1);
  float ms = 0.f;
  if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (rc) return rc;
  if (e != cudaSuccess) return cuda_fail(e, "timed launch loop");
  *avg_ms = ms / static_cast<float>(iters);
  return wtc_check_device_status(nullptr, stream);
}

// Host buffers in, host buffer out.  The call is cut into slabs (row ranges, or batch ranges
// of a batched call) that move through three streams -- copy in, compute, copy out -- so the
// transfer of slab i+1 and the read-back of slab i-1 run under the kernel of slab i and the
// two PCIe directions are busy at the same time.  B goes first, whole.
// ---- calls with host buffers ---------------------------------------------------
// Per host thread: three streams (copies in, kernels, copies back) shared by all calls, and
// two slots of device buffers, so that a second call's operands travel to the device while
// the first call's rows are still on their way back: a caller that keeps two calls in flight
// (submit i+1, then wait for i) keeps both directions of the link busy all the time.
namespace {
constexpr int kMaxSlabs = 16;
constexpr int kHostSlots = 2;
struct HostBuf { void *p = nullptr; size_t cap = 0; };
struct HostSlot {
  HostBuf bufs[4];                    // A, B, Out, workspace
  cudaEvent_t finished = nullptr;     // recorded behind the slot's last copy back
  int *host_status = nullptr;         // pinned: the device status word as the call left it
  int64_t ticket = -1;                // the call in flight in this slot, or -1
};
struct HostSlab { Resolved r; size_t a_off, a_len, o_off, o_len, b_off, b_len; };
struct HostCtx {
  int dev = -1;
  cudaStream_t in = nullptr, run = nullptr, out = nullptr;
  cudaEvent_t a_in[kMaxSlabs] = {}, done[kMaxSlabs] = {};
  HostSlot slot[kHostSlots];
  int64_t next_ticket = 0;
  // slab schedule of the last descriptor
  wtc_chain_desc key; int key_dev = -1; int slab_env = 0; int n = 0; HostSlab slabs[kMaxSlabs];
};
HostCtx &host_ctx() { thread_local HostCtx c; return c; }

int host_wait_slot(HostCtx &hc, HostSlot &sl) {
  if (sl.ticket < 0) return WTC_OK;
  sl.ticket = -1;
  cudaError_t e = cudaEventSynchronize(sl.finished);
  if (e != cudaSuccess) return cuda_fail(e, "waiting for the results");
  const int v = *sl.host_status;
  if (v != 0) cudaMemsetAsync(default_status(), 0, sizeof(int), hc.out);   // reported once, then cleared
  return status_result(v);
}
} // namespace

int wtc_matmul_softmax_host_submit(const wtc_chain_desc *desc, const void *hostA, const void *hostB, void *hostOut, int64_t *ticket) {
  if (!ticket) return fail(WTC_E_ARG, "null ticket pointer");
  *ticket = -1;
  Resolved r;
  int rc = resolve(desc, r);
  if (rc) return rc;
  const wtc_chain_desc &d = r.d;
  if (d.M == 0 || d.N == 0) return WTC_OK;        // nothing to do: ticket -1 is always complete
  if (!hostA || !hostB || !hostOut) return fail(WTC_E_ARG, "null host pointer");
  const size_t in_sz = d.in_dtype == WTC_F16 ? 2 : 4, out_sz = d.out_dtype == WTC_F16 ? 2 : 4;
  const size_t a_bytes = static_cast<size_t>(d.batch) * d.a_batch_stride * in_sz;
  const size_t b_bytes = (r.b_batched ? static_cast<size_t>(d.batch) * d.b_batch_stride : static_cast<size_t>(d.K) * d.ldb) * in_sz;
  const size_t o_bytes = static_cast<size_t>(d.batch) * d.o_batch_stride * out_sz;
  const size_t w_bytes = r.plan.workspace_bytes;

  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  HostCtx &hc = host_ctx();
  if (hc.dev != dev) {
    // first call of this thread on this device (a thread that changes device starts over; what it
    // held on the other device stays allocated until the process ends)
    hc = HostCtx();
    for (cudaStream_t *st : {&hc.in, &hc.run, &hc.out}) {
      e = cudaStreamCreateWithFlags(st, cudaStreamNonBlocking);
      if (e != cudaSuccess) return cuda_fail(e, "cudaStreamCreate");
    }
    for (int i = 0; i < kMaxSlabs && e == cudaSuccess; ++i) {
      e = cudaEventCreateWithFlags(&hc.a_in[i], cudaEventDisableTiming);
      if (e == cudaSuccess) e = cudaEventCreateWithFlags(&hc.done[i], cudaEventDisableTiming);
    }
    for (int i = 0; i < kHostSlots && e == cudaSuccess; ++i) {
      e = cudaEventCreateWithFlags(&hc.slot[i].finished, cudaEventDisableTiming);
      if (e == cudaSuccess) e = cudaHostAlloc(reinterpret_cast<void **>(&hc.slot[i].host_status), sizeof(int), cudaHostAllocDefault);
    }
    if (e != cudaSuccess) return cuda_fail(e, "streams, events and status words of the host-buffer calls");
    hc.dev = dev;
  }
  // the slot's previous call must be over before its buffers are written again
  HostSlot &sl = hc.slot[hc.next_ticket % kHostSlots];
  rc = host_wait_slot(hc, sl);
  if (rc) return rc;
  const size_t want[4] = {a_bytes, b_bytes, o_bytes, w_bytes};
  for (int i = 0; i < 4; ++i) {
    if (sl.bufs[i].cap < want[i]) {
      if (sl.bufs[i].p) cudaFree(sl.bufs[i].p);
      sl.bufs[i].p = nullptr; sl.bufs[i].cap = 0;
      e = cudaMalloc(&sl.bufs[i].p, want[i]);
      if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc (host-buffer entry point)");
      sl.bufs[i].cap = want[i];
    }
  }

  // ---- slabs: rows in multiples of the 128-row tile (whole batches of a batched chain), about
  //      4 MB of A each.  With equal slabs a lone call takes (copy in of everything) + (one slab's
  //      kernels and copy back) + a hand-over between the engines per slab, which was measured at
  //      about 20 us on PCIe 5 x16: two to four slabs are best for 8 MB of A, eight already lose.
  //      A batched B travels with its slab.  The slab schedule of the last descriptor is kept,
  //      so a caller that repeats a shape resolves it once.
  //      When the thread's other slot still has a call in flight the caller overlaps whole calls, and
  //      cutting this one up only adds hand-overs: it then goes in one piece (measured, config 2, two
  //      calls in flight: 245 us per call in one piece, 289 in two slabs, 314 in four).
  int slab_env = 0;
  if (const char *ev = getenv("WTC_HOST_SLABS")) slab_env = atoi(ev) > 0 ? atoi(ev) : 1;
  if (!slab_env)
    for (const HostSlot &other : hc.slot)
      if (&other != &sl && other.ticket >= 0) slab_env = 1;
  if (hc.key_dev != dev || hc.slab_env != slab_env || std::memcmp(&hc.key, &d, sizeof(d)) != 0) {
    hc.key_dev = -1;
    const bool by_batch = d.batch > 1;
    const int64_t units = by_batch ? d.batch : (d.M + wtc::kTcBlockM - 1) / wtc::kTcBlockM;
    int64_t slabs = slab_env ? slab_env : static_cast<int64_t>(a_bytes >> 22);
    if (slabs < 1) slabs = 1;
    if (slabs > kMaxSlabs) slabs = kMaxSlabs;
    if (slabs > units) slabs = units;
    const int64_t per = (units + slabs - 1) / slabs;
    int n = 0;
    for (int64_t u0 = 0; u0 < units; u0 += per, ++n) {
      const int64_t u1 = u0 + per < units ? u0 + per : units;
      HostSlab &hs = hc.slabs[n];
      wtc_chain_desc sd = d;
      hs.b_off = 0; hs.b_len = 0;
      if (by_batch) {
        sd.batch = static_cast<int32_t>(u1 - u0);
        hs.a_off = static_cast<size_t>(u0) * d.a_batch_stride * in_sz;  hs.a_len = static_cast<size_t>(u1 - u0) * d.a_batch_stride * in_sz;
        hs.o_off = static_cast<size_t>(u0) * d.o_batch_stride * out_sz; hs.o_len = static_cast<size_t>(u1 - u0) * d.o_batch_stride * out_sz;
        if (r.b_batched) { hs.b_off = static_cast<size_t>(u0) * d.b_batch_stride * in_sz; hs.b_len = static_cast<size_t>(u1 - u0) * d.b_batch_stride * in_sz; }
        else sd.b_batch_stride = -1;
      } else {
        const int64_t r0 = u0 * wtc::kTcBlockM, r1 = u1 * wtc::kTcBlockM < d.M ? u1 * wtc::kTcBlockM : d.M;
        sd.M = r1 - r0;
        sd.a_batch_stride = 0; sd.o_batch_stride = 0;
        hs.a_off = static_cast<size_t>(r0) * d.lda * in_sz;  hs.a_len = static_cast<size_t>(r1 - r0) * d.lda * in_sz;
        hs.o_off = static_cast<size_t>(r0) * d.ldo * out_sz; hs.o_len = static_cast<size_t>(r1 - r0) * d.ldo * out_sz;
      }
      rc = resolve(&sd, hs.r);
      if (rc) return rc;
    }
    hc.n = n; hc.key = d; hc.slab_env = slab_env; hc.key_dev = dev;
  }

  char *dA = static_cast<char *>(sl.bufs[0].p), *dB = static_cast<char *>(sl.bufs[1].p), *dO = static_cast<char *>(sl.bufs[2].p);
  if (!r.b_batched || d.batch == 1) {
    e = cudaMemcpyAsync(dB, hostB, b_bytes, cudaMemcpyHostToDevice, hc.in);
    if (e != cudaSuccess) return cuda_fail(e, "copy of B to the device");
  }
  for (int n = 0; n < hc.n; ++n) {
    HostSlab &hs = hc.slabs[n];
    e = cudaSuccess;
    if (hs.b_len) e = cudaMemcpyAsync(dB + hs.b_off, static_cast<const char *>(hostB) + hs.b_off, hs.b_len, cudaMemcpyHostToDevice, hc.in);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dA + hs.a_off, static_cast<const char *>(hostA) + hs.a_off, hs.a_len, cudaMemcpyHostToDevice, hc.in);
    if (e == cudaSuccess) e = cudaEventRecord(hc.a_in[n], hc.in);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(hc.run, hc.a_in[n], 0);
    if (e != cudaSuccess) return cuda_fail(e, "copy of the operands to the device");
    rc = launch_resolved(hs.r, dA + hs.a_off, dB + hs.b_off, dO + hs.o_off, sl.bufs[3].p, sl.bufs[3].cap, nullptr, 0, hc.run, nullptr);
    if (rc) return rc;
    e = cudaEventRecord(hc.done[n], hc.run);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(hc.out, hc.done[n], 0);
    if (e == cudaSuccess) e = cudaMemcpyAsync(static_cast<char *>(hostOut) + hs.o_off, dO + hs.o_off, hs.o_len, cudaMemcpyDeviceToHost, hc.out);
    if (e != cudaSuccess) return cuda_fail(e, "copy of the result to the host");
  }
  // the device status word rides back behind the last rows into pinned memory: one wait
  // covers the results and the status (no separate blocking read)
  const int *dev_status = default_status();
  if (!dev_status) return fail(WTC_E_CUDA, "no status word");
  *sl.host_status = 0;
  e = cudaMemcpyAsync(sl.host_status, dev_status, sizeof(int), cudaMemcpyDeviceToHost, hc.out);
  if (e == cudaSuccess) e = cudaEventRecord(sl.finished, hc.out);
  if (e != cudaSuccess) return cuda_fail(e, "copy of the status word");
  sl.ticket = hc.next_ticket++;
  *ticket = sl.ticket;
  return WTC_OK;
}

int wtc_matmul_softmax_host_wait(int64_t ticket) {
  if (ticket < 0) return WTC_OK;
  HostCtx &hc = host_ctx();
  if (ticket >= hc.next_ticket) return fail(WTC_E_ARG, "ticket %lld was not issued on this thread", (long long)ticket);
  HostSlot &sl = hc.slot[ticket % kHostSlots];
  if (sl.ticket != ticket) return WTC_OK;          // already waited for (by the caller, or by a later submit that needed the slot)
  return host_wait_slot(hc, sl);
}

int wtc_matmul_softmax_host(const wtc_chain_desc *desc, const void *hostA, const void *hostB, void *hostOut) {
  int64_t ticket = -1;
#ifdef WTC_BRINGUP
  timespec ts0, ts1, ts2;
  clock_gettime(CLOCK_MONOTONIC, &ts0);
#endif
  int rc = wtc_matmul_softmax_host_submit(desc, hostA, hostB, hostOut, &ticket);
  if (rc) return rc;
#ifdef WTC_BRINGUP
  clock_gettime(CLOCK_MONOTONIC, &ts1);
#endif
  rc = wtc_matmul_softmax_host_wait(ticket);
#ifdef WTC_BRINGUP
  clock_gettime(CLOCK_MONOTONIC, &ts2);
  if (getenv("WTC_HOST_TRACE"))
    fprintf(stderr, "host call: enqueue %.1f us, wait %.1f us\n", (ts1.tv_sec - ts0.tv_sec) * 1e6 + (ts1.tv_nsec - ts0.tv_nsec) * 1e-3,
            (ts2.tv_sec - ts1.tv_sec) * 1e6 + (ts2.tv_nsec - ts1.tv_nsec) * 1e-3);
#endif
  return rc;
}

// ---- the entry point that allocates nothing -----------------------------------
// Scratch for wtc_matmul_softmax_launch_static: one array that lives in the
// library's device image (every GPU that loads the library carries it until the
// process exits): the per-tile (max, sum) pairs of the two-pass schedule.
constexpr size_t kStaticScratchBytes = WTC_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// The array's name is only a host-side handle here; the address kernels can use has to
// be asked for, once per device, with that device current.
unsigned char *static_scratch_for_current_device(int *rc_out) {
  static unsigned char *ptrs[64] = {nullptr};
  *rc_out = WTC_OK;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { *rc_out = cuda_fail(e, "cudaGetDevice"); return nullptr; }
  if (dev < 0 || dev >= 64) { *rc_out = fail(WTC_E_UNSUPPORTED, "device index %d out of range", dev); return nullptr; }
  std::lock_guard<std::mutex> lk(g_mu);
  if (!ptrs[dev]) {
    unsigned char *ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_static_scratch);
    if (e != cudaSuccess || !ptr) { *rc_out = cuda_fail(e, "cudaGetSymbolAddress(static scratch)"); return nullptr; }
    ptrs[dev] = ptr;
  }
  return ptrs[dev];
}

int wtc_matmul_softmax_launch_static(const wtc_chain_desc *desc, const void *A, const void *B, void *Out, void *stream,
                                     int *device_status) {
  Resolved r;
  int rc = resolve(desc, r);
  if (rc) return rc;
  if (r.d.M == 0 || r.d.N == 0) return WTC_OK;        // nothing to compute, as for the other entry points
  // this entry point always runs the two-pass schedule: size the scratch for the tiles it will use
  r.d.flags |= WTC_FLAG_FORCE_TILED;
  rc = resolve(&r.d, r);
  if (rc) return rc;
  if (!r.tc_ok)
    return fail(WTC_E_UNSUPPORTED, "the static-scratch entry point covers the tensor-core two-pass schedule only "
                                   "(f16 operands and output, K, N and row strides multiples of 8)");
  if (!aligned16(A) || !aligned16(B) || !aligned16(Out))
    return fail(WTC_E_UNSUPPORTED, "the static-scratch entry point needs A, B and Out on 16-byte boundaries");
  const size_t need = static_cast<size_t>(r.d.batch) * r.d.M * r.num_nb * sizeof(float2);
  if (need > kStaticScratchBytes)
    return fail(WTC_E_WORKSPACE, "this shape needs %zu bytes of scratch (%d-column tiles); the static scratch holds %zu "
                                 "(use wtc_matmul_softmax_launch with a caller-provided workspace)",
                need, r.bn, kStaticScratchBytes);
  unsigned char *base = static_scratch_for_current_device(&rc);
  if (!base) return rc;
  // the array keeps whatever the previous call left: the (max, sum) pairs are all rewritten
  // before they are read, so nothing has to be cleared
  return launch_resolved(r, A, B, Out, base, kStaticScratchBytes, nullptr, 0, static_cast<cudaStream_t>(stream), device_status);
}

// ---- the row-only chains ---------------------------------------------------------------------
namespace {
int check_row_desc(const wtc_row_chain_desc *d, int64_t &ld_in, int64_t &ld_out) {
  if (!d) return fail(WTC_E_ARG, "null descriptor");
  if (d->struct_size != static_cast<int32_t>(sizeof(wtc_row_chain_desc)))
    return fail(WTC_E_ARG, "descriptor struct_size %d does not match this library (%zu)", d->struct_size, sizeof(wtc_row_chain_desc));
  if (d->kind != WTC_ROW_SOFTMAX && d->kind != WTC_ROW_VARIANCE) return fail(WTC_E_ARG, "unknown row chain kind %d", d->kind);
  if (d->rows < 0 || d->N < 0 || d->N > 0x7fffffff) return fail(WTC_E_ARG, "bad extents rows=%lld N=%lld", (long long)d->rows, (long long)d->N);
  if (d->dtype != WTC_F32 && d->dtype != WTC_F16) return fail(WTC_E_ARG, "unknown dtype %d", d->dtype);
  ld_in = d->ld_in ? d->ld_in : d->N;
  ld_out = d->ld_out ? d->ld_out : d->N;
  if (ld_in < d->N || ld_out < d->N) return fail(WTC_E_ARG, "row stride smaller than the row");
  return WTC_OK;
}
} // namespace

int wtc_row_chain_launch(const wtc_row_chain_desc *desc, const void *X, void *Out, void *stream) {
  int64_t ld_in = 0, ld_out = 0;
  int rc = check_row_desc(desc, ld_in, ld_out);
  if (rc) return rc;
  if (desc->rows == 0 || desc->N == 0) return WTC_OK;
  if (!X || !Out) return fail(WTC_E_ARG, "null operand pointer");
  const int f16 = desc->dtype == WTC_F16;
  cudaError_t e = wtc::launch_row_chain(desc->kind, X, Out, desc->rows, desc->N, ld_in, ld_out, f16, f16, desc->mean_factor,
                                        desc->var_factor, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? WTC_OK : cuda_fail(e, "row chain kernel launch");
}

int wtc_row_chain_time(const wtc_row_chain_desc *desc, const void *X, void *Out, void *stream, int warmup, int iters,
                       float *avg_ms) {
  if (!avg_ms || iters < 1 || warmup < 0) return fail(WTC_E_ARG, "bad timing arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = 0;
  for (int i = 0; i < warmup && rc == 0; ++i) rc = wtc_row_chain_launch(desc, X, Out, stream);
  if (rc) return rc;
  cudaEvent_t e0, e1;
  cudaError_t e = cudaEventCreate(&e0);
  if (e != cudaSuccess) return cuda_fail(e, "cudaEventCreate");
  e = cudaEventCreate(&e1);
  if (e != cudaSuccess) { cudaEventDestroy(e0); return cuda_fail(e, "cudaEventCreate"); }
  cudaEventRecord(e0, s);
  for (int i = 0; i < iters && rc == 0; ++i) rc = wtc_row_chain_launch(desc, X, Out, stream);
  cudaEventRecord(e1, s);
  e = cudaEventSynchronize(e1);
  float ms = 0.f;
  if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (rc) return rc;
  if (e != cudaSuccess) return cuda_fail(e, "timed launch loop");
  *avg_ms = ms / static_cast<float>(iters);
  return WTC_OK;
}

#ifdef WTC_BRINGUP
// Bring-up builds only: a device buffer of grid*48 int64 that the tensor-core kernels stamp
// (see fused_tc_kernel.cu); NULL switches the stamps off.
int wtc_bringup_set_timeline(void *device_buffer) {
  g_timeline = static_cast<long long *>(device_buffer);
  g_timeline_launch = 0;
  return WTC_OK;
}
#endif

} // extern "C"

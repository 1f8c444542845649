// Fused Matmul -> row-Softmax for sm_100a: f16 operands, f32 accumulate in TMEM,
// f16 probabilities.  One persistent, warp-specialised kernel in two flavours:
//
//   CLUSTER = true   a thread-block cluster of ceil(N/BN) CTAs owns 128 complete
//                    rows.  Each CTA contracts its 128 x BN slice, reduces its
//                    local row (max, sum), swaps the pair with its peers through
//                    distributed shared memory and writes normalised f16.
//   CLUSTER = false  independent 128 x BN tiles.  Each writes exp(v - tile max)
//                    as f16 and the per-tile (max, sum); a second, bandwidth-bound
//                    kernel (row_softmax_kernels.cu) rescales the rows.  Used when
//                    a row does not fit one cluster, and for skinny M.
//
// Warp roles (192 threads): warp 0 feeds shared memory with TMA, warp 1 owns TMEM
// and issues tcgen05.mma, warps 2..5 are the softmax epilogue (one thread per row,
// TMEM lane quarter = warp_id % 4).  Two accumulator buffers in TMEM let the
// epilogue of tile i run under the contraction of tile i+1.  The logits never
// leave the SM: TMEM -> registers -> (TMEM) -> swizzled shared -> TMA store.
//
// Operand layouts: A [M,K] is K-major, staged as 128 rows x 128 B with the 128-byte
// swizzle.  B [K,N] has N contiguous, i.e. it is MN-major for the MMA: it is staged
// as BN/64 blocks of (64 k-rows x 128 B), and the instruction descriptor's B-major
// bit asks the tensor core to transpose it.  No operand is pre-transposed.
#include "wtc_kernels.h"
#include "wtc_ptx.cuh"

namespace wtc {

namespace {

constexpr int BM = kTcBlockM;
constexpr int BK = kTcBlockK;
constexpr int kThreads = 192;
constexpr int kEpiThreads = 128;
constexpr int kMaxCluster = 8;

template <int BN, int STAGES, bool CLUSTER>
struct SmemLayout {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BK * BN * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kOutWarpBytes = 2 * 32 * 128;            // two 32-row x 64-col f16 buffers
  static constexpr int kOutBytes = 4 * kOutWarpBytes;
  static constexpr int kStatsBytes = CLUSTER ? 2 * kMaxCluster * BM * 8 : 0;
  static constexpr int kOffOut = STAGES * kStageBytes;
  static constexpr int kOffStats = kOffOut + kOutBytes;
  static constexpr int kOffBars = kOffStats + kStatsBytes;
  static constexpr int kNumBars = 2 * STAGES + 4 + 2;
  static constexpr int kOffTmemSlot = kOffBars + kNumBars * 8;
  static constexpr int kTotal = kOffTmemSlot + 16;
  static constexpr int kDynamic = kTotal + 1024;                 // slack to align the base to 1024 B
};

__device__ __forceinline__ void record_failure(int *status, int code) {
  if (status) atomicCAS(status, 0, code);
}

// Writes one thread's 32 consecutive f16 columns (64 B) into its row of the
// 128-byte-swizzled staging tile.  `half` selects the left or right 64 B of the row.
__device__ __forceinline__ void stage_row_chunk(uint8_t *buf, int lane, int half, const uint32_t (&h)[16]) {
  uint8_t *row = buf + lane * 128;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int phys = ((half * 4 + j) ^ (lane & 7)) * 16;
    *reinterpret_cast<uint4 *>(row + phys) = make_uint4(h[4 * j], h[4 * j + 1], h[4 * j + 2], h[4 * j + 3]);
  }
}

template <int BN, int STAGES, bool CLUSTER>
__global__ void __launch_bounds__(kThreads, 1)
fused_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmO, const TcParams p) {
  using L = SmemLayout<BN, STAGES, CLUSTER>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L::kOffBars);
  uint64_t *full = bars;
  uint64_t *empty = bars + STAGES;
  uint64_t *accum_full = bars + 2 * STAGES;
  uint64_t *accum_empty = bars + 2 * STAGES + 2;
  uint64_t *stats_bar = bars + 2 * STAGES + 4;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + L::kOffTmemSlot);
  float2 *stats = reinterpret_cast<float2 *>(smem + L::kOffStats);  // [2][kMaxCluster][BM]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = CLUSTER ? cluster_ctarank() : 0u;
  const uint32_t cluster_n = CLUSTER ? cluster_nctarank() : 1u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&accum_full[i], 1);
      mbar_init(&accum_empty[i], kEpiThreads);
      mbar_init(&stats_bar[i], cluster_n * kEpiThreads);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); tma_prefetch_desc(&tmO);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 2 * BN); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (CLUSTER) cluster_sync_all();   // every peer's barriers exist before anyone touches them

  // ---- work distribution --------------------------------------------------
  int first, stride;
  if (CLUSTER) { first = blockIdx.x / cluster_n; stride = gridDim.x / cluster_n; }
  else { first = blockIdx.x; stride = gridDim.x; }

  auto decode = [&](int w, int &b, int &rb, int &nb) {
    if (CLUSTER) { b = w / p.num_rb; rb = w - b * p.num_rb; nb = cta_rank; return; }
    const int per_batch = p.num_rb * p.num_nb;
    b = w / per_batch;
    int t = w - b * per_batch;
    // groups of `group_rb` row blocks; inside a group the column block is the
    // slow index, so concurrently running CTAs share B column blocks and the
    // group's A rows stay in L2.
    const int per_group = p.group_rb * p.num_nb;
    const int g = t / per_group;
    t -= g * per_group;
    const int rows_here = min(p.group_rb, p.num_rb - g * p.group_rb);
    nb = t / rows_here;
    rb = g * p.group_rb + (t - nb * rows_here);
  };

  if (warp == 0) {
    // ======================= TMA producer ==================================
    uint32_t n = 0;
    bool ok = true;
    for (int w = first; w < p.num_items && ok; w += stride) {
      int b, rb, nb; decode(w, b, rb, nb);
      for (int kb = 0; kb < p.num_kb; ++kb, ++n) {
        const int s = n % STAGES;
        const uint32_t ph = (n / STAGES) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1)) { record_failure(p.status, WTC_DEV_TIMEOUT_EMPTY); ok = false; break; }
        if (lane == 0) {
          uint8_t *sa = smem + s * L::kStageBytes;
          uint8_t *sb = sa + L::kABytes;
          mbar_expect_tx(&full[s], L::kStageBytes);
          tma_load_3d(sa, &tmA, &full[s], kb * BK, rb * BM, b);
#pragma unroll
          for (int j = 0; j < BN / 64; ++j)
            tma_load_3d(sb + j * (BK * 128), &tmB, &full[s], nb * BN + j * 64, kb * BK, p.b_batched ? b : 0);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // ======================= MMA issuer ====================================
    constexpr uint32_t idesc = umma_idesc_f16_f32(BM, BN, /*a_mn_major=*/0, /*b_mn_major=*/1);
    uint32_t n = 0;
    int it = 0;
    bool ok = true;
    for (int w = first; w < p.num_items && ok; w += stride, ++it) {
      const int ab = it & 1;
      if (!mbar_wait(&accum_empty[ab], ((it >> 1) & 1) ^ 1)) { record_failure(p.status, WTC_DEV_TIMEOUT_TMEM); ok = false; break; }
      tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + ab * BN;
      for (int kb = 0; kb < p.num_kb; ++kb, ++n) {
        const int s = n % STAGES;
        const uint32_t ph = (n / STAGES) & 1;
        if (!mbar_wait(&full[s], ph)) { record_failure(p.status, WTC_DEV_TIMEOUT_FULL); ok = false; break; }
        tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t sa = smem_u32(smem + s * L::kStageBytes);
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = umma_smem_desc_sw128(sa + k * p.geom.a_kstep, p.geom.a_lbo, p.geom.a_sbo);
            const uint64_t db = umma_smem_desc_sw128(sb + k * p.geom.b_kstep, p.geom.b_lbo, p.geom.b_sbo);
            umma_f16_ss(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          umma_commit(&empty[s]);   // frees the stage once these MMAs have read it
        }
        __syncwarp();
      }
      if (ok && lane == 0) umma_commit(&accum_full[ab]);
      __syncwarp();
    }
  } else {
    // ======================= softmax epilogue ==============================
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int row_in_tile = q * 32 + lane;
    uint8_t *stg = smem + L::kOffOut + (warp - 2) * L::kOutWarpBytes;
    const float c2 = p.c2;
    int it = 0;
    uint32_t groups = 0;                    // staging tiles handed to TMA so far (per warp)
    for (int w = first; w < p.num_items; w += stride, ++it) {
      int b, rb, nb; decode(w, b, rb, nb);
      const int ab = it & 1;
      if (!mbar_wait(&accum_full[ab], (it >> 1) & 1)) { record_failure(p.status, WTC_DEV_TIMEOUT_ACCUM); break; }
      tc_fence_after_sync();
      const uint32_t tbase = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + ab * BN;
      const int col0 = nb * BN;
      const int valid = min(BN, p.N - col0);          // columns of this tile inside the matrix
      const int chunks = (valid + 31) >> 5;
      const int row0 = rb * BM + q * 32;              // first row of this warp
      const bool rows_live = row0 < p.M;

      // Stages one 32-column chunk of this warp's 32 rows; every second chunk (or
      // the last one) hands the 32 x 64 staging tile to TMA.  Two tiles alternate:
      // group g uses tile g & 1, and every group commits (possibly empty), so
      // "at most one group still reading" means tile g & 1 is free again.
      auto stage_and_store = [&](int c, int nchunks, const uint32_t (&h)[16]) {
        const int buf = groups & 1;
        if ((c & 1) == 0) {
          if (lane == 0) tma_store_wait_read1();
          __syncwarp();
        }
        stage_row_chunk(stg + buf * 4096, lane, c & 1, h);
        if ((c & 1) == 1 || c == nchunks - 1) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (rows_live) tma_store_3d(&tmO, stg + buf * 4096, col0 + (c >> 1) * 64, row0, b);
            tma_store_commit();
          }
          ++groups;
        }
      };

      uint32_t r[32];
      // ---- pass 1: row maximum of v = s * c2 (log2 domain) ----
      float mx = -INFINITY;
      for (int c = 0; c < chunks; ++c) {
        tmem_ld_32x32b_x32(tbase + c * 32, r);
        tmem_ld_wait();
        const int lim = valid - c * 32;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float s = __uint_as_float(r[i]);
          if (p.round_logits_f16) s = __half2float(__float2half_rn(s));
          const float v = s * c2;
          if (i < lim) mx = fmaxf(mx, v);
        }
      }
      // ---- pass 2: e = 2^(v - mx), row sum ----
      float sum = 0.f;
      for (int c = 0; c < chunks; ++c) {
        tmem_ld_32x32b_x32(tbase + c * 32, r);
        tmem_ld_wait();
        const int lim = valid - c * 32;
        uint32_t h[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float s0 = __uint_as_float(r[i]), s1 = __uint_as_float(r[i + 1]);
          if (p.round_logits_f16) { s0 = __half2float(__float2half_rn(s0)); s1 = __half2float(__float2half_rn(s1)); }
          float e0 = ex2_approx(fmaf(s0, c2, -mx));
          float e1 = ex2_approx(fmaf(s1, c2, -mx));
          if (i >= lim) e0 = 0.f;
          if (i + 1 >= lim) e1 = 0.f;
          sum += e0 + e1;
          if (CLUSTER) { r[i] = __float_as_uint(e0); r[i + 1] = __float_as_uint(e1); }
          else h[i >> 1] = pack_f16x2(e0, e1);
        }
        if (CLUSTER) {
          tmem_st_32x32b_x32(tbase + c * 32, r);   // park e in place of the logits
        } else {
          stage_and_store(c, chunks, h);
        }
      }
      if (!CLUSTER) {
        tc_fence_before_sync();
        mbar_arrive(&accum_empty[ab]);
        const int row = rb * BM + row_in_tile;
        if (row < p.M)
          p.tile_stats[(static_cast<int64_t>(b) * p.M + row) * p.num_nb + nb] = make_float2(mx, sum);
        continue;
      }

      // ---- cluster: swap (max, sum) with the peers that hold the rest of the row ----
      tmem_st_wait();
      const int sbuf = it & 1;
      {
        const uint32_t slot = smem_u32(&stats[(sbuf * kMaxCluster + cta_rank) * BM + row_in_tile]);
        const uint32_t bar = smem_u32(&stats_bar[sbuf]);
        for (uint32_t peer = 0; peer < cluster_n; ++peer) st_cluster_f32x2(map_to_cta(slot, peer), mx, sum);
        for (uint32_t peer = 0; peer < cluster_n; ++peer) mbar_arrive_remote_release(map_to_cta(bar, peer));
      }
      if (!mbar_wait_cluster(&stats_bar[sbuf], (it >> 1) & 1)) { record_failure(p.status, WTC_DEV_TIMEOUT_STATS); break; }
      float gm = mx;
      for (uint32_t peer = 0; peer < cluster_n; ++peer)
        gm = fmaxf(gm, stats[(sbuf * kMaxCluster + peer) * BM + row_in_tile].x);
      float gl = 0.f;
      for (uint32_t peer = 0; peer < cluster_n; ++peer) {
        const float2 st = stats[(sbuf * kMaxCluster + peer) * BM + row_in_tile];
        gl += st.y * ex2_approx(st.x - gm);
      }
      const float f = ex2_approx(mx - gm) / gl;

      // ---- pass 3: p = e * f -> f16 -> swizzled staging -> TMA store ----
      for (int c = 0; c < chunks; ++c) {
        tmem_ld_32x32b_x32(tbase + c * 32, r);
        tmem_ld_wait();
        uint32_t h[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2)
          h[i >> 1] = pack_f16x2(__uint_as_float(r[i]) * f, __uint_as_float(r[i + 1]) * f);
        stage_and_store(c, chunks, h);
      }
      tc_fence_before_sync();
      mbar_arrive(&accum_empty[ab]);
    }
    if (lane == 0) tma_store_wait_all();
  }

  // ---- teardown: nothing in flight, peers done with our shared memory, TMEM freed ----
  if (p.status && *reinterpret_cast<volatile int *>(p.status) != 0) {
    // a wait gave up somewhere: give copies that were already issued time to land
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (CLUSTER) cluster_sync_all();
  if (warp == 1) tmem_dealloc(tmem_base, 2 * BN);
}

template <int BN, int STAGES, bool CLUSTER>
cudaError_t launch_impl(const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmO, const TcParams &p,
                        int cluster_n, int num_sms, cudaStream_t s, TcLaunchInfo *info) {
  using L = SmemLayout<BN, STAGES, CLUSTER>;
  auto kern = fused_tc_kernel<BN, STAGES, CLUSTER>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
  if (e != cudaSuccess) return e;

  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = L::kDynamic;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  int grid;
  if (CLUSTER) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster_n;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.gridDim = dim3(cluster_n, 1, 1);
    int max_clusters = 0;
    e = cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg);
    if (e != cudaSuccess) return e;
    if (max_clusters < 1) return cudaErrorInvalidConfiguration;
    const int clusters = p.num_items < max_clusters ? p.num_items : max_clusters;
    grid = clusters * cluster_n;
  } else {
    grid = p.num_items < num_sms ? p.num_items : num_sms;
    cfg.attrs = nullptr;
    cfg.numAttrs = 0;
  }
  cfg.gridDim = dim3(grid, 1, 1);
  if (info) { info->grid = grid; info->cluster = CLUSTER ? cluster_n : 1; info->smem_bytes = L::kDynamic; info->threads = kThreads; }
  return cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmO, p);
}

} // namespace

cudaError_t launch_fused_cluster(const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmO,
                                 const TcParams &p, int cluster_n, int num_sms, cudaStream_t s,
                                 TcLaunchInfo *info) {
  if (cluster_n < 1 || cluster_n > kMaxCluster) return cudaErrorInvalidValue;
  return launch_impl<kTcBlockN, 3, true>(tmA, tmB, tmO, p, cluster_n, num_sms, s, info);
}

cudaError_t launch_tiled_partial(const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmO,
                                 const TcParams &p, int num_sms, cudaStream_t s, TcLaunchInfo *info) {
  return launch_impl<kTcBlockN, 4, false>(tmA, tmB, tmO, p, 1, num_sms, s, info);
}

} // namespace wtc

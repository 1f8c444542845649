// Fused Matmul -> row-Softmax for sm_100a: f16 operands, f32 accumulate in TMEM,
// f16 probabilities.  One persistent, warp-specialised kernel in two flavours:
//
//   CLUSTER = true   a thread-block cluster of ceil(N/BN) CTAs owns 128 complete
//                    rows.  Each CTA contracts its 128 x BN slice, reduces its
//                    local row (max, sum), sends the pair to its peers' shared
//                    memory (st.async + mbarrier transaction bytes: no fences, no
//                    cluster-wide barrier) and writes normalised f16.
//   CLUSTER = false  independent 128 x BN tiles.  Each writes exp(v - tile max)
//                    as f16 and the per-tile (max, sum); a second, bandwidth-bound
//                    kernel (row_softmax_kernels.cu) rescales the rows.  Used when
//                    a row does not fit one cluster, and for skinny M.
//
// Warp roles (320 threads): warp 0 feeds shared memory with TMA, warp 1 owns TMEM
// and issues tcgen05.mma, warps 2..9 are the softmax epilogue: thread = one row x
// half of the tile's columns (TMEM lane quarter = warp_id % 4, column half =
// (warp_id - 2) / 4).  Two accumulator buffers in TMEM let the epilogue of tile i
// run under the contraction of tile i+1.  The logits never leave the SM:
// TMEM -> registers -> swizzled shared -> TMA store.
//
// Epilogue, per thread: its 128 accumulator values go TMEM -> registers in one go
// and the accumulator buffer is released at once; row extreme, e = 2^(v - max) in
// place (one MUFU per element), the row's (max, sum) exchange -- between the two
// column halves through shared memory, between the CTAs of the cluster through
// st.async -- then p = e * factor, packed to f16, staged 64 columns at a time in
// 128-byte-swizzled shared memory and written with TMA stores.
//
// Other forms of the same kernel (template parameters): RELAY -- twenty warps, an "exp"
// group and a "store" group that work on consecutive tiles at the same time, the exp values
// parked in TMEM between them (chosen when a CTA sees several tiles); PAIR -- two CTAs issue
// one 256-row tcgen05 cta_group::2 MMA; OUT32 -- f32 probabilities; EW = 16 -- a row's
// columns split four ways; OUT_TILES = 0 -- register-to-global stores without staging.
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
// Epilogue warps per CTA: 8 (a thread owns one row x BN/2 columns) or 16 (one row x BN/4:
// four warps per scheduler hide the TMEM-load and barrier latencies the eight-warp form exposes).
constexpr int kThreadsFor(int ew, bool relay = false) { return relay ? 640 : 64 + ew * 32; }
constexpr int kMaxCluster = 8;

// OUT_TILES: 32-row x 64-column f16 staging tiles per epilogue warp (2 = the warp's two
// column groups never wait for each other's TMA read; 1 = smaller, leaves room for a stage).
template <int BN, int STAGES, bool CLUSTER, int OUT_TILES, bool RELAY, bool PAIR, int EW, bool OUT32 = false, bool SINGLE = false>
struct SmemLayout {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BK * BN * 2 / (PAIR ? 2 : 1);     // a CTA pair splits B's columns between its two CTAs
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kHalfCols = RELAY ? BN / 2 : BN * 4 / EW;       // columns per epilogue thread (per step)
  static constexpr int kOutWarpBytes = OUT_TILES * 32 * 64 * 2;      // 0: the epilogue stores straight from registers
  static constexpr int kOutBytes = (RELAY ? 8 : EW) * kOutWarpBytes;   // relay: only the storing group stages
  static constexpr int kPairBytes = 2 * BM * 8;                       // [half][row] float2
  static constexpr int kStatsSets = RELAY ? 4 : 2;                     // relay: a peer may run up to three tiles ahead of this CTA's storing group
  static constexpr int kStatsBytes = CLUSTER ? kStatsSets * kMaxCluster * BM * 8 : 0;
  static constexpr int kOffOut = STAGES * kStageBytes;
  static constexpr int kOffPair = kOffOut + kOutBytes;
  static constexpr int kOffStats = kOffPair + kPairBytes;
  static constexpr int kMhBytes = RELAY ? 2 * 2 * BM * 4 : 0;         // relay: [tile parity][half][row] half-row maxima
  static constexpr int kOffMh = kOffStats + kStatsBytes;
  static constexpr int kOffBars = kOffMh + kMhBytes;
  static constexpr int kNumBars = 2 * STAGES + 4 + 4 + 2;
  static constexpr int kOffTmemSlot = kOffBars + kNumBars * 8;
  static constexpr int kTotal = kOffTmemSlot + 16;
  static constexpr int kDynamic = kTotal;
  static_assert(kDynamic <= 232448, "exceeds the 227 KB of shared memory a CTA may use");
};

__device__ __forceinline__ void record_failure(int *status, int code) {
  if (status) atomicCAS(status, 0, code);
}

// Writes one thread's 32 consecutive f16 columns (64 B) into its row of a
// 128-byte-swizzled 32-row x 64-column staging tile.  `half` selects the left or
// right 64 B of the row.
__device__ __forceinline__ void stage_row_chunk(uint8_t *tile, int lane, int half, const uint32_t (&h)[16]) {
  uint8_t *row = tile + lane * 128;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int phys = ((half * 4 + j) ^ (lane & 7)) * 16;
    *reinterpret_cast<uint4 *>(row + phys) = make_uint4(h[4 * j], h[4 * j + 1], h[4 * j + 2], h[4 * j + 3]);
  }
}

// f32 output: one thread's 32 consecutive f32 columns (128 B) fill its whole row of a
// 128-byte-swizzled 32-row x 32-column staging tile.
__device__ __forceinline__ void stage_row_f32(uint8_t *tile, int lane, const float (&v)[32]) {
  uint8_t *row = tile + lane * 128;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int phys = (j ^ (lane & 7)) * 16;
    *reinterpret_cast<float4 *>(row + phys) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  }
}

__device__ __forceinline__ void stamp(long long *timeline, int slot) {
  if (timeline) timeline[static_cast<size_t>(blockIdx.x) * 16 + slot] = static_cast<long long>(globaltimer_ns());
}

// Second stamp layout (timeline_mode 1): four points of the first four tiles one thread sees.
__device__ __forceinline__ void stamp_tile(const TcParams &p, int seq, int k) {
  if (p.timeline && p.timeline_mode == 1 && seq < 4) stamp(p.timeline, seq * 4 + k);
  if (p.timeline && p.timeline_mode == 3 && seq >= 20 && seq < 24) stamp(p.timeline, (seq - 20) * 4 + k);   // same, steady state
}
// Third layout (timeline_mode 2): eight points of the second and third tile one thread sees.
__device__ __forceinline__ void stamp_fine(const TcParams &p, int seq, int k) {
  if (p.timeline && p.timeline_mode == 2 && (seq == 1 || seq == 2)) stamp(p.timeline, (seq - 1) * 8 + k);
}

template <int BN, int STAGES, bool CLUSTER, int OUT_TILES, bool RELAY, bool PAIR, int EW, bool OUT32 = false, bool SINGLE = false>
__global__ void __launch_bounds__(kThreadsFor(EW, RELAY), 1)
fused_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmO, const TcParams p) {
  using L = SmemLayout<BN, STAGES, CLUSTER, OUT_TILES, RELAY, PAIR, EW, OUT32, SINGLE>;
  constexpr int HC = L::kHalfCols;      // columns per epilogue thread
  constexpr int NCH = HC / 32;          // 32-column chunks per epilogue thread
  constexpr int kEpiThreads = EW * 32;
  constexpr int PARTS = BN / HC;        // threads that share a row (split epilogue)
  static_assert(!RELAY || (EW == 16 && CLUSTER && !PAIR && OUT_TILES == 1 && !OUT32), "relay epilogue: cluster flavour, f16 staged stores, sixteen warps");
  // SINGLE: every CTA owns exactly one tile (the launcher checks it).  Nothing can overlap with a
  // next tile then, so the exp group keeps the first 64 columns of its share in registers and
  // writes them out itself, through staging tiles laid over the operand stages (idle once the
  // tile's accumulator is complete); the store group takes only the last 64 columns.
  static_assert(!SINGLE || (RELAY && STAGES * L::kStageBytes >= 8 * 4096), "single-tile form: relay only");
  static_assert(!OUT32 || (!RELAY && !PAIR && EW == 8 && OUT_TILES >= 1), "f32 output: the eight-warp split epilogue with staged stores");
  static_assert(EW == 8 || (CLUSTER && OUT_TILES == 1 && !PAIR), "sixteen epilogue warps: cluster flavour with staged stores only");
  // The 128-byte swizzle needs the stage buffers on 1024-byte boundaries.  There is no
  // static shared memory in this kernel, so the dynamic window starts aligned; if it ever
  // does not, every thread leaves before any barrier or TMEM state exists.
  extern __shared__ __align__(1024) uint8_t smem[];
  // the first TMA instruction waits for its descriptor: ask for all three before anything else
  if (threadIdx.x == 0) { tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); tma_prefetch_desc(&tmO); }
  if ((smem_u32(smem) & 1023u) != 0) { record_failure(p.status, WTC_DEV_BAD_SMEM_ALIGN); return; }

  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L::kOffBars);
  uint64_t *full = bars;
  uint64_t *empty = bars + STAGES;
  uint64_t *accum_full = bars + 2 * STAGES;
  uint64_t *accum_empty = bars + 2 * STAGES + 2;
  uint64_t *stats_bar = bars + 2 * STAGES + 4;
  uint64_t *xdone = bars + 2 * STAGES + 8;                         // relay: first group -> second group, per accumulator buffer
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + L::kOffTmemSlot);
  float2 *pair = reinterpret_cast<float2 *>(smem + L::kOffPair);    // [2][BM]
  float2 *stats = reinterpret_cast<float2 *>(smem + L::kOffStats);  // [2][kMaxCluster][BM]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Cluster geometry.  PAIR: ranks 2j and 2j+1 form one tcgen05 CTA pair (256 rows x BN
  // columns; the even CTA issues the MMAs); j is the column block.  The CTAs that swap row
  // statistics are the ones with the same rows: same parity when paired.
  constexpr bool CLUSTERED = CLUSTER || PAIR;
  const uint32_t cta_rank = CLUSTERED ? cluster_ctarank() : 0u;
  const uint32_t cluster_size = CLUSTERED ? cluster_nctarank() : 1u;
  const uint32_t pair_rank = PAIR ? (cta_rank & 1u) : 0u;
  const uint32_t leader_rank = PAIR ? (cta_rank & ~1u) : cta_rank;
  const bool is_leader = pair_rank == 0;
  const uint32_t col_rank = PAIR ? (cta_rank >> 1) : cta_rank;               // my column block inside the cluster
  const uint32_t cluster_n = CLUSTER ? (PAIR ? cluster_size / 2 : cluster_size) : 1u;   // CTAs that share my rows

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&accum_full[i], 1);
      mbar_init(&accum_empty[i], (RELAY ? kEpiThreads / 2 : kEpiThreads) * (PAIR ? 2 : 1));
      mbar_init(&xdone[i], kEpiThreads / 2);
    }
    for (int i = 0; i < 4; ++i) mbar_init(&stats_bar[i], 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    if (PAIR) { tmem_alloc_pair(tmem_slot, 2 * BN); tmem_relinquish_pair(); }
    else { tmem_alloc(tmem_slot, 2 * BN); tmem_relinquish(); }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (CLUSTERED) cluster_sync_all();   // every peer's barriers exist before anyone signals them
  // Programmatic dependent launch: everything above overlapped the tail of the previous
  // kernel on the stream; from here on global memory is touched, so wait for that kernel
  // to finish, and let the next one start its own set-up as our CTAs retire.
  grid_dependency_wait();
  grid_launch_dependents();
  if (threadIdx.x == 64 && p.timeline_mode == 0) stamp(p.timeline, 0);

  // ---- work distribution --------------------------------------------------
  int first, stride;
  if (CLUSTERED) { first = blockIdx.x / cluster_size; stride = gridDim.x / cluster_size; }
  else { first = blockIdx.x; stride = gridDim.x; }

  // Work items count "row units": one 128-row block, or one 256-row pair of blocks.
  auto decode = [&](int w, int &b, int &rb, int &nb) {
    int ru;
    if (CLUSTER) { b = w / p.num_ru; ru = w - b * p.num_ru; nb = col_rank; }
    else {
      const int per_batch = p.num_ru * p.num_nb;
      b = w / per_batch;
      int t = w - b * per_batch;
      // groups of `group_rb` row units; inside a group the column block is the slow
      // index, so concurrently running CTAs share B column blocks and the group's A rows
      // stay in L2.
      const int per_group = p.group_rb * p.num_nb;
      const int g = t / per_group;
      t -= g * per_group;
      const int rows_here = min(p.group_rb, p.num_ru - g * p.group_rb);
      nb = t / rows_here;
      ru = g * p.group_rb + (t - nb * rows_here);
    }
    rb = PAIR ? ru * 2 + static_cast<int>(pair_rank) : ru;
  };

  // hands accumulator buffer `ab` back to the MMA warp (of the pair's even CTA)
  auto release_accumulator = [&](int ab) {
    if (PAIR) mbar_arrive_remote_release(map_to_cta(smem_u32(&accum_empty[ab]), leader_rank));
    else mbar_arrive(&accum_empty[ab]);
  };
  // cluster rank of the j-th CTA that holds the same rows as this one
  auto row_peer = [&](uint32_t j) -> uint32_t { return PAIR ? 2 * j + pair_rank : j; };

  // (row max, 1 / row sum) from the pairs the CTAs of the cluster sent for statistics set
  // `set`: all loads first, then a max tree, independent exps, a sum tree.
  auto combine_cluster_stats = [&](int set, int row, float &gm, float &inv_gl) {
    float2 st[kMaxCluster];
#pragma unroll
    for (int j = 0; j < kMaxCluster; ++j)
      st[j] = static_cast<uint32_t>(j) < cluster_n ? stats[(set * kMaxCluster + j) * BM + row] : make_float2(-INFINITY, 0.f);
    gm = fmaxf(fmaxf(max3(st[0].x, st[1].x, st[2].x), max3(st[3].x, st[4].x, st[5].x)), fmaxf(st[6].x, st[7].x));
    float t[kMaxCluster];
#pragma unroll
    for (int j = 0; j < kMaxCluster; ++j) t[j] = st[j].y * ex2_approx(st[j].x - gm);
    inv_gl = rcp_approx(((t[0] + t[1]) + (t[2] + t[3])) + ((t[4] + t[5]) + (t[6] + t[7])));
  };

  // Relay epilogue: register reallocation between aligned groups of four warps.  The exp
  // group needs a whole row share (128 values) in registers, the others need little; each
  // role's code sits under its own reallocation so the allocator sees one budget per region.
  const int relay_role = !RELAY ? 0 : (warp < 4 ? 0 : (warp < 12 ? 1 : 2));
  if (RELAY && relay_role == 1) {
    setmaxnreg_inc<SINGLE ? 160 : 152>();
    // ======================= softmax epilogue, two-stage relay ==============
    // Two groups of eight epilogue warps work on consecutive tiles at the same time.  The
    // first group (warps 4-11, 152 registers a thread after the reallocation above) turns
    // the accumulator into exp values in place in tensor memory and sends the row
    // statistics round the cluster; the second group (warps 12-19, 64 registers) waits for
    // the cluster's statistics, reads the exp values back 32 columns at a time, scales,
    // packs and stores them.  The exchange latency and the store phase of tile i are
    // hidden behind the exp phase of tile i+1.  Warps 2 and 3 only fill up the first
    // warpgroup (register reallocation works on aligned groups of four warps).
    const int q = warp & 3;                       // TMEM lane quarter this warp may touch
    const int row_in_tile = q * 32 + lane;
    const float c2 = p.c2;
    const bool pos = c2 >= 0.f;
    float *mh = reinterpret_cast<float *>(smem + L::kOffMh);   // [2][2][BM]: each half's own maximum, per tile parity
    // ---------------- first group: max, exp in place, statistics out ----------------
    const int half = (warp - 4) >> 2;
    const bool stamper = threadIdx.x == 128;
    float2 *mine = &pair[half * BM + row_in_tile];
    const float2 *other = &pair[(half ^ 1) * BM + row_in_tile];
    for (int it = 0; first + it * stride < p.num_items; ++it) {
      const int w = first + it * stride;
      int b, rb, nb; decode(w, b, rb, nb);
      const int ab = it & 1;
      const uint32_t tile_phase = (it >> 1) & 1;
      const int sset = it & 3;
      if (!mbar_wait(&accum_full[ab], tile_phase)) { record_failure(p.status, WTC_DEV_TIMEOUT_ACCUM); break; }
      tc_fence_after_sync();
      if (stamper && it == 0 && p.timeline_mode == 0) stamp(p.timeline, 1);
      if (stamper) { stamp_tile(p, it, 0); stamp_fine(p, it, 0); }
      const uint32_t tbase = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + ab * BN + half * HC;
      const int col0 = nb * BN + half * HC;
      const int valid = max(0, min(HC, p.N - col0));
      uint32_t r[NCH][32];
      float m_half;
      if (valid == HC && !p.round_logits_f16) {
        // whole share, no rounding: the second half of the loads is in flight while the
        // extreme of the first half is taken
        float m0, m1, m2, m3;
        auto fold = [&](const uint32_t (&v)[32]) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            if (pos) {
              m0 = max3(m0, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
              m1 = max3(m1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
              m2 = max3(m2, __uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
              m3 = max3(m3, __uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
            } else {
              m0 = min3(m0, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
              m1 = min3(m1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
              m2 = min3(m2, __uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
              m3 = min3(m3, __uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
            }
          }
        };
#pragma unroll
        for (int c = 0; c < NCH / 2; ++c) tmem_ld_32x32b_x32(tbase + c * 32, r[c]);
        tmem_ld_wait();
#pragma unroll
        for (int c = NCH / 2; c < NCH; ++c) tmem_ld_32x32b_x32(tbase + c * 32, r[c]);
        m0 = __uint_as_float(r[0][0]); m1 = __uint_as_float(r[0][1]); m2 = __uint_as_float(r[0][2]); m3 = __uint_as_float(r[0][3]);
#pragma unroll
        for (int c = 0; c < NCH / 2; ++c) fold(r[c]);
        tmem_ld_wait();
        if (stamper) stamp_fine(p, it, 1);
#pragma unroll
        for (int c = NCH / 2; c < NCH; ++c) fold(r[c]);
        m_half = (pos ? fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) : fminf(fminf(m0, m1), fminf(m2, m3))) * c2;
      } else {
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          if (c * 32 < valid) tmem_ld_32x32b_x32(tbase + c * 32, r[c]);
          else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[c][i] = 0u;
          }
        }
        tmem_ld_wait();
        if (stamper) stamp_fine(p, it, 1);
        if (p.round_logits_f16) {
#pragma unroll
          for (int c = 0; c < NCH; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) r[c][i] = __float_as_uint(__half2float(__float2half_rn(__uint_as_float(r[c][i]))));
        }
        // ---- extreme of the raw accumulators (max if scale >= 0, else min), four chains ----
        if (valid == HC) {
          float m0 = __uint_as_float(r[0][0]), m1 = __uint_as_float(r[0][1]);
          float m2 = __uint_as_float(r[0][2]), m3 = __uint_as_float(r[0][3]);
          if (pos) {
#pragma unroll
            for (int c = 0; c < NCH; ++c)
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                m0 = max3(m0, __uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1]));
                m1 = max3(m1, __uint_as_float(r[c][i + 2]), __uint_as_float(r[c][i + 3]));
                m2 = max3(m2, __uint_as_float(r[c][i + 4]), __uint_as_float(r[c][i + 5]));
                m3 = max3(m3, __uint_as_float(r[c][i + 6]), __uint_as_float(r[c][i + 7]));
              }
            m_half = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
          } else {
#pragma unroll
            for (int c = 0; c < NCH; ++c)
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                m0 = min3(m0, __uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1]));
                m1 = min3(m1, __uint_as_float(r[c][i + 2]), __uint_as_float(r[c][i + 3]));
                m2 = min3(m2, __uint_as_float(r[c][i + 4]), __uint_as_float(r[c][i + 5]));
                m3 = min3(m3, __uint_as_float(r[c][i + 6]), __uint_as_float(r[c][i + 7]));
              }
            m_half = fminf(fminf(m0, m1), fminf(m2, m3));
          }
          m_half *= c2;
        } else if (valid > 0) {
          float m = __uint_as_float(r[0][0]);
#pragma unroll
          for (int c = 0; c < NCH; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i < valid) m = pos ? fmaxf(m, __uint_as_float(r[c][i])) : fminf(m, __uint_as_float(r[c][i]));
          m_half = m * c2;
        } else {
          m_half = -INFINITY;
        }
      }
      if (stamper) stamp_fine(p, it, 2);
      // ---- e = 2^(v - m_half) in place, row sum; each chunk goes back over its logits ----
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
      if (valid == HC) {
        // (single-tile form: the chunks that go to tensor memory first, so their registers are
        // free while the two chunks this thread keeps are processed and held)
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
          const int c = SINGLE ? (k + 2) % NCH : k;
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float e0 = ex2_approx(fmaf(__uint_as_float(r[c][i]), c2, -m_half));
            const float e1 = ex2_approx(fmaf(__uint_as_float(r[c][i + 1]), c2, -m_half));
            const float e2 = ex2_approx(fmaf(__uint_as_float(r[c][i + 2]), c2, -m_half));
            const float e3 = ex2_approx(fmaf(__uint_as_float(r[c][i + 3]), c2, -m_half));
            s0 += e0; s1 += e1; s2 += e2; s3 += e3;
            r[c][i] = __float_as_uint(e0); r[c][i + 1] = __float_as_uint(e1);
            r[c][i + 2] = __float_as_uint(e2); r[c][i + 3] = __float_as_uint(e3);
          }
          if (!(SINGLE && c < 2)) tmem_st_32x32b_x32(tbase + c * 32, r[c]);
        }
      } else {
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
          const int c = SINGLE ? (k + 2) % NCH : k;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float e = 0.f;
            if (c * 32 + i < valid) e = ex2_approx(fmaf(__uint_as_float(r[c][i]), c2, -m_half));
            s0 += e;
            r[c][i] = __float_as_uint(e);
          }
          if (c * 32 < valid && !(SINGLE && c < 2)) tmem_st_32x32b_x32(tbase + c * 32, r[c]);
        }
      }
      const float sum = (s0 + s1) + (s2 + s3);
      if (stamper && it == 0 && p.timeline_mode == 0) stamp(p.timeline, 2);
      if (stamper) { stamp_tile(p, it, 1); stamp_fine(p, it, 3); }
      // ---- the two halves of a row meet through shared memory, the CTAs through the cluster ----
      *mine = make_float2(m_half, sum);
      mh[((it & 1) * 2 + half) * BM + row_in_tile] = m_half;
      named_bar_sync(1 + q, 64);
      const float2 o = *other;
      named_bar_sync(1 + q, 64);
      if (half == 0) {
        const float lm = fmaxf(m_half, o.x);
        const float ll = (m_half == -INFINITY ? 0.f : sum * ex2_approx(m_half - lm)) +
                         (o.x == -INFINITY ? 0.f : o.y * ex2_approx(o.x - lm));
        const uint32_t slot = smem_u32(&stats[(sset * kMaxCluster + col_rank) * BM + row_in_tile]);
        const uint32_t bar = smem_u32(&stats_bar[sset]);
        for (uint32_t peer = 0; peer < cluster_n; ++peer)
          st_async_f32x2(map_to_cta(slot, row_peer(peer)), lm, ll, map_to_cta(bar, row_peer(peer)));
      }
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&xdone[ab]);                    // exp values parked, maxima published
      if (stamper) stamp_tile(p, it, 2);
      if (SINGLE && valid > 0) {
        // ---- single-tile form: this thread scales, packs and stores its first 64 columns itself ----
        if (!mbar_wait_cluster(&stats_bar[sset], 0)) { record_failure(p.status, WTC_DEV_TIMEOUT_STATS); break; }
        float gm, inv_gl;
        {
          float xs[kMaxCluster];
#pragma unroll
          for (int j = 0; j < kMaxCluster; ++j)
            xs[j] = static_cast<uint32_t>(j) < cluster_n ? stats[(sset * kMaxCluster + j) * BM + row_in_tile].x : -INFINITY;
          gm = fmaxf(fmaxf(max3(xs[0], xs[1], xs[2]), max3(xs[3], xs[4], xs[5])), fmaxf(xs[6], xs[7]));
          float l = 0.f;
#pragma unroll
          for (int j = 0; j < kMaxCluster; ++j)
            if (static_cast<uint32_t>(j) < cluster_n) l += stats[(sset * kMaxCluster + j) * BM + row_in_tile].y * ex2_approx(xs[j] - gm);
          inv_gl = rcp_approx(l);
        }
        const float f = ex2_approx(m_half - gm) * inv_gl;
        uint8_t *xstg = smem + (warp - 4) * 4096;   // over operand stage 0: every stage has been consumed
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t hc[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const __half2 hh = __floats2half2_rn(__uint_as_float(r[c][i]) * f, __uint_as_float(r[c][i + 1]) * f);
            hc[i >> 1] = *reinterpret_cast<const uint32_t *>(&hh);
          }
          stage_row_chunk(xstg, lane, c, hc);       // (columns past `valid` hold zeros: e was 0 there)
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const int row0 = rb * BM + q * 32;
          if (row0 < p.M) tma_store_3d(&tmO, xstg, col0, row0, b);
          tma_store_commit();
          tma_store_wait_all();
        }
      }
    }
  } else if (RELAY && relay_role == 2) {
    setmaxnreg_dec<SINGLE ? 56 : 64>();
    const int q = warp & 3;                       // TMEM lane quarter this warp may touch
    const int row_in_tile = q * 32 + lane;
    float *mh = reinterpret_cast<float *>(smem + L::kOffMh);   // [2][2][BM]: each half's own maximum, per tile parity
    const int yw = warp - 12;
    const int half = yw >> 2;
    const bool lead = threadIdx.x == 384;
    uint8_t *stg = smem + L::kOffOut + yw * L::kOutWarpBytes;
    for (int it = 0; first + it * stride < p.num_items; ++it) {
      const int w = first + it * stride;
      int b, rb, nb; decode(w, b, rb, nb);
      const int ab = it & 1;
      const uint32_t tile_phase = (it >> 1) & 1;
      const int sset = it & 3;
      if (lead) mbar_expect_tx(&stats_bar[sset], cluster_n * BM * 8);
      if (!mbar_wait(&xdone[ab], tile_phase)) { record_failure(p.status, WTC_DEV_TIMEOUT_ACCUM); break; }
      tc_fence_after_sync();
      if (lead) stamp_fine(p, it, 4);
      if (!mbar_wait_cluster(&stats_bar[sset], (it >> 2) & 1)) { record_failure(p.status, WTC_DEV_TIMEOUT_STATS); break; }
      if (lead && it == 0 && p.timeline_mode == 0) stamp(p.timeline, 3);
      if (lead) stamp_fine(p, it, 5);
      float gm, inv_gl;
      combine_cluster_stats(sset, row_in_tile, gm, inv_gl);
      const float f = ex2_approx(mh[((it & 1) * 2 + half) * BM + row_in_tile] - gm) * inv_gl;
      const uint32_t tbase = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + ab * BN + half * HC;
      const int col0 = nb * BN + half * HC;
      const int valid = max(0, min(HC, p.N - col0));
      const int row0 = rb * BM + q * 32;
      const bool rows_live = row0 < p.M;
      // 32 columns at a time through one register buffer (the scheduler's other warps cover
      // the load latency).  The first 64 columns are staged as they are packed, the last 64
      // wait packed in registers, so the accumulator buffer goes back to the MMA warp after
      // the fourth load and before anything waits for a store.
      static_assert(!RELAY || NCH == 4, "relay epilogue: a thread owns 128 columns");
      if (valid == 0 || (SINGLE && valid <= 64)) { tc_fence_before_sync(); release_accumulator(ab); }
      if (lane == 0) tma_store_wait_read();         // the previous tile's store has read the staging tile
      __syncwarp();
      uint32_t h[2][16];
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        uint32_t hc[16];
        if (SINGLE && c < 2) continue;                // the exp group writes these columns itself
        if (c * 32 < valid) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tbase + c * 32, r);
          tmem_ld_wait();
          if ((c + 1) * 32 >= valid) {                // that was my last read of this accumulator buffer
            tc_fence_before_sync();
            release_accumulator(ab);
          }
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const __half2 hh = __floats2half2_rn(__uint_as_float(r[i]) * f, __uint_as_float(r[i + 1]) * f);
            hc[i >> 1] = *reinterpret_cast<const uint32_t *>(&hh);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) hc[i] = 0u;
        }
        if (c < 2 || SINGLE) stage_row_chunk(stg, lane, c & 1, hc);   // single-tile form: nothing in flight, stage straight away
        else {
#pragma unroll
          for (int i = 0; i < 16; ++i) h[c - 2][i] = hc[i];
        }
      }
      if (valid > 0 && !SINGLE) {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (rows_live) tma_store_3d(&tmO, stg, col0, row0, b);
          tma_store_commit();
        }
      }
      if (valid > 64) {
        if (!SINGLE) {
          if (lane == 0) tma_store_wait_read();
          __syncwarp();
          stage_row_chunk(stg, lane, 0, h[0]);
          stage_row_chunk(stg, lane, 1, h[1]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (rows_live) tma_store_3d(&tmO, stg, col0 + 64, row0, b);
          tma_store_commit();
        }
      }
      if (lead && it == 0 && p.timeline_mode == 0) stamp(p.timeline, 4);
      if (lead) { stamp_tile(p, it, 3); stamp_fine(p, it, 7); }
    }
    if (lane == 0) tma_store_wait_all();
    if (lead && p.timeline_mode == 0) stamp(p.timeline, 5);
    
  } else {
  if (RELAY) setmaxnreg_dec<SINGLE ? 40 : 48>();
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
          if (PAIR) {
            // both CTAs of the pair fill their own stage; all bytes are counted on the even CTA's barrier
            if (is_leader) mbar_expect_tx(&full[s], 2 * L::kStageBytes);
            tma_load_3d_pair(sa, &tmA, &full[s], kb * BK, rb * BM, b);
#pragma unroll
            for (int j = 0; j < BN / 128; ++j)
              tma_load_3d_pair(sb + j * (BK * 128), &tmB, &full[s], nb * BN + static_cast<int>(pair_rank) * (BN / 2) + j * 64, kb * BK,
                               p.b_batched ? b : 0);
          } else {
            mbar_expect_tx(&full[s], L::kStageBytes);
            tma_load_3d(sa, &tmA, &full[s], kb * BK, rb * BM, b);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sb + j * (BK * 128), &tmB, &full[s], nb * BN + j * 64, kb * BK, p.b_batched ? b : 0);
          }
          if (n == 0 && p.timeline_mode == 0) stamp(p.timeline, 6);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // ======================= MMA issuer (the even CTA of a pair only) =======
    constexpr uint32_t idesc = umma_idesc_f16_f32(PAIR ? 2 * BM : BM, BN, /*a_mn_major=*/0, /*b_mn_major=*/1);
    const uint16_t pair_mask = static_cast<uint16_t>(3u << leader_rank);
    uint32_t n = 0;
    int it = 0;
    bool ok = true;
    for (int w = first; w < p.num_items && ok && is_leader; w += stride, ++it) {
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
          if (n == 0 && p.timeline_mode == 0) stamp(p.timeline, 7);
          const uint32_t sa = smem_u32(smem + s * L::kStageBytes);
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = umma_smem_desc_sw128(sa + k * p.geom.a_kstep, p.geom.a_lbo, p.geom.a_sbo);
            const uint64_t db = umma_smem_desc_sw128(sb + k * p.geom.b_kstep, p.geom.b_lbo, p.geom.b_sbo);
            if (PAIR) umma_f16_ss_pair(d_tmem, da, db, idesc, (kb | k) != 0);
            else umma_f16_ss(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          // frees the stage (in both CTAs of a pair) once these MMAs have read it
          if (PAIR) umma_commit_pair(&empty[s], pair_mask);
          else umma_commit(&empty[s]);
        }
        __syncwarp();
      }
      if (ok && lane == 0) {
        if (PAIR) umma_commit_pair(&accum_full[ab], pair_mask);
        else umma_commit(&accum_full[ab]);
        if (it == 0 && p.timeline_mode == 0) stamp(p.timeline, 8);
      }
      __syncwarp();
    }
  } else if (!RELAY) {
    // ======================= softmax epilogue ==============================
    const int q = warp & 3;                      // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;            // which part (of PARTS) of the tile's columns
    const int row_in_tile = q * 32 + lane;
    const bool lead = threadIdx.x == 64;         // first epilogue thread: posts expect_tx, stamps
    uint8_t *stg = smem + L::kOffOut + (warp - 2) * L::kOutWarpBytes;   // one 32-row x 64-col f16 tile
    float2 *mine = &pair[half * BM + row_in_tile];
    const float2 *other = &pair[(half ^ 1) * BM + row_in_tile];
    const float c2 = p.c2;
    const bool pos = c2 >= 0.f;
    int it = 0;
    uint32_t gcount = 0;                         // staging groups committed so far by this warp
    for (int w = first; w < p.num_items; w += stride, ++it) {
      int b, rb, nb; decode(w, b, rb, nb);
      const int ab = it & 1;
      const int par = it & 1;
      const uint32_t tile_phase = (it >> 1) & 1;
      if (CLUSTER && lead) mbar_expect_tx(&stats_bar[par], cluster_n * BM * 8);
      if (!mbar_wait(&accum_full[ab], tile_phase)) { record_failure(p.status, WTC_DEV_TIMEOUT_ACCUM); break; }
      tc_fence_after_sync();
      if (lead && it == 0 && p.timeline_mode == 0) stamp(p.timeline, 1);
      if (lead) { stamp_tile(p, it, 0); stamp_fine(p, it, 0); }
      const uint32_t tbase = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + ab * BN + half * HC;
      const int col0 = nb * BN + half * HC;               // first matrix column of this thread
      const int valid = max(0, min(HC, p.N - col0));      // my columns that exist
      const int row0 = rb * BM + q * 32;                  // first row of this warp
      const bool rows_live = row0 < p.M;

      // ---- the thread's whole share of the accumulator row goes to registers at once,
      //      and the accumulator buffer is handed back to the MMA warp straight away ----
      uint32_t r[NCH][32];
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        if (c * 32 < valid) tmem_ld_32x32b_x32(tbase + c * 32, r[c]);
        else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[c][i] = 0u;
        }
      }
      tmem_ld_wait();
      tc_fence_before_sync();
      release_accumulator(ab);
      if (lead && it == 0 && p.timeline_mode == 0) stamp(p.timeline, 14);
      if (lead) stamp_fine(p, it, 1);
      if (p.round_logits_f16) {
#pragma unroll
        for (int c = 0; c < NCH; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) r[c][i] = __float_as_uint(__half2float(__float2half_rn(__uint_as_float(r[c][i]))));
      }

      // ---- extreme of the raw accumulators (max if scale >= 0, else min), four chains ----
      float m_half;
      if (valid == HC) {
        float m0 = __uint_as_float(r[0][0]), m1 = __uint_as_float(r[0][1]);
        float m2 = __uint_as_float(r[0][2]), m3 = __uint_as_float(r[0][3]);
        if (pos) {
#pragma unroll
          for (int c = 0; c < NCH; ++c)
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              m0 = max3(m0, __uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1]));
              m1 = max3(m1, __uint_as_float(r[c][i + 2]), __uint_as_float(r[c][i + 3]));
              m2 = max3(m2, __uint_as_float(r[c][i + 4]), __uint_as_float(r[c][i + 5]));
              m3 = max3(m3, __uint_as_float(r[c][i + 6]), __uint_as_float(r[c][i + 7]));
            }
          m_half = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
        } else {
#pragma unroll
          for (int c = 0; c < NCH; ++c)
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              m0 = min3(m0, __uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1]));
              m1 = min3(m1, __uint_as_float(r[c][i + 2]), __uint_as_float(r[c][i + 3]));
              m2 = min3(m2, __uint_as_float(r[c][i + 4]), __uint_as_float(r[c][i + 5]));
              m3 = min3(m3, __uint_as_float(r[c][i + 6]), __uint_as_float(r[c][i + 7]));
            }
          m_half = fminf(fminf(m0, m1), fminf(m2, m3));
        }
        m_half *= c2;
      } else if (valid > 0) {
        float m = __uint_as_float(r[0][0]);
#pragma unroll
        for (int c = 0; c < NCH; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < valid) m = pos ? fmaxf(m, __uint_as_float(r[c][i])) : fminf(m, __uint_as_float(r[c][i]));
        m_half = m * c2;
      } else {
        m_half = -INFINITY;
      }

      if (lead && it == 0 && p.timeline_mode == 0) stamp(p.timeline, 15);
      if (lead) stamp_fine(p, it, 2);
      // ---- e = 2^(v - m_half) in place, row sum ----
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
      if (valid == HC) {
#pragma unroll
        for (int c = 0; c < NCH; ++c)
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float e0 = ex2_approx(fmaf(__uint_as_float(r[c][i]), c2, -m_half));
            const float e1 = ex2_approx(fmaf(__uint_as_float(r[c][i + 1]), c2, -m_half));
            const float e2 = ex2_approx(fmaf(__uint_as_float(r[c][i + 2]), c2, -m_half));
            const float e3 = ex2_approx(fmaf(__uint_as_float(r[c][i + 3]), c2, -m_half));
            s0 += e0; s1 += e1; s2 += e2; s3 += e3;
            r[c][i] = __float_as_uint(e0); r[c][i + 1] = __float_as_uint(e1);
            r[c][i + 2] = __float_as_uint(e2); r[c][i + 3] = __float_as_uint(e3);
          }
      } else {
#pragma unroll
        for (int c = 0; c < NCH; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float e = 0.f;
            if (c * 32 + i < valid) e = ex2_approx(fmaf(__uint_as_float(r[c][i]), c2, -m_half));
            s0 += e;
            r[c][i] = __float_as_uint(e);
          }
      }
      float sum = (s0 + s1) + (s2 + s3);
      if (lead && it == 0 && p.timeline_mode == 0) stamp(p.timeline, 2);
      if (lead) { stamp_tile(p, it, 1); stamp_fine(p, it, 3); }

      float lm;                                    // tile-row max (log2 domain)
      float2 o = make_float2(-INFINITY, 0.f);      // PARTS == 2: the other half's (max, sum)
      float ll4 = 0.f;                             // PARTS == 4: the row's sum over the four parts (part 0 only)
      if (PARTS == 2) {
        // ---- the two halves of a row meet through shared memory ----
        *mine = make_float2(m_half, sum);
        named_bar_sync(1 + q, 64);
        o = *other;
        named_bar_sync(1 + q, 64);                 // both have read: the slots may be reused
        lm = fmaxf(m_half, o.x);
      } else {
        // ---- four parts of a row: parts 1..3 leave their (max, sum) in their own warp's
        //      staging tile (idle now: its last store has been read), part 0 collects.  Only
        //      part 0 needs the combination; the others just signal and move on. ----
        if (lane == 0) tma_store_wait_read();
        __syncwarp();
        if (half != 0) {
          *reinterpret_cast<float2 *>(stg + lane * 8) = make_float2(m_half, sum);
          named_bar_arrive(1 + q, 128);
          lm = m_half;                             // unused by parts 1..3
        } else {
          named_bar_sync(1 + q, 128);
          lm = m_half;
          float2 part[3];
#pragma unroll
          for (int j = 0; j < 3; ++j) {
            part[j] = *reinterpret_cast<const float2 *>(smem + L::kOffOut + (4 * (j + 1) + ((q + 2) & 3)) * L::kOutWarpBytes + lane * 8);
            lm = fmaxf(lm, part[j].x);
          }
          ll4 = sum * ex2_approx(m_half - lm);
#pragma unroll
          for (int j = 0; j < 3; ++j) ll4 += part[j].x == -INFINITY ? 0.f : part[j].y * ex2_approx(part[j].x - lm);
        }
      }
      float f;                                     // what my e values still have to be multiplied by
      if (CLUSTER) {
        const float ll = PARTS == 4 ? ll4
                                    : (m_half == -INFINITY ? 0.f : sum * ex2_approx(m_half - lm)) +
                                          (o.x == -INFINITY ? 0.f : o.y * ex2_approx(o.x - lm));
        // ... and the CTAs of the cluster through each other's shared memory
        if (half == 0) {
          const uint32_t slot = smem_u32(&stats[(par * kMaxCluster + col_rank) * BM + row_in_tile]);
          const uint32_t bar = smem_u32(&stats_bar[par]);
          for (uint32_t peer = 0; peer < cluster_n; ++peer)
            st_async_f32x2(map_to_cta(slot, row_peer(peer)), lm, ll, map_to_cta(bar, row_peer(peer)));
        }
        if (!mbar_wait_cluster(&stats_bar[par], tile_phase)) { record_failure(p.status, WTC_DEV_TIMEOUT_STATS); break; }
        if (lead && it == 0 && p.timeline_mode == 0) stamp(p.timeline, 3);
        if (lead) { stamp_tile(p, it, 2); stamp_fine(p, it, 4); }
        float gm, inv_gl;
        combine_cluster_stats(par, row_in_tile, gm, inv_gl);
        f = ex2_approx(m_half - gm) * inv_gl;
      } else {
        f = ex2_approx(m_half - lm);               // tiled: values relative to the tile max, not normalised
      }

      if (lead) stamp_fine(p, it, 5);              // row statistics combined, factor known
      // ---- p = e * f -> f16 -> global memory ----
      float sum_r = 0.f;                           // tiled: sum of what is actually stored
      if (OUT32) {
        // f32 probabilities: 32 columns (one 128-byte row) per staging tile and TMA store
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          if (c * 32 < valid) {
            uint8_t *tile = stg + (OUT_TILES == 2 ? (gcount & 1) * 4096 : 0);
            if (lane == 0) { if (OUT_TILES == 2) tma_store_wait_read1(); else tma_store_wait_read(); }
            __syncwarp();
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) { v[i] = __uint_as_float(r[c][i]) * f; if (!CLUSTER) sum_r += v[i]; }
            stage_row_f32(tile, lane, v);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (rows_live) tma_store_3d(&tmO, tile, col0 + c * 32, row0, b);
              tma_store_commit();
            }
            ++gcount;
          }
        }
      } else if (OUT_TILES == 0) {
        // straight from registers: each thread owns 256 contiguous bytes of its row
        const int row = rb * BM + row_in_tile;
        __half *orow = static_cast<__half *>(p.out) + static_cast<long long>(b) * p.o_batch_stride + static_cast<long long>(row) * p.ldo + col0;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          if (c * 32 < valid) {
            uint32_t h[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const __half2 hh = __floats2half2_rn(__uint_as_float(r[c][i]) * f, __uint_as_float(r[c][i + 1]) * f);
              if (!CLUSTER) { const float2 back = __half22float2(hh); sum_r += back.x + back.y; }
              h[i >> 1] = *reinterpret_cast<const uint32_t *>(&hh);
            }
            if (row < p.M) st_global_row32(orow + c * 32, h, p.out_align32, valid - c * 32);
          }
        }
      } else {
        // 128-byte-swizzled staging tiles in shared memory, written out by TMA.
        if (OUT_TILES * 2 >= NCH) {
          // the warp's whole share of the tile fits its staging tiles: pack and stage
          // everything, then ONE proxy fence and warp barrier, then all stores back to back
          if (lane == 0) tma_store_wait_read();    // the previous tile's stores have read the staging tiles
          __syncwarp();
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            if (c * 32 < valid) {
              uint32_t h[16];
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                const __half2 hh = __floats2half2_rn(__uint_as_float(r[c][i]) * f, __uint_as_float(r[c][i + 1]) * f);
                if (!CLUSTER) { const float2 back = __half22float2(hh); sum_r += back.x + back.y; }
                h[i >> 1] = *reinterpret_cast<const uint32_t *>(&hh);
              }
              stage_row_chunk(stg + (c >> 1) * 4096, lane, c & 1, h);
            }
          }
          if (lead) stamp_fine(p, it, 6);          // packed and staged
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (rows_live) {
#pragma unroll
              for (int g = 0; g < NCH / 2; ++g)
                if (g * 64 < valid) tma_store_3d(&tmO, stg + g * 4096, col0 + g * 64, row0, b);
            }
            tma_store_commit();
          }
        } else {
          // fewer staging tiles than column groups: 64 columns at a time through one tile
#pragma unroll
          for (int g = 0; g < NCH / 2; ++g) {
            if (g * 64 < valid) {
              if (lane == 0) tma_store_wait_read();
              __syncwarp();
#pragma unroll
              for (int hc = 0; hc < 2; ++hc) {
                const int c = g * 2 + hc;
                uint32_t h[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                  const __half2 hh = __floats2half2_rn(__uint_as_float(r[c][i]) * f, __uint_as_float(r[c][i + 1]) * f);
                  if (!CLUSTER) { const float2 back = __half22float2(hh); sum_r += back.x + back.y; }
                  h[i >> 1] = *reinterpret_cast<const uint32_t *>(&hh);
                }
                stage_row_chunk(stg, lane, hc, h);
              }
              if (lead && g == NCH / 2 - 1) stamp_fine(p, it, 6);
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                if (rows_live) tma_store_3d(&tmO, stg, col0 + g * 64, row0, b);
                tma_store_commit();
              }
            }
          }
        }
      }
      if (!CLUSTER) {
        // tile statistics: max of the tile row, sum of the stored values of both halves
        mine->y = sum_r;
        named_bar_sync(1 + q, 64);
        const int row = rb * BM + row_in_tile;
        if (half == 0 && row < p.M)
          p.tile_stats[(static_cast<int64_t>(b) * p.M + row) * p.num_nb + nb] = make_float2(lm, sum_r + other->y);
        named_bar_sync(1 + q, 64);
      }
      if (lead && it == 0 && p.timeline_mode == 0) stamp(p.timeline, 4);
      if (lead) { stamp_tile(p, it, 3); stamp_fine(p, it, 7); }
    }
    if (lane == 0) tma_store_wait_all();
    if (lead && p.timeline_mode == 0) stamp(p.timeline, 5);
  }

  }   // warps 0-3 of the relay form, every warp of the others

  // ---- teardown: nothing in flight, peers done with our shared memory, TMEM freed ----
  if (p.status && *reinterpret_cast<volatile int *>(p.status) != 0) {
    // a wait gave up somewhere: give copies that were already issued time to land
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (CLUSTERED) cluster_sync_all();
  if (warp == 1) { if (PAIR) tmem_dealloc_pair(tmem_base, 2 * BN); else tmem_dealloc(tmem_base, 2 * BN); }
}

template <int BN, int STAGES, bool CLUSTER, int OUT_TILES, bool RELAY, bool PAIR, int EW, bool OUT32 = false, bool SINGLE = false>
cudaError_t launch_impl(const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmO, TcParams p,
                        int cluster_n, int num_sms, cudaStream_t s, TcLaunchInfo *info) {
  using L = SmemLayout<BN, STAGES, CLUSTER, OUT_TILES, RELAY, PAIR, EW, OUT32, SINGLE>;
  auto kern = fused_tc_kernel<BN, STAGES, CLUSTER, OUT_TILES, RELAY, PAIR, EW, OUT32, SINGLE>;
  static bool attr_set = false;   // per template instance
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  // work items: row units (128 rows, or 256 for a CTA pair) x (column blocks when tiled)
  p.num_ru = PAIR ? (p.num_rb + 1) / 2 : p.num_rb;
  p.num_items = p.batch * p.num_ru * (CLUSTER ? 1 : p.num_nb);
  const int cluster_size = (CLUSTER ? cluster_n : 1) * (PAIR ? 2 : 1);

  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kThreadsFor(EW, RELAY), 1, 1);
  cfg.dynamicSmemBytes = L::kDynamic;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  int nattr = 0;
  if (p.use_pdl) {
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  int grid;
  if (CLUSTER || PAIR) {   // always a cluster launch for these variants, even for a cluster of one
    attr[nattr].id = cudaLaunchAttributeClusterDimension;
    attr[nattr].val.clusterDim.x = cluster_size;
    attr[nattr].val.clusterDim.y = 1;
    attr[nattr].val.clusterDim.z = 1;
    ++nattr;
    cfg.attrs = attr;
    cfg.numAttrs = nattr;
    static int max_clusters_cache[2 * kMaxCluster + 1] = {0};   // per template instance, by cluster size
    if (!max_clusters_cache[cluster_size]) {
      cfg.gridDim = dim3(cluster_size, 1, 1);
      int mc = 0;
      cudaError_t e = cudaOccupancyMaxActiveClusters(&mc, kern, &cfg);
      if (e != cudaSuccess) return e;
      if (mc < 1) return cudaErrorInvalidConfiguration;
      max_clusters_cache[cluster_size] = mc;
    }
    const int max_clusters = max_clusters_cache[cluster_size];
    if (SINGLE && p.num_items > max_clusters) return cudaErrorNotSupported;   // some CTA would own two tiles: the caller takes another form
    const int clusters = p.num_items < max_clusters ? p.num_items : max_clusters;
    grid = clusters * cluster_size;
  } else {
    grid = p.num_items < num_sms ? p.num_items : num_sms;
    cfg.attrs = nattr ? attr : nullptr;
    cfg.numAttrs = nattr;
  }
  cfg.gridDim = dim3(grid, 1, 1);
  if (info) { info->grid = grid; info->cluster = cluster_size; info->smem_bytes = L::kDynamic; info->threads = kThreadsFor(EW, RELAY); }
  return cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmO, p);
}

} // namespace

// Variant choice.  pair: two CTAs share one 256-row MMA (a third less L2 operand traffic per
// flop).  Measured on B200 the contraction runs at the same rate either way, and an
// eight-CTA cluster fits the chip only 15 times, so the cluster flavour pairs only on
// request; the tiled flavour (clusters of two) pairs when the K loop is long.  relay: sixteen
// epilogue warps in two groups that overlap consecutive tiles (cluster flavour, f16, staged
// stores).  store: swizzled staging + TMA stores by default, direct register stores on request.
cudaError_t launch_fused_cluster(const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmO,
                                 const TcParams &p, int bn, int cluster_n, int num_sms, cudaStream_t s,
                                 TcLaunchInfo *info) {
  if (cluster_n < 1 || cluster_n > kMaxCluster) return cudaErrorInvalidValue;
  if (p.out_f32)
    return bn == 128 ? launch_impl<128, 4, true, 2, false, false, 8, true>(tmA, tmB, tmO, p, cluster_n, num_sms, s, info)
                     : launch_impl<kTcBlockN, 3, true, 2, false, false, 8, true>(tmA, tmB, tmO, p, cluster_n, num_sms, s, info);
  // 128-column tiles (a tile choice of best.json): the default schedule only
  if (bn == 128) return launch_impl<128, 4, true, 2, false, false, 8>(tmA, tmB, tmO, p, cluster_n, num_sms, s, info);
  const bool pair = p.pair_mode == 2 && 2 * cluster_n <= kMaxCluster;
  const bool tma = p.store_mode == 1;
  if (pair) {
    if (tma) return launch_impl<kTcBlockN, 4, true, 2, false, true, 8>(tmA, tmB, tmO, p, cluster_n, num_sms, s, info);
    return launch_impl<kTcBlockN, 6, true, 0, false, true, 8>(tmA, tmB, tmO, p, cluster_n, num_sms, s, info);
  }
  if (tma) {
    // the relay pays when a CTA sees several tiles: its two groups then overlap
    const int resident = num_sms / cluster_n;
    const int tiles_per_cta = (p.batch * p.num_rb + resident - 1) / (resident > 0 ? resident : 1);
    const bool relay = p.epilogue_mode == 2 || (p.epilogue_mode == 0 && tiles_per_cta >= kRelayMinTiles);
    if (relay) return launch_impl<kTcBlockN, 3, true, 1, true, false, 16>(tmA, tmB, tmO, p, cluster_n, num_sms, s, info);
    // one tile per CTA: the single-tile relay form (both groups share the tile's store phase), unless
    // a form was asked for; it declines (before launching) when the clusters do not all fit at once
    if (p.epilogue_mode == 0 && p.epilogue_warps != 16) {
      const cudaError_t e = launch_impl<kTcBlockN, 3, true, 1, true, false, 16, false, true>(tmA, tmB, tmO, p, cluster_n, num_sms, s, info);
      if (e != cudaErrorNotSupported) return e;
    }
    // sixteen epilogue warps (a row's columns split four ways) on request: measured on B200 it
    // does not beat eight (the exp and pack phases are bound by the special-function unit)
    if (p.epilogue_warps == 16)
      return launch_impl<kTcBlockN, 3, true, 1, false, false, 16>(tmA, tmB, tmO, p, cluster_n, num_sms, s, info);
    return launch_impl<kTcBlockN, 3, true, 2, false, false, 8>(tmA, tmB, tmO, p, cluster_n, num_sms, s, info);
  }
  return launch_impl<kTcBlockN, 4, true, 0, false, false, 8>(tmA, tmB, tmO, p, cluster_n, num_sms, s, info);
}

cudaError_t launch_tiled_partial(const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmO,
                                 const TcParams &p, int bn, int num_sms, cudaStream_t s, TcLaunchInfo *info) {
  if (p.out_f32)
    return bn == 128 ? launch_impl<128, 6, false, 1, false, false, 8, true>(tmA, tmB, tmO, p, 1, num_sms, s, info)
                     : launch_impl<kTcBlockN, 4, false, 1, false, false, 8, true>(tmA, tmB, tmO, p, 1, num_sms, s, info);
  if (bn == 128) return launch_impl<128, 6, false, 1, false, false, 8>(tmA, tmB, tmO, p, 1, num_sms, s, info);
  const bool pair = p.pair_mode == 2 || (p.pair_mode == 0 && p.num_rb >= 2 && p.num_kb >= 8);
  const bool tma = p.store_mode == 1;
  if (pair) {
    if (tma) return launch_impl<kTcBlockN, 6, false, 1, false, true, 8>(tmA, tmB, tmO, p, 1, num_sms, s, info);
    return launch_impl<kTcBlockN, 6, false, 0, false, true, 8>(tmA, tmB, tmO, p, 1, num_sms, s, info);
  }
  if (tma) return launch_impl<kTcBlockN, 4, false, 1, false, false, 8>(tmA, tmB, tmO, p, 1, num_sms, s, info);
  return launch_impl<kTcBlockN, 4, false, 0, false, false, 8>(tmA, tmB, tmO, p, 1, num_sms, s, info);
}

} // namespace wtc

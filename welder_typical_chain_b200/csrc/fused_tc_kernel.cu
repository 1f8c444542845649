// Fused Matmul -> row-Softmax for sm_100a: f16 operands, f32 accumulate in TMEM,
// f16 (or f32) probabilities.  One persistent, warp-specialised kernel in two flavours:
//
//   CLUSTER = true   a thread-block cluster of ceil(N/BN) CTAs owns 128 complete
//                    rows.  Each CTA contracts its 128 x BN slice, reduces its
//                    local row (max, sum), sends the pair to its peers' shared
//                    memory (st.async + mbarrier transaction bytes: no fences, no
//                    cluster-wide barrier in the loop) and writes normalised values.
//   CLUSTER = false  independent 128 x BN tiles.  Each writes exp(v - tile max)
//                    as f16 and the per-tile (max, sum); a second, bandwidth-bound
//                    kernel (row_softmax_kernels.cu) rescales the rows.  Used when
//                    a row does not fit one cluster, and for skinny M.
//
// Warp roles: ONE thread of warp 0 feeds shared memory with TMA (its warp only helps to
// request the first stages of the first tile, one box per lane), ONE thread of warp 1
// issues tcgen05.mma (warp 1 also owns the TMEM allocation), the remaining warps are the
// softmax epilogue.  The two single-thread loops are kept as short as possible: the tensor
// pipe holds only a few instructions ahead, so every cycle the issuing thread spends on
// anything else is a cycle the pipe idles (measured on B200: 4 MMAs of 128x256x16 take
// 512 cycles; a loop that waits, builds descriptors from scratch and re-converges its warp
// per K block ran at 740).  Hence: descriptors advanced by additions, the next stage's
// barrier probed while the current MMAs drain, no warp-wide instruction inside the loop.
//
// Epilogue forms (template parameter EPI):
//   EPI_SPLIT   eight warps; thread = one row x half of the tile's columns (TMEM lane
//               quarter = warp_id % 4).  The thread's 128 accumulators go TMEM -> registers
//               in one go and the accumulator buffer is released at once; row extreme,
//               e = 2^(v - max) in place (one MUFU per element), the (max, sum) exchange --
//               between the two halves through shared memory, between the CTAs of the
//               cluster through st.async -- then p = e * factor, packed, staged in
//               128-byte-swizzled shared memory and written with TMA stores.
//   EPI_RELAY   sixteen warps in two groups that work on consecutive tiles at the same
//               time: an "exp" group turns the accumulator into exp values in place in
//               tensor memory and sends the row statistics, a "store" group scales, packs
//               and stores them.  Chosen when a CTA sees several tiles.
//   EPI_SINGLE  for launches in which every CTA owns exactly one tile (nothing can overlap
//               with a next tile): sixteen warps, thread = one row x a quarter of the tile's
//               columns, values in registers from the TMEM load to the staging tile; the
//               staging tiles lie over the (by then idle) operand stages, which buys a
//               fourth operand stage.
// PAIR: two CTAs issue one 256-row tcgen05 cta_group::2 MMA (tiled flavour, long K).
// OUT32: f32 probabilities.
// KD, TM: K depth of a pipeline stage (64; 32 or 128 on request) and rows of a tile (128;
// 64 on request, tcgen05.mma with M = 64) -- the schedule's tileK and tileM.
//
// Operand layouts: A [M,K] is K-major, staged as TM rows x 128 B with the 128-byte
// swizzle (64-byte rows and swizzle for 32-deep stages, two 128-byte blocks side by side
// for 128-deep ones).  B [K,N] has N contiguous, i.e. it is MN-major for the MMA: it is
// staged as BN/64 blocks of (KD k-rows x 128 B), and the instruction descriptor's B-major
// bit asks the tensor core to transpose it.  No operand is pre-transposed.
#include "wtc_kernels.h"
#include "wtc_ptx.cuh"

namespace wtc {

namespace {

constexpr int BM = kTcBlockM;
constexpr int kMaxCluster = 8;
enum : int { EPI_SPLIT = 0, EPI_RELAY = 1, EPI_SINGLE = 2 };
constexpr int kThreadsFor(int epi) { return epi == EPI_SPLIT ? 320 : (epi == EPI_RELAY ? 640 : 576); }

// UMMA shared-memory descriptor geometry (bytes).
//   A (K-major, 128-byte swizzle): 8-row groups are 1024 B apart; one 16-wide K step is 32 B.
//   B (MN-major, 128-byte swizzle): 64-column blocks are (k-rows of a stage) * 128 B apart
//   (leading: 8192 B for 64-deep stages), 8-k-row groups are 1024 B apart (stride); one
//   16-deep K step is 16 * 128 B.
constexpr uint32_t kALbo = 16, kASbo = 1024, kAKstep = 32;
constexpr uint32_t kBSbo = 1024, kBKstep = 2048;

// KD: the K depth of one pipeline stage (the schedule's tileK): 64 by default; 32 and 128 for
// the eight-warp epilogue forms.  A's 128 rows are then staged as 64-byte rows with the 64-byte
// swizzle (32), or as two 128-byte-swizzled blocks of 64 columns side by side (128); B's
// 64-column blocks simply have KD k-rows.
// TM: rows of a tile (the schedule's tileM): 128, or 64 (tcgen05.mma with M = 64, whose
// accumulator rows lie in lanes 0-15 of each 32-lane quarter of tensor memory) in the same family.
template <int BN, int STAGES, bool CLUSTER, int EPI, bool PAIR, bool OUT32, int KD = kTcBlockK, int TM = kTcBlockM>
struct SmemLayout {
  static constexpr bool RELAY = EPI == EPI_RELAY;
  static constexpr bool SINGLE = EPI == EPI_SINGLE;
  static_assert(KD == 32 || KD == 64 || KD == 128, "stage depth: 32, 64 or 128");
  static_assert(KD == 64 || (EPI == EPI_SPLIT && !PAIR && !OUT32), "other stage depths: eight-warp epilogue, unpaired, f16 output");
  static_assert(TM == 128 || (TM == 64 && EPI == EPI_SPLIT && !PAIR && !OUT32), "64-row tiles: eight-warp epilogue, unpaired, f16 output");
  static constexpr int kABytes = TM * KD * 2;
  static constexpr int kBBytes = KD * BN * 2 / (PAIR ? 2 : 1);     // a CTA pair splits B's columns between its two CTAs
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kHalfCols = SINGLE ? BN / 4 : BN / 2;         // columns per epilogue thread
  // 32-row x 64-column f16 (32 x 32 f32) staging tiles per storing warp: two let a warp's
  // column groups go out without waiting for each other's TMA read; the tiled flavour and
  // the relay take one and spend the room on operand stages
  static constexpr int kOutTiles = RELAY ? (STAGES <= 2 ? 2 : 1) : ((SINGLE || !CLUSTER) ? 1 : 2);
  static constexpr int kOutWarpBytes = kOutTiles * 4096;
  static constexpr int kOutBytes = SINGLE ? 0 : 8 * kOutWarpBytes;   // single-tile form: staging lies over the operand stages
  static constexpr int kPairBytes = (SINGLE ? 4 : 2) * BM * 8;        // [part][row] float2
  // statistics sets: a peer's exp group may run up to three tiles ahead of this CTA's store group
  static constexpr int kStatsSets = SINGLE ? 1 : (RELAY ? 4 : 2);
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
  static_assert(!SINGLE || STAGES * kStageBytes >= 16 * 4096, "single-tile form: sixteen staging tiles over the operand stages");
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

// Bring-up builds (-DWTC_BRINGUP) stamp the phases of each CTA's first tile; the default
// build carries no stamps.
#ifdef WTC_BRINGUP
__device__ __forceinline__ void stamp(long long *timeline, int slot) {
  if (timeline) {
    long long *t = timeline + static_cast<size_t>(blockIdx.x) * 48;
    t[slot] = static_cast<long long>(globaltimer_ns());
    t[24 + slot] = clock64();
  }
}
#define WTC_STAMP(p, slot) stamp((p).timeline, slot)
#else
#define WTC_STAMP(p, slot) ((void)0)
#endif
// stamp slots
enum : int { TS_ENTRY = 0, TS_SETUP = 1, TS_DEPS = 2, TS_TMA0 = 3, TS_FULL0 = 4, TS_MMA_DONE = 5, TS_ACCUM = 6, TS_EXP = 7,
             TS_STATS = 8, TS_STAGED = 9, TS_STORED = 10, TS_EXIT = 11, TS_LOADED = 12, TS_MAX = 13, TS_TEARDOWN = 14, TS_CLSYNC = 15, TS_MMA_READY = 16, TS_PACKED = 17, TS_PRODUCER_END = 18,
             TS_R_ACCUM8 = 19, TS_R_EXP8 = 20, TS_R_ACCUM9 = 21, TS_R_XDONE8 = 22, TS_R_STORED8 = 23 };

// ---- extreme of 32 raw accumulators folded into four running chains ----
template <bool POS>
__device__ __forceinline__ void fold_extreme(const uint32_t (&v)[32], float &m0, float &m1, float &m2, float &m3) {
#pragma unroll
  for (int i = 0; i < 32; i += 8) {
    if (POS) {
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
}

// max (scale >= 0) or min (scale < 0) of a thread's NCH x 32 raw accumulators of which the
// first `valid` exist, times c2: the row share's largest logit in the log2 domain
template <int NCH>
__device__ __forceinline__ float share_extreme(const uint32_t (&r)[NCH][32], int valid, float c2) {
  const bool pos = c2 >= 0.f;
  if (valid == NCH * 32) {
    float m0 = __uint_as_float(r[0][0]), m1 = __uint_as_float(r[0][1]);
    float m2 = __uint_as_float(r[0][2]), m3 = __uint_as_float(r[0][3]);
    if (pos) {
#pragma unroll
      for (int c = 0; c < NCH; ++c) fold_extreme<true>(r[c], m0, m1, m2, m3);
      return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * c2;
    }
#pragma unroll
    for (int c = 0; c < NCH; ++c) fold_extreme<false>(r[c], m0, m1, m2, m3);
    return fminf(fminf(m0, m1), fminf(m2, m3)) * c2;
  }
  if (valid <= 0) return -INFINITY;
  float m = __uint_as_float(r[0][0]);
#pragma unroll
  for (int c = 0; c < NCH; ++c)
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (c * 32 + i < valid) m = pos ? fmaxf(m, __uint_as_float(r[c][i])) : fminf(m, __uint_as_float(r[c][i]));
  return m * c2;
}

// 32 values times f, rounded to f16 pairs
__device__ __forceinline__ void scale_pack(const uint32_t (&r)[32], float f, uint32_t (&h)[16]) {
#pragma unroll
  for (int i = 0; i < 32; i += 2) h[i >> 1] = pack_f16x2(__uint_as_float(r[i]) * f, __uint_as_float(r[i + 1]) * f);
}

template <int BN, int STAGES, bool CLUSTER, int EPI, bool PAIR, bool OUT32, int KD, int TM>
__global__ void __launch_bounds__(kThreadsFor(EPI), 1)
fused_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmO, const TcParams p) {
  using L = SmemLayout<BN, STAGES, CLUSTER, EPI, PAIR, OUT32, KD, TM>;
  constexpr int BK = KD;                // K depth of a stage
  constexpr int A_BOXES = KD == 128 ? 2 : 1;   // A's copies per stage: a box is at most one swizzle span (64 columns) wide
  constexpr bool RELAY = L::RELAY;
  constexpr bool SINGLE = L::SINGLE;
  constexpr int OUT_TILES = L::kOutTiles;
  constexpr int HC = L::kHalfCols;      // columns per epilogue thread
  constexpr int NCH = HC / 32;          // 32-column chunks per epilogue thread
  constexpr int kEpiThreads = (RELAY || SINGLE) ? 512 : 256;
  static_assert(!(RELAY || SINGLE) || (CLUSTER && !PAIR && !OUT32 && BN == 256 && TM == 128), "sixteen-warp epilogues: cluster flavour, 128 x 256 tiles, f16 staged stores");
  static_assert(!OUT32 || !PAIR, "f32 output: unpaired CTAs");
  static_assert(!PAIR || !CLUSTER, "CTA pairs: tiled flavour only");
  // The 128-byte swizzle needs the stage buffers on 1024-byte boundaries.  There is no
  // static shared memory in this kernel, so the dynamic window starts aligned; if it ever
  // does not, every thread leaves before any barrier or TMEM state exists.
  extern __shared__ __align__(1024) uint8_t smem[];
  // the first TMA instruction waits for its descriptor: ask for all three before anything else
  if (threadIdx.x == 0) { tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); tma_prefetch_desc(&tmO); WTC_STAMP(p, TS_ENTRY); }
  if ((smem_u32(smem) & 1023u) != 0) { record_failure(p.status, WTC_DEV_BAD_SMEM_ALIGN); return; }

  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L::kOffBars);
  uint64_t *full = bars;
  uint64_t *empty = bars + STAGES;
  uint64_t *accum_full = bars + 2 * STAGES;
  uint64_t *accum_empty = bars + 2 * STAGES + 2;
  uint64_t *stats_bar = bars + 2 * STAGES + 4;
  uint64_t *xdone = bars + 2 * STAGES + 8;                         // relay: exp group -> store group, per accumulator buffer
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + L::kOffTmemSlot);
  float2 *pair = reinterpret_cast<float2 *>(smem + L::kOffPair);    // [2][BM]
  float2 *stats = reinterpret_cast<float2 *>(smem + L::kOffStats);  // [sets][kMaxCluster][BM]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Cluster geometry.  PAIR: ranks 0 and 1 form one tcgen05 CTA pair (256 rows x BN
  // columns; the even CTA issues the MMAs).
  constexpr bool CLUSTERED = CLUSTER || PAIR;
  const uint32_t cta_rank = CLUSTERED ? cluster_ctarank() : 0u;
  const uint32_t cluster_size = CLUSTERED ? cluster_nctarank() : 1u;
  const uint32_t pair_rank = PAIR ? (cta_rank & 1u) : 0u;
  const uint32_t leader_rank = PAIR ? (cta_rank & ~1u) : cta_rank;
  const bool is_leader = pair_rank == 0;
  const uint32_t col_rank = cta_rank;                                // my column block inside the cluster (cluster flavour)
  const uint32_t cluster_n = CLUSTER ? cluster_size : 1u;           // CTAs that share my rows

  // ---- work distribution (needs nothing but special registers and parameters) ----
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

  // one K block of operands into stage s (unpaired CTAs)
  auto load_stage = [&](uint32_t s, int kb, int rb, int nb, int b, int bb) {
    uint8_t *sa = smem + s * L::kStageBytes;
    uint8_t *sb = sa + L::kABytes;
    mbar_expect_tx(&full[s], L::kStageBytes);
    tma_load_3d(sa, &tmA, &full[s], kb * BK, rb * TM, b);
    if (A_BOXES == 2) tma_load_3d(sa + TM * 128, &tmA, &full[s], kb * BK + 64, rb * TM, b);
    if (p.b_blocks) tma_load_4d(sb, &tmB, &full[s], 0, kb * BK, nb * (BN / 64), bb);
    else {
#pragma unroll
      for (int j = 0; j < BN / 64; ++j)
        tma_load_3d(sb + j * (BK * 128), &tmB, &full[s], nb * BN + j * 64, kb * BK, bb);
    }
  };

  // ---- set-up.  Under programmatic dependent launch this CTA is resident a microsecond or two
  // before the previous kernel on the stream is complete: everything that touches no global
  // memory happens now (barriers, tensor memory, the cluster barrier's arrival), and ONLY the
  // producer warp then waits for the previous kernel -- the MMA thread and the epilogue warps
  // go straight to their shared-memory barriers, so the first MMA issues as soon as the first
  // stage lands.  (They write global memory only after an accumulator is complete, which cannot
  // happen before the producer's loads, which come after its wait.)
  const int early = PAIR ? 0 : (p.num_kb < STAGES ? p.num_kb : STAGES);   // stages of the first tile the producer warp requests in one go
  if (warp == 0) {
    if (lane == 0) {
      for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
      for (int i = 0; i < 2; ++i) {
        mbar_init(&accum_full[i], 1);
        mbar_init(&accum_empty[i], (RELAY ? kEpiThreads / 2 : kEpiThreads) * (PAIR ? 2 : 1));   // relay: the store group hands it back
        mbar_init(&xdone[i], kEpiThreads / 2);
      }
      for (int i = 0; i < 4; ++i) mbar_init(&stats_bar[i], 1);
      mbar_fence_init();
    }
    __syncwarp();
  }
  if (warp == 1) {
    if (PAIR) { tmem_alloc_pair(tmem_slot, 2 * BN); tmem_relinquish_pair(); }
    else { tmem_alloc(tmem_slot, 2 * BN); tmem_relinquish(); }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Every peer's barriers must exist before anyone signals them.  A CTA pair signals from its
  // main loop, so it completes the cluster barrier here; the cluster flavour signals only from
  // the epilogue (row statistics), so its threads arrive now and wait where they first need it.
  if (CLUSTERED) cluster_arrive_release();
  if (PAIR) cluster_wait_acquire();
  if (threadIdx.x == 0) WTC_STAMP(p, TS_SETUP);
  grid_launch_dependents();            // the next kernel on the stream may start its own set-up as our CTAs retire

  // While the producer waits for the previous kernel, warp 2 (an epilogue warp, idle until the
  // first accumulator is complete) asks for the first tile's operands to be brought into L2.
  // Shared memory may not be filled yet (the operands may be that kernel's output), but an L2
  // prefetch is harmless, and turns the cold start of the pipeline into L2 hits.  The first
  // TMA instruction of a launch stalls its thread until the tensor map has been fetched
  // (well over a microsecond), and each further one costs its thread a hundred cycles or
  // more, which is why this is neither the producer's job nor part of the set-up that the
  // whole CTA waits for.
  // The CTAs that share a panel split its K blocks: A[rb] among the cluster, B[nb] among the clusters.
  if (CLUSTER && !PAIR && KD == kTcBlockK && warp == 2 && first < p.num_items) {
    int b, rb, nb; decode(first, b, rb, nb);
    const int bb = p.b_batched ? b : 0;
    const int cl = static_cast<int>(cluster_n);
    const int groups = stride < p.num_kb ? stride : p.num_kb;
    for (int base = 0; base < p.num_kb; base += 4) {
      const int kb = base + lane;
      if (lane < 4 && kb < p.num_kb) {
        if (kb % cl == nb || kb < early) tma_prefetch_l2_3d(&tmA, kb * BK, rb * TM, b);
        if (kb % groups == first % groups || kb < early) {
          if (p.b_blocks) tma_prefetch_l2_4d(&tmB, 0, kb * BK, nb * (BN / 64), bb);
          else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_prefetch_l2_3d(&tmB, nb * BN + j * 64, kb * BK, bb);
          }
        }
      }
      __syncwarp();
    }
  }

  // hands accumulator buffer `ab` back to the MMA thread (of the pair's even CTA)
  auto release_accumulator = [&](int ab) {
    if (PAIR) mbar_arrive_remote_release(map_to_cta(smem_u32(&accum_empty[ab]), leader_rank));
    else mbar_arrive(&accum_empty[ab]);
  };

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

  // Relay epilogue: warps 0-3 are the producer, the MMA issuer and two idle warps (the two
  // groups below are aligned groups of four warps each), warps 4-11 the exp group, warps
  // 12-19 the store group.
  const int relay_role = !RELAY ? 0 : (warp < 4 ? 0 : (warp < 12 ? 1 : 2));
  bool cluster_waited = PAIR;     // this thread has completed the set-up's cluster barrier
  if (RELAY && relay_role == 1) {
    // register reallocation between aligned groups of four warps: this group holds a whole
    // row share (128 values) in registers: 152 a thread here, 64 in the store group (one
    // 16-column chunk in flight, one being packed), 48 in warps 0-3 (they need little)
    setmaxnreg_inc<152>();
    cluster_wait_acquire();
    cluster_waited = true;
    // ======================= softmax epilogue, two-stage relay: exp group ==============
    // Two groups of eight epilogue warps work on consecutive tiles at the same time.  This
    // group turns a tile's accumulator into exp values in place in tensor memory and sends
    // the row statistics round the cluster; the store group waits for the cluster's
    // statistics, reads the exp values back 16 columns at a time (the next chunk's load in
    // flight while one is scaled and packed), and stores them.  The exchange latency and
    // the store phase of tile i are hidden behind the exp phase of tile i+1.
    const int q = warp & 3;                       // TMEM lane quarter this warp may touch
    const int row_in_tile = q * 32 + lane;
    const float c2 = p.c2;
    float *mh = reinterpret_cast<float *>(smem + L::kOffMh);   // [2 tile parity][2 half][BM]: each half's own maximum
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
      if (stamper && it == 0) WTC_STAMP(p, TS_ACCUM);
      if (stamper && it == 8) WTC_STAMP(p, TS_R_ACCUM8);
      if (stamper && it == 9) WTC_STAMP(p, TS_R_ACCUM9);
      const uint32_t tbase = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + ab * BN + half * HC;
      const int col0 = nb * BN + half * HC;
      const int valid = max(0, min(HC, p.N - col0));
      uint32_t r[NCH][32];
      float m_half;
      if (valid == HC && !p.round_logits_f16) {
        // whole share, no rounding: the second half of the loads is in flight while the
        // extreme of the first half is taken
        const bool pos = c2 >= 0.f;
#pragma unroll
        for (int c = 0; c < NCH / 2; ++c) tmem_ld_32x32b_x32(tbase + c * 32, r[c]);
        tmem_ld_wait();
#pragma unroll
        for (int c = NCH / 2; c < NCH; ++c) tmem_ld_32x32b_x32(tbase + c * 32, r[c]);
        float m0 = __uint_as_float(r[0][0]), m1 = __uint_as_float(r[0][1]), m2 = __uint_as_float(r[0][2]), m3 = __uint_as_float(r[0][3]);
        if (pos) {
#pragma unroll
          for (int c = 0; c < NCH / 2; ++c) fold_extreme<true>(r[c], m0, m1, m2, m3);
        } else {
#pragma unroll
          for (int c = 0; c < NCH / 2; ++c) fold_extreme<false>(r[c], m0, m1, m2, m3);
        }
        tmem_ld_wait();
        if (pos) {
#pragma unroll
          for (int c = NCH / 2; c < NCH; ++c) fold_extreme<true>(r[c], m0, m1, m2, m3);
        } else {
#pragma unroll
          for (int c = NCH / 2; c < NCH; ++c) fold_extreme<false>(r[c], m0, m1, m2, m3);
        }
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
        if (p.round_logits_f16) {
#pragma unroll
          for (int c = 0; c < NCH; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) r[c][i] = __float_as_uint(__half2float(__float2half_rn(__uint_as_float(r[c][i]))));
        }
        m_half = share_extreme<NCH>(r, valid, c2);
      }
      // ---- e = 2^(v - m_half) in place, row sum; each chunk goes back over its logits ----
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
      if (valid == HC) {
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
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
          tmem_st_32x32b_x32(tbase + c * 32, r[c]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float e = 0.f;
            if (c * 32 + i < valid) e = ex2_approx(fmaf(__uint_as_float(r[c][i]), c2, -m_half));
            s0 += e;
            r[c][i] = __float_as_uint(e);
          }
          if (c * 32 < valid) tmem_st_32x32b_x32(tbase + c * 32, r[c]);
        }
      }
      const float sum = (s0 + s1) + (s2 + s3);
      if (stamper && it == 0) WTC_STAMP(p, TS_EXP);
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
          st_async_f32x2(map_to_cta(slot, peer), lm, ll, map_to_cta(bar, peer));
      }
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&xdone[ab]);                    // exp values parked, maxima published
      if (stamper && it == 8) WTC_STAMP(p, TS_R_EXP8);
    }
  } else if (RELAY && relay_role == 2) {
    setmaxnreg_dec<64>();
    cluster_wait_acquire();
    cluster_waited = true;
    // ======================= softmax epilogue, two-stage relay: store group ==============
    const int q = warp & 3;                       // TMEM lane quarter this warp may touch
    const int row_in_tile = q * 32 + lane;
    const float *mh = reinterpret_cast<const float *>(smem + L::kOffMh);
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
      if (p.operands_ready && it == 0) grid_dependency_wait();   // the store group is the relay's only writer of global memory
      if (lead && it == 8) WTC_STAMP(p, TS_R_XDONE8);
      const uint32_t tbase = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + ab * BN + half * HC;
      const int col0 = nb * BN + half * HC;
      const int valid = max(0, min(HC, p.N - col0));
      const int row0 = rb * BM + q * 32;
      const bool rows_live = row0 < p.M;
      // 16 columns at a time through two small register buffers: the next chunk's load is in
      // flight while one is scaled, packed and staged; the first is on its way from tensor
      // memory while the cluster's statistics arrive
      constexpr int NC16 = HC / 16;
      uint32_t r[2][16];
      if (valid > 0) tmem_ld_32x32b_x16(tbase, r[0]);
      else { tc_fence_before_sync(); release_accumulator(ab); }
      if (!mbar_wait_cluster(&stats_bar[sset], (it >> 2) & 1)) { record_failure(p.status, WTC_DEV_TIMEOUT_STATS); break; }
      float gm, inv_gl;
      combine_cluster_stats(sset, row_in_tile, gm, inv_gl);
      const float f = ex2_approx(mh[((it & 1) * 2 + half) * BM + row_in_tile] - gm) * inv_gl;
      if (lane == 0) tma_store_wait_read();         // the previous tile's stores have read the staging tiles
      __syncwarp();
#pragma unroll
      for (int c = 0; c < NC16; ++c) {
        uint8_t *tile = stg + (OUT_TILES == 2 ? (c >> 2) * 4096 : 0);
        if (c * 16 < valid) {
          tmem_ld_wait();
          if ((c + 1) * 16 < valid && c + 1 < NC16) tmem_ld_32x32b_x16(tbase + (c + 1) * 16, r[(c + 1) & 1]);
          else { tc_fence_before_sync(); release_accumulator(ab); }   // that was my last read of this accumulator buffer
          if (OUT_TILES == 1 && c == 4) {           // one staging tile: the first store must have read it
            if (lane == 0) tma_store_wait_read();
            __syncwarp();
          }
          uint8_t *row = tile + lane * 128;
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const uint32_t (&v)[16] = r[c & 1];
            const uint4 h = make_uint4(pack_f16x2(__uint_as_float(v[8 * j]) * f, __uint_as_float(v[8 * j + 1]) * f),
                                       pack_f16x2(__uint_as_float(v[8 * j + 2]) * f, __uint_as_float(v[8 * j + 3]) * f),
                                       pack_f16x2(__uint_as_float(v[8 * j + 4]) * f, __uint_as_float(v[8 * j + 5]) * f),
                                       pack_f16x2(__uint_as_float(v[8 * j + 6]) * f, __uint_as_float(v[8 * j + 7]) * f));
            *reinterpret_cast<uint4 *>(row + ((((c & 3) * 2 + j) ^ (lane & 7)) * 16)) = h;   // 128-byte swizzle
          }
        }
        if ((c & 3) == 3 && (c - 3) * 16 < valid) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (rows_live) tma_store_3d(&tmO, tile, col0 + (c >> 2) * 64, row0, b);
            tma_store_commit();
          }
        }
      }
      if (lead && it == 0) WTC_STAMP(p, TS_STAGED);
      if (lead && it == 8) WTC_STAMP(p, TS_R_STORED8);
    }
    if (lane == 0) tma_store_wait_read();
  } else if (SINGLE && warp >= 2) {
    // ======================= softmax epilogue, sixteen warps, one tile per CTA ==============
    // Thread = one row x a quarter (64) of the tile's columns: TMEM lane quarter = warp_id % 4,
    // column quarter = (warp_id - 2) / 4.  Everything stays in registers between the TMEM load
    // and the staging tile; with four warps per scheduler the exponentials of the whole tile
    // run at the special-function unit's rate, and all sixteen warps share the store phase.
    cluster_wait_acquire();
    cluster_waited = true;
    const int q = warp & 3;
    const int part = (warp - 2) >> 2;
    const int row_in_tile = q * 32 + lane;
    const bool lead = threadIdx.x == 64;
    const float c2 = p.c2;
    if (first < p.num_items) {
      int b, rb, nb; decode(first, b, rb, nb);
      if (lead) mbar_expect_tx(&stats_bar[0], cluster_n * BM * 8);
      if (!mbar_wait(&accum_full[0], 0)) record_failure(p.status, WTC_DEV_TIMEOUT_ACCUM);
      else {
        tc_fence_after_sync();
        if (p.operands_ready) grid_dependency_wait();
        if (lead) WTC_STAMP(p, TS_ACCUM);
        const uint32_t tbase = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + part * HC;
        const int col0 = nb * BN + part * HC;
        const int valid = max(0, min(HC, p.N - col0));
        const int row0 = rb * BM + q * 32;
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
        if (lead) WTC_STAMP(p, TS_LOADED);
        if (p.round_logits_f16) {
#pragma unroll
          for (int c = 0; c < NCH; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) r[c][i] = __float_as_uint(__half2float(__float2half_rn(__uint_as_float(r[c][i]))));
        }
        const float m_part = share_extreme<NCH>(r, valid, c2);
        if (lead) WTC_STAMP(p, TS_MAX);
        // ---- e = 2^(v - m_part) in place, row sum ----
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
        if (valid == HC) {
#pragma unroll
          for (int c = 0; c < NCH; ++c)
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const float e0 = ex2_approx(fmaf(__uint_as_float(r[c][i]), c2, -m_part));
              const float e1 = ex2_approx(fmaf(__uint_as_float(r[c][i + 1]), c2, -m_part));
              const float e2 = ex2_approx(fmaf(__uint_as_float(r[c][i + 2]), c2, -m_part));
              const float e3 = ex2_approx(fmaf(__uint_as_float(r[c][i + 3]), c2, -m_part));
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
              if (c * 32 + i < valid) e = ex2_approx(fmaf(__uint_as_float(r[c][i]), c2, -m_part));
              s0 += e;
              r[c][i] = __float_as_uint(e);
            }
        }
        const float sum = (s0 + s1) + (s2 + s3);
        if (lead) WTC_STAMP(p, TS_EXP);
        // ---- the four quarters of a row meet through shared memory, the CTAs through the cluster ----
        pair[part * BM + row_in_tile] = make_float2(m_part, sum);
        named_bar_sync(1 + q, 128);
        float2 pq[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) pq[j] = pair[j * BM + row_in_tile];
        const float lm = fmaxf(fmaxf(pq[0].x, pq[1].x), fmaxf(pq[2].x, pq[3].x));
        if (part == 0) {
          float ll = 0.f;
#pragma unroll
          for (int j = 0; j < 4; ++j) ll += pq[j].x == -INFINITY ? 0.f : pq[j].y * ex2_approx(pq[j].x - lm);
          const uint32_t slot = smem_u32(&stats[col_rank * BM + row_in_tile]);
          const uint32_t bar = smem_u32(&stats_bar[0]);
          for (uint32_t peer = 0; peer < cluster_n; ++peer)
            st_async_f32x2(map_to_cta(slot, peer), lm, ll, map_to_cta(bar, peer));
        }
        if (!mbar_wait_cluster(&stats_bar[0], 0)) record_failure(p.status, WTC_DEV_TIMEOUT_STATS);
        else {
          if (lead) WTC_STAMP(p, TS_STATS);
          float gm, inv_gl;
          combine_cluster_stats(0, row_in_tile, gm, inv_gl);
          const float f = ex2_approx(m_part - gm) * inv_gl;
          // ---- p = e * f -> f16 -> this warp's staging tile (over the idle operand stages) -> one TMA store ----
          uint8_t *stg = smem + (warp - 2) * 4096;
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            uint32_t h[16];
            scale_pack(r[c], f, h);                  // (columns past `valid` hold zeros: e was 0 there)
            stage_row_chunk(stg, lane, c, h);
          }
          if (lead) WTC_STAMP(p, TS_PACKED);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (valid > 0 && row0 < p.M) tma_store_3d(&tmO, stg, col0, row0, b);
            tma_store_commit();
            if (lead) WTC_STAMP(p, TS_STAGED);
            tma_store_wait_read();
          }
          if (lead) WTC_STAMP(p, TS_STORED);
        }
      }
    }
  } else {
  if (RELAY) setmaxnreg_dec<48>();
  if (warp == 0) {
    // ======================= TMA producer ====================================
    // programmatic dependent launch: the operands may be the previous kernel's output -- unless the
    // caller has said they are not; then only the stores wait (see the epilogues)
    if (!p.operands_ready) grid_dependency_wait();
    if (lane == 0) WTC_STAMP(p, TS_DEPS);
    if (!PAIR && first < p.num_items) {
      // the first stages of the first tile, one box per lane (box 0 of a stage is A's, the
      // others are B's 64-column blocks): twenty copies leave in the time of one
      int b, rb, nb; decode(first, b, rb, nb);
      const int bb = p.b_batched ? b : 0;
      if (lane == 0)
        for (int s = 0; s < early; ++s) mbar_expect_tx(&full[s], L::kStageBytes);
      __syncwarp();
      const int boxes = A_BOXES + (p.b_blocks ? 1 : BN / 64);
      for (int t = lane; t < early * boxes; t += 32) {
        const int st = t / boxes, j = t - st * boxes;
        uint8_t *sa = smem + st * L::kStageBytes;
        if (j < A_BOXES) tma_load_3d(sa + j * (TM * 128), &tmA, &full[st], st * BK + j * 64, rb * TM, b);
        else if (p.b_blocks) tma_load_4d(sa + L::kABytes, &tmB, &full[st], 0, st * BK, nb * (BN / 64), bb);
        else tma_load_3d(sa + L::kABytes + (j - A_BOXES) * (BK * 128), &tmB, &full[st], nb * BN + (j - A_BOXES) * 64, st * BK, bb);
      }
      if (lane == 0) WTC_STAMP(p, TS_TMA0);
    }
    if (lane == 0) {
      // the rest, one thread: (the first `early` stages of the first tile are already on their way)
      uint32_t s = early == STAGES ? 0 : early, ph = early == STAGES ? 1 : 0;
      bool ok = true;
      for (int w = first; w < p.num_items && ok; w += stride) {
        int b, rb, nb; decode(w, b, rb, nb);
        const int bb = p.b_batched ? b : 0;
        for (int kb = (w == first ? early : 0); kb < p.num_kb; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1)) { record_failure(p.status, WTC_DEV_TIMEOUT_EMPTY); ok = false; break; }
          if (PAIR) {
            // both CTAs of the pair fill their own stage; all bytes are counted on the even CTA's barrier
            uint8_t *sa = smem + s * L::kStageBytes;
            uint8_t *sb = sa + L::kABytes;
            if (is_leader) mbar_expect_tx(&full[s], 2 * L::kStageBytes);
            tma_load_3d_pair(sa, &tmA, &full[s], kb * BK, rb * BM, b);
            if (p.b_blocks) tma_load_4d_pair(sb, &tmB, &full[s], 0, kb * BK, nb * (BN / 64) + static_cast<int>(pair_rank) * (BN / 128), bb);
            else {
#pragma unroll
              for (int j = 0; j < BN / 128; ++j)
                tma_load_3d_pair(sb + j * (BK * 128), &tmB, &full[s], nb * BN + static_cast<int>(pair_rank) * (BN / 2) + j * 64, kb * BK, bb);
            }
            if (w == first && kb == 0) WTC_STAMP(p, TS_TMA0);
          } else {
            load_stage(s, kb, rb, nb, b, bb);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      WTC_STAMP(p, TS_PRODUCER_END);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ======================= MMA issuer: one thread (of the even CTA of a pair) =======
    if (is_leader && elect_one()) {
      constexpr uint32_t idesc = umma_idesc_f16_f32(PAIR ? 2 * BM : TM, BN, /*a_mn_major=*/0, /*b_mn_major=*/1);
      const uint16_t pair_mask = static_cast<uint16_t>(3u << leader_rank);
      // everything of the two operand descriptors but the address, which is added per stage
      // (A with 64-byte rows: 64-byte swizzle, 8-row groups 512 B apart; B's 64-column blocks are KD k-rows apart)
      const uint64_t a_desc0 = KD == 32 ? umma_smem_desc_sw64(smem_u32(smem), kALbo, kASbo / 2) : umma_smem_desc_sw128(smem_u32(smem), kALbo, kASbo);
      const uint64_t b_desc0 = umma_smem_desc_sw128(smem_u32(smem) + L::kABytes, KD * 128, kBSbo);
      uint32_t s = 0, ph = 0;
      uint32_t landed = 0;            // the next stage's barrier was already seen complete
      WTC_STAMP(p, TS_MMA_READY);
      int it = 0;
      bool ok = true;
      for (int w = first; w < p.num_items && ok; w += stride, ++it) {
        const int ab = it & 1;
        if (!mbar_wait(&accum_empty[ab], ((it >> 1) & 1) ^ 1)) { record_failure(p.status, WTC_DEV_TIMEOUT_TMEM); ok = false; break; }
        tc_fence_after_sync();
        if (it == 8) WTC_STAMP(p, TS_LOADED);
        const uint32_t d_tmem = tmem_base + ab * BN;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!landed && !mbar_wait(&full[s], ph)) { record_failure(p.status, WTC_DEV_TIMEOUT_FULL); ok = false; break; }
          tc_fence_after_sync();
          if (it == 0 && kb == 0) WTC_STAMP(p, TS_FULL0);
          uint64_t da = a_desc0 + ((s * L::kStageBytes) >> 4);
          uint64_t db = b_desc0 + ((s * L::kStageBytes) >> 4);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            if (PAIR) umma_f16_ss_pair(d_tmem, da, db, idesc, (kb | k) != 0);
            else umma_f16_ss(d_tmem, da, db, idesc, (kb | k) != 0);
            da += (k == 3 ? TM * 128 - 3 * kAKstep : kAKstep) >> 4;   // after four steps: the second 64-column block of a 128-deep stage
            db += kBKstep >> 4;
          }
          // while those MMAs drain: has the next stage landed already?  (The ring runs on
          // across tiles, so "next" is the same barrier whichever tile it belongs to.)
          const uint32_t s1 = s + 1 == STAGES ? 0 : s + 1;
          const uint32_t ph1 = s1 == 0 ? ph ^ 1 : ph;
          landed = mbar_try_wait(&full[s1], ph1);
          // frees the stage (in both CTAs of a pair) once these MMAs have read it
          if (PAIR) umma_commit_pair(&empty[s], pair_mask);
          else umma_commit(&empty[s]);
          s = s1; ph = ph1;
        }
        if (ok) {
          if (PAIR) umma_commit_pair(&accum_full[ab], pair_mask);
          else umma_commit(&accum_full[ab]);
          if (it == 0) WTC_STAMP(p, TS_MMA_DONE);
          if (it == 8) WTC_STAMP(p, TS_MAX);
        }
      }
    }
    __syncwarp();
  } else if (!RELAY && !SINGLE) {
    // ======================= softmax epilogue, eight warps ==================
    if (CLUSTER) { cluster_wait_acquire(); cluster_waited = true; }
    const int q = warp & 3;                      // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;            // which half of the tile's columns
    // (64-row tiles: the accumulator's rows are in lanes 0-15 of each quarter; the other lanes run
    //  along on whatever their lanes hold, in statistics slots 64.. that no row uses, and store nothing)
    const bool lane_live = TM == 128 || lane < 16;
    const int row_in_tile = TM == 128 ? q * 32 + lane : (lane < 16 ? q * 16 + lane : 48 + q * 16 + lane);
    const bool lead = threadIdx.x == 64;         // first epilogue thread: posts expect_tx, stamps
    uint8_t *stg = smem + L::kOffOut + (warp - 2) * L::kOutWarpBytes;
    float2 *mine = &pair[half * BM + row_in_tile];
    const float2 *other = &pair[(half ^ 1) * BM + row_in_tile];
    const float c2 = p.c2;
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
      if (p.operands_ready && it == 0) grid_dependency_wait();   // nothing of this warp has touched global memory yet
      if (lead && it == 0) WTC_STAMP(p, TS_ACCUM);
      const uint32_t tbase = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + ab * BN + half * HC;
      const int col0 = nb * BN + half * HC;               // first matrix column of this thread
      const int valid = max(0, min(HC, p.N - col0));      // my columns that exist
      const int row0 = rb * TM + q * (TM / 4);            // first row of this warp
      const bool rows_live = row0 < p.M;

      // ---- the thread's whole share of the accumulator row goes to registers at once,
      //      and the accumulator buffer is handed back to the MMA thread straight away ----
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
      if (lead && it == 0) WTC_STAMP(p, TS_LOADED);
      if (p.round_logits_f16) {
#pragma unroll
        for (int c = 0; c < NCH; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) r[c][i] = __float_as_uint(__half2float(__float2half_rn(__uint_as_float(r[c][i]))));
      }
      if (OUT32 && !CLUSTER && p.logits_only) {
        // the unfused baseline's first kernel: scale * A . B as f32 logits, nothing else
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          if (c * 32 < valid) {
            if (lane == 0) tma_store_wait_read();
            __syncwarp();
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[c][i]) * p.scale;
            stage_row_f32(stg, lane, v);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (rows_live) tma_store_3d(&tmO, stg, col0 + c * 32, row0, b);
              tma_store_commit();
            }
          }
        }
        continue;
      }
      const float m_half = share_extreme<NCH>(r, valid, c2);
      if (lead && it == 0) WTC_STAMP(p, TS_MAX);

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
      const float sum = (s0 + s1) + (s2 + s3);
      if (lead && it == 0) WTC_STAMP(p, TS_EXP);

      // ---- the two halves of a row meet through shared memory ----
      *mine = make_float2(m_half, sum);
      named_bar_sync(1 + q, 64);
      const float2 o = *other;
      named_bar_sync(1 + q, 64);                 // both have read: the slots may be reused
      const float lm = fmaxf(m_half, o.x);       // tile-row max (log2 domain)
      float f;                                     // what my e values still have to be multiplied by
      if (CLUSTER) {
        const float ll = (m_half == -INFINITY ? 0.f : sum * ex2_approx(m_half - lm)) +
                         (o.x == -INFINITY ? 0.f : o.y * ex2_approx(o.x - lm));
        // ... and the CTAs of the cluster through each other's shared memory
        if (half == 0) {
          const uint32_t slot = smem_u32(&stats[(par * kMaxCluster + col_rank) * BM + row_in_tile]);
          const uint32_t bar = smem_u32(&stats_bar[par]);
          for (uint32_t peer = 0; peer < cluster_n; ++peer)
            st_async_f32x2(map_to_cta(slot, peer), lm, ll, map_to_cta(bar, peer));
        }
        if (!mbar_wait_cluster(&stats_bar[par], tile_phase)) { record_failure(p.status, WTC_DEV_TIMEOUT_STATS); break; }
        if (lead && it == 0) WTC_STAMP(p, TS_STATS);
        float gm, inv_gl;
        combine_cluster_stats(par, row_in_tile, gm, inv_gl);
        f = ex2_approx(m_half - gm) * inv_gl;
      } else {
        f = ex2_approx(m_half - lm);               // tiled: values relative to the tile max, not normalised
      }

      // ---- p = e * f -> output type -> 128-byte-swizzled staging tiles -> TMA stores ----
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
      } else if (OUT_TILES * 2 >= NCH) {
        // the warp's whole share of the tile fits its staging tiles: pack and stage
        // everything, then ONE proxy fence and warp barrier, then all stores back to back
        if (lane == 0) tma_store_wait_read();    // the previous tile's stores have read the staging tiles
        __syncwarp();
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          if (c * 32 < valid) {
            uint32_t h[16];
            scale_pack(r[c], f, h);
            if (!CLUSTER) {
#pragma unroll
              for (int i = 0; i < 16; ++i) { const float2 back = __half22float2(*reinterpret_cast<const __half2 *>(&h[i])); sum_r += back.x + back.y; }
            }
            stage_row_chunk(stg + (c >> 1) * 4096, lane, c & 1, h);
          }
        }
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
              scale_pack(r[c], f, h);
              if (!CLUSTER) {
#pragma unroll
                for (int i = 0; i < 16; ++i) { const float2 back = __half22float2(*reinterpret_cast<const __half2 *>(&h[i])); sum_r += back.x + back.y; }
              }
              stage_row_chunk(stg, lane, hc, h);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (rows_live) tma_store_3d(&tmO, stg, col0 + g * 64, row0, b);
              tma_store_commit();
            }
          }
        }
      }
      if (!CLUSTER) {
        // tile statistics: max of the tile row, sum of the stored values of both halves
        mine->y = sum_r;
        named_bar_sync(1 + q, 64);
        const int row = rb * TM + row_in_tile;
        if (half == 0 && lane_live && row < p.M)
          p.tile_stats[(static_cast<int64_t>(b) * p.M + row) * p.num_nb + nb] = make_float2(lm, sum_r + other->y);
        named_bar_sync(1 + q, 64);
      }
      if (lead && it == 0) WTC_STAMP(p, TS_STAGED);
    }
    if (lane == 0) tma_store_wait_read();
    if (lead) WTC_STAMP(p, TS_STORED);
  }

  }   // warps 0-3 of the relay form, warps 0-1 of the single-tile form, every warp of the split form

  // ---- teardown: nothing in flight, peers done with our shared memory, TMEM freed ----
  if (p.status && *reinterpret_cast<volatile int *>(p.status) != 0) {
    // a wait gave up somewhere: give copies that were already issued time to land
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  if (threadIdx.x == 0) WTC_STAMP(p, TS_TEARDOWN);
  if (CLUSTER && !cluster_waited) cluster_wait_acquire();   // (whole warps: the role split is by warp)
  tc_fence_before_sync();
  __syncthreads();
  if (CLUSTERED) cluster_sync_all();
  if (threadIdx.x == 0) WTC_STAMP(p, TS_CLSYNC);
  if (warp == 1) { if (PAIR) tmem_dealloc_pair(tmem_base, 2 * BN); else tmem_dealloc(tmem_base, 2 * BN); }
  if (threadIdx.x == 0) WTC_STAMP(p, TS_EXIT);
}

// Per-device launch facts of one kernel instance: the dynamic shared memory opt-in and how
// many clusters of each size the device holds at once.
struct DeviceFacts {
  bool attr_set = false;
  int max_clusters[2 * kMaxCluster + 1] = {0};
  int registers = 0;
};

template <int BN, int STAGES, bool CLUSTER, int EPI, bool PAIR, bool OUT32, int KD, int TM>
cudaError_t launch_impl(const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmO, TcParams p,
                        int cluster_n, int num_sms, cudaStream_t s, TcLaunchInfo *info) {
  using L = SmemLayout<BN, STAGES, CLUSTER, EPI, PAIR, OUT32, KD, TM>;
  auto kern = fused_tc_kernel<BN, STAGES, CLUSTER, EPI, PAIR, OUT32, KD, TM>;
  static DeviceFacts facts[64];   // per template instance, per device
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  DeviceFacts &df = facts[dev];
  if (!df.attr_set) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
    if (e != cudaSuccess) return e;
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, kern) == cudaSuccess) df.registers = fa.numRegs;
    df.attr_set = true;
  }
  // work items: row units (128 rows, or 256 for a CTA pair) x (column blocks when tiled)
  p.num_ru = PAIR ? (p.num_rb + 1) / 2 : p.num_rb;
  p.num_items = p.batch * p.num_ru * (CLUSTER ? 1 : p.num_nb);
  const int cluster_size = (CLUSTER ? cluster_n : 1) * (PAIR ? 2 : 1);

  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kThreadsFor(EPI), 1, 1);
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
    if (!df.max_clusters[cluster_size]) {
      cfg.gridDim = dim3(cluster_size, 1, 1);
      int mc = 0;
      e = cudaOccupancyMaxActiveClusters(&mc, kern, &cfg);
      if (e != cudaSuccess) return e;
      if (mc < 1) return cudaErrorInvalidConfiguration;
      df.max_clusters[cluster_size] = mc;
    }
    const int max_clusters = df.max_clusters[cluster_size];
    if (EPI == EPI_SINGLE && p.num_items > max_clusters) return cudaErrorNotSupported;   // some CTA would own two tiles: the caller takes another form
    const int clusters = p.num_items < max_clusters ? p.num_items : max_clusters;
    grid = clusters * cluster_size;
  } else {
    grid = p.num_items < num_sms ? p.num_items : num_sms;
    cfg.attrs = nattr ? attr : nullptr;
    cfg.numAttrs = nattr;
  }
  cfg.gridDim = dim3(grid, 1, 1);
  if (info) {
    info->grid = grid; info->cluster = cluster_size; info->smem_bytes = L::kDynamic; info->threads = kThreadsFor(EPI);
    info->stages = STAGES; info->registers = df.registers;
  }
  return cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmO, p);
}

} // namespace

// Every instantiated variant, once: X(BN, STAGES, CLUSTER, EPI, PAIR, OUT32, KD, TM).
#define WTC_TC_VARIANTS(X)                                                                                \
  X(128, 4, true, EPI_SPLIT, false, true, 64, 128) X(kTcBlockN, 3, true, EPI_SPLIT, false, true, 64, 128)            \
  X(128, 4, true, EPI_SPLIT, false, false, 64, 128) X(kTcBlockN, 3, true, EPI_SPLIT, false, false, 64, 128)          \
  X(kTcBlockN, 2, true, EPI_RELAY, false, false, 64, 128) X(kTcBlockN, 3, true, EPI_RELAY, false, false, 64, 128)    \
  X(kTcBlockN, 4, true, EPI_SINGLE, false, false, 64, 128)                                                      \
  X(128, 6, false, EPI_SPLIT, false, true, 64, 128) X(kTcBlockN, 4, false, EPI_SPLIT, false, true, 64, 128)          \
  X(128, 6, false, EPI_SPLIT, false, false, 64, 128) X(kTcBlockN, 4, false, EPI_SPLIT, false, false, 64, 128)        \
  X(kTcBlockN, 6, false, EPI_SPLIT, true, false, 64, 128)                                                       \
  /* other stage depths (the schedule's tileK): eight-warp epilogue, f16 output */                        \
  X(128, 8, true, EPI_SPLIT, false, false, 32, 128) X(kTcBlockN, 6, true, EPI_SPLIT, false, false, 32, 128)          \
  X(128, 12, false, EPI_SPLIT, false, false, 32, 128) X(kTcBlockN, 8, false, EPI_SPLIT, false, false, 32, 128)       \
  X(128, 2, true, EPI_SPLIT, false, false, 128, 128)                                                            \
  X(128, 3, false, EPI_SPLIT, false, false, 128, 128) X(kTcBlockN, 2, false, EPI_SPLIT, false, false, 128, 128)       \
  /* 64-row tiles (the schedule's tileM = 64), stage depth 32 or 64 */                                         \
  X(128, 4, true, EPI_SPLIT, false, false, 64, 64) X(kTcBlockN, 3, true, EPI_SPLIT, false, false, 64, 64)      \
  X(128, 6, false, EPI_SPLIT, false, false, 64, 64) X(kTcBlockN, 4, false, EPI_SPLIT, false, false, 64, 64)    \
  X(128, 8, true, EPI_SPLIT, false, false, 32, 64) X(kTcBlockN, 6, true, EPI_SPLIT, false, false, 32, 64)      \
  X(128, 12, false, EPI_SPLIT, false, false, 32, 64) X(kTcBlockN, 8, false, EPI_SPLIT, false, false, 32, 64)

// Form choice.  Cluster flavour: f32 probabilities and 128-column tiles take the split
// epilogue; 256-column f16 tiles take the relay when a CTA sees several tiles (its two groups
// then overlap; a short K loop needs no third operand stage: the room goes to a second staging
// tile per storing warp), the single-tile form when every cluster fits the chip at once, the
// split form otherwise or on request.  Tiled flavour: two CTAs share one 256-row MMA (a third
// less L2 operand traffic per flop) when the K loop is long and there are two row blocks.
bool tc_stage_depth_legal(bool tiled, int bn, bool out_f32, int kd, int tm) {
  if (tm != kTcBlockM && (tm != 64 || out_f32 || kd == 128)) return false;
  if (kd == kTcBlockK) return true;
  if (out_f32 || (kd != 32 && kd != 128)) return false;
  return kd == 32 || bn == 128 || tiled;     // 128-deep stages of 256-column tiles leave no room for a cluster's statistics
}

TcVariant tc_choose_variant(bool tiled, int bn, bool out_f32, int batch, int num_rb, int num_kb, int cluster_n,
                            int epilogue_mode, int pair_mode, int num_sms, int resident, int kd, int tm) {
  if ((kd != kTcBlockK || tm != kTcBlockM) && tc_stage_depth_legal(tiled, bn, out_f32, kd, tm)) {
    // as many stages as keep the default's K depth in flight (more than its bytes, with 64-row tiles)
    const int st_cl = bn == 128 ? (kd == 32 ? 8 : (kd == 64 ? 4 : 2)) : (kd == 32 ? 6 : 3);
    const int st_ti = bn == 128 ? (kd == 32 ? 12 : (kd == 64 ? 6 : 3)) : (kd == 32 ? 8 : (kd == 64 ? 4 : 2));
    return tiled ? TcVariant{bn == 128 ? 128 : kTcBlockN, st_ti, 0, EPI_SPLIT, 0, 0, kd, tm}
                 : TcVariant{bn == 128 ? 128 : kTcBlockN, st_cl, 1, EPI_SPLIT, 0, 0, kd, tm};
  }
  if (tiled) {
    if (out_f32) return bn == 128 ? TcVariant{128, 6, 0, EPI_SPLIT, 0, 1, kTcBlockK, kTcBlockM} : TcVariant{kTcBlockN, 4, 0, EPI_SPLIT, 0, 1, kTcBlockK, kTcBlockM};
    if (bn == 128) return TcVariant{128, 6, 0, EPI_SPLIT, 0, 0, kTcBlockK, kTcBlockM};
    const bool pair = num_rb >= 2 && (pair_mode == 2 || (pair_mode == 0 && num_kb >= 8));
    return pair ? TcVariant{kTcBlockN, 6, 0, EPI_SPLIT, 1, 0, kTcBlockK, kTcBlockM} : TcVariant{kTcBlockN, 4, 0, EPI_SPLIT, 0, 0, kTcBlockK, kTcBlockM};
  }
  if (out_f32) return bn == 128 ? TcVariant{128, 4, 1, EPI_SPLIT, 0, 1, kTcBlockK, kTcBlockM} : TcVariant{kTcBlockN, 3, 1, EPI_SPLIT, 0, 1, kTcBlockK, kTcBlockM};
  if (bn == 128) return TcVariant{128, 4, 1, EPI_SPLIT, 0, 0, kTcBlockK, kTcBlockM};
  const int per_round = num_sms / (cluster_n > 0 ? cluster_n : 1);
  const int units = batch * num_rb;
  const int tiles_per_cta = (units + per_round - 1) / (per_round > 0 ? per_round : 1);
  const bool relay = epilogue_mode == kEpilogueRelay || (epilogue_mode == kEpilogueAuto && tiles_per_cta >= kRelayMinTiles);
  if (relay) return TcVariant{kTcBlockN, num_kb <= 3 ? 2 : 3, 1, EPI_RELAY, 0, 0, kTcBlockK, kTcBlockM};
  if (epilogue_mode == kEpilogueAuto && units <= resident) return TcVariant{kTcBlockN, 4, 1, EPI_SINGLE, 0, 0, kTcBlockK, kTcBlockM};
  return TcVariant{kTcBlockN, 3, 1, EPI_SPLIT, 0, 0, kTcBlockK, kTcBlockM};
}

int tc_variant_smem_bytes(const TcVariant &v) {
#define X(BN, ST, CL, EP, PA, O32, KD, TM) \
  if (v.bn == BN && v.stages == ST && (v.cluster != 0) == CL && v.epi == EP && (v.pair != 0) == PA && (v.out32 != 0) == O32 && v.kd == KD && v.tm == TM) \
    return SmemLayout<BN, ST, CL, EP, PA, O32, KD, TM>::kDynamic;
  WTC_TC_VARIANTS(X)
#undef X
  return 0;
}

int tc_variant_threads(const TcVariant &v) { return kThreadsFor(v.epi); }

namespace {
cudaError_t launch_variant(const TcVariant &v, const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmO,
                           const TcParams &p, int cluster_n, int num_sms, cudaStream_t s, TcLaunchInfo *info) {
#define X(BN, ST, CL, EP, PA, O32, KD, TM) \
  if (v.bn == BN && v.stages == ST && (v.cluster != 0) == CL && v.epi == EP && (v.pair != 0) == PA && (v.out32 != 0) == O32 && v.kd == KD && v.tm == TM) \
    return launch_impl<BN, ST, CL, EP, PA, O32, KD, TM>(tmA, tmB, tmO, p, cluster_n, num_sms, s, info);
  WTC_TC_VARIANTS(X)
#undef X
  return cudaErrorInvalidConfiguration;
}
} // namespace

cudaError_t launch_fused_cluster(const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmO,
                                 const TcParams &p, int bn, int cluster_n, int num_sms, cudaStream_t s,
                                 TcLaunchInfo *info) {
  if (cluster_n < 1 || cluster_n > kMaxCluster) return cudaErrorInvalidValue;
  // the single-tile form is tried whenever one tile per CTA is possible at all; it declines
  // (before launching) when the clusters do not all fit the chip at once, and the split form runs
  TcVariant v = tc_choose_variant(false, bn, p.out_f32 != 0, p.batch, p.num_rb, p.num_kb, cluster_n, p.epilogue_mode, p.pair_mode,
                                  num_sms, /*resident=*/1 << 30, p.stage_k ? p.stage_k : kTcBlockK, p.tile_rows ? p.tile_rows : kTcBlockM);
  if (v.epi == EPI_SINGLE) {
    const cudaError_t e = launch_variant(v, tmA, tmB, tmO, p, cluster_n, num_sms, s, info);
    if (e != cudaErrorNotSupported) return e;
    v = TcVariant{kTcBlockN, 3, 1, EPI_SPLIT, 0, 0, kTcBlockK, kTcBlockM};
  }
  return launch_variant(v, tmA, tmB, tmO, p, cluster_n, num_sms, s, info);
}

cudaError_t launch_tiled_partial(const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmO,
                                 const TcParams &p, int bn, int num_sms, cudaStream_t s, TcLaunchInfo *info) {
  const TcVariant v = tc_choose_variant(true, bn, p.out_f32 != 0, p.batch, p.num_rb, p.num_kb, 1, p.epilogue_mode, p.pair_mode, num_sms, 0,
                                        p.stage_k ? p.stage_k : kTcBlockK, p.tile_rows ? p.tile_rows : kTcBlockM);
  return launch_variant(v, tmA, tmB, tmO, p, 1, num_sms, s, info);
}

} // namespace wtc

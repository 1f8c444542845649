// Host-visible declarations of the kernel launchers.  The launch layer
// (wtc_launch.cu) is the only caller.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace wtc {

// Epilogue forms of the tensor-core kernel (TcParams::epilogue_mode; 0 lets the launcher choose).
enum : int { kEpilogueAuto = 0, kEpilogueSplit = 1, kEpilogueRelay = 2 };

struct TcParams {
  int batch, M, N, K;
  int num_rb;      // row blocks of 128 per batch
  int num_nb;      // column blocks of BN per row
  int num_kb;      // K blocks of 64
  int num_ru;      // row units per batch: row blocks, or pairs of row blocks (set by the launcher)
  int num_items;   // work items: cluster mode batch*num_rb, tiled mode batch*num_rb*num_nb
  int b_batched;   // B has its own batch dimension
  int b_blocks;    // tmB is the rank-4 view [batch][N/64][K][64] (N a multiple of 64): one copy per stage instead of one per 64 columns
  int group_rb;    // tiled mode: row blocks per rasterisation group
  int out_f32;     // f32 probabilities (else f16)
  int pair_mode;   // tiled flavour: 0 choose, 1 never pair CTAs, 2 pair whenever the shape allows
  int epilogue_mode;  // cluster flavour: kEpilogue*
  int use_pdl;     // launch with programmatic stream serialisation
  int operands_ready;  // A and B do not depend on earlier work on the stream: only the stores wait for it
  int round_logits_f16;  // chain spelled with an f16 matmul result: round s to f16 before the softmax
  int stage_k;     // K depth of a pipeline stage (0: 64)
  int tile_rows;   // rows of a tile (0: 128)
  int logits_only; // tiled flavour, f32 output: store scale * A . B and stop (the unfused baseline's first kernel)
  float scale;     // the chain's scale factor
  float c2;        // scale * log2(e)
  float2 *tile_stats;    // tiled mode: [batch*M][num_nb] (max in log2 domain, sum of 2^(v-max))
  int *status;     // device status word (0 = ok)
#ifdef WTC_BRINGUP
  long long *timeline;   // optional [grid][48] stamps of each CTA's first tile: %globaltimer ns in 0..23, clock64 in 24..47
#endif
};

struct TcLaunchInfo {
  int grid, cluster, smem_bytes, threads, stages, registers;
};

// One instantiation of the tensor-core kernel template: column tile, operand stages, flavour
// (cluster / tiled), epilogue form (0 split, 1 relay, 2 single tile), CTA pairing, f32 output.
struct TcVariant {
  int bn, stages, cluster, epi, pair, out32;
  int kd;    // K depth of one pipeline stage: 64, or the schedule's tileK when it is 32 or 128 and legal
  int tm;    // rows of a tile: 128, or the schedule's tileM when it is 64 and legal
};
// The variant the launchers below take for a call, worked out without a device: `resident` is how
// many clusters of `cluster_n` CTAs the chip holds at once (the launchers ask the runtime; a plan
// made without a device uses the figures measured on a 148-SM part).
TcVariant tc_choose_variant(bool tiled, int bn, bool out_f32, int batch, int num_rb, int num_kb, int cluster_n,
                            int epilogue_mode, int pair_mode, int num_sms, int resident, int kd = 64, int tm = 128);
// Whether this stage depth and tile height have a kernel for this flavour, column tile and output type.
bool tc_stage_depth_legal(bool tiled, int bn, bool out_f32, int kd, int tm = 128);
// Dynamic shared memory and threads per CTA of a variant (0 if it is not instantiated).
int tc_variant_smem_bytes(const TcVariant &v);
int tc_variant_threads(const TcVariant &v);

// Fused cluster kernel: a cluster of ceil(N/BN) CTAs owns 128 full rows, exchanges
// per-row (max, sum) through distributed shared memory and writes probabilities.
cudaError_t launch_fused_cluster(const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmO,
                                 const TcParams &p, int bn, int cluster_n, int num_sms, cudaStream_t s,
                                 TcLaunchInfo *info);
// Tiled kernel: independent 128 x BN tiles write exp(v - tile max) and per-tile
// (max, sum); rescale_rows() then normalises the rows.
cudaError_t launch_tiled_partial(const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmO,
                                 const TcParams &p, int bn, int num_sms, cudaStream_t s, TcLaunchInfo *info);

// rows = batch*M.  tile_stats [rows][num_nb].  row_stats_out (optional) receives
// the per-row combination over this launch's tiles.  global_stats (optional):
// [num_parts][rows] (max, sum) pairs covering the WHOLE row (all N shards); when
// given, rows are normalised against their combination instead of the local one.
cudaError_t launch_row_stats(const float2 *tile_stats, float2 *row_stats_out, int64_t rows, int num_nb,
                             cudaStream_t s);
cudaError_t launch_rescale_rows(void *out, int out_f32, int64_t rows, int N, int64_t ld_out, int BN, int num_nb,
                                const float2 *tile_stats, const float2 *global_stats, int num_parts,
                                cudaStream_t s);

// For both operands in one launch: dst[b][r][c] (dense f16: row stride cols, batch stride rows * cols)
// = round-to-nearest-even of src[b * batch_stride + r * ld + c] (f32).
cudaError_t launch_round_to_f16(const float *A, void *dstA, int batchA, int64_t rowsA, int64_t colsA, int64_t ldA, int64_t strideA,
                                const float *B, void *dstB, int batchB, int64_t rowsB, int64_t colsB, int64_t ldB, int64_t strideB,
                                cudaStream_t s);

// The four softmax passes of the unfused baseline on logits C32[rows, N] already in global
// memory: row max -> exp -> row sum -> divide (intermediates E[rows, N], mx[rows], sum[rows]).
cudaError_t launch_softmax_passes(const float *C32, float *E, float *mx, float *sum, void *Out, int64_t rows, int64_t rows_per_batch,
                                  int N, int64_t ldo, int64_t o_batch_stride, int out_f16, cudaStream_t s);

// Row-only chains (row_chain_kernels.cu).  kind 0: Out = softmax_row(X); kind 1: Out[i, :] =
// c2 * sum_j (X[i,j] - c1 * sum_j X[i,j])^2.  Row strides in elements.
cudaError_t launch_row_chain(int kind, const void *X, void *Out, int64_t rows, int64_t N, int64_t ld_in, int64_t ld_out, int in_f16,
                             int out_f16, float c1, float c2, cudaStream_t s);

// SIMT kernels: any shape, f32 or f16 operands, f32 or f16 output.
struct SimtParams {
  int batch, M, N, K;
  int64_t lda, ldb, ldo;
  int64_t a_batch_stride, b_batch_stride, o_batch_stride;
  int in_f16, out_f16;
  int acc_mode;  // 0 f32 accumulate, 1 round the finished sum to f16 (f16 matmul result)
  float scale;
};
cudaError_t launch_simt_fused(const void *A, const void *B, void *Out, const SimtParams &p, cudaStream_t s);
// Unfused five-kernel pipeline: matmul -> row max -> exp -> row sum -> divide,
// with C32[M,N], max[M], E[M,N], sum[M] in global memory (workspace).
cudaError_t launch_simt_unfused(const void *A, const void *B, void *Out, void *workspace, const SimtParams &p,
                                cudaStream_t s);
size_t simt_unfused_workspace_bytes(const SimtParams &p);

constexpr int kTcBlockM = 128;
// Tiles per CTA from which the relay epilogue is chosen unless a form is asked for: with one tile
// per CTA its two groups cannot overlap (measured equal to the split form on config 2).
constexpr int kRelayMinTiles = 2;
constexpr int kTcBlockK = 64;
constexpr int kTcBlockN = 256;

} // namespace wtc

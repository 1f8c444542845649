/*
 * wtc_launch.h -- thin C-ABI launch layer for the fused Matmul -> row-Softmax
 * chain  Out[b,M,N] = softmax_row(scale * A[b,M,K] . B[b,K,N])  on sm_100a.
 *
 * This is the device boundary of the chain.  In the reference the same boundary
 * is the `welder-profiler` tool, which JIT-loads the PTX embedded in
 * 05.out.nvvm.runnable.mlir and launches it through the CUDA driver API
 * (backend/welder/compiler/solver/WelderProfiler.cpp:296-303 context/stream,
 * :321-340 buffers, :359-428 module load, :752-793 warm-up + timed launch loop).
 * Here the kernels are precompiled for sm_100a and the host side (runner,
 * harness, bindings) reaches them only through the entry points below.
 *
 * Rules of the ABI: plain C types; every pointer named "device" is a CUDA device
 * pointer owned by the caller; calls are asynchronous on `stream` unless stated;
 * return 0 on success, a negative WTC_E_* code otherwise (wtc_last_error() gives
 * the text for the calling thread); no exceptions cross the boundary; there is no
 * CPU fallback -- without a usable CUDA device every launch fails with
 * WTC_E_CUDA.
 */
#ifndef WTC_LAUNCH_H
#define WTC_LAUNCH_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WTC_ABI_VERSION 2

/* element types */
#define WTC_F32 0
#define WTC_F16 1

/* variants: the reference compiles the same chain twice -- one fused kernel, or a
 * five-kernel baseline with intermediates in global memory
 * (compiler/transform/BuildCutEdgesTransformCommon.cpp:27-34). */
#define WTC_VARIANT_FUSED 0
#define WTC_VARIANT_BASELINE 1

/* flags */
#define WTC_FLAG_FORCE_SIMT 0x1   /* never use the tensor-core kernels            */
#define WTC_FLAG_FORCE_TILED 0x2  /* two-pass tiled kernel even if a cluster fits  */
/* f32 operands in memory, rounded to f16 (round to nearest even, arith.truncf) before the
 * contraction: the chain of mlir_pipeline/matmul_softmax_chain_f16_matmul.mlir:18-44 in the
 * reference.  Needs in_dtype = WTC_F32.  The rounded copies live in the workspace
 * (wtc_matmul_softmax_workspace_bytes counts them); the single-GPU entry points only. */
#define WTC_FLAG_MATMUL_F16 0x4
/* Schedule overrides, for experiments and for the tests that run every kernel form:
 * the launch layer normally picks the epilogue form and the CTA pairing by shape. */
#define WTC_FLAG_EPILOGUE_SPLIT 0x8  /* cluster flavour: eight epilogue warps share a tile            */
#define WTC_FLAG_EPILOGUE_RELAY 0x10 /* cluster flavour: two warp groups relay consecutive tiles      */
#define WTC_FLAG_NO_PAIR 0x20        /* tiled flavour: never pair CTAs for tcgen05 cta_group::2       */
#define WTC_FLAG_PAIR 0x40           /* tiled flavour: pair CTAs whenever there are two row blocks    */
/* The caller promises that A and B are not written by work that is still running earlier on the
 * stream (they were resident before, or the caller ordered them itself).  The tensor-core kernels
 * are launched behind one another with programmatic stream serialisation; by default their loads
 * wait until the previous launch on the stream is complete, because its output may be this
 * launch's operands.  With this flag only the stores wait (the previous launch may still read or
 * write the output buffer), and the loads of one call run under the tail of the one before. */
#define WTC_FLAG_OPERANDS_READY 0x80

/* error codes */
#define WTC_OK 0
#define WTC_E_ARG (-1)        /* null pointer, bad size, unknown dtype ...            */
#define WTC_E_UNSUPPORTED (-2)/* a legal request no kernel here covers               */
#define WTC_E_WORKSPACE (-3)  /* workspace missing or too small                      */
#define WTC_E_CUDA (-4)       /* a CUDA call failed (no device, launch error ...)    */
#define WTC_E_DEVICE (-5)     /* a kernel reported a non-zero device status word     */

/* Which kernel family a descriptor resolves to (wtc_plan_query). */
#define WTC_KERNEL_SIMT_FUSED 0
#define WTC_KERNEL_TC_CLUSTER 1   /* tcgen05, cluster of CTAs per 128 rows, one launch   */
#define WTC_KERNEL_TC_TILED 2     /* tcgen05 tiles + row rescale, two launches           */
#define WTC_KERNEL_SIMT_UNFUSED 3 /* five launches (baseline variant, f32 chains)        */
#define WTC_KERNEL_TC_UNFUSED 4   /* baseline variant of f16 chains: the tcgen05 contraction
                                     writes f32 logits to global memory, four more kernels
                                     do max / exp / sum / divide                         */

/*
 * The chain, as the compiler front-end recognised it.  Strides are in elements;
 * 0 means dense (lda = K, ldb = N, ldo = N, batch strides = rows * ld).
 * b_batch_stride < 0 means one B shared by every batch.
 * tile_* carry the tile choice of best.json (tileM/tileN/tileK,
 * compiler/include/wtc/scheduler/Search.h:11-17); 0 lets the library choose.
 * As in the reference's fused mode the softmax row is never cut: tile_n < N
 * selects a multi-CTA (cluster) or two-pass schedule, not a narrower softmax.
 */
typedef struct wtc_chain_desc {
  int32_t struct_size; /* sizeof(wtc_chain_desc) */
  int32_t batch;
  int64_t M, N, K;
  int64_t lda, ldb, ldo;
  int64_t a_batch_stride, b_batch_stride, o_batch_stride;
  int32_t in_dtype;  /* WTC_F32 | WTC_F16 (A and B) */
  int32_t out_dtype; /* WTC_F32 | WTC_F16 */
  int32_t acc_dtype; /* WTC_F32, or WTC_F16 when the chain spells an f16 matmul result */
  float scale;
  int32_t tile_m, tile_n, tile_k;
  int32_t variant; /* WTC_VARIANT_* */
  int32_t flags;   /* WTC_FLAG_* */
} wtc_chain_desc;

typedef struct wtc_plan_info {
  int32_t kernel;       /* WTC_KERNEL_* */
  int32_t launches;     /* kernel launches per call */
  int32_t tile_m, tile_n, tile_k; /* tile actually used (after legalisation) */
  int32_t cluster_n;    /* CTAs per cluster along N (1 if none) */
  int32_t grid, threads, smem_bytes; /* main kernel; grid is 0 until a device is known */
  int32_t tmem_columns; /* tensor-memory columns allocated per CTA */
  int32_t stages;       /* shared-memory pipeline depth */
  int32_t tile_substituted; /* 1 if a requested tile_* was not legal and was replaced */
  size_t workspace_bytes;
  /* compiler facts of the main kernel's template instance (0 where not recorded) */
  int32_t registers;    /* registers per thread at launch */
  int32_t spill_bytes;  /* bytes of spill stores in the whole kernel (all warp roles) */
  int32_t stack_bytes;  /* local-memory stack frame */
  int32_t reserved;
} wtc_plan_info;

/* ABI version of the loaded library (== WTC_ABI_VERSION of its build). */
int wtc_abi_version(void);

/* Text of the last error on this thread ("" if none).  Never NULL. */
const char *wtc_last_error(void);

/* Resolve a descriptor to a kernel plan without touching the device. */
int wtc_plan_query(const wtc_chain_desc *desc, wtc_plan_info *out);

/* Scratch memory (global memory beyond inputs and outputs) a launch needs. */
int wtc_matmul_softmax_workspace_bytes(const wtc_chain_desc *desc, size_t *bytes);

/*
 * Launch the chain.  A, B, Out, workspace: device pointers.  stream: a
 * cudaStream_t (NULL = default stream).  device_status: optional device pointer
 * to one int32 the caller zeroed; kernels store a non-zero code there instead of
 * trapping when a bounded wait gives up (read it after synchronising, or use
 * wtc_check_device_status).  Replaces the launch loop body of
 * WelderProfiler.cpp:773-786.
 */
int wtc_matmul_softmax_launch(const wtc_chain_desc *desc, const void *A, const void *B, void *Out,
                              void *workspace, size_t workspace_bytes, void *stream, int *device_status);

/*
 * N-sharded use (one shard of the columns per GPU): `partial` runs the chain on
 * this shard's columns, leaving un-normalised exp() values in Out and the
 * shard's per-row (max, sum) pairs -- maxima in the log2 domain -- in
 * row_stats[batch*M] (device, 2 floats per row).  After the shards' row_stats
 * have been gathered into all_stats[num_parts][batch*M] (device), `finish`
 * normalises Out against the whole row.  The reference has no counterpart: it is
 * single-GPU (WelderProfiler.cpp:296-303).
 */
int wtc_matmul_softmax_partial_launch(const wtc_chain_desc *desc, const void *A, const void *B, void *Out,
                                      void *workspace, size_t workspace_bytes, void *row_stats,
                                      void *stream, int *device_status);
int wtc_matmul_softmax_finish_launch(const wtc_chain_desc *desc, void *Out, const void *workspace,
                                     const void *all_stats, int32_t num_parts, void *stream);

/*
 * Whole call with HOST buffers: copies A and B to the device, launches, copies
 * Out back and synchronises.  Device buffers are cached per thread between calls.
 * Large calls are cut into row (or batch) ranges that move through three streams, so
 * both PCIe directions and the kernels overlap; pinned host memory makes the copies
 * asynchronous, pageable memory works but serialises them.
 * This is what a host-side caller of the reference would otherwise do around the
 * profiler's cuMemcpyHtoD / launch / dump sequence (WelderProfiler.cpp:601-677,
 * :808-864).
 */
int wtc_matmul_softmax_host(const wtc_chain_desc *desc, const void *hostA, const void *hostB, void *hostOut);

/*
 * The same call in two halves, for callers with a stream of chains: submit
 * enqueues the copies and kernels and returns a ticket; wait blocks until that
 * call's results (and its device status) are in host memory.  A thread has two
 * slots of device buffers: with two calls in flight (submit i+1, then wait i) the
 * operands of one call travel to the device while the rows of the other travel
 * back, and the link is busy in both directions all the time.  A third submit
 * first waits for the oldest call itself.  The host buffers of a call must stay
 * valid, and hostOut unread, until its wait returns.  Tickets belong to the
 * thread that issued them; waiting twice, or for a ticket of -1 (an empty call),
 * returns WTC_OK at once.  wtc_matmul_softmax_host is submit followed by wait.
 */
int wtc_matmul_softmax_host_submit(const wtc_chain_desc *desc, const void *hostA, const void *hostB, void *hostOut,
                                   int64_t *ticket);
int wtc_matmul_softmax_host_wait(int64_t ticket);

/*
 * Same chain, for callers that must not allocate device memory.  (No counterpart
 * in the reference: its profiler allocates every buffer itself with cuMemAlloc.)
 *
 * Some hosts of this library cannot call cudaMalloc at the point where they need
 * the chain: an inference server that handed all of HBM to its own pool at start
 * up, a step loop that must not hit the device-wide synchronisation an
 * allocation implies, a plugin running under a memory budget it may not exceed.
 * This entry point runs the two-pass tiled schedule with its scratch -- the
 * per-tile (max, sum) pairs -- in an array that is part of the library image:
 * WTC_STATIC_SCRATCH_BYTES (16 MiB) on every GPU that loads the library, held
 * until the process exits.  It calls no cudaMalloc, cudaFree or allocating
 * library routine; the caller still provides A, B and Out (device pointers).
 *
 * Limits and rules:
 *  - f16 operands and output on the tensor-core path only (K, N and the row
 *    strides multiples of 8; A, B and Out on 16-byte boundaries), and
 *    batch * M * ceil(N/tile) * 8 bytes of scratch must fit (tile = 256 columns,
 *    128 for rows of at most 128 columns): WTC_E_UNSUPPORTED / WTC_E_WORKSPACE
 *    otherwise, with the sizes in wtc_last_error().  Empty shapes return WTC_OK.
 *  - The first call on each device looks the array's device address up (with
 *    that device current), and, like the first launch of any kernel of the
 *    library, makes the CUDA runtime load the library's device image -- the
 *    16 MiB array included.  A host whose pool already owns HBM should make that
 *    first call at start-up, before it hands the memory out.
 *  - Every call on a device shares the one array.  Calls whose kernels may
 *    overlap on the GPU (two streams, two threads) race on it: serialise them.
 *    Nothing is assumed about what the previous call left there.
 *  - device_status: as for wtc_matmul_softmax_launch.  With NULL the kernels
 *    report into the library's own status word -- also a word of the library
 *    image, never allocated -- which wtc_check_device_status(NULL, stream) reads
 *    and then clears.
 */
#define WTC_STATIC_SCRATCH_BYTES (16u << 20)
int wtc_matmul_softmax_launch_static(const wtc_chain_desc *desc, const void *A, const void *B, void *Out,
                                     void *stream, int *device_status);

/*
 * The two row-only chains among the reference's backend inputs, which share this operator's
 * row-statistics machinery but have no contraction in front:
 *   WTC_ROW_SOFTMAX   Out[i,:] = softmax(X[i,:])   (max -> exp(x - max) -> sum -> divide;
 *                     backend/welder/mlir_pipeline/softmax_row_chain.mlir:10-75)
 *   WTC_ROW_VARIANCE  Out[i,j] = var_factor * sum_j (X[i,j] - mean_factor * sum_j X[i,j])^2 for every j
 *                     (two dependent row reductions and a broadcast;
 *                     backend/welder/mlir_pipeline/layernorm_variance_chain.mlir:12-104)
 * The reference compiles them with its backend tools and runs them with welder-profiler; here
 * each is one fused kernel.  X and Out are device pointers to `rows` rows of N elements of
 * `dtype` (WTC_F32 or WTC_F16; arithmetic in f32), row strides ld_in / ld_out in elements
 * (0 = dense).  Asynchronous on `stream`; needs no workspace.
 */
#define WTC_ROW_SOFTMAX 0
#define WTC_ROW_VARIANCE 1
typedef struct wtc_row_chain_desc {
  int32_t struct_size; /* sizeof(wtc_row_chain_desc) */
  int32_t kind;        /* WTC_ROW_* */
  int64_t rows, N;
  int64_t ld_in, ld_out;
  int32_t dtype;       /* WTC_F32 | WTC_F16 */
  float mean_factor;   /* WTC_ROW_VARIANCE: the chain's 1/N constants, as written in its input */
  float var_factor;
  int32_t reserved;
} wtc_row_chain_desc;
int wtc_row_chain_launch(const wtc_row_chain_desc *desc, const void *X, void *Out, void *stream);
/* Timed loop of the same launch (warm-up, then `iters` launches between two CUDA events). */
int wtc_row_chain_time(const wtc_row_chain_desc *desc, const void *X, void *Out, void *stream, int warmup, int iters,
                       float *avg_ms);

/* Synchronise `stream`, read a device status word, 0 if clean else WTC_E_DEVICE.
 * device_status NULL reads the library's own per-device word (the one kernels use when a
 * launch was given no status pointer) and clears it after a non-zero report; a caller's
 * word is the caller's to clear.  Allocates nothing. */
int wtc_check_device_status(const int *device_status, void *stream);

/*
 * Timed launch loop with CUDA events on `stream`: `warmup` untimed launches, then
 * `iters` back-to-back launches between two events; *avg_ms = elapsed / iters.
 * Same method as WelderProfiler.cpp:752-793.
 */
int wtc_matmul_softmax_time(const wtc_chain_desc *desc, const void *A, const void *B, void *Out,
                            void *workspace, size_t workspace_bytes, void *stream, int warmup, int iters,
                            float *avg_ms);

/*
 * Environment, read once when the library first needs it:
 *   WTC_HOST_SLABS=n   pieces the host-buffer entry point cuts a call into (default: by size, at most 8)
 *   WTC_NO_PDL=1       no programmatic dependent launch
 */

#ifdef __cplusplus
}
#endif
#endif /* WTC_LAUNCH_H */

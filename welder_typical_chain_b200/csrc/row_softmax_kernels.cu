// Bandwidth-bound companions of the tiled kernel: combine per-tile (max, sum)
// pairs into per-row statistics and rescale the stored exp(v - tile max) values
// into probabilities.  All maxima are in the log2 domain (v = scale*log2(e)*s).
#include "wtc_kernels.h"
#include "wtc_ptx.cuh"

namespace wtc {
namespace {

__device__ __forceinline__ float2 lse_combine(float2 a, float2 b) {
  // (max, sum) pairs of disjoint column sets -> pair of their union
  const float m = fmaxf(a.x, b.x);
  if (m == -INFINITY) return make_float2(m, 0.f);
  return make_float2(m, a.y * ex2_approx(a.x - m) + b.y * ex2_approx(b.x - m));
}

__device__ __forceinline__ float2 warp_lse(float2 v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float2 other = make_float2(__shfl_xor_sync(0xffffffffu, v.x, o), __shfl_xor_sync(0xffffffffu, v.y, o));
    v = lse_combine(v, other);
  }
  return v;
}

// one warp per row
__global__ void row_stats_kernel(const float2 *__restrict__ tile_stats, float2 *__restrict__ row_stats,
                                 int64_t rows, int num_nb) {
  grid_dependency_wait();
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float2 v = make_float2(-INFINITY, 0.f);
  for (int t = lane; t < num_nb; t += 32) v = lse_combine(v, tile_stats[row * num_nb + t]);
  v = warp_lse(v);
  if (lane == 0) row_stats[row] = v;
}

// One CTA per row, or -- when there are few rows -- gridDim.y CTAs per row, each taking `chunk`
// columns (a multiple of 256) after working out the row's total for itself.
__global__ void __launch_bounds__(256)
rescale_rows_kernel(void *__restrict__ out_v, int out_f32, int N, int64_t ld_out, int BN, int num_nb,
                    const float2 *__restrict__ tile_stats, const float2 *__restrict__ global_stats,
                    int num_parts, int64_t rows, int chunk) {
  extern __shared__ float factor[];          // [num_nb]
  __shared__ float2 warp_part[8];
  __shared__ float2 row_total;
  grid_dependency_wait();                    // launched behind the tiled kernel with programmatic serialisation
  const int64_t row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  float2 v = make_float2(-INFINITY, 0.f);
  if (global_stats) {
    for (int t = threadIdx.x; t < num_parts; t += blockDim.x) v = lse_combine(v, global_stats[static_cast<int64_t>(t) * rows + row]);
  } else {
    for (int t = threadIdx.x; t < num_nb; t += blockDim.x) v = lse_combine(v, tile_stats[row * num_nb + t]);
  }
  v = warp_lse(v);
  if (lane == 0) warp_part[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float2 t = lane < (blockDim.x >> 5) ? warp_part[lane] : make_float2(-INFINITY, 0.f);
    t = warp_lse(t);
    if (lane == 0) row_total = t;
  }
  __syncthreads();
  const float gm = row_total.x;
  const float inv = 1.0f / row_total.y;
  for (int t = threadIdx.x; t < num_nb; t += blockDim.x)
    factor[t] = ex2_approx(tile_stats[row * num_nb + t].x - gm) * inv;
  __syncthreads();
  const int c0 = blockIdx.y * chunk;                       // my columns: [c0, c1)
  const int c1 = min(N, c0 + chunk);

  if (out_f32) {
    float *frow = static_cast<float *>(out_v) + row * ld_out;
    if ((N % 4 == 0) && (ld_out % 4 == 0) && ((reinterpret_cast<uintptr_t>(out_v) & 15) == 0) && (BN % 4 == 0)) {
      float4 *o4 = reinterpret_cast<float4 *>(frow);
      for (int j = c0 / 4 + threadIdx.x; j < c1 / 4; j += blockDim.x) {
        const float fct = factor[(j * 4) / BN];
        float4 x = o4[j];
        x.x *= fct; x.y *= fct; x.z *= fct; x.w *= fct;
        o4[j] = x;
      }
    } else {
      for (int j = c0 + threadIdx.x; j < c1; j += blockDim.x) frow[j] *= factor[j / BN];
    }
    return;
  }
  __half *out = static_cast<__half *>(out_v);
  __half *orow = out + row * ld_out;
  const bool vec_ok = (N % 8 == 0) && (ld_out % 8 == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0) && (BN % 8 == 0);
  if (vec_ok) {
    uint4 *o4 = reinterpret_cast<uint4 *>(orow);
    for (int j = c0 / 8 + threadIdx.x; j < c1 / 8; j += blockDim.x) {
      const float f = factor[(j * 8) / BN];
      uint4 x = o4[j];
      __half2 *h = reinterpret_cast<__half2 *>(&x);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 t = __half22float2(h[i]);
        h[i] = __floats2half2_rn(t.x * f, t.y * f);
      }
      o4[j] = x;
    }
  } else {
    for (int j = c0 + threadIdx.x; j < c1; j += blockDim.x)
      orow[j] = __float2half_rn(__half2float(orow[j]) * factor[j / BN]);
  }
}

} // namespace

cudaError_t launch_row_stats(const float2 *tile_stats, float2 *row_stats_out, int64_t rows, int num_nb,
                             cudaStream_t s) {
  if (rows <= 0) return cudaSuccess;
  const int warps = 8;
  const unsigned grid = static_cast<unsigned>((rows + warps - 1) / warps);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(warps * 32, 1, 1);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, row_stats_kernel, tile_stats, row_stats_out, rows, num_nb);
}

cudaError_t launch_rescale_rows(void *out, int out_f32, int64_t rows, int N, int64_t ld_out, int BN, int num_nb,
                                const float2 *tile_stats, const float2 *global_stats, int num_parts,
                                cudaStream_t s) {
  if (rows <= 0) return cudaSuccess;
  // few rows (skinny problems): several CTAs per row so that the pass still fills the chip
  // (16 rows x 32000 columns: one CTA per row takes 12 us, sixteen per row 3 us)
  int splits = 1, chunk = N;
  if (rows < 2 * 148 && N > 4096) {
    const int want = static_cast<int>((2 * 148 + rows - 1) / rows);
    const int by_size = (N + 2047) / 2048;
    splits = want < by_size ? want : by_size;
    chunk = ((N + splits - 1) / splits + 255) / 256 * 256;
    splits = (N + chunk - 1) / chunk;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(rows), static_cast<unsigned>(splits), 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.dynamicSmemBytes = num_nb * sizeof(float);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, rescale_rows_kernel, out, out_f32, N, ld_out, BN, num_nb, tile_stats,
                            global_stats, num_parts, rows, chunk);
}

// ---- f32 -> f16 rounding of both operands (the chain that truncates its f32 arguments) --------
namespace {
struct RoundJob {
  const float *src; __half *dst;
  int64_t rows, cols, ld, batch_stride, work;   // work: quads (vec) or elements
  int vec;
};

__device__ __forceinline__ void round_one(const RoundJob &j, int64_t q) {
  if (j.vec) {
    const int64_t per_row = j.cols >> 2;
    const int64_t row = q / per_row, c = (q - row * per_row) << 2;
    const int64_t b = row / j.rows, r = row - b * j.rows;
    const float4 v = *reinterpret_cast<const float4 *>(j.src + b * j.batch_stride + r * j.ld + c);
    const __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t *>(&lo);
    o.y = *reinterpret_cast<const uint32_t *>(&hi);
    *reinterpret_cast<uint2 *>(j.dst + row * j.cols + c) = o;
  } else {
    const int64_t row = q / j.cols, c = q - row * j.cols;
    const int64_t b = row / j.rows, r = row - b * j.rows;
    j.dst[q] = __float2half_rn(j.src[b * j.batch_stride + r * j.ld + c]);
  }
}

// One launch rounds A and B: one thread per four consecutive columns of a row (or per element
// when the rows are not 16-byte friendly), the work items of A first, then B's.  Launched with
// programmatic stream serialisation: the chain's kernel behind it starts its set-up as soon as
// these CTAs are resident, and waits for them to finish before its first load.
__global__ void round_to_f16_kernel(const RoundJob a, const RoundJob b) {
  grid_dependency_wait();                    // the operands may be the previous kernel's output
  grid_launch_dependents();
  const int64_t total = a.work + b.work;
  for (int64_t q = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; q < total;
       q += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    if (q < a.work) round_one(a, q);
    else round_one(b, q - a.work);
  }
}

RoundJob make_job(const float *src, void *dst, int batch, int64_t rows, int64_t cols, int64_t ld, int64_t batch_stride) {
  RoundJob j;
  j.src = src; j.dst = static_cast<__half *>(dst);
  j.rows = rows; j.cols = cols; j.ld = ld; j.batch_stride = batch_stride;
  const int64_t total = static_cast<int64_t>(batch) * rows * cols;
  j.vec = (cols % 4 == 0) && (ld % 4 == 0) && (batch_stride % 4 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0) &&
          ((reinterpret_cast<uintptr_t>(dst) & 7) == 0);
  j.work = j.vec ? total / 4 : total;
  return j;
}
} // namespace

cudaError_t launch_round_to_f16(const float *A, void *dstA, int batchA, int64_t rowsA, int64_t colsA, int64_t ldA, int64_t strideA,
                                const float *B, void *dstB, int batchB, int64_t rowsB, int64_t colsB, int64_t ldB, int64_t strideB,
                                cudaStream_t s) {
  const RoundJob a = make_job(A, dstA, batchA, rowsA, colsA, ldA, strideA);
  const RoundJob b = make_job(B, dstB, batchB, rowsB, colsB, ldB, strideB);
  const int64_t work = a.work + b.work;
  if (work == 0) return cudaSuccess;
  const int64_t blocks = (work + 255) / 256;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(blocks < 148 * 16 ? blocks : 148 * 16), 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, round_to_f16_kernel, a, b);
}

} // namespace wtc

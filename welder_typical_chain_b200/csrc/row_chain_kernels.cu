// The two row-only chains of the reference's backend inputs, as single fused kernels:
//
//   row softmax       Out[i,:] = softmax(X[i,:])                      (max -> exp(x - max) -> sum -> divide;
//                     backend/welder/mlir_pipeline/softmax_row_chain.mlir:10-75)
//   row variance      Out[i,j] = c2 * sum_j (A[i,j] - c1 * sum_j A[i,j])^2 for every j
//                     (sum -> mean -> squared differences -> sum -> variance -> broadcast;
//                     backend/welder/mlir_pipeline/layernorm_variance_chain.mlir:12-104)
//
// Both are bandwidth-bound: every element is read once and written once.  A row is owned by
// one warp (N <= 2048: the row lives in the warp's registers between the passes, 128-bit
// loads and stores when the rows allow) or by one 256-thread CTA (longer rows: the row is
// re-read from L2 for the second and third pass).  f32 or f16 elements (input and output of
// the same type); the arithmetic is f32.
#include "wtc_kernels.h"
#include "wtc_ptx.cuh"

namespace wtc {
namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kWarpRowMax = 2048;            // longest row a warp keeps in registers (64 values a lane)

__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <bool F16> __device__ __forceinline__ float load_elem(const void *p, int64_t i) {
  return F16 ? __half2float(static_cast<const __half *>(p)[i]) : static_cast<const float *>(p)[i];
}
template <bool F16> __device__ __forceinline__ void store_elem(void *p, int64_t i, float v) {
  if (F16) static_cast<__half *>(p)[i] = __float2half_rn(v);
  else static_cast<float *>(p)[i] = v;
}

// ---- block-wide reductions for the long-row kernels -------------------------------------------
__device__ __forceinline__ float block_reduce(float v, bool is_max, float *scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = is_max ? warp_max_f(v) : warp_sum_f(v);
  __syncthreads();                       // scratch may still be read from the previous reduction
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = lane < (blockDim.x >> 5) ? scratch[lane] : (is_max ? -INFINITY : 0.f);
  t = is_max ? warp_max_f(t) : warp_sum_f(t);
  return t;
}

// KIND 0: softmax, 1: variance.  One warp per row, row in registers (strided by lane: element j
// of the row is value j / 32 of lane j % 32, so a warp's loads are contiguous).  PER = values a
// lane holds (rows of up to 32 * PER elements); the loops are fully unrolled over it.
template <int KIND, bool IN16, bool OUT16, int PER>
__global__ void __launch_bounds__(256) row_chain_warp_kernel(const void *__restrict__ X, void *__restrict__ Out, int64_t rows, int N,
                                                             int64_t ld_in, int64_t ld_out, float c1, float c2) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int64_t in0 = row * ld_in, out0 = row * ld_out;
  float v[PER];
  if (KIND == 0) {
    float m = -INFINITY;
#pragma unroll
    for (int t = 0; t < PER; ++t) {
      const int j = t * 32 + lane;
      v[t] = j < N ? load_elem<IN16>(X, in0 + j) : -INFINITY;
      m = fmaxf(m, v[t]);
    }
    m = warp_max_f(m);
    float s = 0.f;
#pragma unroll
    for (int t = 0; t < PER; ++t) {
      v[t] = ex2_approx((v[t] - m) * kLog2e);     // exp(x - max); -inf padding gives 0
      s += v[t];
    }
    s = warp_sum_f(s);
    const float inv = 1.0f / s;
#pragma unroll
    for (int t = 0; t < PER; ++t) {
      const int j = t * 32 + lane;
      if (j < N) store_elem<OUT16>(Out, out0 + j, v[t] * inv);
    }
  } else {
    float s = 0.f;
#pragma unroll
    for (int t = 0; t < PER; ++t) {
      const int j = t * 32 + lane;
      v[t] = j < N ? load_elem<IN16>(X, in0 + j) : 0.f;
      s += v[t];
    }
    const float mean = warp_sum_f(s) * c1;
    float q = 0.f;
#pragma unroll
    for (int t = 0; t < PER; ++t) {
      const int j = t * 32 + lane;
      const float d = v[t] - mean;
      if (j < N) q += d * d;
    }
    const float var = warp_sum_f(q) * c2;
#pragma unroll
    for (int t = 0; t < PER; ++t) {
      const int j = t * 32 + lane;
      if (j < N) store_elem<OUT16>(Out, out0 + j, var);
    }
  }
}

// One CTA per row, any length: three passes over the row (the second and third come from L2).
template <int KIND, bool IN16, bool OUT16>
__global__ void __launch_bounds__(256) row_chain_block_kernel(const void *__restrict__ X, void *__restrict__ Out, int N, int64_t ld_in,
                                                              int64_t ld_out, float c1, float c2) {
  __shared__ float scratch[8];
  const int64_t in0 = static_cast<int64_t>(blockIdx.x) * ld_in, out0 = static_cast<int64_t>(blockIdx.x) * ld_out;
  if (KIND == 0) {
    float m = -INFINITY;
    for (int j = threadIdx.x; j < N; j += blockDim.x) m = fmaxf(m, load_elem<IN16>(X, in0 + j));
    m = block_reduce(m, true, scratch);
    float s = 0.f;
    for (int j = threadIdx.x; j < N; j += blockDim.x) s += ex2_approx((load_elem<IN16>(X, in0 + j) - m) * kLog2e);
    s = block_reduce(s, false, scratch);
    const float inv = 1.0f / s;
    for (int j = threadIdx.x; j < N; j += blockDim.x)
      store_elem<OUT16>(Out, out0 + j, ex2_approx((load_elem<IN16>(X, in0 + j) - m) * kLog2e) * inv);
  } else {
    float s = 0.f;
    for (int j = threadIdx.x; j < N; j += blockDim.x) s += load_elem<IN16>(X, in0 + j);
    const float mean = block_reduce(s, false, scratch) * c1;
    float q = 0.f;
    for (int j = threadIdx.x; j < N; j += blockDim.x) { const float d = load_elem<IN16>(X, in0 + j) - mean; q += d * d; }
    const float var = block_reduce(q, false, scratch) * c2;
    for (int j = threadIdx.x; j < N; j += blockDim.x) store_elem<OUT16>(Out, out0 + j, var);
  }
}

template <int KIND, bool IN16, bool OUT16>
cudaError_t launch_typed(const void *X, void *Out, int64_t rows, int N, int64_t ld_in, int64_t ld_out, float c1, float c2, cudaStream_t s) {
  if (N <= kWarpRowMax) {
    const int64_t blocks = (rows + 7) / 8;
    if (blocks > 0x7fffffff) return cudaErrorInvalidConfiguration;
    const unsigned g = static_cast<unsigned>(blocks);
    if (N <= 256) row_chain_warp_kernel<KIND, IN16, OUT16, 8><<<g, 256, 0, s>>>(X, Out, rows, N, ld_in, ld_out, c1, c2);
    else if (N <= 1024) row_chain_warp_kernel<KIND, IN16, OUT16, 32><<<g, 256, 0, s>>>(X, Out, rows, N, ld_in, ld_out, c1, c2);
    else row_chain_warp_kernel<KIND, IN16, OUT16, 64><<<g, 256, 0, s>>>(X, Out, rows, N, ld_in, ld_out, c1, c2);
  } else {
    if (rows > 0x7fffffff) return cudaErrorInvalidConfiguration;
    row_chain_block_kernel<KIND, IN16, OUT16><<<static_cast<unsigned>(rows), 256, 0, s>>>(X, Out, N, ld_in, ld_out, c1, c2);
  }
  return cudaGetLastError();
}

} // namespace

cudaError_t launch_row_chain(int kind, const void *X, void *Out, int64_t rows, int64_t N, int64_t ld_in, int64_t ld_out, int in_f16,
                             int out_f16, float c1, float c2, cudaStream_t s) {
  if (rows <= 0 || N <= 0) return cudaSuccess;
  if (N > 0x7fffffff) return cudaErrorInvalidValue;
  const int n = static_cast<int>(N);
#define WTC_ROW_CASE(K, I, O) if (kind == K && (in_f16 != 0) == I && (out_f16 != 0) == O) return launch_typed<K, I, O>(X, Out, rows, n, ld_in, ld_out, c1, c2, s);
  WTC_ROW_CASE(0, false, false) WTC_ROW_CASE(0, true, true) WTC_ROW_CASE(1, false, false) WTC_ROW_CASE(1, true, true)
#undef WTC_ROW_CASE
  return cudaErrorInvalidValue;
}

} // namespace wtc

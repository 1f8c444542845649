// The two row-only chains of the reference's backend inputs, as single fused kernels:
//
//   row softmax       Out[i,:] = softmax(X[i,:])                      (max -> exp(x - max) -> sum -> divide;
//                     backend/welder/mlir_pipeline/softmax_row_chain.mlir:10-75)
//   row variance      Out[i,j] = c2 * sum_j (A[i,j] - c1 * sum_j A[i,j])^2 for every j
//                     (sum -> mean -> squared differences -> sum -> variance -> broadcast;
//                     backend/welder/mlir_pipeline/layernorm_variance_chain.mlir:12-104)
//
// Both are bandwidth-bound: every element is read once and written once, with 16-byte loads and
// stores (8 f16 or 4 f32 a lane) whenever the rows start on 16-byte boundaries and N is a
// multiple of the vector.  A row is owned by one warp (N <= 2048: 64 values a lane) or by one
// CTA of up to 512 threads (f32 rows up to 32768, f16 rows up to 65536 elements: 16 to 128 values
// a thread; f16 rows beyond 16384 elements stay packed as loaded); in both the row lives in
// registers between the passes.  Longer or unaligned rows take a CTA per row that re-reads the row (from
// L2) for the second and third pass.  f32 or f16 elements (input and output of the same type);
// the arithmetic is f32.
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

// ---- 16-byte vectors: 8 f16 or 4 f32 ----------------------------------------------------------
template <bool F16> struct VecOf { static constexpr int N = F16 ? 8 : 4; };

template <bool F16> __device__ __forceinline__ void load_vec(const void *base, int64_t elem, float (&v)[VecOf<F16>::N]) {
  if (F16) {
    const uint4 q = *reinterpret_cast<const uint4 *>(static_cast<const __half *>(base) + elem);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  } else {
    const float4 q = *reinterpret_cast<const float4 *>(static_cast<const float *>(base) + elem);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
  }
}
template <bool F16> __device__ __forceinline__ void store_vec(void *base, int64_t elem, const float (&v)[VecOf<F16>::N]) {
  if (F16) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = pack_f16x2(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4 *>(static_cast<__half *>(base) + elem) = make_uint4(w[0], w[1], w[2], w[3]);
  } else {
    *reinterpret_cast<float4 *>(static_cast<float *>(base) + elem) = make_float4(v[0], v[1], v[2], v[3]);
  }
}

// The chain on a row that is spread over a group of threads (a warp, or a CTA), NV vectors a
// thread: vector t of thread `tid` is vector number t * group + tid of the row, so that the
// group's loads are contiguous.  `reduce(x, is_max)` reduces over the group.
template <int KIND, bool F16, int NV, typename Reduce>
__device__ __forceinline__ void chain_on_row(const void *X, void *Out, int64_t in0, int64_t out0, int N, int tid, int group, float c1, float c2,
                                             Reduce reduce) {
  constexpr int V = VecOf<F16>::N;
  float v[NV][V];
  // all loads first: NV independent 16-byte requests a thread
#pragma unroll
  for (int t = 0; t < NV; ++t) {
    const int j = (t * group + tid) * V;
    if (j < N) load_vec<F16>(X, in0 + j, v[t]);
    else {
#pragma unroll
      for (int e = 0; e < V; ++e) v[t][e] = KIND == 0 ? -INFINITY : 0.f;
    }
  }
  if (KIND == 0) {
    float m = -INFINITY;
#pragma unroll
    for (int t = 0; t < NV; ++t)
#pragma unroll
      for (int e = 0; e < V; ++e) m = fmaxf(m, v[t][e]);
    m = reduce(m, true);
    const float mb = m * kLog2e;
    float s = 0.f;
#pragma unroll
    for (int t = 0; t < NV; ++t)
#pragma unroll
      for (int e = 0; e < V; ++e) {
        v[t][e] = ex2_approx(fmaf(v[t][e], kLog2e, -mb));     // exp(x - max); -inf padding gives 0
        s += v[t][e];
      }
    s = reduce(s, false);
    const float inv = 1.0f / s;
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      const int j = (t * group + tid) * V;
      if (j < N) {
#pragma unroll
        for (int e = 0; e < V; ++e) v[t][e] *= inv;
        store_vec<F16>(Out, out0 + j, v[t]);
      }
    }
  } else {
    float s = 0.f;
#pragma unroll
    for (int t = 0; t < NV; ++t)
#pragma unroll
      for (int e = 0; e < V; ++e) s += v[t][e];
    const float mean = reduce(s, false) * c1;
    float q = 0.f;
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      const int j = (t * group + tid) * V;
      if (j < N) {
#pragma unroll
        for (int e = 0; e < V; ++e) { const float d = v[t][e] - mean; q += d * d; }
      }
    }
    const float var = reduce(q, false) * c2;
    float o[V];
#pragma unroll
    for (int e = 0; e < V; ++e) o[e] = var;
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      const int j = (t * group + tid) * V;
      if (j < N) store_vec<F16>(Out, out0 + j, o);
    }
  }
}

// The same for long f16 rows with the row kept as it was loaded (8 halves in four registers
// instead of eight f32 values): half the registers, so that two 512-thread CTAs fit an SM and the
// phases of different rows overlap.  The exponentials are taken twice (once for the sum, once
// for the result); the special-function unit has the headroom, the memory system does not.
template <int KIND, int NV, typename Reduce>
__device__ __forceinline__ void chain_on_row_packed(const void *X, void *Out, int64_t in0, int64_t out0, int N, int tid, int group, float c1,
                                                    float c2, Reduce reduce) {
  const __half *x = static_cast<const __half *>(X);
  uint4 raw[NV];
#pragma unroll
  for (int t = 0; t < NV; ++t) {
    const int j = (t * group + tid) * 8;
    raw[t] = j < N ? *reinterpret_cast<const uint4 *>(x + in0 + j) : make_uint4(0u, 0u, 0u, 0u);
  }
  auto unpack = [](const uint4 &q, float (&v)[8]) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  };
  if (KIND == 0) {
    float m = -INFINITY;
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      if ((t * group + tid) * 8 < N) {
        float v[8]; unpack(raw[t], v);
#pragma unroll
        for (int e = 0; e < 8; ++e) m = fmaxf(m, v[e]);
      }
    }
    m = reduce(m, true);
    const float mb = m * kLog2e;
    float s = 0.f;
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      if ((t * group + tid) * 8 < N) {
        float v[8]; unpack(raw[t], v);
#pragma unroll
        for (int e = 0; e < 8; ++e) s += ex2_approx(fmaf(v[e], kLog2e, -mb));
      }
    }
    s = reduce(s, false);
    const float inv = 1.0f / s;
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      const int j = (t * group + tid) * 8;
      if (j < N) {
        float v[8]; unpack(raw[t], v);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = ex2_approx(fmaf(v[e], kLog2e, -mb)) * inv;
        store_vec<true>(Out, out0 + j, v);
      }
    }
  } else {
    float s = 0.f;
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      float v[8]; unpack(raw[t], v);             // (padding vectors are zeros)
#pragma unroll
      for (int e = 0; e < 8; ++e) s += v[e];
    }
    const float mean = reduce(s, false) * c1;
    float q = 0.f;
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      if ((t * group + tid) * 8 < N) {
        float v[8]; unpack(raw[t], v);
#pragma unroll
        for (int e = 0; e < 8; ++e) { const float d = v[e] - mean; q += d * d; }
      }
    }
    const float var = reduce(q, false) * c2;
    float o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = var;
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      const int j = (t * group + tid) * 8;
      if (j < N) store_vec<true>(Out, out0 + j, o);
    }
  }
}

// One warp per row (eight rows a CTA), the row in the warp's registers.
template <int KIND, bool F16, int NV>
__global__ void __launch_bounds__(256) row_chain_warp_kernel(const void *__restrict__ X, void *__restrict__ Out, int64_t rows, int N,
                                                             int64_t ld_in, int64_t ld_out, float c1, float c2) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  chain_on_row<KIND, F16, NV>(X, Out, row * ld_in, row * ld_out, N, threadIdx.x & 31, 32, c1, c2,
                              [](float x, bool is_max) { return is_max ? warp_max_f(x) : warp_sum_f(x); });
}

// One CTA of up to 512 threads per row, the row in the CTA's registers (NV vectors a thread).
template <int KIND, bool F16, int NV>
__global__ void __launch_bounds__(512) row_chain_cta_kernel(const void *__restrict__ X, void *__restrict__ Out, int N, int64_t ld_in,
                                                             int64_t ld_out, float c1, float c2) {
  __shared__ float scratch[32];
  chain_on_row<KIND, F16, NV>(X, Out, static_cast<int64_t>(blockIdx.x) * ld_in, static_cast<int64_t>(blockIdx.x) * ld_out, N, threadIdx.x,
                              blockDim.x, c1, c2, [&](float x, bool is_max) { return block_reduce(x, is_max, scratch); });
}

template <int KIND, int NV>
__global__ void __launch_bounds__(512, 2) row_chain_cta_packed_kernel(const void *__restrict__ X, void *__restrict__ Out, int N, int64_t ld_in,
                                                                     int64_t ld_out, float c1, float c2) {
  __shared__ float scratch[32];
  chain_on_row_packed<KIND, NV>(X, Out, static_cast<int64_t>(blockIdx.x) * ld_in, static_cast<int64_t>(blockIdx.x) * ld_out, N, threadIdx.x,
                                blockDim.x, c1, c2, [&](float x, bool is_max) { return block_reduce(x, is_max, scratch); });
}

// One CTA per row, any length and alignment: three passes over the row (the second and third come from L2).
template <int KIND, bool IN16, bool OUT16>
__global__ void __launch_bounds__(256) row_chain_block_kernel(const void *__restrict__ X, void *__restrict__ Out, int N, int64_t ld_in,
                                                              int64_t ld_out, float c1, float c2) {
  __shared__ float scratch[32];
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

template <int KIND, bool F16>
cudaError_t launch_typed(const void *X, void *Out, int64_t rows, int N, int64_t ld_in, int64_t ld_out, float c1, float c2, cudaStream_t s) {
  constexpr int V = VecOf<F16>::N;
  constexpr int ES = F16 ? 2 : 4;
  const bool vec = N % V == 0 && (ld_in * ES) % 16 == 0 && (ld_out * ES) % 16 == 0 &&
                   (reinterpret_cast<uintptr_t>(X) & 15) == 0 && (reinterpret_cast<uintptr_t>(Out) & 15) == 0;
  if (rows > 0x7fffffff) return cudaErrorInvalidConfiguration;
  if (vec && N <= kWarpRowMax) {
    const unsigned g = static_cast<unsigned>((rows + 7) / 8);
    const int nv = (N + 32 * V - 1) / (32 * V);            // vectors a lane
    constexpr int kMaxNv = 64 / V;                          // 64 values a lane at most
    if (nv <= 1) row_chain_warp_kernel<KIND, F16, 1><<<g, 256, 0, s>>>(X, Out, rows, N, ld_in, ld_out, c1, c2);
    else if (nv <= 2) row_chain_warp_kernel<KIND, F16, 2><<<g, 256, 0, s>>>(X, Out, rows, N, ld_in, ld_out, c1, c2);
    else if (nv <= 4) row_chain_warp_kernel<KIND, F16, 4><<<g, 256, 0, s>>>(X, Out, rows, N, ld_in, ld_out, c1, c2);
    else if (nv <= 8 || kMaxNv == 8) row_chain_warp_kernel<KIND, F16, 8><<<g, 256, 0, s>>>(X, Out, rows, N, ld_in, ld_out, c1, c2);
    else row_chain_warp_kernel<KIND, F16, kMaxNv><<<g, 256, 0, s>>>(X, Out, rows, N, ld_in, ld_out, c1, c2);
  } else if (vec && N <= 512 * 16 * V) {
    // as many threads as the row needs with 4, 8 or 16 vectors a thread, in whole warps, 512 at most
    const unsigned g = static_cast<unsigned>(rows);
    auto threads_for = [&](int nv) { return (((N + nv * V - 1) / (nv * V)) + 31) & ~31; };
    if (threads_for(4) <= 512) row_chain_cta_kernel<KIND, F16, 4><<<g, threads_for(4), 0, s>>>(X, Out, N, ld_in, ld_out, c1, c2);
    else if (F16 && threads_for(8) <= 512) row_chain_cta_packed_kernel<KIND, 8><<<g, threads_for(8), 0, s>>>(X, Out, N, ld_in, ld_out, c1, c2);
    else if (F16) row_chain_cta_packed_kernel<KIND, 16><<<g, threads_for(16), 0, s>>>(X, Out, N, ld_in, ld_out, c1, c2);
    else if (threads_for(8) <= 512) row_chain_cta_kernel<KIND, F16, 8><<<g, threads_for(8), 0, s>>>(X, Out, N, ld_in, ld_out, c1, c2);
    else row_chain_cta_kernel<KIND, F16, 16><<<g, threads_for(16), 0, s>>>(X, Out, N, ld_in, ld_out, c1, c2);
  } else {
    row_chain_block_kernel<KIND, F16, F16><<<static_cast<unsigned>(rows), 256, 0, s>>>(X, Out, N, ld_in, ld_out, c1, c2);
  }
  return cudaGetLastError();
}

} // namespace

cudaError_t launch_row_chain(int kind, const void *X, void *Out, int64_t rows, int64_t N, int64_t ld_in, int64_t ld_out, int in_f16,
                             int out_f16, float c1, float c2, cudaStream_t s) {
  if (rows <= 0 || N <= 0) return cudaSuccess;
  if (N > 0x7fffffff) return cudaErrorInvalidValue;
  if ((in_f16 != 0) != (out_f16 != 0)) return cudaErrorInvalidValue;
  const int n = static_cast<int>(N);
  if (kind == 0) return in_f16 ? launch_typed<0, true>(X, Out, rows, n, ld_in, ld_out, c1, c2, s) : launch_typed<0, false>(X, Out, rows, n, ld_in, ld_out, c1, c2, s);
  if (kind == 1) return in_f16 ? launch_typed<1, true>(X, Out, rows, n, ld_in, ld_out, c1, c2, s) : launch_typed<1, false>(X, Out, rows, n, ld_in, ld_out, c1, c2, s);
  return cudaErrorInvalidValue;
}

} // namespace wtc

// SIMT kernels for what the tensor-core path does not take: f32 chains (tcgen05
// has no f32 MMA), shapes whose row strides are not 16-byte multiples, and the
// unfused five-kernel pipeline the A/B harness compares the fused kernel with.
// k is accumulated in ascending order in f32, like a scalar loop nest.
#include "wtc_kernels.h"

#include <cuda_fp16.h>

namespace wtc {
namespace {

constexpr int kSimtThreads = 256;
constexpr int kKChunk = 64;

template <bool F16>
__device__ __forceinline__ float ld_elem(const void *p, int64_t i) {
  if (F16) return __half2float(static_cast<const __half *>(p)[i]);
  return static_cast<const float *>(p)[i];
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// logits tile of R rows x N columns: thread t owns columns t, t+256, ...
// shared: As[R][kKChunk] then S[R][N]
template <int R, bool F16>
__device__ __forceinline__ void matmul_rows(const void *A, const void *B, const SimtParams &p, int64_t a_off,
                                            int64_t b_off, int row0, int rows, float *As, float *S) {
  for (int j0 = 0; j0 < p.N; j0 += kSimtThreads) {
    const int j = j0 + threadIdx.x;
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.f;
    for (int k0 = 0; k0 < p.K; k0 += kKChunk) {
      const int kc = min(kKChunk, p.K - k0);
      __syncthreads();
      for (int i = threadIdx.x; i < R * kKChunk; i += kSimtThreads) {
        const int r = i / kKChunk, k = i - r * kKChunk;
        As[i] = (r < rows && k < kc) ? ld_elem<F16>(A, a_off + static_cast<int64_t>(row0 + r) * p.lda + k0 + k) : 0.f;
      }
      __syncthreads();
      if (j < p.N) {
        // sixteen independent loads of B's column are in flight before the first is used (a thread
        // walks down one column: without this the loop is a chain of L2 round trips); k stays ascending
        int k = 0;
        for (; k + 16 <= kc; k += 16) {
          float bv[16];
#pragma unroll
          for (int u = 0; u < 16; ++u) bv[u] = ld_elem<F16>(B, b_off + static_cast<int64_t>(k0 + k + u) * p.ldb + j);
#pragma unroll
          for (int u = 0; u < 16; ++u) {
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r] = fmaf(As[r * kKChunk + k + u], bv[u], acc[r]);
          }
        }
        for (; k < kc; ++k) {
          const float bv = ld_elem<F16>(B, b_off + static_cast<int64_t>(k0 + k) * p.ldb + j);
#pragma unroll
          for (int r = 0; r < R; ++r) acc[r] = fmaf(As[r * kKChunk + k], bv, acc[r]);
        }
      }
    }
    if (j < p.N) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float s = acc[r];
        if (p.acc_mode == 1) s = __half2float(__float2half_rn(s));
        S[static_cast<int64_t>(r) * p.N + j] = s * p.scale;
      }
    }
  }
  __syncthreads();
}

template <int R, bool F16>
__global__ void __launch_bounds__(kSimtThreads)
simt_fused_kernel(const void *__restrict__ A, const void *__restrict__ B, void *__restrict__ Out, const SimtParams p) {
  extern __shared__ float sm[];
  float *As = sm;
  float *S = sm + R * kKChunk;
  const int blocks_per_batch = (p.M + R - 1) / R;
  const int b = blockIdx.x / blocks_per_batch;
  const int row0 = (blockIdx.x - b * blocks_per_batch) * R;
  const int rows = min(R, p.M - row0);
  matmul_rows<R, F16>(A, B, p, b * p.a_batch_stride, b * p.b_batch_stride, row0, rows, As, S);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = warp; r < rows; r += kSimtThreads / 32) {
    float *s = S + static_cast<int64_t>(r) * p.N;
    float mx = -3.4028235e38f;
    for (int j = lane; j < p.N; j += 32) mx = fmaxf(mx, s[j]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int j = lane; j < p.N; j += 32) { const float e = expf(s[j] - mx); s[j] = e; sum += e; }
    sum = warp_sum(sum);
    const int64_t o = b * p.o_batch_stride + static_cast<int64_t>(row0 + r) * p.ldo;
    if (p.out_f16) {
      __half *out = static_cast<__half *>(Out) + o;
      for (int j = lane; j < p.N; j += 32) out[j] = __float2half_rn(s[j] / sum);
    } else {
      float *out = static_cast<float *>(Out) + o;
      for (int j = lane; j < p.N; j += 32) out[j] = s[j] / sum;
    }
  }
}

// ---- the unfused pipeline ----------------------------------------------------
template <int R, bool F16>
__global__ void __launch_bounds__(kSimtThreads)
unfused_matmul_kernel(const void *__restrict__ A, const void *__restrict__ B, float *__restrict__ C32, const SimtParams p) {
  extern __shared__ float sm[];
  float *As = sm;
  const int blocks_per_batch = (p.M + R - 1) / R;
  const int b = blockIdx.x / blocks_per_batch;
  const int row0 = (blockIdx.x - b * blocks_per_batch) * R;
  const int rows = min(R, p.M - row0);
  // write straight to global: S points at this block's rows of C32 (row stride N)
  float *S = C32 + (static_cast<int64_t>(b) * p.M + row0) * p.N;
  // rows beyond `rows` must not be written: matmul_rows writes R rows, so guard here
  if (rows == R) {
    matmul_rows<R, F16>(A, B, p, b * p.a_batch_stride, b * p.b_batch_stride, row0, rows, As, S);
  } else {
    for (int r = 0; r < rows; ++r) {
      SimtParams q = p;
      matmul_rows<1, F16>(A, B, q, b * p.a_batch_stride, b * p.b_batch_stride, row0 + r, 1, As, S + static_cast<int64_t>(r) * p.N);
    }
  }
}

__global__ void rowmax_kernel(const float *__restrict__ C32, float *__restrict__ mx, int64_t rows, int N) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float m = -3.4028235e38f;
  for (int j = lane; j < N; j += 32) m = fmaxf(m, C32[row * N + j]);
  m = warp_max(m);
  if (lane == 0) mx[row] = m;
}
__global__ void exp_kernel(const float *__restrict__ C32, const float *__restrict__ mx, float *__restrict__ E, int64_t total, int N) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    E[i] = expf(C32[i] - mx[i / N]);
}
__global__ void rowsum_kernel(const float *__restrict__ E, float *__restrict__ sum, int64_t rows, int N) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float s = 0.f;
  for (int j = lane; j < N; j += 32) s += E[row * N + j];
  s = warp_sum(s);
  if (lane == 0) sum[row] = s;
}
__global__ void div_kernel(const float *__restrict__ E, const float *__restrict__ sum, void *__restrict__ Out, int64_t rows_per_batch,
                           int64_t total, int N, int64_t ldo, int64_t o_batch_stride, int out_f16) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / N; const int j = static_cast<int>(i - row * N);
    const int64_t b = row / rows_per_batch, r = row - b * rows_per_batch;
    const float v = E[i] / sum[row];
    const int64_t o = b * o_batch_stride + r * ldo + j;
    if (out_f16) static_cast<__half *>(Out)[o] = __float2half_rn(v);
    else static_cast<float *>(Out)[o] = v;
  }
}

int pick_rows(const SimtParams &p, size_t smem_limit) {
  // largest R in {16,8,4,2,1} whose logits tile fits shared memory; small problems trade rows
  // per CTA for more CTAs (latency-bound: fill the 148 SMs before deepening the per-CTA work)
  int best = 0;
  for (int R = 16; R >= 1; R >>= 1) {
    const size_t need = (static_cast<size_t>(R) * kKChunk + static_cast<size_t>(R) * p.N) * sizeof(float);
    if (need > smem_limit) continue;
    if (!best) best = R;
    const int64_t blocks = static_cast<int64_t>(p.batch) * ((p.M + R - 1) / R);
    if (blocks >= 148) return R;
    best = R;
  }
  return best;
}

// The opt-in to more than 48 KB of dynamic shared memory is per kernel instance and per device:
// it is raised once to the largest window this instance has been asked for there, not on every call.
template <int R, bool IN16>
cudaError_t fused_r_window(size_t smem) {
  static size_t granted[64] = {0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (smem > granted[dev]) {
    e = cudaFuncSetAttribute(simt_fused_kernel<R, IN16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    granted[dev] = smem;
  }
  return cudaSuccess;
}

template <int R>
cudaError_t launch_fused_r(const void *A, const void *B, void *Out, const SimtParams &p, cudaStream_t s) {
  const size_t smem = (static_cast<size_t>(R) * kKChunk + static_cast<size_t>(R) * p.N) * sizeof(float);
  const int64_t blocks = static_cast<int64_t>(p.batch) * ((p.M + R - 1) / R);
  if (blocks > 0x7fffffff) return cudaErrorInvalidConfiguration;
  cudaError_t e;
  if (p.in_f16) {
    e = fused_r_window<R, true>(smem);
    if (e != cudaSuccess) return e;
    simt_fused_kernel<R, true><<<static_cast<unsigned>(blocks), kSimtThreads, smem, s>>>(A, B, Out, p);
  } else {
    e = fused_r_window<R, false>(smem);
    if (e != cudaSuccess) return e;
    simt_fused_kernel<R, false><<<static_cast<unsigned>(blocks), kSimtThreads, smem, s>>>(A, B, Out, p);
  }
  return cudaGetLastError();
}

} // namespace

cudaError_t launch_simt_fused(const void *A, const void *B, void *Out, const SimtParams &p, cudaStream_t s) {
  if (p.batch <= 0 || p.M <= 0 || p.N <= 0) return cudaSuccess;
  const int R = pick_rows(p, 200 * 1024);
  switch (R) {
    case 16: return launch_fused_r<16>(A, B, Out, p, s);
    case 8: return launch_fused_r<8>(A, B, Out, p, s);
    case 4: return launch_fused_r<4>(A, B, Out, p, s);
    case 2: return launch_fused_r<2>(A, B, Out, p, s);
    case 1: return launch_fused_r<1>(A, B, Out, p, s);
    default: return cudaErrorInvalidValue;  // one row of logits does not fit shared memory
  }
}

size_t simt_unfused_workspace_bytes(const SimtParams &p) {
  const size_t rows = static_cast<size_t>(p.batch) * p.M;
  // C32[rows,N], E[rows,N], max[rows], sum[rows]
  return (2 * rows * p.N + 2 * rows) * sizeof(float);
}

cudaError_t launch_simt_unfused(const void *A, const void *B, void *Out, void *workspace, const SimtParams &p,
                                cudaStream_t s) {
  if (p.batch <= 0 || p.M <= 0 || p.N <= 0) return cudaSuccess;
  const int64_t rows = static_cast<int64_t>(p.batch) * p.M;
  const int64_t total = rows * p.N;
  float *C32 = static_cast<float *>(workspace);
  float *E = C32 + total;
  float *mx = E + total;
  float *sum = mx + rows;
  constexpr int R = 8;
  const size_t smem = static_cast<size_t>(R) * kKChunk * sizeof(float);
  const int64_t blocks = static_cast<int64_t>(p.batch) * ((p.M + R - 1) / R);
  if (blocks > 0x7fffffff) return cudaErrorInvalidConfiguration;
  if (p.in_f16) unfused_matmul_kernel<R, true><<<static_cast<unsigned>(blocks), kSimtThreads, smem, s>>>(A, B, C32, p);
  else unfused_matmul_kernel<R, false><<<static_cast<unsigned>(blocks), kSimtThreads, smem, s>>>(A, B, C32, p);
  return launch_softmax_passes(C32, E, mx, sum, Out, rows, p.M, p.N, p.ldo, p.o_batch_stride, p.out_f16, s);
}

cudaError_t launch_softmax_passes(const float *C32, float *E, float *mx, float *sum, void *Out, int64_t rows, int64_t rows_per_batch,
                                  int N, int64_t ldo, int64_t o_batch_stride, int out_f16, cudaStream_t s) {
  const int64_t total = rows * N;
  const unsigned row_grid = static_cast<unsigned>((rows + 7) / 8);
  const unsigned ew_grid = static_cast<unsigned>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
  rowmax_kernel<<<row_grid, 256, 0, s>>>(C32, mx, rows, N);
  exp_kernel<<<ew_grid, 256, 0, s>>>(C32, mx, E, total, N);
  rowsum_kernel<<<row_grid, 256, 0, s>>>(E, sum, rows, N);
  div_kernel<<<ew_grid, 256, 0, s>>>(E, sum, Out, rows_per_batch, total, N, ldo, o_batch_stride, out_f16);
  return cudaGetLastError();
}

} // namespace wtc

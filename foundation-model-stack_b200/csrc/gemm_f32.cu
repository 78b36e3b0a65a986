// y[M, N] = x[M, K] . w[N, K]^T (+ bias[N]) in true float32: FFMA on the CUDA cores, no tensor-core mode,
// no reduced-precision product.  Each output element is one sequential sum over k, in the same order
// whatever M is, so a row's result does not depend on what else is in the batch.
// 64 x 64 output tile per block of 256 threads, 16-wide k steps through shared memory, 4 x 4 per thread.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                       const float* __restrict__ bias, float* __restrict__ y, int M,
                                                       int N, int K) {
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tm = (tid / 16) * TM, tn = (tid % 16) * TN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  // each thread loads 4 consecutive k of one row of each operand tile
  const int lr = tid / 4;        // 0..63: row within the tile
  const int lk = (tid % 4) * 4;  // 0,4,8,12
  const bool vec = (K % 4) == 0;
  for (int k0 = 0; k0 < K; k0 += BK) {
    float xv[4] = {0.f, 0.f, 0.f, 0.f}, wv[4] = {0.f, 0.f, 0.f, 0.f};
    const int gm = m0 + lr, gn = n0 + lr, gk = k0 + lk;
    if (gm < M) {
      if (vec && gk + 3 < K) {
        const float4 v = *reinterpret_cast<const float4*>(x + (size_t)gm * K + gk);
        xv[0] = v.x; xv[1] = v.y; xv[2] = v.z; xv[3] = v.w;
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (gk + i < K) xv[i] = x[(size_t)gm * K + gk + i];
      }
    }
    if (gn < N) {
      if (vec && gk + 3 < K) {
        const float4 v = *reinterpret_cast<const float4*>(w + (size_t)gn * K + gk);
        wv[0] = v.x; wv[1] = v.y; wv[2] = v.z; wv[3] = v.w;
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (gk + i < K) wv[i] = w[(size_t)gn * K + gk + i];
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      xs[lk + i][lr] = xv[i];
      ws[lk + i][lr] = wv[i];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = xs[k][tm + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = ws[k][tn + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + tm + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tn + j;
      if (gn < N && FMS_IN((size_t)gm * N + gn, (size_t)M * N)) y[(size_t)gm * N + gn] = acc[i][j] + (bias ? bias[gn] : 0.f);
    }
  }
}

// Few rows (a decode step): the tiles above would be nearly empty and their loop, which waits for memory at every
// step of 16 k, takes 20 times what the weights' bytes need.  Here a thread owns one column of y (one row of w) for
// all rows of x, reads its row of w 16 bytes at a time with two batches of loads in flight, and takes x from shared
// memory.  Every element is still one sequential fmaf chain over k = 0, 1, 2, ..., so the result is bit for bit the
// tiled kernel's.
constexpr int FEW_ROWS = 8, FEW_THREADS = 64, FEW_BATCH = 16;  // rows at most; columns a block; float4 a batch

__global__ void __launch_bounds__(FEW_THREADS) gemm_f32_few_rows_kernel(const float* __restrict__ x,
                                                                        const float* __restrict__ w,
                                                                        const float* __restrict__ bias,
                                                                        float* __restrict__ y, int M, int N, int K) {
  __shared__ float4 xs[FEW_ROWS][FEW_BATCH];
  const int n = blockIdx.x * FEW_THREADS + threadIdx.x;
  const int k4 = K / 4;  // K is a multiple of 4 here
  const float4* wrow = reinterpret_cast<const float4*>(w + (size_t)min(n, N - 1) * K);
  float acc[FEW_ROWS];
#pragma unroll
  for (int m = 0; m < FEW_ROWS; ++m) acc[m] = 0.f;
  float4 cur[FEW_BATCH], nxt[FEW_BATCH];
#pragma unroll
  for (int u = 0; u < FEW_BATCH; ++u) cur[u] = u < k4 ? wrow[u] : make_float4(0.f, 0.f, 0.f, 0.f);
  for (int k0 = 0; k0 < k4; k0 += FEW_BATCH) {
#pragma unroll
    for (int u = 0; u < FEW_BATCH; ++u)  // the next batch of this row of w, while this one is used
      nxt[u] = k0 + FEW_BATCH + u < k4 ? wrow[k0 + FEW_BATCH + u] : make_float4(0.f, 0.f, 0.f, 0.f);
    __syncthreads();  // the batch of x before this one has been used by everyone
    for (int i = threadIdx.x; i < FEW_ROWS * FEW_BATCH; i += FEW_THREADS) {
      const int m = i / FEW_BATCH, u = i % FEW_BATCH;
      xs[m][u] = (m < M && k0 + u < k4) ? reinterpret_cast<const float4*>(x + (size_t)m * K)[k0 + u]
                                        : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __syncthreads();
    const int live = min(FEW_BATCH, k4 - k0);  // beyond K nothing is added: a chain must not see extra terms
#pragma unroll
    for (int u = 0; u < FEW_BATCH; ++u) {
      if (u >= live) break;
      const float4 wv = cur[u];
#pragma unroll
      for (int m = 0; m < FEW_ROWS; ++m) {
        const float4 xv = xs[m][u];
        acc[m] = fmaf(xv.x, wv.x, acc[m]);
        acc[m] = fmaf(xv.y, wv.y, acc[m]);
        acc[m] = fmaf(xv.z, wv.z, acc[m]);
        acc[m] = fmaf(xv.w, wv.w, acc[m]);
      }
    }
#pragma unroll
    for (int u = 0; u < FEW_BATCH; ++u) cur[u] = nxt[u];
  }
  if (n < N) {
    const float b = bias ? bias[n] : 0.f;
#pragma unroll
    for (int m = 0; m < FEW_ROWS; ++m)
      if (m < M && FMS_IN((size_t)m * N + n, (size_t)M * N)) y[(size_t)m * N + n] = acc[m] + b;
  }
}
}  // namespace

FMS_API int fms_gemm_f32(const float* x, const float* w, const float* bias, float* y, int M, int N, int K,
                         cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return fms_fail("gemm_f32: K %d", K);
  if (M <= FEW_ROWS && K % 4 == 0 && K >= 4) {
    gemm_f32_few_rows_kernel<<<(N + FEW_THREADS - 1) / FEW_THREADS, FEW_THREADS, 0, stream>>>(x, w, bias, y, M, N, K);
    return fms_launch_status("gemm_f32");
  }
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return fms_fail("gemm_f32: %d rows are more than one launch takes", M);
  gemm_f32_kernel<<<grid, 256, 0, stream>>>(x, w, bias, y, M, N, K);
  return fms_launch_status("gemm_f32");
}

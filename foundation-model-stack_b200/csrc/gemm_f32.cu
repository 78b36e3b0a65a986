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

// Few rows (a decode step: up to 64): the tiles above would be nearly empty and their loop, which waits for memory
// at every step of 16 k, takes 20 times what the weights' bytes need.  Here a block owns 32 columns of y (32 rows of w)
// and a thread one of them for ROWS / MSPLIT of the rows of x (MSPLIT warps; 4 where the matrix has few rows and the
// multiprocessors would else have too few warps, 2 where it has many).  The block brings its rows of w and all rows of x,
// 64 k at a time, into shared memory by 16-byte asynchronous copies in which 16 lanes cover 256 contiguous bytes of
// one row (four such stages a block, and up to five blocks a multiprocessor), and each thread then walks its own row
// there.  Every element is still one sequential fmaf chain over k = 0, 1, 2, ..., so the result is bit for bit the tiled
// kernel's.  (A thread that read its row of w straight from global memory, 16 bytes a lane and a row apart from its
// neighbour's, got 0.7 TB/s out of the memory system.)
constexpr int FEW_MAX_ROWS = 64, FEW_WROWS = 32, FEW_KT = 64, FEW_STAGES = 4, FEW_PAD = 4;
constexpr int FEW_WSTRIDE = FEW_KT + FEW_PAD;

template <int ROWS>
constexpr size_t few_smem() {
  return (size_t)FEW_STAGES * (FEW_WROWS * FEW_WSTRIDE + ROWS * FEW_KT) * sizeof(float);
}

__device__ __forceinline__ void few_copy16(void* smem, const void* gmem, bool valid) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0: the destination is filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}

template <int ROWS, int MSPLIT>
__global__ void __launch_bounds__(FEW_WROWS * MSPLIT) gemm_f32_few_rows_kernel(const float* __restrict__ x,
                                                                               const float* __restrict__ w,
                                                                               const float* __restrict__ bias,
                                                                               float* __restrict__ y, int M, int N, int K) {
  extern __shared__ __align__(16) float few_smem_base[];
  constexpr int THREADS = FEW_WROWS * MSPLIT, MPT = ROWS / MSPLIT;
  constexpr int STAGE_FLOATS = FEW_WROWS * FEW_WSTRIDE + ROWS * FEW_KT;
  const int tid = threadIdx.x, row = tid % FEW_WROWS, m0 = (tid / FEW_WROWS) * MPT;
  const int n0 = blockIdx.x * FEW_WROWS;
  const int steps = (K + FEW_KT - 1) / FEW_KT;  // K is a multiple of 4 here

  auto issue = [&](int step) {
    if (step < steps) {
      float* ws = few_smem_base + (size_t)(step % FEW_STAGES) * STAGE_FLOATS;
      float* xs = ws + FEW_WROWS * FEW_WSTRIDE;
      const int k0 = step * FEW_KT;
#pragma unroll
      for (int c = tid; c < FEW_WROWS * (FEW_KT / 4); c += THREADS) {
        const int r = c / (FEW_KT / 4), piece = c % (FEW_KT / 4);
        const int k = k0 + 4 * piece;
        const int n = min(n0 + r, N - 1);  // rows beyond N repeat the last one; their results are not stored
        few_copy16(ws + r * FEW_WSTRIDE + 4 * piece, w + (size_t)n * K + min(k, K - 4), k < K);
      }
#pragma unroll
      for (int c = tid; c < ROWS * (FEW_KT / 4); c += THREADS) {
        const int m = c / (FEW_KT / 4), piece = c % (FEW_KT / 4);
        const int k = k0 + 4 * piece;
        few_copy16(xs + m * FEW_KT + 4 * piece, x + (size_t)min(m, M - 1) * K + min(k, K - 4), m < M && k < K);
      }
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");  // an empty group keeps the count of groups in step
  };

  float acc[MPT];
#pragma unroll
  for (int i = 0; i < MPT; ++i) acc[i] = 0.f;
#pragma unroll
  for (int s = 0; s < FEW_STAGES - 1; ++s) issue(s);
  for (int step = 0; step < steps; ++step) {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(FEW_STAGES - 2) : "memory");  // this step's stage has arrived
    __syncthreads();  // ... for every thread, and everyone is done with the stage that is filled next
    issue(step + FEW_STAGES - 1);
    const float* ws = few_smem_base + (size_t)(step % FEW_STAGES) * STAGE_FLOATS + row * FEW_WSTRIDE;
    const float* xs = few_smem_base + (size_t)(step % FEW_STAGES) * STAGE_FLOATS + FEW_WROWS * FEW_WSTRIDE + m0 * FEW_KT;
    const int live = min(FEW_KT / 4, (K - step * FEW_KT) / 4);  // beyond K nothing is added: a chain sees no extra terms
    if (m0 < M) {  // a warp whose rows of x do not exist has nothing to add
#pragma unroll (MPT <= 4 ? 4 : 2)
      for (int u = 0; u < live; ++u) {
        const float4 wv = *reinterpret_cast<const float4*>(ws + 4 * u);
#pragma unroll
        for (int i = 0; i < MPT; ++i) {
          const float4 xv = *reinterpret_cast<const float4*>(xs + i * FEW_KT + 4 * u);
          acc[i] = fmaf(xv.x, wv.x, acc[i]);
          acc[i] = fmaf(xv.y, wv.y, acc[i]);
          acc[i] = fmaf(xv.z, wv.z, acc[i]);
          acc[i] = fmaf(xv.w, wv.w, acc[i]);
        }
      }
    }
  }
  const int n = n0 + row;
  if (n < N) {
    const float b = bias ? bias[n] : 0.f;
#pragma unroll
    for (int i = 0; i < MPT; ++i)
      if (m0 + i < M && FMS_IN((size_t)(m0 + i) * N + n, (size_t)M * N)) y[(size_t)(m0 + i) * N + n] = acc[i] + b;
  }
}

template <int ROWS, int MSPLIT>
int launch_few_rows(const float* x, const float* w, const float* bias, float* y, int M, int N, int K, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_f32_few_rows_kernel<ROWS, MSPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)few_smem<ROWS>());
    if (e != cudaSuccess) return fms_fail("gemm_f32: %zu bytes of shared memory refused: %s", few_smem<ROWS>(), cudaGetErrorString(e));
    configured = true;
  }
  gemm_f32_few_rows_kernel<ROWS, MSPLIT><<<(N + FEW_WROWS - 1) / FEW_WROWS, FEW_WROWS * MSPLIT, few_smem<ROWS>(), stream>>>(
      x, w, bias, y, M, N, K);
  return fms_launch_status("gemm_f32");
}

template <int ROWS>
int launch_few_rows_for(const float* x, const float* w, const float* bias, float* y, int M, int N, int K, cudaStream_t stream) {
  const int blocks = (N + FEW_WROWS - 1) / FEW_WROWS;
  if (blocks < 4 * 148) return launch_few_rows<ROWS, 4>(x, w, bias, y, M, N, K, stream);
  return launch_few_rows<ROWS, 2>(x, w, bias, y, M, N, K, stream);
}
}  // namespace

FMS_API int fms_gemm_f32(const float* x, const float* w, const float* bias, float* y, int M, int N, int K,
                         cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return fms_fail("gemm_f32: K %d", K);
  if (M <= FEW_MAX_ROWS && K % 4 == 0 && K >= 4) {
    if (M <= 8) return launch_few_rows_for<8>(x, w, bias, y, M, N, K, stream);
    if (M <= 16) return launch_few_rows_for<16>(x, w, bias, y, M, N, K, stream);
    if (M <= 32) return launch_few_rows_for<32>(x, w, bias, y, M, N, K, stream);
    return launch_few_rows_for<64>(x, w, bias, y, M, N, K, stream);
  }
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return fms_fail("gemm_f32: %d rows are more than one launch takes", M);
  gemm_f32_kernel<<<grid, 256, 0, stream>>>(x, w, bias, y, M, N, K);
  return fms_launch_status("gemm_f32");
}

// Shared helpers of the sm_100a kernels: dtype codes, conversions, reductions, error reporting.
//
// Every library built from these sources exports plain C functions that take raw device pointers,
// sizes and a CUDA stream, launch on that stream and return 0 or an error code; fms_last_error() gives
// the text.  No function allocates device memory or synchronises.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#define FMS_API extern "C" __attribute__((visibility("default")))

enum FmsDtype { FMS_F32 = 0, FMS_BF16 = 1, FMS_NONE = -1 };

static char g_fms_error[512] = "";

static inline int fms_fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_fms_error, sizeof(g_fms_error), fmt, ap);
  va_end(ap);
  return 1;
}

static inline int fms_launch_status(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fms_fail("%s: launch failed: %s", what, cudaGetErrorString(e));
  return 0;
}

FMS_API const char* fms_last_error() { return g_fms_error; }

// ---- conversions ------------------------------------------------------------------------------------
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---- reductions -------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a thread block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Dispatch on a runtime dtype code.
#define FMS_DISPATCH_DTYPE(code, T, ...)                     \
  do {                                                       \
    if ((code) == FMS_F32) {                                 \
      typedef float T;                                       \
      __VA_ARGS__;                                           \
    } else if ((code) == FMS_BF16) {                         \
      typedef __nv_bfloat16 T;                               \
      __VA_ARGS__;                                           \
    } else {                                                 \
      return fms_fail("unsupported dtype code %d", (int)(code)); \
    }                                                        \
  } while (0)

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

// ---- bounds-checked build ---------------------------------------------------------------------------
// Compiled with -DFMS_DEBUG_BOUNDS (environment variable FMS_B200_DEBUG_BOUNDS=1 when the library is built),
// FMS_IN(index, extent) is false for an index outside [0, extent) and records the first such index of the process
// (source line, index, extent) in a word of the library that fms_debug_bounds() reads and clears; the access is
// then skipped, nothing traps and the context stays usable.  An extent <= 0 means "not known here": only a
// negative index is caught.  Without the flag FMS_IN is the constant true and costs nothing.  This stands in for
// a memory checker on machines where none can be run.
#ifdef FMS_DEBUG_BOUNDS
__device__ int g_fms_bounds[4] = {0, 0, 0, 0};  // violations, then line, index and extent of the first
__device__ __forceinline__ bool fms_index_ok(long long i, long long n, int line) {
  if (i >= 0 && (n <= 0 || i < n)) return true;
  if (atomicAdd(&g_fms_bounds[0], 1) == 0) {
    g_fms_bounds[1] = line;
    g_fms_bounds[2] = (int)(i > 0x7fffffffLL ? 0x7fffffffLL : (i < -0x7fffffffLL ? -0x7fffffffLL : i));
    g_fms_bounds[3] = (int)(n > 0x7fffffffLL ? 0x7fffffffLL : n);
  }
  return false;
}
#define FMS_IN(i, n) fms_index_ok((long long)(i), (long long)(n), __LINE__)
// out[0..3]: violations since the last call, line, index, extent of the first.  Synchronises the device.
FMS_API int fms_debug_bounds(int* out) {
  int zero[4] = {0, 0, 0, 0};
  if (cudaMemcpyFromSymbol(out, g_fms_bounds, sizeof(zero)) != cudaSuccess) return fms_fail("debug_bounds: read failed");
  if (out[0] != 0 && cudaMemcpyToSymbol(g_fms_bounds, zero, sizeof(zero)) != cudaSuccess) return fms_fail("debug_bounds: reset failed");
  return 0;
}
#else
#define FMS_IN(i, n) true
FMS_API int fms_debug_bounds(int* out) {  // not a checked build
  (void)out;
  return -1;
}
#endif

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

// ---- programmatic dependent launch ------------------------------------------------------------------
// Kernels of a step are launched so that a kernel may start while the one before it is still draining.
// Every kernel calls pdl_launch_dependents() early (the next kernel may be scheduled once all blocks of this
// one have done so) and pdl_wait() before it reads what an earlier kernel wrote or writes anything at all;
// only loads of constant data (weights) may come before pdl_wait().
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

#include <stdlib.h>
static inline bool fms_pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("FMS_B200_PDL");
    enabled = (e && e[0] == '0') ? 0 : 1;
  }
  return enabled == 1;
}

// Launches `kernel` on `stream`; with programmatic stream serialization unless FMS_B200_PDL=0.
template <typename... KArgs, typename... Args>
static inline cudaError_t fms_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = fms_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---- mbarrier and bulk copies (sm_90+) ---------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(void* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(void* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Waits for the phase with the given parity to complete; gives up after a bounded number of polls and returns
// false (the caller records the failure and goes on, so that no kernel can hang).
__device__ __forceinline__ bool mbar_wait(void* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (int i = 0; i < (1 << 22); ++i) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
// bytes: a multiple of 16; both addresses 16-byte aligned; completion is counted on the mbarrier
__device__ __forceinline__ void bulk_copy_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, void* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

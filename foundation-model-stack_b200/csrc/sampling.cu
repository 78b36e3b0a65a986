// Picking the next token from float32 logits, one thread block per row.
//   argmax:  the largest logit, the lowest index among equals        (fms/utils/generation.py:328)
//   sample:  logits / temperature; with top_k, everything below the k-th largest value is dropped;
//            softmax in float32; one draw                            (fms/utils/generation.py:318-326)
// The draw is the inverse CDF at a uniform number u in [0, 1) that is a hash of (seed, request, step), so
// a request draws the same tokens alone and in any batch.  The reference draws with torch.multinomial from
// the global generator instead; the distribution is the same.
#include "common.cuh"

namespace {
constexpr int THREADS = 1024;
constexpr int WARPS = THREADS / 32;

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__device__ __forceinline__ float uniform01(uint64_t seed, uint64_t request, uint64_t step) {
  uint64_t z = mix64(seed);
  z = mix64(z ^ request);
  z = mix64(z ^ step);
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(THREADS) argmax_kernel(const float* __restrict__ logits, int* __restrict__ out,
                                                         int vocab) {
  __shared__ float best_v[WARPS];
  __shared__ int best_i[WARPS];
  pdl_launch_dependents();
  pdl_wait();
  const float* x = logits + (size_t)blockIdx.x * vocab;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  if ((vocab & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    // 16 bytes a load, four loads on their way before the first comparison: the row is one block's to read, so
    // what counts is how many bytes that block keeps in flight
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const int n4 = vocab >> 2;
    for (int i0 = threadIdx.x; i0 < n4; i0 += 4 * THREADS) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        v[u] = i0 + u * THREADS < n4 ? x4[i0 + u * THREADS] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = 4 * (i0 + u * THREADS);
        const float e[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (e[j] > bv || (e[j] == bv && i + j < bi)) { bv = e[j]; bi = i + j; }
      }
    }
  } else {
    for (int i = threadIdx.x; i < vocab; i += THREADS) {
      const float v = x[i];
      if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = best_v[lane];
    bi = best_i[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0 && FMS_IN(bi == 0x7fffffff ? 0 : bi, vocab)) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;  // a row of NaN or -inf only: token 0
  }
}

// floats to unsigned keys with the same order
__device__ __forceinline__ uint32_t order_key(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float warp_inclusive_scan(float v, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  return v;
}

__global__ void __launch_bounds__(THREADS) sample_kernel(const float* __restrict__ logits, int* __restrict__ out,
                                                         int vocab, float temperature, int top_k, uint64_t seed,
                                                         const int* __restrict__ requests, int step) {
  __shared__ float red[WARPS];
  __shared__ unsigned int hist[256];
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining;
  __shared__ float seg_sum[WARPS];
  __shared__ float s_max;
  const float* x = logits + (size_t)blockIdx.x * vocab;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // 1. the largest logit
  float mx = -INFINITY;
  for (int i = tid; i < vocab; i += THREADS) mx = fmaxf(mx, x[i]);
  mx = warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  if (warp == 0) {
    float t = warp_max(red[lane]);
    if (lane == 0) s_max = t;
  }
  __syncthreads();
  mx = s_max;

  // 2. the k-th largest logit by radix selection over the ordered keys, 8 bits a pass
  uint32_t kth_key = 0;
  if (top_k > 0 && top_k < vocab) {
    if (tid == 0) { s_prefix = 0; s_remaining = top_k; }
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      if (tid < 256) hist[tid] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const uint32_t high_mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      for (int i = tid; i < vocab; i += THREADS) {
        const uint32_t key = order_key(x[i]);
        if ((key & high_mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xff], 1u);
      }
      __syncthreads();
      if (tid == 0) {
        int remaining = s_remaining;
        int bin = 255;
        for (; bin > 0; --bin) {
          if ((int)hist[bin] >= remaining) break;
          remaining -= (int)hist[bin];
        }
        s_prefix = prefix | ((uint32_t)bin << shift);
        s_remaining = remaining;
      }
      __syncthreads();
    }
    kth_key = s_prefix;
  }

  // 3. each warp owns a contiguous segment; its sum is taken in the order of the later walk
  const int seg = ((vocab + WARPS - 1) / WARPS + 31) / 32 * 32;
  const int begin = warp * seg, end = min(vocab, begin + seg);
  const float inv_t = 1.0f / temperature;
  float running = 0.f;
  for (int base = begin; base < end; base += 32) {
    const int i = base + lane;
    float p = 0.f;
    if (i < end) {
      const float v = x[i];
      if (order_key(v) >= kth_key && v != -INFINITY) p = expf((v - mx) * inv_t);
    }
    running += __shfl_sync(0xffffffffu, warp_inclusive_scan(p, lane), 31);
  }
  if (lane == 0) seg_sum[warp] = running;
  __syncthreads();

  // 4. inverse CDF: the first index whose running sum exceeds u * total
  if (warp == 0) {
    const float mine = seg_sum[lane];
    const float incl = warp_inclusive_scan(mine, lane);
    const float total = __shfl_sync(0xffffffffu, incl, 31);
    const float u = uniform01(seed, (uint64_t)(uint32_t)requests[blockIdx.x], (uint64_t)(uint32_t)step);
    const float target = u * total;
    // the first segment whose inclusive sum exceeds the target (the last non-empty one if rounding leaves none)
    const unsigned ballot = __ballot_sync(0xffffffffu, incl > target && mine > 0.f);
    int w = ballot ? __ffs(ballot) - 1 : -1;
    if (w < 0) {
      const unsigned nonempty = __ballot_sync(0xffffffffu, mine > 0.f);
      w = nonempty ? 31 - __clz(nonempty) : 0;
    }
    float base_sum = __shfl_sync(0xffffffffu, incl - mine, w);
    const int b = w * seg, e = min(vocab, b + seg);
    int chosen = -1, last_kept = -1;
    for (int base = b; base < e && chosen < 0; base += 32) {
      const int i = base + lane;
      float p = 0.f;
      if (i < e) {
        const float v = x[i];
        if (order_key(v) >= kth_key && v != -INFINITY) p = expf((v - mx) * inv_t);
      }
      const float cum = base_sum + warp_inclusive_scan(p, lane);
      const unsigned hit = __ballot_sync(0xffffffffu, p > 0.f && cum > target);
      const unsigned kept = __ballot_sync(0xffffffffu, p > 0.f);
      if (kept) last_kept = base + 31 - __clz(kept);
      if (hit) chosen = base + __ffs(hit) - 1;
      base_sum = __shfl_sync(0xffffffffu, cum, 31);
    }
    if (chosen < 0) chosen = last_kept >= 0 ? last_kept : 0;
    if (lane == 0 && FMS_IN(chosen, vocab)) out[blockIdx.x] = chosen;
  }
}
}  // namespace

FMS_API int fms_argmax(const float* logits, int* out, int rows, int vocab, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return fms_fail("argmax: vocab %d", vocab);
  fms_launch(argmax_kernel, dim3(rows), dim3(THREADS), 0, stream, logits, out, vocab);
  return fms_launch_status("argmax");
}

FMS_API int fms_sample(const float* logits, int* out, int rows, int vocab, float temperature, int top_k,
                       unsigned long long seed, const int* requests, int step, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return fms_fail("sample: vocab %d", vocab);
  if (!(temperature > 0.f)) return fms_fail("sample: temperature %g must be positive", (double)temperature);
  if (top_k < 0) return fms_fail("sample: top_k %d", top_k);
  sample_kernel<<<rows, THREADS, 0, stream>>>(logits, out, vocab, temperature, top_k, (uint64_t)seed, requests, step);
  return fms_launch_status("sample");
}

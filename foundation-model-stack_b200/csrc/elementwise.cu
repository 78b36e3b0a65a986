// Memory-bound kernels of a decoder step: embedding rows, residual add + RMSNorm in one pass, gated
// activation, and rotary position encoding fused with the write of keys and values into the block cache.
// All arithmetic is float32; inputs and outputs are float32 or bfloat16.
#include "common.cuh"

// ---------------------------------------------------------------------------------------------------
// embedding: out[t, :] = scale * float(table[tokens[t], :])    (reference: fms/models/llama.py:332; scale 1)
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ void embed_load8(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void embed_load8(const __nv_bfloat16* p, float* v) {
  const uint4 t = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    v[2 * k] = __uint_as_float(w[k] << 16);
    v[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
  }
}

template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ table, const int* __restrict__ tokens, float* __restrict__ out,
                                  int dim, int vocab, float scale, int* __restrict__ error_flag) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int tok = tokens[t];
  const bool ok = tok >= 0 && tok < vocab;
  if (!ok && threadIdx.x == 0 && error_flag) atomicExch(error_flag, 1);
  const T* src = table + (size_t)(ok ? tok : 0) * dim;
  float* dst = out + (size_t)t * dim;
  if ((dim & 7) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    // 8 values a thread and step: 16 bytes in for bfloat16 (two loads for float32), two 16-byte stores out
    for (int d = 8 * threadIdx.x; d < dim; d += 8 * blockDim.x) {
      float v[8];
      embed_load8(src + d, v);
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
      if (ok) {
        a = make_float4(scale * v[0], scale * v[1], scale * v[2], scale * v[3]);
        b = make_float4(scale * v[4], scale * v[5], scale * v[6], scale * v[7]);
      }
      *reinterpret_cast<float4*>(dst + d) = a;
      *reinterpret_cast<float4*>(dst + d + 4) = b;
    }
    return;
  }
  for (int d = threadIdx.x; d < dim; d += blockDim.x) dst[d] = ok ? scale * to_f32(src[d]) : 0.f;
}

FMS_API int fms_embed_rows(const void* table, int table_dtype, const int* tokens, float* out, int n_tokens, int dim,
                           int vocab, float scale, int* error_flag, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (dim <= 0 || vocab <= 0) return fms_fail("embed_rows: dim %d, vocab %d", dim, vocab);
  const int threads = dim >= 1024 ? 256 : 128;
  FMS_DISPATCH_DTYPE(table_dtype, T,
                     fms_launch(embed_rows_kernel<T>, dim3(n_tokens), dim3(threads), 0, stream, (const T*)table, tokens,
                                out, dim, vocab, scale, error_flag));
  return fms_launch_status("embed_rows");
}

// ---------------------------------------------------------------------------------------------------
// residual add + RMSNorm                                     (reference: fms/modules/layernorm.py:56-69)
//   x = residual[src] + delta[src]       float32; written back to residual unless rows are gathered
//   out[r] = gain * x * rsqrt(mean(x^2) + eps)
// One thread block per output row; the row is read twice (the second time from cache).
// ---------------------------------------------------------------------------------------------------
template <typename T, typename TG>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const TG* __restrict__ gain, float eps, T* __restrict__ out,
                                   const int* __restrict__ rows, int dim, int residual_rows) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  if (!FMS_IN(src, residual_rows)) return;  // the whole block alike
  float* res = residual + (size_t)src * dim;
  const T* del = delta ? delta + (size_t)src * dim : nullptr;
  float ss = 0.f;
  if (rows == nullptr) {
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
      float x = res[d];
      if (del) {
        x += to_f32(del[d]);
        res[d] = x;
      }
      ss += x * x;
    }
  } else {
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
      float x = res[d] + (del ? to_f32(del[d]) : 0.f);
      ss += x * x;
    }
  }
  const float total = block_sum(ss, scratch);
  const float inv = rsqrtf(total / (float)dim + eps);
  T* o = out + (size_t)r * dim;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    float x = res[d];
    if (rows != nullptr && del) x += to_f32(del[d]);
    o[d] = from_f32<T>(to_f32(gain[d]) * (x * inv));
  }
}

// The same for rows whose width is a multiple of 4 and at most 4 * NCHUNK * blockDim: each thread keeps its
// part of the row in registers, all loads are issued before the first store, nothing is read twice.
__device__ __forceinline__ void load4(const float* p, float* v) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float* v) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
  v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
}
__device__ __forceinline__ void store4(float* p, const float* v) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float* v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<uint32_t*>(&a);
  t.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = t;
}

template <typename T, typename TG, int NCHUNK>
__global__ void add_rmsnorm_regs_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                        const TG* __restrict__ gain, float eps, T* __restrict__ out,
                                        const int* __restrict__ rows, int dim, int residual_rows) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const int nvec = dim >> 2;
  float x[NCHUNK][4], dl[NCHUNK][4], g[NCHUNK][4];
#pragma unroll
  for (int j = 0; j < NCHUNK; ++j) {  // the gain is a weight: it can be read before the kernel before this one is done
    const int c = threadIdx.x + j * blockDim.x;
    if (c < nvec) load4(gain + 4 * c, g[j]);
  }
  pdl_wait();
  const int src = rows ? rows[r] : r;
  if (!FMS_IN(src, residual_rows)) return;  // the whole block alike
  float* res = residual + (size_t)src * dim;
  const T* del = delta ? delta + (size_t)src * dim : nullptr;
#pragma unroll
  for (int j = 0; j < NCHUNK; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    if (c < nvec) {
      load4(res + 4 * c, x[j]);
      if (del) load4(del + 4 * c, dl[j]);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < NCHUNK; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    if (c < nvec) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (del) x[j][e] += dl[j][e];
        ss += x[j][e] * x[j][e];
      }
      if (del && rows == nullptr) store4(res + 4 * c, x[j]);
    }
  }
  const float total = block_sum(ss, scratch);
  const float inv = rsqrtf(total / (float)dim + eps);
  T* o = out + (size_t)r * dim;
#pragma unroll
  for (int j = 0; j < NCHUNK; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    if (c < nvec) {
      float y[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) y[e] = g[j][e] * (x[j][e] * inv);
      store4(o + 4 * c, y);
    }
  }
}

// residual_rows: rows of the residual stream (and of delta), which the entries of `rows` index; used by the
// bounds-checked build only (0: not known)
FMS_API int fms_add_rmsnorm(float* residual, const void* delta, const void* gain, int gain_dtype, float eps, void* out,
                            int dtype, const int* rows, int n_rows, int dim, int residual_rows, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (dim <= 0) return fms_fail("add_rmsnorm: dim %d", dim);
  if (dim % 4 == 0 && dim <= 4 * 4 * 1024) {
    // up to 4 chunks of 4 values per thread; few rows: more threads per row, so that each has one chunk
    const int nvec = dim / 4;
    int threads = 128;
    while (threads < 1024 && threads * (n_rows <= 64 ? 1 : 4) < nvec) threads *= 2;
    const int nchunk = (nvec + threads - 1) / threads;
    FMS_DISPATCH_DTYPE(dtype, T, FMS_DISPATCH_DTYPE(gain_dtype, TG, {
      if (nchunk <= 1)
        fms_launch(add_rmsnorm_regs_kernel<T, TG, 1>, dim3(n_rows), dim3(threads), 0, stream, residual, (const T*)delta,
                   (const TG*)gain, eps, (T*)out, rows, dim, residual_rows);
      else if (nchunk <= 2)
        fms_launch(add_rmsnorm_regs_kernel<T, TG, 2>, dim3(n_rows), dim3(threads), 0, stream, residual, (const T*)delta,
                   (const TG*)gain, eps, (T*)out, rows, dim, residual_rows);
      else
        fms_launch(add_rmsnorm_regs_kernel<T, TG, 4>, dim3(n_rows), dim3(threads), 0, stream, residual, (const T*)delta,
                   (const TG*)gain, eps, (T*)out, rows, dim, residual_rows);
    }));
    return fms_launch_status("add_rmsnorm");
  }
  const int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
  FMS_DISPATCH_DTYPE(dtype, T, FMS_DISPATCH_DTYPE(gain_dtype, TG,
                     fms_launch(add_rmsnorm_kernel<T, TG>, dim3(n_rows), dim3(threads), 0, stream, residual,
                                (const T*)delta, (const TG*)gain, eps, (T*)out, rows, dim, residual_rows)));
  return fms_launch_status("add_rmsnorm");
}

// ---------------------------------------------------------------------------------------------------
// gated activation: out[n, f] = act(gu[n, f]) * gu[n, hidden + f]   (fms/modules/feedforward.py:291-292)
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ float activate(float g, int act) {
  switch (act) {
    case 0: return g / (1.f + expf(-g));                                               // silu
    case 1: return 0.5f * g * (1.f + erff(g * 0.70710678118654752f));                  // gelu
    case 2: return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));  // gelu-tanh
    default: return fmaxf(g, 0.f);                                                     // relu
  }
}

template <typename T>
__global__ void gated_activation_kernel(const T* __restrict__ gu, T* __restrict__ out, int hidden, int act,
                                        size_t total) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t n = i / hidden;
    const int f = (int)(i - n * hidden);
    const float g = to_f32(gu[n * 2 * hidden + f]);
    const float u = to_f32(gu[n * 2 * hidden + hidden + f]);
    out[i] = from_f32<T>(activate(g, act) * u);
  }
}

// bfloat16 rows whose width is a multiple of 8: 8 values (16 bytes) of gate and of up per thread
__global__ void gated_activation_vec_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                            int hidden, int act, int n_rows) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = hidden >> 3;
  const long total = (long)n_rows * per_row;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int n = (int)(i / per_row), f = (int)(i - (long)n * per_row) * 8;
    const uint4 gv = *reinterpret_cast<const uint4*>(gu + (size_t)n * 2 * hidden + f);
    const uint4 uv = *reinterpret_cast<const uint4*>(gu + (size_t)n * 2 * hidden + hidden + f);
    const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
    uint32_t ow[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float g0 = __uint_as_float(gw[k] << 16), g1 = __uint_as_float(gw[k] & 0xffff0000u);
      const float u0 = __uint_as_float(uw[k] << 16), u1 = __uint_as_float(uw[k] & 0xffff0000u);
      __nv_bfloat162 r = __floats2bfloat162_rn(activate(g0, act) * u0, activate(g1, act) * u1);
      ow[k] = *reinterpret_cast<uint32_t*>(&r);
    }
    *reinterpret_cast<uint4*>(out + (size_t)n * hidden + f) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
}

FMS_API int fms_gated_activation(const void* gu, void* out, int dtype, int n_rows, int hidden, int act,
                                 cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (hidden <= 0 || act < 0 || act > 3) return fms_fail("gated_activation: hidden %d, act %d", hidden, act);
  const int threads = 256;
  if (dtype == FMS_BF16 && hidden % 8 == 0) {
    const long total = (long)n_rows * (hidden / 8);
    const int blocks = (int)((total + threads - 1) / threads < 148 * 32 ? (total + threads - 1) / threads : 148 * 32);
    fms_launch(gated_activation_vec_kernel, dim3(blocks), dim3(threads), 0, stream, (const __nv_bfloat16*)gu,
               (__nv_bfloat16*)out, hidden, act, n_rows);
    return fms_launch_status("gated_activation");
  }
  const size_t total = (size_t)n_rows * hidden;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  FMS_DISPATCH_DTYPE(dtype, T,
                     gated_activation_kernel<T><<<blocks, threads, 0, stream>>>((const T*)gu, (T*)out, hidden, act,
                                                                                total));
  return fms_launch_status("gated_activation");
}

// ---------------------------------------------------------------------------------------------------
// rotary encoding + cache write
//   qkv[t] = [q heads | k heads | v heads], each head `head_dim` wide     (fms/modules/attention.py:653-657)
//   q, k: adjacent pairs (2i, 2i+1) rotated by angle = position * inv_freq[i], float32
//                                                                    (fms/modules/positions.py:438-456)
//   positions[t]: the token's place in its sequence's cache; position_ids[t]: the position that the rotation sees
//   (null: the same; they differ for a sequence that does not start at position 0)
//   rotated q -> q_out[t]; rotated k and v -> the cache block of the token's slot and position
// grid (token, head), one thread per pair.
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_store_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, const float* __restrict__ inv_freq,
                                  const int* __restrict__ positions, const int* __restrict__ position_ids,
                                  const int* __restrict__ token_seq,
                                  const int* __restrict__ slots, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                  const int* __restrict__ table, int table_stride, int block_tokens, int nheads,
                                  int kvheads, int head_dim, int write_cache, int* __restrict__ error_flag, int n_seqs,
                                  int table_rows, int pool_blocks) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int head = blockIdx.y;  // 0..nheads-1: q; then k heads; then v heads
  const int i = threadIdx.x;    // pair index
  if (i >= head_dim / 2) return;
  const int pos = positions[t];
  const int width = (nheads + 2 * kvheads) * head_dim;
  const T* src = qkv + (size_t)t * width + (size_t)head * head_dim;
  float x0 = to_f32(src[2 * i]), x1 = to_f32(src[2 * i + 1]);
  const bool is_v = head >= nheads + kvheads;
  if (!is_v && inv_freq != nullptr) {
    const float angle = (float)(position_ids ? position_ids[t] : pos) * inv_freq[i];
    float s, c;
    sincosf(angle, &s, &c);
    const float r0 = c * x0 - s * x1;
    const float r1 = s * x0 + c * x1;
    x0 = r0;
    x1 = r1;
  }
  if (head < nheads) {
    T* dst = q_out + (size_t)t * nheads * head_dim + (size_t)head * head_dim;
    dst[2 * i] = from_f32<T>(x0);
    dst[2 * i + 1] = from_f32<T>(x1);
    return;
  }
  if (!write_cache) return;
  const int seq = token_seq[t];
  if (!FMS_IN(seq, n_seqs)) return;
  const int slot = slots[seq];
  if (!FMS_IN(slot, table_rows) || !FMS_IN(pos / block_tokens, table_stride)) return;
  const int blk = table[(size_t)slot * table_stride + pos / block_tokens];
  if (blk < 0) {
    if (i == 0 && error_flag) atomicExch(error_flag, 2);
    return;
  }
  if (!FMS_IN(blk, pool_blocks)) return;
  const int kvh = is_v ? head - nheads - kvheads : head - nheads;
  T* base = is_v ? v_cache : k_cache;
  T* dst = base + (((size_t)blk * kvheads + kvh) * block_tokens + (pos % block_tokens)) * head_dim;
  dst[2 * i] = from_f32<T>(x0);
  dst[2 * i + 1] = from_f32<T>(x1);
}

// bfloat16, many tokens: one block per token, a thread per 16-byte piece (8 values = 4 pairs) of a head.  The
// angle of a pair is the same for every head of the token: its sine and cosine are taken once, into shared memory.
constexpr int ROPE_VEC_MAX_PAIRS = 1024;  // head_dim / 2 that the table in shared memory holds

__global__ void rope_store_vec_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                                      const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                      const int* __restrict__ position_ids, const int* __restrict__ token_seq,
                                      const int* __restrict__ slots,
                                      __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                      const int* __restrict__ table, int table_stride, int block_tokens, int nheads,
                                      int kvheads, int head_dim, int write_cache, int* __restrict__ error_flag,
                                      int n_seqs, int table_rows, int pool_blocks) {
  extern __shared__ float2 sincos_of_pair[];  // [head_dim / 2]: (sin, cos)
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int pieces = head_dim >> 3;
  const int total = (nheads + 2 * kvheads) * pieces;
  const size_t width = (size_t)(nheads + 2 * kvheads) * head_dim;
  int blk = 0;
  if (write_cache) {
    const int seq = token_seq[t];
    const int slot = FMS_IN(seq, n_seqs) ? slots[seq] : -1;
    if (slot >= 0 && FMS_IN(slot, table_rows) && FMS_IN(pos / block_tokens, table_stride)) {
      blk = table[(size_t)slot * table_stride + pos / block_tokens];
      if (blk < 0 && threadIdx.x == 0 && error_flag) atomicExch(error_flag, 2);
      if (blk >= 0 && !FMS_IN(blk, pool_blocks)) blk = -1;
    } else {
      blk = -1;
    }
  }
  if (inv_freq != nullptr) {
    const float turned_by = (float)(position_ids ? position_ids[t] : pos);
    for (int i = threadIdx.x; i < head_dim / 2; i += blockDim.x) {
      float sn, cs;
      sincosf(turned_by * inv_freq[i], &sn, &cs);
      sincos_of_pair[i] = make_float2(sn, cs);
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int head = i / pieces, piece = i - head * pieces;
    const uint4 v = *reinterpret_cast<const uint4*>(qkv + (size_t)t * width + (size_t)head * head_dim + piece * 8);
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
    const bool is_v = head >= nheads + kvheads;
    if (!is_v && inv_freq != nullptr) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float x0 = __uint_as_float(w[k] << 16), x1 = __uint_as_float(w[k] & 0xffff0000u);
        const float2 sc = sincos_of_pair[piece * 4 + k];
        __nv_bfloat162 r = __floats2bfloat162_rn(sc.y * x0 - sc.x * x1, sc.x * x0 + sc.y * x1);
        w[k] = *reinterpret_cast<uint32_t*>(&r);
      }
    }
    const uint4 o = make_uint4(w[0], w[1], w[2], w[3]);
    if (head < nheads) {
      *reinterpret_cast<uint4*>(q_out + ((size_t)t * nheads + head) * head_dim + piece * 8) = o;
    } else if (write_cache && blk >= 0) {
      const int kvh = is_v ? head - nheads - kvheads : head - nheads;
      __nv_bfloat16* base = is_v ? v_cache : k_cache;
      *reinterpret_cast<uint4*>(base + (((size_t)blk * kvheads + kvh) * block_tokens + (pos % block_tokens)) * head_dim +
                                piece * 8) = o;
    }
  }
}

FMS_API int fms_rope_store(const void* qkv, int dtype, void* q_out, const float* inv_freq, const int* positions,
                           const int* position_ids, const int* token_seq, const int* slots, void* k_cache, void* v_cache, const int* table,
                           int table_stride, int block_tokens, int n_tokens, int nheads, int kvheads, int head_dim,
                           int write_cache, int* error_flag, int n_seqs, int table_rows, int pool_blocks,
                           cudaStream_t stream) {
  // n_seqs, table_rows, pool_blocks: extents of slots, of the table and of the cache, for the bounds-checked build (0: not known)
  if (n_tokens <= 0) return 0;
  if (head_dim <= 0 || head_dim % 2 || head_dim > 2048) return fms_fail("rope_store: head_dim %d", head_dim);
  if (dtype == FMS_BF16 && head_dim % 8 == 0 && n_tokens >= 64 && head_dim / 2 <= ROPE_VEC_MAX_PAIRS) {
    const int total = (nheads + 2 * kvheads) * (head_dim / 8);
    const int threads = total >= 256 ? 256 : ((total + 31) / 32) * 32;
    fms_launch(rope_store_vec_kernel, dim3(n_tokens), dim3(threads), (size_t)(head_dim / 2) * sizeof(float2), stream,
               (const __nv_bfloat16*)qkv,
               (__nv_bfloat16*)q_out, inv_freq, positions, position_ids, token_seq, slots, (__nv_bfloat16*)k_cache,
               (__nv_bfloat16*)v_cache, table, table_stride, block_tokens, nheads, kvheads, head_dim, write_cache,
               error_flag, n_seqs, table_rows, pool_blocks);
    return fms_launch_status("rope_store");
  }
  dim3 grid(n_tokens, nheads + 2 * kvheads);
  const int threads = ((head_dim / 2 + 31) / 32) * 32;
  FMS_DISPATCH_DTYPE(dtype, T,
                     fms_launch(rope_store_kernel<T>, grid, dim3(threads), 0, stream, (const T*)qkv, (T*)q_out, inv_freq,
                                positions, position_ids, token_seq, slots, (T*)k_cache, (T*)v_cache, table, table_stride,
                                block_tokens,
                                nheads, kvheads, head_dim, write_cache, error_flag, n_seqs, table_rows, pool_blocks));
  return fms_launch_status("rope_store");
}

// ---------------------------------------------------------------------------------------------------
// (sin, cos) of every token's rotation angles, once a step for all layers that rotate by the same frequencies:
//   out[t, i] = (sin, cos)(position(t) * inv_freq[i]),  position = position_ids[t] if given, else positions[t]
// the float32 product and sincosf of the rotation kernels themselves, so a kernel that reads the table turns by the
// very angles one that takes them itself would
// ---------------------------------------------------------------------------------------------------
__global__ void rotary_table_kernel(const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                    const int* __restrict__ position_ids, float2* __restrict__ out, int n_tokens, int half) {
  pdl_launch_dependents();
  pdl_wait();
  const long total = (long)n_tokens * half;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int t = (int)(i / half), p = (int)(i - (long)t * half);
    float sn, cs;
    sincosf((float)(position_ids ? position_ids[t] : positions[t]) * inv_freq[p], &sn, &cs);
    out[i] = make_float2(sn, cs);
  }
}

FMS_API int fms_rotary_table(const float* inv_freq, const int* positions, const int* position_ids, void* out, int n_tokens,
                             int half, cudaStream_t stream) {
  if (n_tokens <= 0 || half <= 0) return 0;
  const long total = (long)n_tokens * half;
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  fms_launch(rotary_table_kernel, dim3(blocks), dim3(256), 0, stream, inv_freq, positions, position_ids, (float2*)out,
             n_tokens, half);
  return fms_launch_status("rotary_table");
}

// ---------------------------------------------------------------------------------------------------
// start of a decode step: every sequence's new token sits at its current length, which then grows by one; the
// position its encoding sees is that place plus the offset at which the sequence started (offsets null: none)
// ---------------------------------------------------------------------------------------------------
__global__ void decode_advance_kernel(int* __restrict__ positions, int* __restrict__ lengths,
                                      const int* __restrict__ offsets, int* __restrict__ position_ids,
                                      const int* __restrict__ slots, int spare_slot, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    // a row that only fills the step up to a size with a captured graph sits in the cache's spare slot and stays at
    // its first position, whatever the array held
    const int len = (slots != nullptr && slots[i] == spare_slot) ? 0 : lengths[i];
    positions[i] = len;
    lengths[i] = len + 1;
    if (offsets != nullptr) position_ids[i] = len + offsets[i];
  }
}

// slots, spare_slot: rows whose slot is spare_slot restart at position 0 every step (slots null: no such rows)
FMS_API int fms_decode_advance(int* positions, int* lengths, const int* offsets, int* position_ids, const int* slots,
                               int spare_slot, int n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((offsets == nullptr) != (position_ids == nullptr)) return fms_fail("decode_advance: offsets without position_ids");
  fms_launch(decode_advance_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, positions, lengths, offsets, position_ids,
             slots, spare_slot, n);
  return fms_launch_status("decode_advance");
}

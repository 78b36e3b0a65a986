// Grouped-query causal softmax attention over the block cache, for one head size (HEAD_DIM, given at
// compile time: the library is built once per head size a model needs).  (fms/modules/attention.py:215-294 is
// the formula.)  This file holds the float32 kernels (all arithmetic in float32 on the CUDA cores), the merge of
// decode splits and the entry points; the bfloat16 kernels are in attention_mma.cuh (mma.sync: prefill for any
// head size, decode), attention_tc.cuh (tcgen05: prefill for head sizes 64 and 128) and attention_stream.cuh
// (decode with much to read, head sizes 64 and 128: persistent warps fed by TMA).
//
//   prefill:  any number of new tokens per sequence; the query at position p sees cached positions
//             max(0, p - window + 1)..p.  Keys and values of the new tokens are already in the cache.
//   decode:   one query per sequence; the keys are cut into splits of 256 positions (a fixed size, so
//             that a sequence's arithmetic depends on its own length only), one thread block per
//             (sequence, key/value head, split) or, with much to read, persistent warps that draw such
//             units from a counter; then a second kernel combines the splits.
//
// Cache layout: keys, values [blocks, kv_heads, 64, HEAD_DIM]; table[slot, p / 64] is the block of
// position p.  Rows of a block beyond the sequence's length hold garbage and are never used: masked
// scores are set to -inf by selection and their values are skipped or zeroed, not multiplied by 0.
#include <cuda.h>

#include <algorithm>

#include "common.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<head size>"
#endif
static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 256, "head size: a multiple of 16 up to 256");

namespace {
constexpr int HD = HEAD_DIM;
constexpr int BLK = 64;           // tokens per cache block
constexpr int SPLIT = 256;        // keys per decode split
constexpr int GC = 8;             // query heads of one kv head handled by one decode block
constexpr int TQ = 16;            // query rows per prefill block

template <typename T> struct Vec;  // 16-byte vectors
template <> struct Vec<float> { static constexpr int N = 4; };

template <typename T> __device__ __forceinline__ void load_vec(const T* p, float* out);
template <> __device__ __forceinline__ void load_vec<float>(const float* p, float* out) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}

struct AttnArgs {
  const void* q;        // [tokens, nheads * HD]
  void* out;            // [tokens, nheads * HD]
  const void* keys;     // cache
  const void* values;
  const int* table;
  int table_stride;
  const int* slots;      // [seqs]
  const int* first_row;  // [seqs + 1]
  const int* len_after;  // [seqs]
  int nheads, kvheads;
  float scale;
  int window;
  int table_rows;   // slots the table has rows for, and blocks in the cache: extents that only the bounds-checked
  int pool_blocks;  // build looks at (0: not known)
};

// The cache block that holds key block kb of the sequence in `slot`; negative: none (a block given back behind a
// window, or, in the bounds-checked build, an index outside the table or the cache, which is recorded).
__device__ __forceinline__ int block_of(const AttnArgs& a, int slot, int kb) {
  if (!FMS_IN(slot, a.table_rows) || !FMS_IN(kb, a.table_stride)) return -1;
  const int blk = a.table[(size_t)slot * a.table_stride + kb];
  if (blk >= 0 && !FMS_IN(blk, a.pool_blocks)) return -1;
  return blk;
}

// ---------------------------------------------------------------------------------------------------
// prefill: grid (query tiles, heads), 128 threads; thread (r = tid / 8, c = tid % 8) owns row r of the
// tile, scores of keys c, c+8, ... and output columns c, c+8, ...
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) attn_prefill_kernel(AttnArgs a, const int* __restrict__ tiles) {
  extern __shared__ float smem[];
  float* qs = smem;                        // [TQ][HD + 1]
  float* ks = qs + TQ * (HD + 1);          // [BLK][HD + 1]
  float* vs = ks + BLK * (HD + 1);         // [BLK][HD]
  float* ps = vs + BLK * HD;               // [TQ][BLK + 1]

  const int tid = threadIdx.x, r = tid >> 3, c = tid & 7;
  const int seq = tiles[2 * blockIdx.x], r0 = tiles[2 * blockIdx.x + 1];
  const int head = blockIdx.y;
  const int kvh = head / (a.nheads / a.kvheads);
  const int row_begin = a.first_row[seq];
  const int n_new = a.first_row[seq + 1] - row_begin;
  const int len = a.len_after[seq];
  const int len_before = len - n_new;
  const int slot = a.slots[seq];
  const int rows_here = min(TQ, n_new - r0);
  const T* q = (const T*)a.q;
  const T* kc = (const T*)a.keys;
  const T* vc = (const T*)a.values;

  for (int i = tid; i < TQ * HD; i += 128) {
    const int rr = i / HD, d = i - rr * HD;
    qs[rr * (HD + 1) + d] =
        rr < rows_here ? to_f32(q[(size_t)(row_begin + r0 + rr) * a.nheads * HD + (size_t)head * HD + d]) : 0.f;
  }
  const int p_first = len_before + r0;
  const int p_last = p_first + rows_here - 1;
  const int my_pos = p_first + r;
  const bool row_ok = r < rows_here;
  const int kb_lo = a.window > 0 ? max(0, p_first - a.window + 1) / BLK : 0;
  const int kb_hi = p_last / BLK;

  float m = -INFINITY, l = 0.f;
  float acc[HD / 8];
#pragma unroll
  for (int j = 0; j < HD / 8; ++j) acc[j] = 0.f;

  for (int kb = kb_lo; kb <= kb_hi; ++kb) {
    const int blk = block_of(a, slot, kb);
    if (blk < 0) continue;  // uniform over the block: a block that left the window
    __syncthreads();
    const T* kbase = kc + ((size_t)blk * a.kvheads + kvh) * BLK * HD;
    const T* vbase = vc + ((size_t)blk * a.kvheads + kvh) * BLK * HD;
    constexpr int VN = Vec<T>::N;
    for (int i = tid; i < BLK * HD / VN; i += 128) {
      const int key = (i * VN) / HD, d = (i * VN) - key * HD;
      const bool valid = kb * BLK + key < len;
      float kv[VN], vv[VN];
      if (valid) {
        load_vec<T>(kbase + (size_t)key * HD + d, kv);
        load_vec<T>(vbase + (size_t)key * HD + d, vv);
      }
#pragma unroll
      for (int e = 0; e < VN; ++e) {
        ks[key * (HD + 1) + d + e] = valid ? kv[e] : 0.f;
        vs[key * HD + d + e] = valid ? vv[e] : 0.f;
      }
    }
    __syncthreads();
    float s[8];
    float tile_max = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int key = c + 8 * i;
      const int kpos = kb * BLK + key;
      float dot = 0.f;
      const float* qr = qs + r * (HD + 1);
      const float* kr = ks + key * (HD + 1);
#pragma unroll 8
      for (int d = 0; d < HD; ++d) dot = fmaf(qr[d], kr[d], dot);
      const bool visible = row_ok && kpos <= my_pos && (a.window <= 0 || kpos > my_pos - a.window);
      s[i] = visible ? dot * a.scale : -INFINITY;
      tile_max = fmaxf(tile_max, s[i]);
    }
    tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
    tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
    tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 4));
    const float m_new = fmaxf(m, tile_max);
    const float m_use = m_new == -INFINITY ? 0.f : m_new;
    const float alpha = m == -INFINITY ? 0.f : expf(m - m_use);
    float psum = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float p = s[i] == -INFINITY ? 0.f : expf(s[i] - m_use);
      psum += p;
      ps[r * (BLK + 1) + c + 8 * i] = p;
    }
    psum += __shfl_xor_sync(0xffffffffu, psum, 1);
    psum += __shfl_xor_sync(0xffffffffu, psum, 2);
    psum += __shfl_xor_sync(0xffffffffu, psum, 4);
    l = l * alpha + psum;
    m = m_new;
    __syncwarp();  // the 8 threads of a row are in one warp; ps[r] is read only by them
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) acc[j] *= alpha;
    const float* pr = ps + r * (BLK + 1);
    for (int key = 0; key < BLK; ++key) {
      const float p = pr[key];
      const float* vr = vs + key * HD + c;
#pragma unroll
      for (int j = 0; j < HD / 8; ++j) acc[j] = fmaf(p, vr[8 * j], acc[j]);
    }
  }
  if (row_ok) {
    T* o = (T*)a.out + (size_t)(row_begin + r0 + r) * a.nheads * HD + (size_t)head * HD;
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) o[c + 8 * j] = from_f32<T>(acc[j] * inv);
  }
}

// ---------------------------------------------------------------------------------------------------
// decode: grid (sequences, kv heads * head chunks, splits), 128 threads.  One block handles up to GC
// query heads of one kv head over one split of the keys and writes an unnormalised partial result
// (m, l, o) per head; attn_combine_kernel merges the splits.
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) attn_decode_kernel(AttnArgs a, float* __restrict__ part_o,
                                                          float* __restrict__ part_ml, int n_splits) {
  constexpr int VN = Vec<T>::N;
  constexpr int NCH = HD / VN;        // 16-byte chunks per row
  constexpr int TPR = NCH;            // threads per value row
  constexpr int RP = 128 / TPR;       // value rows in flight
  __shared__ float qs[GC][HD];
  __shared__ float ss[GC][BLK];
  __shared__ float sm[GC], sl[GC], salpha[GC];
  __shared__ float red[RP][GC][HD];

  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  const int seq = blockIdx.x, split = blockIdx.z;
  const int group = a.nheads / a.kvheads;
  const int chunks = (group + GC - 1) / GC;
  const int kvh = blockIdx.y / chunks, chunk = blockIdx.y - kvh * chunks;
  const int g0 = chunk * GC;
  const int ng = min(GC, group - g0);   // heads handled here
  const int len = a.len_after[seq];
  const int pos = len - 1;              // the query's position
  const int kstart = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  const int k_lo = max(kstart, split * SPLIT), k_hi = min(len, (split + 1) * SPLIT);
  if (k_lo >= k_hi) return;
  const int slot = a.slots[seq];
  const int row = a.first_row[seq];
  const T* q = (const T*)a.q + (size_t)row * a.nheads * HD + (size_t)(kvh * group + g0) * HD;
  const T* kc = (const T*)a.keys;
  const T* vc = (const T*)a.values;

  for (int i = tid; i < GC * HD; i += 128) {
    const int g = i / HD, d = i - g * HD;
    qs[g][d] = g < ng ? to_f32(q[(size_t)g * HD + d]) * a.scale : 0.f;
  }
  if (tid < GC) { sm[tid] = -INFINITY; sl[tid] = 0.f; salpha[tid] = 0.f; }
  float acc[GC][VN];
#pragma unroll
  for (int g = 0; g < GC; ++g)
#pragma unroll
    for (int e = 0; e < VN; ++e) acc[g][e] = 0.f;
  __syncthreads();

  const int key_of = tid >> 1, half = tid & 1;     // phase 1: two threads per key
  const int rg = tid / TPR, cv = tid - rg * TPR;   // phase 3: TPR threads per value row
  const int warp = tid >> 5, lane = tid & 31;

  for (int kb = k_lo / BLK; kb * BLK < k_hi; ++kb) {
    const int blk = block_of(a, slot, kb);
    if (blk < 0) continue;  // cannot happen for positions inside the window; skip rather than read
    const T* kbase = kc + ((size_t)blk * a.kvheads + kvh) * BLK * HD;
    const T* vbase = vc + ((size_t)blk * a.kvheads + kvh) * BLK * HD;
    // phase 1: scores
    {
      const int kpos = kb * BLK + key_of;
      const bool valid = kpos >= k_lo && kpos < k_hi;
      float dot[GC];
#pragma unroll
      for (int g = 0; g < GC; ++g) dot[g] = 0.f;
      if (valid) {
        for (int ch = half; ch < NCH; ch += 2) {
          float kx[VN];
          load_vec<T>(kbase + (size_t)key_of * HD + ch * VN, kx);
#pragma unroll
          for (int g = 0; g < GC; ++g)
#pragma unroll
            for (int e = 0; e < VN; ++e) dot[g] = fmaf(kx[e], qs[g][ch * VN + e], dot[g]);
        }
      }
#pragma unroll
      for (int g = 0; g < GC; ++g) {
        const float other = __shfl_xor_sync(0xffffffffu, dot[g], 1);
        if (half == 0) ss[g][key_of] = valid ? dot[g] + other : -INFINITY;
      }
    }
    __syncthreads();
    // phase 2: running softmax per head; warp w takes heads w, w + 4
    for (int g = warp; g < ng; g += 4) {
      const float s0 = ss[g][lane], s1 = ss[g][lane + 32];
      const float tile_max = warp_max(fmaxf(s0, s1));
      const float m_old = sm[g];
      const float m_new = fmaxf(m_old, tile_max);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float p0 = s0 == -INFINITY ? 0.f : expf(s0 - m_use);
      const float p1 = s1 == -INFINITY ? 0.f : expf(s1 - m_use);
      const float psum = warp_sum(p0 + p1);
      ss[g][lane] = p0;
      ss[g][lane + 32] = p1;
      if (lane == 0) {
        const float alpha = m_old == -INFINITY ? 0.f : expf(m_old - m_use);
        salpha[g] = alpha;
        sl[g] = sl[g] * alpha + psum;
        sm[g] = m_new;
      }
    }
    __syncthreads();
    // phase 3: values
    if (rg < RP) {
#pragma unroll
      for (int g = 0; g < GC; ++g) {
        const float alpha = g < ng ? salpha[g] : 0.f;
#pragma unroll
        for (int e = 0; e < VN; ++e) acc[g][e] *= alpha;
      }
      for (int key = rg; key < BLK; key += RP) {
        const int kpos = kb * BLK + key;
        if (kpos < k_lo || kpos >= k_hi) continue;
        float vx[VN];
        load_vec<T>(vbase + (size_t)key * HD + cv * VN, vx);
#pragma unroll
        for (int g = 0; g < GC; ++g) {
          const float p = ss[g][key];
#pragma unroll
          for (int e = 0; e < VN; ++e) acc[g][e] = fmaf(p, vx[e], acc[g][e]);
        }
      }
    }
    __syncthreads();
  }
  // sum the row groups in a fixed order and write the partial result
  if (rg < RP) {
#pragma unroll
    for (int g = 0; g < GC; ++g)
#pragma unroll
      for (int e = 0; e < VN; ++e) red[rg][g][cv * VN + e] = acc[g][e];
  }
  __syncthreads();
  for (int i = tid; i < ng * HD; i += 128) {
    const int g = i / HD, d = i - g * HD;
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < RP; ++k) sum += red[k][g][d];
    const int head = kvh * group + g0 + g;
    const size_t at = ((size_t)seq * a.nheads + head) * n_splits + split;
    if (FMS_IN(at, (size_t)gridDim.x * a.nheads * n_splits)) part_o[at * HD + d] = sum;
  }
  if (tid < ng) {
    const int head = kvh * group + g0 + tid;
    const size_t at = ((size_t)seq * a.nheads + head) * n_splits + split;
    if (FMS_IN(at, (size_t)gridDim.x * a.nheads * n_splits)) {
      part_ml[at * 2] = sm[tid];
      part_ml[at * 2 + 1] = sl[tid];
    }
  }
}

// One block per (sequence, head), one thread per value of the head.  Everything the block reads is asked for at
// once, before anything is known: the length, the (maximum, sum) pairs of all splits the launch is sized for, and
// the partial outputs of the first COMBINE_EARLY splits.  What belongs to splits without keys was never written
// and is never used (selected away, not multiplied by zero).  So the kernel costs one trip to memory, not three in
// a row (length, then pairs, then outputs).  The sums run over the live splits in ascending order.
constexpr int COMBINE_EARLY = 8, COMBINE_MAX_SPLITS = 128;

template <typename T>
__global__ void attn_combine_kernel(AttnArgs a, const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    int n_splits, int* __restrict__ reset = nullptr, int* __restrict__ error_flag = nullptr) {
  __shared__ float2 sml[COMBINE_MAX_SPLITS];
  pdl_launch_dependents();
  pdl_wait();
  // the kernel before this one is done: its work counter (if it has one) is put back for the next launch
  if (reset != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *reset = 0;
  const int seq = blockIdx.x, head = blockIdx.y, d = threadIdx.x;
  const float* ml = part_ml + ((size_t)seq * a.nheads + head) * n_splits * 2;
  const float* po = part_o + ((size_t)seq * a.nheads + head) * n_splits * HD;
  const bool staged = n_splits <= COMBINE_MAX_SPLITS;
  const int len = a.len_after[seq];
  const int row0 = a.first_row[seq];
  float2 mine = make_float2(0.f, 0.f);
  if (staged)
    for (int i = d; i < n_splits; i += HD) {
      mine = reinterpret_cast<const float2*>(ml)[i];
      sml[i] = mine;
    }
  float early[COMBINE_EARLY];
#pragma unroll
  for (int i = 0; i < COMBINE_EARLY; ++i) early[i] = i < n_splits ? po[(size_t)i * HD + d] : 0.f;
  const int pos = len - 1;
  const int kstart = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  int s_lo = kstart / SPLIT, s_hi = pos / SPLIT;
  if (s_hi >= n_splits) {
    // a sequence longer than the launch's splits cover (the caller's n_splits is too small): nothing beyond the
    // scratch is read, the keys past the last split are left out, and the flag says so where there is one
    if (error_flag != nullptr && threadIdx.x == 0) atomicExch(error_flag, 8);
    s_hi = n_splits - 1;
    s_lo = min(s_lo, s_hi);
  }
  __syncthreads();
  auto pair_of = [&](int s) { return staged ? sml[s] : make_float2(ml[2 * s], ml[2 * s + 1]); };
  float m = -INFINITY;
  for (int s = s_lo; s <= s_hi; ++s) m = fmaxf(m, pair_of(s).x);
  float total = 0.f;
  for (int s = s_lo; s <= s_hi; ++s) total += pair_of(s).y * expf(pair_of(s).x - m);
  const float inv = total > 0.f ? 1.f / total : 0.f;
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < COMBINE_EARLY; ++i)
    if (i >= s_lo && i <= s_hi) sum += early[i] * expf(pair_of(i).x - m);
  for (int s = max(s_lo, COMBINE_EARLY); s <= s_hi; ++s) sum += po[(size_t)s * HD + d] * expf(pair_of(s).x - m);
  T* o = (T*)a.out + (size_t)row0 * a.nheads * HD + (size_t)head * HD;
  o[d] = from_f32<T>(sum * inv);
}

#include "attention_mma.cuh"

#if HEAD_DIM == 64 || HEAD_DIM == 128
#define FMS_ATTENTION_TC 1
#include "attention_tc.cuh"
#include "attention_stream.cuh"
#else
#define FMS_ATTENTION_TC 0
#endif

#if FMS_ATTENTION_TC
// whether bfloat16 prefill takes the tcgen05 kernel (head sizes 64 and 128; FMS_B200_ATTN_TC=0 turns it off)
static bool prefill_on_tcgen05() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("FMS_B200_ATTN_TC");
    on = (FMS_ATTENTION_TC && !(e && e[0] == '0')) ? 1 : 0;
  }
  return on == 1;
}
#endif

int check_args(const char* what, int nheads, int kvheads, int head_dim, int block_tokens) {
  if (head_dim != HD) return fms_fail("%s: this library is built for head size %d, not %d", what, HD, head_dim);
  if (block_tokens != BLK) return fms_fail("%s: cache blocks of %d tokens, %d expected", what, block_tokens, BLK);
  if (nheads <= 0 || kvheads <= 0 || nheads % kvheads) return fms_fail("%s: %d heads over %d kv heads", what, nheads, kvheads);
  return 0;
}

// Launches the decode kernels (splits, then combine) with the given scratch.  float32: CUDA-core kernel;
// bfloat16: tensor-core kernel.  Both entry points below go through here.
long g_stream_launches = 0;  // launches (or captures) of the streaming decode kernel by this process, for tests
#if FMS_ATTENTION_TC
constexpr long STREAM_FROM_BLOCKS = 1800;  // cache blocks of 64 keys (times kv heads) from which decode streams
// whether decode steps with much to read take the streaming kernel (FMS_B200_ATTN_STREAM=0 turns it off)
bool decode_streams() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("FMS_B200_ATTN_STREAM");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}
int multiprocessors() {
  static int n = 0;
  if (n == 0) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0)
      n = 148;
  }
  return n;
}
#endif

// (sequence, kv head) pairs up to which decode attention takes pieces of 32 keys on 8 warps a split
// (FMS_B200_ATTN_PIECES: another number; 0: never).  Measured in the decode step of the 8B sizes (8 kv heads,
// contexts of 128 to 2,048), 8 warps against 4: one sequence 3.145 against 3.229 ms, two 3.262 / 3.355, four 3.296 /
// 3.425, six 3.340 / 3.415, eight 3.591 / 3.500: with 64 pairs the blocks of 256 threads no longer all fit at once.
static int decode_pieces_up_to() {
  static int n = -1;
  if (n < 0) {
    const char* e = getenv("FMS_B200_ATTN_PIECES");
    n = e ? atoi(e) : 48;
  }
  return n;
}

int launch_decode(const char* what, const AttnArgs& a, int dtype, int n_seqs, int n_splits, float* part_o,
                  float* part_ml, int pool_blocks, long total_len, int* work_counter, int* error_flag, cudaStream_t stream) {
  if (n_splits <= 0 || n_splits > 65535) return fms_fail("%s: %d splits", what, n_splits);
  const int group = a.nheads / a.kvheads;
  if (a.nheads > 65535) return fms_fail("%s: %d heads", what, a.nheads);
  if (dtype == FMS_F32) {
    const int chunks = (group + GC - 1) / GC;
    fms_launch(attn_decode_kernel<float>, dim3(n_seqs, a.kvheads * chunks, n_splits), dim3(128), 0, stream, a, part_o,
               part_ml, n_splits);
    fms_launch(attn_combine_kernel<float>, dim3(n_seqs, a.nheads), dim3(HD), 0, stream, a,
               (const float*)part_o, (const float*)part_ml, n_splits, (int*)nullptr, error_flag);
  } else if (dtype == FMS_BF16) {
    // Few (sequence, kv head) pairs: four warps share a split, each with one block of 64 keys in flight, which
    // is quickest when the GPU is not full.  Many: one warp per block with a small footprint, so that several
    // blocks of threads fit on a multiprocessor and one's loads overlap another's arithmetic.
    const int chunks = (group + GROWS - 1) / GROWS;
    const long units = (long)n_seqs * a.kvheads * chunks;
#if FMS_ATTENTION_TC
    // Much to read (measured: from about 60 MB of keys and values on, whatever the batch): bytes decide, and
    // persistent warps that keep their requests in flight across the units stream them quickest.  Below that a
    // block of threads per unit, with its early hints, has the shorter chain.
    const long key_blocks = (long)(total_len / BLK) * a.kvheads * chunks;  // what the launch will read, in cache blocks
    if (key_blocks >= STREAM_FROM_BLOCKS && n_splits > 1 && pool_blocks > 0 && work_counter != nullptr && error_flag != nullptr &&
        units * n_splits < 0x40000000L && decode_streams()) {
      CUtensorMap map_k, map_v;
      const long rows = (long)pool_blocks * a.kvheads * BLK;
      if (make_map(&map_k, a.keys, rows, HD, BLK) || make_map(&map_v, a.values, rows, HD, BLK)) return 1;
      static bool configured_stream = false;
      if (!configured_stream) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SR_SMEM);
        if (e != cudaSuccess) return fms_fail("%s: %zu bytes of shared memory refused: %s", what, SR_SMEM, cudaGetErrorString(e));
        configured_stream = true;
      }
      const long all_units = units * n_splits;
      const int blocks = (int)std::min<long>(multiprocessors(), (all_units + SR_WARPS - 1) / SR_WARPS);
      ++g_stream_launches;
      fms_launch(attn_decode_stream_kernel, dim3(blocks), dim3((SR_WARPS + 1) * 32), SR_SMEM, stream, map_k, map_v, a,
                 part_o, part_ml, n_seqs, n_splits, work_counter, error_flag);
      fms_launch(attn_combine_kernel<__nv_bfloat16>, dim3(n_seqs, a.nheads), dim3(HD), 0, stream, a,
                 (const float*)part_o, (const float*)part_ml, n_splits, work_counter, error_flag);
      return fms_launch_status(what);
    }
#endif
    // Very few (up to six sequences of 8 kv heads): eight warps share a split, each with one piece of 32 keys: the
    // shortest chain a block can have, while all blocks still fit on the GPU at once.
    const int nw = units >= 512 ? 1 : (units >= 192 ? 2 : (units <= decode_pieces_up_to() ? 8 : 4));
    const int wk = nw == 8 ? 32 : BLK;
    const size_t smem = (size_t)nw * wk * ROWB;
    auto kernel = nw == 1 ? attn_decode_mma_kernel<1, BLK>
                          : (nw == 2 ? attn_decode_mma_kernel<2, BLK>
                                     : (nw == 4 ? attn_decode_mma_kernel<4, BLK> : attn_decode_mma_kernel<8, 32>));
    static bool configured[4] = {false, false, false, false};
    const int slot = nw == 1 ? 0 : (nw == 2 ? 1 : (nw == 4 ? 2 : 3));
    if (!configured[slot]) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return fms_fail("%s: %zu bytes of shared memory refused: %s", what, smem, cudaGetErrorString(e));
      configured[slot] = true;
    }
    // the early L2 hints pay only while the GPU is not full of key and value traffic anyway
    fms_launch(kernel, dim3(n_seqs, a.kvheads * chunks, n_splits), dim3(nw * 32), smem, stream, a, part_o, part_ml,
               n_splits, nw >= 4 ? pool_blocks : 0);
    if (n_splits > 1)  // with one split the kernel above has written the result itself
      fms_launch(attn_combine_kernel<__nv_bfloat16>, dim3(n_seqs, a.nheads), dim3(HD), 0, stream, a,
                 (const float*)part_o, (const float*)part_ml, n_splits, (int*)nullptr, error_flag);
  } else {
    return fms_fail("%s: unsupported dtype code %d", what, dtype);
  }
  return fms_launch_status(what);
}
}  // namespace

FMS_API int fms_attn_head_dim() { return HD; }
FMS_API long fms_attn_stream_launches() { return g_stream_launches; }
FMS_API int fms_attn_split_tokens() { return SPLIT; }
// Positions of one sequence that a prefill block takes (the host cuts the new tokens into such tiles).
FMS_API int fms_attn_prefill_tile_positions(int dtype, int nheads, int kvheads) {
  if (dtype == FMS_BF16 && kvheads > 0 && nheads % kvheads == 0) {
#if FMS_ATTENTION_TC
    if (prefill_on_tcgen05()) return tc_positions_per_block(nheads / kvheads);
#endif
    return prefill_positions_per_block(nheads / kvheads);
  }
  return TQ;
}

FMS_API int fms_attention_prefill(const void* q, void* out, int dtype, const void* keys, const void* values,
                                  const int* table, int table_stride, int block_tokens, const int* slots,
                                  const int* first_row, const int* len_after, const int* tiles, int n_tiles,
                                  int nheads, int kvheads, int head_dim, float scale, int window, int pool_blocks,
                                  int table_rows, int* error_flag, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (check_args("attention_prefill", nheads, kvheads, head_dim, block_tokens)) return 1;
  AttnArgs a{q, out, keys, values, table, table_stride, slots, first_row, len_after, nheads, kvheads, scale, window,
             table_rows, pool_blocks};
  if (nheads > 65535) return fms_fail("attention_prefill: %d heads", nheads);
  if (!(scale > 0.f)) return fms_fail("attention_prefill: the scale of the scores is %g; it must be positive", (double)scale);
#if FMS_ATTENTION_TC
  if (dtype == FMS_BF16 && prefill_on_tcgen05()) {
    // the cache as a matrix [blocks * kv heads * 64 positions, head size], loaded in boxes of 64 x 64
    CUtensorMap map_k, map_v;
    const long rows = (long)pool_blocks * kvheads * BLK;
    if (make_map(&map_k, keys, rows, HD, BLK) || make_map(&map_v, values, rows, HD, BLK)) return 1;
    static bool configured_tc = false;
    if (!configured_tc) {
      cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM);
      if (e != cudaSuccess) return fms_fail("attention_prefill: shared memory of %zu bytes refused: %s", TC_SMEM, cudaGetErrorString(e));
      configured_tc = true;
    }
    const int group = nheads / kvheads;
    const int gh = tc_heads_per_block(group);
    const long blocks = (long)n_tiles * kvheads * ((group + gh - 1) / gh);
    if (blocks > 0x7fffffffL) return fms_fail("attention_prefill: %ld thread blocks", blocks);
    fms_launch(attn_prefill_tc_kernel, dim3((unsigned)blocks), dim3(192), TC_SMEM, stream, map_k, map_v, a, tiles, n_tiles,
               error_flag);
    return fms_launch_status("attention_prefill");
  }
#endif
  if (dtype == FMS_BF16) {
    constexpr size_t smem = (size_t)2 * 2 * BLK * ROWB;
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(attn_prefill_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return fms_fail("attention_prefill: shared memory of %zu bytes refused: %s", smem, cudaGetErrorString(e));
      configured = true;
    }
    const int group = nheads / kvheads;
    const int gh = prefill_heads_per_block(group);
    fms_launch(attn_prefill_mma_kernel, dim3(n_tiles, kvheads * ((group + gh - 1) / gh)), dim3(PF_WARPS * 32), smem,
               stream, a, tiles);
    return fms_launch_status("attention_prefill");
  }
  if (dtype != FMS_F32) return fms_fail("attention_prefill: unsupported dtype code %d", dtype);
  const size_t smem = (size_t)(TQ * (HD + 1) + BLK * (HD + 1) + BLK * HD + TQ * (BLK + 1)) * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fms_fail("attention_prefill: shared memory of %zu bytes refused: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  attn_prefill_kernel<float><<<dim3(n_tiles, nheads), 128, smem, stream>>>(a, tiles);
  return fms_launch_status("attention_prefill");
}

// part_o: float [seqs, nheads, n_splits, HD]; part_ml: float [seqs, nheads, n_splits, 2]; both scratch.
// pool_blocks: blocks in the cache (bounds the early L2 hints and the streaming kernel's tensor maps; 0 turns both
// off).  table_rows: slots the table has rows for (looked at by the bounds-checked build only; 0: not known).  total_len: cached tokens of all sequences together as far as the host knows (0: unknown), by which the
// kernel is chosen.  work_counter: one int that is 0 between launches, from which the streaming kernel's warps draw their
// units; error_flag: where a kernel records that a wait ran out (either null: the streaming kernel is not used).
// n_splits * 256 must cover every len_after (they live on the device, so the host cannot check it): a longer sequence
// loses its keys beyond that, sets error flag 8 where there is a flag, and reads nothing outside the scratch.
FMS_API int fms_attention_decode(const void* q, void* out, int dtype, const void* keys, const void* values,
                                 const int* table, int table_stride, int block_tokens, const int* slots,
                                 const int* first_row, const int* len_after, int n_seqs, int n_splits, float* part_o,
                                 float* part_ml, int nheads, int kvheads, int head_dim, float scale, int window,
                                 int pool_blocks, int table_rows, long total_len, int* work_counter, int* error_flag,
                                 cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (check_args("attention_decode", nheads, kvheads, head_dim, block_tokens)) return 1;
  if (!(scale > 0.f)) return fms_fail("attention_decode: the scale of the scores is %g; it must be positive", (double)scale);
  AttnArgs a{q, out, keys, values, table, table_stride, slots, first_row, len_after, nheads, kvheads, scale, window,
             table_rows, pool_blocks};
  return launch_decode("attention_decode", a, dtype, n_seqs, n_splits, part_o, part_ml, pool_blocks, total_len, work_counter, error_flag, stream);
}

// ---------------------------------------------------------------------------------------------------
// The same decode attention for callers that cannot allocate: scratch inside the library image.
// Declaration, limit and rules of use: attention_no_alloc.h.
// ---------------------------------------------------------------------------------------------------
#include "attention_no_alloc.h"

#include <mutex>

namespace {
static __device__ __align__(256) unsigned char g_decode_scratch[FMS_NO_ALLOC_SCRATCH_BYTES];
constexpr int MAX_DEVICES = 64;
float* g_scratch_address[MAX_DEVICES] = {};  // per device, filled by the first call on that device
std::mutex g_scratch_mutex;

// The device address of g_decode_scratch on the current device; nullptr with fms_last_error() set.
float* scratch_on_current_device() {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= MAX_DEVICES) {
    fms_fail("attention_decode_no_alloc: no usable current device (%s)", cudaGetErrorString(e));
    return nullptr;
  }
  std::lock_guard<std::mutex> guard(g_scratch_mutex);
  if (g_scratch_address[device] == nullptr) {
    void* address = nullptr;
    e = cudaGetSymbolAddress(&address, g_decode_scratch);
    if (e != cudaSuccess || address == nullptr) {
      fms_fail("attention_decode_no_alloc: cudaGetSymbolAddress failed on device %d: %s", device, cudaGetErrorString(e));
      return nullptr;
    }
    g_scratch_address[device] = static_cast<float*>(address);
  }
  return g_scratch_address[device];
}
}  // namespace

FMS_API int fms_attention_decode_no_alloc(const void* q, void* out, int dtype, const void* keys, const void* values,
                                          const int* table, int table_stride, int block_tokens, const int* slots,
                                          const int* first_row, const int* len_after, int n_seqs, int n_splits,
                                          int nheads, int kvheads, int head_dim, float scale, int window,
                                          cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (check_args("attention_decode_no_alloc", nheads, kvheads, head_dim, block_tokens)) return 1;
  if (!(scale > 0.f)) return fms_fail("attention_decode_no_alloc: the scale of the scores is %g; it must be positive", (double)scale);
  if (n_splits <= 0 || n_splits > 65535) return fms_fail("attention_decode_no_alloc: %d splits", n_splits);
  const size_t entries = (size_t)n_seqs * (size_t)nheads * (size_t)n_splits;
  const size_t need = entries * (size_t)(HD + 2) * sizeof(float);
  if (need > (size_t)FMS_NO_ALLOC_SCRATCH_BYTES)
    return fms_fail("attention_decode_no_alloc: %d sequences x %d heads x %d splits need %zu bytes of scratch, the "
                    "built-in array holds %u; use fms_attention_decode with scratch of your own",
                    n_seqs, nheads, n_splits, need, (unsigned)FMS_NO_ALLOC_SCRATCH_BYTES);
  float* scratch = scratch_on_current_device();
  if (scratch == nullptr) return 1;
  float* part_o = scratch;                  // [seqs, nheads, n_splits, HD]
  float* part_ml = scratch + entries * HD;  // [seqs, nheads, n_splits, 2]
  AttnArgs a{q, out, keys, values, table, table_stride, slots, first_row, len_after, nheads, kvheads, scale, window, 0, 0};
  return launch_decode("attention_decode_no_alloc", a, dtype, n_seqs, n_splits, part_o, part_ml, 0, 0, nullptr, nullptr, stream);
}

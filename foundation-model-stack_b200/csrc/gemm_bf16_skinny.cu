// y[M, N] = x[M, K] . w[N, K]^T (+ bias) for few rows (M <= 8): the products of a decode step, which read
// every weight once and are bound by memory bandwidth.  bfloat16 operands, float32 accumulation on the
// tensor cores (mma.sync m16n8k16: 16 weight rows x 8 batch rows per instruction), float32 or bfloat16 out.
//
// Work split: a block of 8 warps owns RT tiles of weight rows; the warps share the K dimension in interleaved
// chunks of 32 and their partial sums are added in shared memory in a fixed order, so the result does not
// depend on timing nor on M.  A lane copies 16 contiguous bytes (8 values) of a weight row and of an x row per
// chunk with cp.async into a ring in shared memory that only it reads back, several chunks ahead of use; the
// two mma of a chunk use these values in the order in which they lie in memory, which is a permutation of the
// instruction's k index that is the same for both operands and so leaves the sum as it is.
//
// A tile's two halves (mma rows 0-7 and 8-15) are
//   ROWS16: weight rows r..r+7 and r+8..r+15;
//   QKV_ROPE: as ROWS16 for the fused [q; k; v] projection of an attention layer; the epilogue rotates the pairs
//           (2i, 2i+1) of the q and k heads by the token's position (float32 angles, fms/modules/positions.py:438-456),
//           writes q to its own buffer and k and v into the token's place in the block cache, so that neither the
//           [M, N] product nor a second kernel is needed;
//   GLU8:   rows r..r+7 of the gate and of the up matrix of a fused [gate; up] weight; the epilogue writes
//           act(gate) * up (fms/modules/feedforward.py:291-292) without the [M, 2 hidden] round trip.
//
// The weights of the first ring stages are requested before the kernel waits for the kernel before it
// (programmatic dependent launch): weights do not depend on it, so the stream of weights from memory does
// not stop between the kernels of a step.
#include "common.cuh"

namespace {
constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
enum Mode { ROWS16 = 0, QKV_ROPE = 1, GLU8 = 2 };

// What the QKV_ROPE epilogue needs beyond the product (unused by the other modes).
struct RopeArgs {
  __nv_bfloat16* q_out;        // [M, nheads * head_dim]
  const float* inv_freq;       // [head_dim / 2], or null: nothing is rotated
  const int* positions;        // [M] each token's place in its sequence's cache
  const int* position_ids;     // [M] the position the rotation sees, or null: the same
  const int* token_seq;        // [M] index into slots
  const int* slots;
  __nv_bfloat16* k_cache;      // [blocks, kvheads, block_tokens, head_dim]
  __nv_bfloat16* v_cache;
  const int* table;            // [slots, table_stride]
  int table_stride, block_tokens, nheads, kvheads, head_dim, write_cache;
  int* error_flag;
  int n_seqs, table_rows, pool_blocks;  // extents of slots, of the table and of the cache, for the bounds-checked build
};

__device__ __forceinline__ void mma_bf16(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 16 bytes global -> shared without passing through registers; `valid` false writes zeros instead.
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid, bool keep_in_l1) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  if (keep_in_l1)
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
  else
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ float activate(float g, int act) {
  switch (act) {
    case 0: return g / (1.f + expf(-g));
    case 1: return 0.5f * g * (1.f + erff(g * 0.70710678118654752f));
    case 2: return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    default: return fmaxf(g, 0.f);
  }
}

// NT: tiles of 8 batch rows (M <= 8 NT).  RT: tiles per block.  D: ring stages.
template <int NT, int RT, int MODE, int D, typename TOut>
__global__ void __launch_bounds__(THREADS) linear_skinny_kernel(const __nv_bfloat16* __restrict__ x,
                                                                const __nv_bfloat16* __restrict__ w,
                                                                const __nv_bfloat16* __restrict__ bias,
                                                                TOut* __restrict__ y, int M, int N, int K, int hidden,
                                                                int act, RopeArgs rope) {
  constexpr int HALVES = 2;                           // weight rows a lane reads per tile
  constexpr int TILE_ROWS = MODE == GLU8 ? 8 : 16;    // output rows (or gate/up pairs) per tile
  constexpr int WL = RT * HALVES;                     // weight pieces per stage
  constexpr int LOADS = WL + NT;
  __shared__ float red[WARPS][RT][NT][32][4];
  extern __shared__ uint4 ring[];
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int n_rows = MODE == GLU8 ? 2 * hidden : N;  // rows of w

  const __nv_bfloat16* wp[RT][2];
#pragma unroll
  for (int t = 0; t < RT; ++t) {
    const int r0 = (blockIdx.x * RT + t) * TILE_ROWS + g;
    wp[t][0] = w + (size_t)min(r0, n_rows - 1) * K + 8 * c;
    wp[t][1] = w + (size_t)min(MODE == GLU8 ? hidden + r0 : r0 + 8, n_rows - 1) * K + 8 * c;
  }
  const __nv_bfloat16* xp[NT];
  bool xok[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    xok[j] = j * 8 + g < M;
    xp[j] = x + (size_t)(xok[j] ? j * 8 + g : 0) * K + 8 * c;
  }
  float acc[RT][NT][4];
#pragma unroll
  for (int t = 0; t < RT; ++t)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[t][j][e] = 0.f;

  // Each thread streams its own 16-byte pieces through a private ring of D stages in shared memory: a stage
  // holds, for one chunk of 32 k, the thread's WL pieces of weight rows and NT pieces of x rows.  A thread
  // reads back only what it copied itself, so no barrier is needed.
  const int chunks = (K + 31) / 32;
  const int my_chunks = chunks > warp ? (chunks - warp + WARPS - 1) / WARPS : 0;
  auto issue_w = [&](int i) {
    if (i < my_chunks) {
      const int k0 = (warp + i * WARPS) * 32;
      const bool kok = k0 + 8 * c + 8 <= K;  // K is a multiple of 8: a lane's 8 values are all inside or all outside
      uint4* st = ring + (size_t)(i % D) * LOADS * THREADS + threadIdx.x;
#pragma unroll
      for (int t = 0; t < RT; ++t)
#pragma unroll
        for (int h = 0; h < HALVES; ++h) cp_async16(st + (t * HALVES + h) * THREADS, wp[t][h] + (kok ? k0 : 0), kok, false);
    }
  };
  auto issue_x = [&](int i) {
    if (i < my_chunks) {
      const int k0 = (warp + i * WARPS) * 32;
      const bool kok = k0 + 8 * c + 8 <= K;
      uint4* st = ring + (size_t)(i % D) * LOADS * THREADS + threadIdx.x;
#pragma unroll
      for (int j = 0; j < NT; ++j) cp_async16(st + (WL + j) * THREADS, xp[j] + (kok ? k0 : 0), kok && xok[j], true);
    }
  };
#pragma unroll
  for (int i = 0; i < D; ++i) issue_w(i);  // weights: before the wait for the kernel that produces x
  cp_async_commit();
  pdl_wait();
#pragma unroll
  for (int i = 0; i < D; ++i) issue_x(i);
  cp_async_commit();
  cp_async_wait<0>();
  for (int i = 0; i < my_chunks; ++i) {
    cp_async_wait<D - 1>();
    const uint4* st = ring + (size_t)(i % D) * LOADS * THREADS + threadIdx.x;
    uint4 a[RT][2], b[NT];
#pragma unroll
    for (int t = 0; t < RT; ++t) {
      a[t][0] = st[(t * HALVES) * THREADS];
      a[t][1] = st[(t * HALVES + 1) * THREADS];
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) b[j] = st[(WL + j) * THREADS];
#pragma unroll
    for (int t = 0; t < RT; ++t)
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        mma_bf16(acc[t][j], a[t][0].x, a[t][1].x, a[t][0].y, a[t][1].y, b[j].x, b[j].y);
        mma_bf16(acc[t][j], a[t][0].z, a[t][1].z, a[t][0].w, a[t][1].w, b[j].z, b[j].w);
      }
    issue_w(i + D);  // into the stage just consumed
    issue_x(i + D);
    cp_async_commit();
  }
  cp_async_wait<0>();

#pragma unroll
  for (int t = 0; t < RT; ++t)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) red[warp][t][j][lane][e] = acc[t][j][e];
  __syncthreads();
  // warp w of the first RT * NT warps sums one (tile, batch tile) over the 8 warps, in order
  for (int item = warp; item < RT * NT; item += WARPS) {
    const int t = item / NT, j = item % NT;
    float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ww = 0; ww < WARPS; ++ww)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[e] += red[ww][t][j][lane][e];
#pragma unroll
    for (int e = 0; e < 4; ++e) red[0][t][j][lane][e] = s[e];
  }
  __syncthreads();
  // epilogue: element e of a lane is (mma row g + 8 (e / 2), batch row 2 c + (e % 2)) of its tile
  if (MODE == GLU8) {
    for (int i = threadIdx.x; i < RT * NT * 32 * 2; i += THREADS) {
      const int t = i / (NT * 64), j = (i / 64) % NT, l = (i / 2) % 32, e = i % 2;
      const int row = (blockIdx.x * RT + t) * 8 + (l >> 2);
      const int m = j * 8 + 2 * (l & 3) + e;
      if (row < hidden && m < M) {
        float gate = red[0][t][j][l][e], up = red[0][t][j][l][e + 2];
        if (bias) {
          gate += __bfloat162float(bias[row]);
          up += __bfloat162float(bias[hidden + row]);
        }
        if (FMS_IN((size_t)m * hidden + row, (size_t)M * hidden)) y[(size_t)m * hidden + row] = from_f32<TOut>(activate(gate, act) * up);
      }
    }
  } else if (MODE == QKV_ROPE) {
    // one (tile, pair of rows, token) per step: rows 2p and 2p + 1 of the tile are a pair of one head
    static_assert(MODE != QKV_ROPE || NT == 1, "the fused projection is for up to 8 tokens");
    for (int i = threadIdx.x; i < RT * 8 * 8; i += THREADS) {
      const int t = i / 64, p = (i / 8) % 8, m = i % 8;
      const int r0 = (blockIdx.x * RT + t) * TILE_ROWS + 2 * p;
      if (r0 >= N || m >= M) continue;
      // element (row rr, token m) of the tile lies with lane (rr % 8) * 4 + m / 2 as element (rr / 8) * 2 + m % 2
      float x0 = red[0][t][0][((2 * p) & 7) * 4 + (m >> 1)][((2 * p) >> 3) * 2 + (m & 1)];
      float x1 = red[0][t][0][((2 * p + 1) & 7) * 4 + (m >> 1)][((2 * p + 1) >> 3) * 2 + (m & 1)];
      if (bias) {
        x0 += __bfloat162float(bias[r0]);
        x1 += __bfloat162float(bias[r0 + 1]);
      }
      const int head = r0 / rope.head_dim, d = r0 - head * rope.head_dim;
      const bool is_v = head >= rope.nheads + rope.kvheads;
      const int pos = rope.positions[m];
      if (!is_v && rope.inv_freq != nullptr) {
        float sn, cs;
        sincosf((float)(rope.position_ids ? rope.position_ids[m] : pos) * rope.inv_freq[d >> 1], &sn, &cs);
        const float r = cs * x0 - sn * x1;
        x1 = sn * x0 + cs * x1;
        x0 = r;
      }
      const __nv_bfloat162 out = __floats2bfloat162_rn(x0, x1);
      if (head < rope.nheads) {
        *reinterpret_cast<__nv_bfloat162*>(rope.q_out + ((size_t)m * rope.nheads + head) * rope.head_dim + d) = out;
      } else if (rope.write_cache) {
        const int seq = rope.token_seq[m];
        if (!FMS_IN(seq, rope.n_seqs)) continue;
        const int slot = rope.slots[seq];
        if (!FMS_IN(slot, rope.table_rows) || !FMS_IN(pos / rope.block_tokens, rope.table_stride)) continue;
        const int blk = rope.table[(size_t)slot * rope.table_stride + pos / rope.block_tokens];
        if (blk < 0) {
          if (rope.error_flag) atomicExch(rope.error_flag, 2);
          continue;
        }
        if (!FMS_IN(blk, rope.pool_blocks)) continue;
        const int kvh = is_v ? head - rope.nheads - rope.kvheads : head - rope.nheads;
        __nv_bfloat16* base = is_v ? rope.v_cache : rope.k_cache;
        *reinterpret_cast<__nv_bfloat162*>(
            base + (((size_t)blk * rope.kvheads + kvh) * rope.block_tokens + (pos % rope.block_tokens)) * rope.head_dim + d) = out;
      }
    }
  } else {
    constexpr int EL = 4;
    for (int i = threadIdx.x; i < RT * NT * 32 * EL; i += THREADS) {
      const int t = i / (NT * 32 * EL), j = (i / (32 * EL)) % NT, l = (i / EL) % 32, e = i % EL;
      const int row = (blockIdx.x * RT + t) * TILE_ROWS + (l >> 2) + 8 * (e >> 1);
      const int m = j * 8 + 2 * (l & 3) + (e & 1);
      if (row < N && m < M) {
        float v = red[0][t][j][l][e];
        if (bias) v += __bfloat162float(bias[row]);
        if (FMS_IN((size_t)m * N + row, (size_t)M * N)) y[(size_t)m * N + row] = from_f32<TOut>(v);
      }
    }
  }
}

template <int NT, int RT, int MODE, typename TOut>
int launch_typed(const void* x, const void* w, const void* bias, void* y, int M, int N, int K, int hidden, int act,
                 cudaStream_t stream, const RopeArgs& rope = RopeArgs{}) {
  constexpr int LOADS = RT * 2 + NT;
  constexpr int D = LOADS <= 2 ? 7 : (LOADS == 3 ? 5 : (LOADS == 4 ? 4 : 3));  // 56 to 72 KB of ring per block
  constexpr size_t smem = (size_t)D * LOADS * THREADS * sizeof(uint4);
  auto kernel = linear_skinny_kernel<NT, RT, MODE, D, TOut>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fms_fail("linear_bf16_skinny: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  constexpr int TILE_ROWS = MODE == GLU8 ? 8 : 16;
  const int rows = MODE == GLU8 ? hidden : N;
  const int blocks = (rows + TILE_ROWS * RT - 1) / (TILE_ROWS * RT);
  cudaError_t e = fms_launch(kernel, dim3(blocks), dim3(THREADS), smem, stream, (const __nv_bfloat16*)x,
                             (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, (TOut*)y, M, N, K, hidden, act, rope);
  if (e != cudaSuccess) return fms_fail("linear_bf16_skinny: launch failed: %s", cudaGetErrorString(e));
  return 0;
}

template <int NT, int RT, int MODE>
int launch(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M, int N, int K, int hidden,
           int act, cudaStream_t stream) {
  if (out_dtype == FMS_F32) return launch_typed<NT, RT, MODE, float>(x, w, bias, y, M, N, K, hidden, act, stream);
  return launch_typed<NT, RT, MODE, __nv_bfloat16>(x, w, bias, y, M, N, K, hidden, act, stream);
}
}  // namespace

// More rows than the 8 columns of one mma would make every block read twice as much of x as of w (a block owns 16
// rows of w and all of x); from 9 rows on the caller takes another product.
FMS_API int fms_linear_skinny_max_rows() { return 8; }

// y [M, N] (out_dtype) = x [M, K] w[N, K]^T + bias.  M <= 8, K a multiple of 8, all bfloat16 inputs.
FMS_API int fms_linear_bf16_skinny(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M, int N,
                                   int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 8) return fms_fail("linear_bf16_skinny: %d rows, at most 8", M);
  if (K <= 0 || K % 8) return fms_fail("linear_bf16_skinny: K %d must be a positive multiple of 8", K);
  if (out_dtype != FMS_F32 && out_dtype != FMS_BF16) return fms_fail("linear_bf16_skinny: out dtype %d", out_dtype);
  // very many weight rows: 32 rows a block, which halves the re-reading of x
  if (N < 16384) return launch<1, 1, ROWS16>(x, w, bias, y, out_dtype, M, N, K, 0, 0, stream);
  return launch<1, 2, ROWS16>(x, w, bias, y, out_dtype, M, N, K, 0, 0, stream);
}

// The fused projection of an attention layer for up to 8 tokens: [q | k | v] = x [M, K] w[(nheads + 2 kvheads) head_dim, K]^T
// + bias; q and k rotated by each token's position; q -> q_out [M, nheads head_dim], k and v -> the token's place in
// the block cache (write_cache 0: q only).  A token whose position has no block sets error flag 2 and is skipped.
FMS_API int fms_qkv_rope_store_bf16_skinny(const void* x, const void* w, const void* bias, void* q_out,
                                           const float* inv_freq, const int* positions, const int* position_ids,
                                           const int* token_seq, const int* slots, void* k_cache, void* v_cache, const int* table,
                                           int table_stride, int block_tokens, int M, int K, int nheads, int kvheads,
                                           int head_dim, int write_cache, int* error_flag, int n_seqs, int table_rows,
                                           int pool_blocks, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (M > 8) return fms_fail("qkv_rope_store_bf16_skinny: %d rows, at most 8", M);
  if (K <= 0 || K % 8) return fms_fail("qkv_rope_store_bf16_skinny: K %d must be a positive multiple of 8", K);
  if (nheads <= 0 || kvheads <= 0 || head_dim <= 0 || head_dim % 2 || block_tokens <= 0)
    return fms_fail("qkv_rope_store_bf16_skinny: %d heads, %d kv heads, head size %d, blocks of %d", nheads, kvheads,
                    head_dim, block_tokens);
  const long rows = (long)(nheads + 2 * kvheads) * head_dim;
  if (rows > 0x7fffffffL) return fms_fail("qkv_rope_store_bf16_skinny: %ld rows of w", rows);
  const RopeArgs rope{(__nv_bfloat16*)q_out, inv_freq, positions, position_ids, token_seq, slots, (__nv_bfloat16*)k_cache,
                      (__nv_bfloat16*)v_cache, table, table_stride, block_tokens, nheads, kvheads, head_dim, write_cache,
                      error_flag, n_seqs, table_rows, pool_blocks};
  if (rows < 16384) return launch_typed<1, 1, QKV_ROPE, __nv_bfloat16>(x, w, bias, nullptr, M, (int)rows, K, 0, 0, stream, rope);
  return launch_typed<1, 2, QKV_ROPE, __nv_bfloat16>(x, w, bias, nullptr, M, (int)rows, K, 0, 0, stream, rope);
}

// y [M, hidden] = act(x w_gate^T + b_gate) * (x w_up^T + b_up) with w = [gate; up] of 2 hidden rows.
FMS_API int fms_glu_bf16_skinny(const void* x, const void* w, const void* bias, void* y, int M, int hidden, int K,
                                int act, cudaStream_t stream) {
  if (M <= 0 || hidden <= 0) return 0;
  if (M > 8) return fms_fail("glu_bf16_skinny: %d rows, at most 8", M);
  if (K <= 0 || K % 8) return fms_fail("glu_bf16_skinny: K %d must be a positive multiple of 8", K);
  if (act < 0 || act > 3) return fms_fail("glu_bf16_skinny: activation %d", act);
  return launch<1, 2, GLU8>(x, w, bias, y, FMS_BF16, M, 2 * hidden, K, hidden, act, stream);
}

// y[M, N] = x[M, K] . w[N, K]^T for 9 to 256 rows of x (decode steps of many sequences, short prompts): bfloat16
// operands, float32 accumulation in tensor memory on the tcgen05 tensor cores, with the operands swapped so that
// the WEIGHTS fill the instruction's 128 rows and the tokens are its columns (16 to 256): a step of this size is
// bound by reading w once, and nothing of the instruction is wasted on padding rows.
//
// Of the products of a layer the library hands the gated feed-forward one to this kernel by default (9 to 64 rows),
// where it is ahead of the library's product plus an activation kernel; the others it can take on request.
//
// A thread block owns 128 rows of w (one tile) for a slice of K; the KS blocks that share a tile (KS = 1, 2, 4
// or 8, chosen from the matrix's shape alone so that two blocks a multiprocessor are there to stream) form a thread
// block CLUSTER and add their partial sums through distributed shared memory, in a fixed order, before the epilogue:
// no partial sum goes through global memory and no second kernel is needed.
//
//   warp 0   one lane issues the TMA loads: per step of 64 k a 128 x 64 box of w (GLU: 64 gate rows and the 64 up
//            rows that belong to them) and a [tokens] x 64 box of x, 128-byte swizzle, into one of 3 to 6 stages.  The
//            first stages' boxes of w are asked for BEFORE griddepcontrol.wait: weights do not depend on the kernel
//            before, so they stream in while it drains.
//   warp 1   allocates tensor memory; one lane waits for a stage, issues 4 tcgen05.mma (128 x tokens x 16), commits
//            them to the stage's "empty" barrier, and after the last step to the "accumulator ready" barrier.
//   warps 2-5  read the accumulator (lane = row of w = column of y) and put it into shared memory, over the stages
//            that are no longer needed; after the cluster's barrier each block adds, for its share of the tokens, the
//            partial sums of all blocks (rank 0, 1, ... in this order) and runs the epilogue on them:
//              plain   (+ bias) -> y, bfloat16 or float32
//              GLU     act(gate + bias) * (up + bias) -> y [M, hidden]          (fms/modules/feedforward.py:288-297)
//              QKV     (+ bias), q and k rotated by the token's position (adjacent pairs, float32 angles,
//                      fms/modules/positions.py:438-456), q -> q_out, k and v -> the token's place in the block cache
//
// Every wait on an mbarrier is bounded; on a time-out the block records error 4, skips its work, still meets the
// cluster's barriers and frees its tensor memory.  Rows beyond M, N and K are zeros on the way in (TMA) and are not
// stored.  K must be a multiple of 8 (16-byte row pitch).  The k order of the sums depends on the matrix's shape
// only, never on how many rows of x there are, so a token's result does not depend on the rest of the batch.
#include <cuda.h>

#include "common.cuh"

namespace {
constexpr int TILE_ROWS = 128, TILE_K = 64, UMMA_K = 16, MAX_TOKENS = 256, MAX_STAGES = 12, MAX_KS = 8;
constexpr int W_BYTES = TILE_ROWS * TILE_K * 2;
constexpr int THREADS = 192;

#include "tcgen05.cuh"

__device__ __forceinline__ float activate(float g, int act) {
  switch (act) {
    case 0: return g / (1.f + expf(-g));
    case 1: return 0.5f * g * (1.f + erff(g * 0.70710678118654752f));
    case 2: return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    default: return fmaxf(g, 0.f);
  }
}

enum Mode { PLAIN = 0, GLU = 1, QKV_ROPE = 2 };

struct MidArgs {
  int mode;
  void* out;            // PLAIN: [M, N] bfloat16 or float32; GLU: [M, hidden] bfloat16; QKV_ROPE: q_out [M, nheads * head_dim]
  const void* bias;     // bfloat16 [N] (GLU: [2 hidden]) or null
  int out_f32, hidden, act;
  int n_tokens;         // columns of the instruction: M rounded up to a multiple of 16
  int stages, ks;
  // QKV_ROPE
  const float* inv_freq;      // [head_dim / 2] or null: nothing is rotated
  const int* positions;       // [M] each token's place in its sequence's cache
  const int* position_ids;    // [M] the position the rotation sees, or null: the same
  const int* token_seq;       // [M] index into slots
  const int* slots;
  __nv_bfloat16* k_cache;     // [blocks, kvheads, block_tokens, head_dim]
  __nv_bfloat16* v_cache;
  const int* table;           // [table_rows, table_stride]
  int table_stride, block_tokens, nheads, kvheads, head_dim, write_cache;
  int n_seqs, table_rows, pool_blocks;  // extents, for the bounds-checked build
};

__device__ __forceinline__ float ld_cluster_f32(uint32_t local_addr, uint32_t rank) {
  float v;
  asm volatile("{\n.reg .b32 remote;\nmapa.shared::cluster.u32 remote, %1, %2;\nld.shared::cluster.f32 %0, [remote];\n}\n"
               : "=f"(v)
               : "r"(local_addr), "r"(rank)
               : "memory");
  return v;
}

__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t local_addr, uint32_t rank) {
  float4 v;
  asm volatile(
      "{\n.reg .b32 remote;\nmapa.shared::cluster.u32 remote, %4, %5;\nld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [remote];\n}\n"
      : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
      : "r"(local_addr), "r"(rank)
      : "memory");
  return v;
}

// Grid (ks, tiles); clusters of ks blocks along x.  Block (r, t) takes the k steps [r * per, (r + 1) * per) of tile t.
__global__ void __launch_bounds__(THREADS) gemm_mid_kernel(const __grid_constant__ CUtensorMap map_w,
                                                           const __grid_constant__ CUtensorMap map_x, MidArgs p, int M, int N,
                                                           int K, int* __restrict__ error_flag) {
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
  const int x_bytes = p.n_tokens * TILE_K * 2, stage_bytes = W_BYTES + x_bytes, stages = p.stages;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)stages * stage_bytes);
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* acc_full = empty + MAX_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  __shared__ int failed_flag;
  volatile int* failed = &failed_flag;

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ks = p.ks, rank = ks > 1 ? (int)cluster_rank() : 0;
  const int tile = blockIdx.y;
  const int row_step = p.mode == GLU ? TILE_ROWS / 2 : TILE_ROWS;  // output columns of a tile
  const int n0 = tile * row_step;
  const int k_steps_all = (K + TILE_K - 1) / TILE_K;
  const int per = (k_steps_all + ks - 1) / ks;
  const int step_lo = min(rank * per, k_steps_all), step_hi = min(step_lo + per, k_steps_all);
  const int k_steps = step_hi - step_lo;  // may be 0 for the last ranks of a short K: their partial sum is zero
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < p.n_tokens) tmem_cols *= 2;

  if (threadIdx.x == 0) {
    failed_flag = 0;
    for (int s = 0; s < MAX_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      auto load_w = [&](int i) {  // the tile's rows of w for local step i
        const int s = i % stages;
        unsigned char* a = smem + (size_t)s * stage_bytes;
        mbar_arrive_expect_tx(&full[s], stage_bytes);
        const int kc = (step_lo + i) * TILE_K;
        if (p.mode == GLU) {
          tma_load_2d(a, &map_w, kc, n0, &full[s]);
          tma_load_2d(a + W_BYTES / 2, &map_w, kc, p.hidden + n0, &full[s]);
        } else {
          tma_load_2d(a, &map_w, kc, n0, &full[s]);
        }
      };
      auto load_x = [&](int i) {
        const int s = i % stages;
        tma_load_2d(smem + (size_t)s * stage_bytes + W_BYTES, &map_x, (step_lo + i) * TILE_K, 0, &full[s]);
      };
      const int early = min(stages, k_steps);
      for (int i = 0; i < early; ++i) load_w(i);  // weights: independent of the kernel before
      pdl_wait();                                  // x is what the kernel before wrote
      for (int i = 0; i < early; ++i) load_x(i);
      for (int i = early; i < k_steps && !*failed; ++i) {
        if (!wait_or_abort(&empty[i % stages], ((i / stages) & 1) ^ 1, failed)) break;
        load_w(i);
        load_x(i);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc = umma_idesc(TILE_ROWS, p.n_tokens);
      for (int i = 0; i < k_steps; ++i) {
        const int s = i % stages;
        if (!wait_or_abort(&full[s], (i / stages) & 1, failed)) break;
        tc_fence_after();
        const uint32_t a = smem_u32(smem + (size_t)s * stage_bytes), b = a + W_BYTES;
#pragma unroll
        for (int kk = 0; kk < TILE_K / UMMA_K; ++kk)
          umma(tmem, umma_desc(a + kk * UMMA_K * 2), umma_desc(b + kk * UMMA_K * 2), idesc, i > 0 || kk > 0);
        tc_commit(&empty[s]);
      }
      tc_commit(acc_full);  // arrives when everything issued so far is done (at once if there was nothing)
    }
  }
  // The partial sums of this block as float32 [128 rows][n_tokens + 4] in shared memory, over the stages (every
  // copy into them has landed and every mma that read them is done once the accumulator is ready).  The stride keeps
  // rows 16-byte aligned and lets the lanes of a warp write 16 bytes each without meeting in a bank.
  float* red = reinterpret_cast<float*>(smem);
  const int red_stride = p.n_tokens + 4;
  if (warp >= 2) {
    pdl_wait();  // these warps read and write what other kernels of the step touch (the error flag, y, the cache)
    const int quarter = warp & 3;
    const bool ok = wait_or_abort(acc_full, 0, failed);
    tc_fence_after();
    const int row = quarter * 32 + lane;
    const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16);
    for (int c0 = 0; c0 < p.n_tokens; c0 += 16) {
      float v[16];
      if (ok && k_steps > 0) {
        tmem_load_16(taddr + c0, v);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < 16; j += 4)
        *reinterpret_cast<float4*>(red + row * red_stride + c0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    }
    tc_fence_before();
  }
  __syncthreads();
  if (ks > 1) cluster_sync_all();  // every block's partial sums are in its shared memory

  // ---- the sum over the cluster and the epilogue: this block's share of the tokens (a multiple of 4), all 128 rows;
  // a thread takes four tokens of a row at a time ----
  if (warp >= 2) {
    const int e = threadIdx.x - 64;                       // 0..127
    const int share = ((p.n_tokens + ks - 1) / ks + 3) / 4 * 4;
    const int t_lo = rank * share, t_hi = min(t_lo + share, p.n_tokens);
    const uint32_t red_addr = smem_u32(red);
    auto total4 = [&](int row, int t, float* out) {       // tokens t..t+3 of a row, summed in the fixed order rank 0, 1, ...
      if (ks == 1) {
        const float4 v = *reinterpret_cast<const float4*>(red + row * red_stride + t);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
        return;
      }
      float4 v[MAX_KS];
      const uint32_t at = red_addr + (uint32_t)(row * red_stride + t) * 4u;
#pragma unroll
      for (int r = 0; r < MAX_KS; ++r)  // all loads on their way before the first sum
        if (r < ks) v[r] = ld_cluster_f32x4(at, (uint32_t)r);
      out[0] = out[1] = out[2] = out[3] = 0.f;
#pragma unroll
      for (int r = 0; r < MAX_KS; ++r)
        if (r < ks) {
          out[0] += v[r].x; out[1] += v[r].y; out[2] += v[r].z; out[3] += v[r].w;
        }
    };
    const __nv_bfloat16* bias = (const __nv_bfloat16*)p.bias;
    if (p.mode == GLU) {
      // rows 0..63 of the tile are gate rows n0 + i, rows 64..127 the up rows that belong to them; thread e takes
      // output column e % 64 and every second group of four tokens
      const int i = e & 63, f = n0 + i;
      const float bg = (bias && f < p.hidden) ? __bfloat162float(bias[f]) : 0.f;
      const float bu = (bias && f < p.hidden) ? __bfloat162float(bias[p.hidden + f]) : 0.f;
      __nv_bfloat16* y = (__nv_bfloat16*)p.out;
      for (int t = t_lo + 4 * (e >> 6); t < t_hi; t += 8) {
        float g[4], u[4];
        total4(i, t, g);
        total4(64 + i, t, u);
        if (f < p.hidden) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (t + j < M && FMS_IN((size_t)(t + j) * p.hidden + f, (size_t)M * p.hidden))
              y[(size_t)(t + j) * p.hidden + f] = __float2bfloat16_rn(activate(g[j] + bg, p.act) * (u[j] + bu));
        }
      }
    } else {
      // thread e takes row e of the tile: the lanes of a warp write neighbouring columns of y; the partner of a
      // rotary pair (rows 2 i, 2 i + 1) is the neighbouring lane
      const int n = n0 + e;
      const float b0 = (bias && n < N) ? __bfloat162float(bias[n]) : 0.f;
      const int head = n / max(p.head_dim, 1), d = n - head * max(p.head_dim, 1);
      const bool rope = p.mode == QKV_ROPE;
      const bool is_q = head < p.nheads, is_v = head >= p.nheads + p.kvheads;
      const float freq = (rope && !is_v && p.inv_freq != nullptr && n < N) ? p.inv_freq[d >> 1] : 0.f;
      for (int t = t_lo; t < t_hi; t += 4) {
        float v[4];
        total4(e, t, v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float x = v[j] + b0;
          const int tok = t + j;
          const bool live = tok < M && n < N;
          if (!rope) {
            if (live && FMS_IN((size_t)tok * N + n, (size_t)M * N)) {
              if (p.out_f32) ((float*)p.out)[(size_t)tok * N + n] = x;
              else ((__nv_bfloat16*)p.out)[(size_t)tok * N + n] = __float2bfloat16_rn(x);
            }
            continue;
          }
          const float other = __shfl_xor_sync(0xffffffffu, x, 1);  // every lane takes part, live or not
          if (!live) continue;
          const int pos = p.positions[tok];
          if (!is_v && p.inv_freq != nullptr) {
            float sn, cs;
            sincosf((float)(p.position_ids ? p.position_ids[tok] : pos) * freq, &sn, &cs);
            x = (e & 1) ? sn * other + cs * x : cs * x - sn * other;  // odd row: sin x0 + cos x1; even: cos x0 - sin x1
          }
          const __nv_bfloat16 o = __float2bfloat16_rn(x);
          if (is_q) {
            ((__nv_bfloat16*)p.out)[((size_t)tok * p.nheads + head) * p.head_dim + d] = o;
          } else if (p.write_cache) {
            const int seq = p.token_seq[tok];
            if (!FMS_IN(seq, p.n_seqs)) continue;
            const int slot = p.slots[seq];
            if (!FMS_IN(slot, p.table_rows) || !FMS_IN(pos / p.block_tokens, p.table_stride)) continue;
            const int blk = p.table[(size_t)slot * p.table_stride + pos / p.block_tokens];
            if (blk < 0) {
              if (error_flag) atomicExch(error_flag, 2);
              continue;
            }
            if (!FMS_IN(blk, p.pool_blocks)) continue;
            const int kvh = is_v ? head - p.nheads - p.kvheads : head - p.nheads;
            __nv_bfloat16* base = is_v ? p.v_cache : p.k_cache;
            base[(((size_t)blk * p.kvheads + kvh) * p.block_tokens + (pos % p.block_tokens)) * p.head_dim + d] = o;
          }
        }
      }
    }
  }
  if (ks > 1) cluster_sync_all();  // nobody leaves while another block still reads its shared memory
  __syncthreads();
  if (threadIdx.x == 0 && *failed && error_flag) atomicExch(error_flag, 4);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, tmem_cols);
  }
}

// Blocks that share a tile: from the matrix's shape alone.  Enough blocks for two a multiprocessor to be there to
// stream (296 on 148 multiprocessors), at least 4 steps of 64 k a block.
int choose_ks(int tiles, int K) {
  const int k_steps = (K + TILE_K - 1) / TILE_K;
  int ks = 1;
  while (ks < MAX_KS && tiles * ks * 2 <= 320 && k_steps / (ks * 2) >= 4) ks *= 2;
  const char* e = getenv("FMS_B200_MID_KS");
  if (e && (e[0] == '1' || e[0] == '2' || e[0] == '4' || e[0] == '8')) ks = e[0] - '0';
  return ks;
}

int launch_mid(const char* what, const void* x, const void* w, MidArgs p, int M, int N, int K, int rows_of_w,
               int* error_flag, cudaStream_t stream) {
  if (M > MAX_TOKENS) return fms_fail("%s: %d rows of x, at most %d", what, M, MAX_TOKENS);
  if (K <= 0 || K % 8) return fms_fail("%s: K %d must be a positive multiple of 8", what, K);
  p.n_tokens = (M + 15) / 16 * 16;
  const int row_step = p.mode == GLU ? TILE_ROWS / 2 : TILE_ROWS;
  const int outputs = p.mode == GLU ? p.hidden : N;
  const int tiles = (outputs + row_step - 1) / row_step;
  if (tiles > 65535) return fms_fail("%s: %d tiles of rows of w", what, tiles);
  p.ks = choose_ks(tiles, K);
  const int stage_bytes = W_BYTES + p.n_tokens * TILE_K * 2;
  // two blocks a multiprocessor, one where the tokens are many
  int budget = p.n_tokens <= 128 ? 104 : 200;  // KB: two blocks a multiprocessor (measured ahead of three with fewer stages)
  if (tiles * p.ks <= 148) budget = 200;  // a block a multiprocessor at most: all of its shared memory for stages
  if (const char* e = getenv("FMS_B200_MID_SMEM_KB")) budget = atoi(e);
  int stages = budget * 1024 / stage_bytes;
  stages = stages < 3 ? 3 : (stages > MAX_STAGES ? MAX_STAGES : stages);
  const size_t red_bytes = (size_t)TILE_ROWS * (p.n_tokens + 4) * sizeof(float);
  while ((size_t)stages * stage_bytes < red_bytes) ++stages;  // the sums go over the stages
  if (stages > MAX_STAGES) return fms_fail("%s: no room for the sums of %d tokens", what, p.n_tokens);
  p.stages = stages;
  const size_t smem = (size_t)stages * stage_bytes + 1024 + 256;
  CUtensorMap map_w, map_x;
  if (make_map(&map_w, w, rows_of_w, K, p.mode == GLU ? TILE_ROWS / 2 : TILE_ROWS)) return 1;
  if (make_map(&map_x, x, M, K, p.n_tokens)) return 1;
  static size_t configured = 0;
  if (configured < smem) {
    cudaError_t e = cudaFuncSetAttribute(gemm_mid_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);
    if (e != cudaSuccess) return fms_fail("%s: shared memory refused: %s", what, cudaGetErrorString(e));
    configured = 225 * 1024;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.ks, tiles);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = p.ks;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = fms_pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_mid_kernel, map_w, map_x, p, M, N, K, error_flag);
  if (e != cudaSuccess) return fms_fail("%s: launch failed: %s", what, cudaGetErrorString(e));
  return fms_launch_status(what);
}
}  // namespace

// The most rows of x these kernels take.
FMS_API int fms_gemm_bf16_mid_max_rows() { return MAX_TOKENS; }

// y [M, N] (bfloat16, or float32 with out_dtype FMS_F32) = x [M, K] w[N, K]^T + bias.
FMS_API int fms_linear_bf16_mid(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M, int N, int K,
                                int* error_flag, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (out_dtype != FMS_F32 && out_dtype != FMS_BF16) return fms_fail("linear_bf16_mid: out dtype %d", out_dtype);
  MidArgs p = {};
  p.mode = PLAIN;
  p.out = y;
  p.bias = bias;
  p.out_f32 = out_dtype == FMS_F32;
  return launch_mid("linear_bf16_mid", x, w, p, M, N, K, N, error_flag, stream);
}

// y [M, hidden] = act(x w_gate^T + b_gate) * (x w_up^T + b_up) with w = [gate; up] of 2 hidden rows.
FMS_API int fms_glu_bf16_mid(const void* x, const void* w, const void* bias, void* y, int M, int hidden, int K, int act,
                             int* error_flag, cudaStream_t stream) {
  if (M <= 0 || hidden <= 0) return 0;
  if (act < 0 || act > 3) return fms_fail("glu_bf16_mid: activation %d", act);
  MidArgs p = {};
  p.mode = GLU;
  p.out = y;
  p.bias = bias;
  p.hidden = hidden;
  p.act = act;
  return launch_mid("glu_bf16_mid", x, w, p, M, 2 * hidden, K, 2 * hidden, error_flag, stream);
}

// The fused projection of an attention layer: [q | k | v] = x w^T + bias; q and k rotated by each token's position;
// q -> q_out [M, nheads head_dim], k and v -> the token's place in the block cache (write_cache 0: q only).  A token
// whose position has no block sets error flag 2 and is skipped.
FMS_API int fms_qkv_rope_store_bf16_mid(const void* x, const void* w, const void* bias, void* q_out, const float* inv_freq,
                                        const int* positions, const int* position_ids, const int* token_seq,
                                        const int* slots, void* k_cache, void* v_cache, const int* table, int table_stride,
                                        int block_tokens, int M, int K, int nheads, int kvheads, int head_dim,
                                        int write_cache, int* error_flag, int n_seqs, int table_rows, int pool_blocks,
                                        cudaStream_t stream) {
  if (M <= 0) return 0;
  if (nheads <= 0 || kvheads <= 0 || head_dim <= 0 || head_dim % 2 || block_tokens <= 0)
    return fms_fail("qkv_rope_store_bf16_mid: %d heads, %d kv heads, head size %d, blocks of %d", nheads, kvheads, head_dim,
                    block_tokens);
  const long rows = (long)(nheads + 2 * kvheads) * head_dim;
  if (rows > 0x7fffffffL) return fms_fail("qkv_rope_store_bf16_mid: %ld rows of w", rows);
  MidArgs p = {};
  p.mode = QKV_ROPE;
  p.out = q_out;
  p.bias = bias;
  p.inv_freq = inv_freq;
  p.positions = positions;
  p.position_ids = position_ids;
  p.token_seq = token_seq;
  p.slots = slots;
  p.k_cache = (__nv_bfloat16*)k_cache;
  p.v_cache = (__nv_bfloat16*)v_cache;
  p.table = table;
  p.table_stride = table_stride;
  p.block_tokens = block_tokens;
  p.nheads = nheads;
  p.kvheads = kvheads;
  p.head_dim = head_dim;
  p.write_cache = write_cache;
  p.n_seqs = n_seqs;
  p.table_rows = table_rows;
  p.pool_blocks = pool_blocks;
  return launch_mid("qkv_rope_store_bf16_mid", x, w, p, M, (int)rows, K, (int)rows, error_flag, stream);
}

// y[M, N] = x[M, K] . w[N, K]^T for many rows (prefill): bfloat16 operands, float32 accumulation in tensor
// memory, on the fifth-generation tensor cores of sm_100a (tcgen05.mma issued by one thread, operands brought
// into shared memory by TMA, the accumulator read back with tcgen05.ld for the epilogue).
//
// A tile of y is 128 x TN (128 rows of x against TN rows of w; TN a multiple of 16 up to 256) — or, in the GLU
// variant, a 128 x TN/2 tile of act(x w_gate^T) * (x w_up^T), whose TN accumulator columns are TN/2 gate and the
// TN/2 matching up rows of a fused [gate; up] weight (fms/modules/feedforward.py:288-297).  One persistent thread
// block per multiprocessor walks over the tiles.  TN is chosen per product so that the tiles fill whole rounds of
// the multiprocessors: 256 tiles of 128 x 256 on 148 multiprocessors are two rounds of which the second is 3/4
// idle, 592 tiles of 128 x 112 are exactly four.
//
//   warp 0   one lane issues the TMA loads: per step of 64 k, a 128 x 64 box of x and a TN x 64 box of w (GLU: two
//            of TN/2 rows), 128-byte swizzle, into one of 4 to 8 stages, completion counted on the stage's "full"
//            mbarrier
//   warp 1   allocates all 512 columns of tensor memory (two accumulators); one lane waits for "full", issues 4
//            tcgen05.mma (128 x TN x 16 each) on the stage and commits them to the stage's "empty" mbarrier;
//            after a tile's last step it commits to that accumulator's "ready" mbarrier
//   warps 2-5  wait for an accumulator, read their 32 rows of it 32 columns at a time, convert, store, and
//            give the accumulator back, while the mma warp already works on the next tile in the other one
//
// Every wait on an mbarrier is bounded: on a time-out the block records error 4 in the error flag, skips the
// rest of its work and still frees its tensor memory.  Rows and columns beyond M, N and K are filled with zeros
// by TMA on the way in and are not stored on the way out.  K must be a multiple of 8 (16-byte row pitch).
#include <cuda.h>

#include "common.cuh"

namespace {
constexpr int TILE_M = 128, MAX_TILE_N = 256, TILE_K = 64, MAX_STAGES = 8, UMMA_K = 16;
constexpr int A_BYTES = TILE_M * TILE_K * 2;
constexpr int THREADS = 192;
constexpr int RING_BYTES = 192 * 1024;  // of the stages together
constexpr size_t SMEM_BYTES = (size_t)RING_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;

#include "tcgen05.cuh"

__device__ __forceinline__ float activate(float g, int act) {
  switch (act) {
    case 0: return g / (1.f + expf(-g));
    case 1: return 0.5f * g * (1.f + erff(g * 0.70710678118654752f));
    case 2: return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    default: return fmaxf(g, 0.f);
  }
}

struct Epilogue {
  void* out;          // [M, N] bfloat16 or float32; GLU: [M, hidden] bfloat16
  const void* bias;   // bfloat16 [N] (GLU: [2 hidden]) or null
  int out_f32;        // plain only
  int glu;            // 1: the first half of the accumulator's columns are gate rows, the second the matching up rows
  int hidden;         // GLU: rows of the gate matrix
  int act;
  int tile_n;         // accumulator columns of a tile: rows of w per tile (GLU: gate and up together)
  int stages;
  // The fused projection of an attention layer (qkv 1): rows of w are [q heads | k heads | v heads]; q and k are
  // rotated by each token's position (adjacent pairs, float32 angles, fms/modules/positions.py:438-456), q goes to
  // `out` [M, nheads * head_dim], k and v into the token's place in the block cache.
  int qkv;
  const float2* sincos;       // [M, head_dim / 2] (sin, cos) of every token's rotation angles, or null: nothing is rotated
  const int* positions;       // [M] each token's place in its sequence's cache
  const int* token_seq;       // [M] index into slots
  const int* slots;
  __nv_bfloat16* k_cache;     // [blocks, kvheads, block_tokens, head_dim]
  __nv_bfloat16* v_cache;
  const int* table;           // [table_rows, table_stride]
  int table_stride, block_tokens, nheads, kvheads, head_dim, write_cache;
  int n_seqs, table_rows, pool_blocks;  // extents, for the bounds-checked build
  int* error_flag;
};

// One thread's row of a tile's accumulator (tensor-memory address `taddr`, lane = row), `tile_n` output columns
// from column n0 on: bias, the GLU product, conversion, store.  Every lane of the warp must call it.
__device__ __forceinline__ void store_rows(const Epilogue& ep, uint32_t taddr, int row, int n0, int tile_n, int M, int N) {
  const __nv_bfloat16* bias = (const __nv_bfloat16*)ep.bias;
  // the fused projection: what this thread's token needs for the rotation and for its place in the cache, once a tile
  int pos = 0, blk = -1;
  if (ep.qkv && row < M) {
    pos = ep.positions[row];
    if (ep.write_cache && n0 + tile_n > ep.nheads * ep.head_dim) {  // the tile holds columns of k or v
      const int seq = ep.token_seq[row];
      if (FMS_IN(seq, ep.n_seqs)) {
        const int slot = ep.slots[seq];
        if (FMS_IN(slot, ep.table_rows) && FMS_IN(pos / ep.block_tokens, ep.table_stride)) {
          blk = ep.table[(size_t)slot * ep.table_stride + pos / ep.block_tokens];
          if (blk < 0 && ep.error_flag) atomicExch(ep.error_flag, 2);
          if (blk >= 0 && !FMS_IN(blk, ep.pool_blocks)) blk = -1;
        }
      }
    }
  }
  // 16 columns at a time (every lane loads: tensor-memory loads are warp-wide; only rows inside M store)
  for (int c0 = 0; c0 < tile_n; c0 += 16) {
    float v[16];
    tmem_load_16(taddr + c0, v);
    const int ncols = ep.glu ? ep.hidden : N, col0 = n0 + c0;
    if (ep.glu) {
      float u[16];
      tmem_load_16(taddr + tile_n + c0, u);
#pragma unroll
      for (int jj = 0; jj < 16; ++jj) {
        float gv = v[jj], uv = u[jj];
        if (bias && col0 + jj < ncols) {
          gv += __bfloat162float(bias[col0 + jj]);
          uv += __bfloat162float(bias[ep.hidden + col0 + jj]);
        }
        v[jj] = activate(gv, ep.act) * uv;
      }
    } else if (bias) {
#pragma unroll
      for (int jj = 0; jj < 16; ++jj)
        if (col0 + jj < ncols) v[jj] += __bfloat162float(bias[col0 + jj]);
    }
    if (row >= M || col0 >= ncols) continue;  // nothing of these 16 columns lies inside y
    if (ep.qkv) {
      // 16 columns of one head (head sizes are multiples of 16, and so is col0): 8 rotary pairs
      const int head = col0 / ep.head_dim, d0 = col0 - head * ep.head_dim;
      const bool is_q = head < ep.nheads, is_v = head >= ep.nheads + ep.kvheads;
      if (!is_v && ep.sincos != nullptr) {
        // the step's table of (sin, cos): 64 contiguous bytes of this token's row
        float2 sc[8];
        const float4* t = reinterpret_cast<const float4*>(ep.sincos + (size_t)row * (ep.head_dim >> 1) + (d0 >> 1));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 two = t[j];
          sc[2 * j] = make_float2(two.x, two.y);
          sc[2 * j + 1] = make_float2(two.z, two.w);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float sn = sc[j].x, cs = sc[j].y;
          const float x0 = v[2 * j], x1 = v[2 * j + 1];
          v[2 * j] = cs * x0 - sn * x1;
          v[2 * j + 1] = sn * x0 + cs * x1;
        }
      }
      __nv_bfloat16* o;
      if (is_q) {
        o = (__nv_bfloat16*)ep.out + ((size_t)row * ep.nheads + head) * ep.head_dim + d0;
      } else {
        if (!ep.write_cache || blk < 0) continue;
        const int kvh = is_v ? head - ep.nheads - ep.kvheads : head - ep.nheads;
        o = (is_v ? ep.v_cache : ep.k_cache) +
            (((size_t)blk * ep.kvheads + kvh) * ep.block_tokens + (pos % ep.block_tokens)) * ep.head_dim + d0;
      }
#pragma unroll
      for (int jj = 0; jj < 16; jj += 8) {
        uint32_t pk[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          __nv_bfloat162 t = __floats2bfloat162_rn(v[jj + 2 * q], v[jj + 2 * q + 1]);
          pk[q] = *reinterpret_cast<uint32_t*>(&t);
        }
        *reinterpret_cast<uint4*>(o + jj) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      continue;
    }
    if (!FMS_IN((size_t)row * ncols + col0, (size_t)M * ncols)) continue;
    if (ep.out_f32) {
      float* o = (float*)ep.out + (size_t)row * ncols + col0;
#pragma unroll
      for (int jj = 0; jj < 16; ++jj)
        if (col0 + jj < ncols) o[jj] = v[jj];
    } else {
      __nv_bfloat16* o = (__nv_bfloat16*)ep.out + (size_t)row * ncols + col0;
      if (col0 + 16 <= ncols && (ncols % 8) == 0) {
#pragma unroll
        for (int jj = 0; jj < 16; jj += 8) {
          uint32_t pk[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            __nv_bfloat162 t = __floats2bfloat162_rn(v[jj + 2 * q], v[jj + 2 * q + 1]);
            pk[q] = *reinterpret_cast<uint32_t*>(&t);
          }
          *reinterpret_cast<uint4*>(o + jj) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
      } else {
#pragma unroll
        for (int jj = 0; jj < 16; ++jj)
          if (col0 + jj < ncols) o[jj] = __float2bfloat16_rn(v[jj]);
      }
    }
  }
}

// Persistent: block b computes tiles b, b + gridDim.x, ...; tiles are numbered with the row index fastest, so
// that the blocks running at the same time share few tiles of w.  The accumulator is double-buffered in tensor
// memory (2 x 256 columns, of which TN are used): the epilogue of a tile runs while the mma of the block's next
// tile are issued.
// Barriers that a consumer gives back ("empty") are waited for with the opposite parity, which a freshly
// initialised mbarrier satisfies at once.
__global__ void __launch_bounds__(THREADS, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                             const __grid_constant__ CUtensorMap map_b, Epilogue ep, int M,
                                                             int N, int K, int* __restrict__ error_flag) {
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
  const int b_bytes = ep.tile_n * TILE_K * 2, stage_bytes = A_BYTES + b_bytes, stages = ep.stages;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)RING_BYTES);
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* acc_full = empty + MAX_STAGES;   // [2]
  uint64_t* acc_empty = acc_full + 2;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  __shared__ int failed_flag;
  volatile int* failed = &failed_flag;

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_n = ep.glu ? ep.tile_n / 2 : ep.tile_n;  // output columns of a tile
  const int tiles_m = (M + TILE_M - 1) / TILE_M, tiles_n = (N + tile_n - 1) / tile_n;
  const int n_tiles = tiles_m * tiles_n;
  const int k_steps = (K + TILE_K - 1) / TILE_K;

  if (threadIdx.x == 0) {
    failed_flag = 0;
    for (int s = 0; s < MAX_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);  // one arrival per epilogue warp
    }
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 2 * MAX_TILE_N);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // everything above (barriers, tensor memory) overlaps the end of the kernel before; x may be read only now
  pdl_wait();

  if (warp == 0) {
    if (elect_one()) {
      int it = 0;  // steps issued so far, over all tiles
      for (int tile = blockIdx.x; tile < n_tiles && !*failed; tile += gridDim.x) {
        const int m0 = (tile % tiles_m) * TILE_M, n0 = (tile / tiles_m) * tile_n;
        for (int i = 0; i < k_steps; ++i, ++it) {
          const int s = it % stages;
          if (!wait_or_abort(&empty[s], ((it / stages) & 1) ^ 1, failed)) break;
          unsigned char* a = smem + (size_t)s * stage_bytes;
          unsigned char* b = a + A_BYTES;
          mbar_arrive_expect_tx(&full[s], stage_bytes);
          tma_load_2d(a, &map_a, i * TILE_K, m0, &full[s]);
          // the tile's rows of w: a whole range in one box, or the gate rows and the up rows that belong to them
          tma_load_2d(b, &map_b, i * TILE_K, n0, &full[s]);
          if (ep.glu) tma_load_2d(b + b_bytes / 2, &map_b, i * TILE_K, ep.hidden + n0, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc = umma_idesc(TILE_M, ep.tile_n);
      int it = 0, j = 0;
      for (int tile = blockIdx.x; tile < n_tiles && !*failed; tile += gridDim.x, ++j) {
        const int acc = j & 1;
        if (!wait_or_abort(&acc_empty[acc], ((j >> 1) & 1) ^ 1, failed)) break;  // the epilogue has read this buffer
        tc_fence_after();
        const uint32_t d = tmem + acc * MAX_TILE_N;
        for (int i = 0; i < k_steps; ++i, ++it) {
          const int s = it % stages;
          if (!wait_or_abort(&full[s], (it / stages) & 1, failed)) break;
          tc_fence_after();
          const uint32_t a = smem_u32(smem + (size_t)s * stage_bytes), b = a + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < TILE_K / UMMA_K; ++kk)
            umma(d, umma_desc(a + kk * UMMA_K * 2), umma_desc(b + kk * UMMA_K * 2), idesc, i > 0 || kk > 0);
          tc_commit(&empty[s]);  // the stage may be filled again once these mma have read it
        }
        tc_commit(&acc_full[acc]);  // arrives when everything issued so far is done
      }
    }
  } else {
    // epilogue warps 2..5 own the accumulator rows 32 (warp % 4) .. + 31
    const int quarter = warp & 3;
    int j = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++j) {
      const int acc = j & 1;
      const int m0 = (tile % tiles_m) * TILE_M, n0 = (tile / tiles_m) * tile_n;
      if (!wait_or_abort(&acc_full[acc], (j >> 1) & 1, failed)) break;
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t taddr = tmem + acc * MAX_TILE_N + ((uint32_t)(quarter * 32) << 16);
      store_rows(ep, taddr, row, n0, tile_n, M, N);
      // this warp has read its part of the buffer: give it back to the mma warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
    }
    tc_fence_before();
  }
  __syncthreads();
  if (threadIdx.x == 0 && *failed && error_flag) atomicExch(error_flag, 4);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 2 * MAX_TILE_N);
  }
}

// The same product by pairs of thread blocks (a cluster of two, tcgen05 cta_group::2): a pair owns a tile of 256
// rows of x by TN rows of w.  Each block of the pair brings its own 128 rows of x and its half of the rows of w
// (GLU: block 0 the gate rows, block 1 the up rows) into its own shared memory, so a multiprocessor takes in a
// third less per flop than with tiles of 128 x 256 of its own, and that intake is what limits the kernel.  Block 0
// issues the mma for both (256 x TN x 16) and counts the arriving bytes of both on its "full" barriers; the
// commits go to the "empty" and "accumulator ready" barriers of both blocks (one commit each); each block's epilogue reads its own
// tensor memory (its 128 rows) and gives the accumulator back on block 0's barrier.  No block leaves before its
// partner has (cluster barrier at the end).
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
    gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, Epilogue ep,
                        int M, int N, int K, int* __restrict__ error_flag) {
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
  const int b_rows = ep.tile_n / 2;  // rows of w that this block loads
  const int b_bytes = b_rows * TILE_K * 2, stage_bytes = A_BYTES + b_bytes, stages = ep.stages;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)RING_BYTES);
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* acc_full = empty + MAX_STAGES;   // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  __shared__ int failed_flag;
  volatile int* failed = &failed_flag;

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int tile_n = ep.glu ? ep.tile_n / 2 : ep.tile_n;  // output columns of a tile
  const int tiles_m = (M + 2 * TILE_M - 1) / (2 * TILE_M), tiles_n = (N + tile_n - 1) / tile_n;
  const int n_tiles = tiles_m * tiles_n;
  const int k_steps = (K + TILE_K - 1) / TILE_K;
  const int pair = blockIdx.x / 2, pairs = gridDim.x / 2;

  if (threadIdx.x == 0) {
    failed_flag = 0;
    for (int s = 0; s < MAX_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 8);  // one arrival per epilogue warp of either block (used in block 0)
    }
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, 2 * MAX_TILE_N);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the partner's barriers exist before anything is sent to them
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();

  if (warp == 0) {
    if (elect_one()) {
      int it = 0;
      for (int tile = pair; tile < n_tiles && !*failed; tile += pairs) {
        const int m0 = (tile % tiles_m) * 2 * TILE_M + (int)rank * TILE_M, n0 = (tile / tiles_m) * tile_n;
        const int w_row = ep.glu ? (leader ? n0 : ep.hidden + n0) : n0 + (int)rank * b_rows;
        for (int i = 0; i < k_steps; ++i, ++it) {
          const int s = it % stages;
          if (!wait_or_abort(&empty[s], ((it / stages) & 1) ^ 1, failed)) break;
          unsigned char* a = smem + (size_t)s * stage_bytes;
          if (leader) mbar_arrive_expect_tx(&full[s], 2 * stage_bytes);  // the bytes of both blocks
          tma_load_2d_pair(a, &map_a, i * TILE_K, m0, &full[s]);
          tma_load_2d_pair(a + A_BYTES, &map_b, i * TILE_K, w_row, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (leader && elect_one()) {
      const uint32_t idesc = umma_idesc(2 * TILE_M, ep.tile_n);
      int it = 0, j = 0;
      for (int tile = pair; tile < n_tiles && !*failed; tile += pairs, ++j) {
        const int acc = j & 1;
        if (!wait_or_abort(&acc_empty[acc], ((j >> 1) & 1) ^ 1, failed)) break;  // both epilogues have read this buffer
        tc_fence_after();
        const uint32_t d = tmem + acc * MAX_TILE_N;
        for (int i = 0; i < k_steps; ++i, ++it) {
          const int s = it % stages;
          if (!wait_or_abort(&full[s], (it / stages) & 1, failed)) break;
          tc_fence_after();
          const uint32_t a = smem_u32(smem + (size_t)s * stage_bytes), b = a + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < TILE_K / UMMA_K; ++kk)
            umma_pair(d, umma_desc(a + kk * UMMA_K * 2), umma_desc(b + kk * UMMA_K * 2), idesc, i > 0 || kk > 0);
          tc_commit_pair(&empty[s]);
        }
        tc_commit_pair(&acc_full[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;
    int j = 0;
    for (int tile = pair; tile < n_tiles; tile += pairs, ++j) {
      const int acc = j & 1;
      const int m0 = (tile % tiles_m) * 2 * TILE_M + (int)rank * TILE_M, n0 = (tile / tiles_m) * tile_n;
      if (!wait_or_abort(&acc_full[acc], (j >> 1) & 1, failed)) break;
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t taddr = tmem + acc * MAX_TILE_N + ((uint32_t)(quarter * 32) << 16);
      store_rows(ep, taddr, row, n0, tile_n, M, N);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (leader) mbar_arrive(&acc_empty[acc]);
        else mbar_arrive_remote(&acc_empty[acc], 0);
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  cluster_sync_all();  // nothing is sent to a block that has left
  if (threadIdx.x == 0 && *failed && error_flag) atomicExch(error_flag, 4);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem, 2 * MAX_TILE_N);
  }
}

int multiprocessors() {
  static int sms = 0;
  if (sms == 0) {
    int device = 0;
    cudaGetDevice(&device);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) sms = 148;
  }
  return sms;
}

// The tile width (accumulator columns) for a product with `cols` output columns a tile row: the one whose tiles
// cost least in whole rounds of the `units` that work at the same time (multiprocessors, or pairs of them).
// A pair's tile costs, measured, 1.0 at 256 columns and 0.56 + 0.0014 TN below (the tensor cores limit the widest
// tile, what a multiprocessor takes in per step the others); a single block's tile costs as its intake per step
// of 64 k: 128 rows of x, TN rows of w and a constant.  step: 16 (GLU: 32, so that a half is a multiple of 16).
int choose_tile_n(int tiles_m, int cols, bool glu, bool pair, int units) {
  static int forced = -1;
  if (forced < 0) {
    const char* e = getenv("FMS_B200_TC_TILE_N");
    forced = e ? atoi(e) : 0;
  }
  const int step = glu ? 32 : 16;
  if (forced >= 64 && forced <= MAX_TILE_N && forced % step == 0) return forced;
  long best_cost = -1;
  int best = MAX_TILE_N;
  for (int tn = MAX_TILE_N; tn >= 64; tn -= step) {
    const int out = glu ? tn / 2 : tn;
    const long tiles = (long)tiles_m * ((cols + out - 1) / out);
    const long tile_cost = pair ? (tn == MAX_TILE_N ? 10000 : 5600 + 14 * tn) : (TILE_M + tn + 64);
    const long cost = ((tiles + units - 1) / units) * tile_cost;
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = tn;
    }
  }
  return best;
}

bool pairs_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("FMS_B200_TC_PAIR");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

int launch(const void* x, const void* w, int w_rows, Epilogue ep, int M, int N, int K, int* error_flag,
           cudaStream_t stream) {
  if (K <= 0 || K % 8) return fms_fail("gemm_tc: K %d must be a positive multiple of 8", K);
  if (((uintptr_t)x | (uintptr_t)w) & 15) return fms_fail("gemm_tc: operands must be 16-byte aligned");
  const int sms = multiprocessors();
  const bool pair = pairs_enabled() && M > TILE_M && sms >= 2;
  const int tiles_m = pair ? (M + 2 * TILE_M - 1) / (2 * TILE_M) : (M + TILE_M - 1) / TILE_M;
  const int units = pair ? sms / 2 : sms;
  ep.tile_n = choose_tile_n(tiles_m, N, ep.glu != 0, pair, units);
  const int b_rows = pair ? ep.tile_n / 2 : ep.tile_n;  // rows of w in a block's stage
  const int stage_bytes = A_BYTES + b_rows * TILE_K * 2;
  ep.stages = RING_BYTES / stage_bytes < MAX_STAGES ? RING_BYTES / stage_bytes : MAX_STAGES;
  CUtensorMap map_a, map_b;
  if (make_map(&map_a, x, M, K) || make_map(&map_b, w, w_rows, K, (ep.glu || pair) ? ep.tile_n / 2 : ep.tile_n)) return 1;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemm_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) return fms_fail("gemm_tc: %zu bytes of shared memory refused: %s", SMEM_BYTES, cudaGetErrorString(e));
    configured = true;
  }
  const int out = ep.glu ? ep.tile_n / 2 : ep.tile_n;
  const long tiles = (long)((N + out - 1) / out) * tiles_m;
  const int busy = (int)(tiles < units ? tiles : units);  // one persistent block (or pair) per multiprocessor (pair)
  if (pair)
    fms_launch(gemm_tc_pair_kernel, dim3(2 * busy), dim3(THREADS), SMEM_BYTES, stream, map_a, map_b, ep, M, N, K, error_flag);
  else
    fms_launch(gemm_tc_kernel, dim3(busy), dim3(THREADS), SMEM_BYTES, stream, map_a, map_b, ep, M, N, K, error_flag);
  return fms_launch_status("gemm_tc");
}
}  // namespace

// y [M, N] (bfloat16 or float32) = x [M, K] w[N, K]^T + bias; x, w, bias bfloat16.
FMS_API int fms_gemm_bf16_tc(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M, int N, int K,
                             int* error_flag, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (out_dtype != FMS_F32 && out_dtype != FMS_BF16) return fms_fail("gemm_tc: out dtype %d", out_dtype);
  Epilogue ep = {};
  ep.out = y;
  ep.bias = bias;
  ep.out_f32 = out_dtype == FMS_F32 ? 1 : 0;
  return launch(x, w, N, ep, M, N, K, error_flag, stream);
}

// y [M, hidden] bfloat16 = act(x w_gate^T + b_gate) * (x w_up^T + b_up), w = [gate; up] of 2 hidden rows.
FMS_API int fms_glu_bf16_tc(const void* x, const void* w, const void* bias, void* y, int M, int hidden, int K, int act,
                            int* error_flag, cudaStream_t stream) {
  if (M <= 0 || hidden <= 0) return 0;
  if (act < 0 || act > 3) return fms_fail("glu_tc: activation %d", act);
  Epilogue ep = {};
  ep.out = y;
  ep.bias = bias;
  ep.glu = 1;
  ep.hidden = hidden;
  ep.act = act;
  return launch(x, w, 2 * hidden, ep, M, hidden, K, error_flag, stream);
}

// The fused projection of an attention layer for many tokens: [q | k | v] = x w^T + bias; q and k rotated by each
// token's position; q -> q_out [M, nheads head_dim], k and v -> the token's place in the block cache (write_cache 0: q
// only).  head_dim must be a multiple of 16.  A token whose position has no block sets error flag 2 and is skipped.
// sincos: (sin, cos) of every token's rotation angles, [M, head_dim / 2] float2, 16-byte aligned, as fms_rotary_table
// (elementwise.cu) makes it once a step for all layers; null: nothing is rotated.  (Taking them in the epilogue with
// sincosf made the epilogue longer than the tile's products: a prefill of 2,048 tokens lost 1.3 ms to it.)
FMS_API int fms_qkv_rope_store_bf16_tc(const void* x, const void* w, const void* bias, void* q_out, const void* sincos,
                                       const int* positions, const int* token_seq,
                                       const int* slots, void* k_cache, void* v_cache, const int* table, int table_stride,
                                       int block_tokens, int M, int K, int nheads, int kvheads, int head_dim,
                                       int write_cache, int* error_flag, int n_seqs, int table_rows, int pool_blocks,
                                       cudaStream_t stream) {
  if (M <= 0) return 0;
  if (nheads <= 0 || kvheads <= 0 || head_dim <= 0 || head_dim % 16 || block_tokens <= 0)
    return fms_fail("qkv_rope_store_bf16_tc: %d heads, %d kv heads, head size %d (a multiple of 16), blocks of %d", nheads,
                    kvheads, head_dim, block_tokens);
  const long rows = (long)(nheads + 2 * kvheads) * head_dim;
  if (rows > 0x7fffffffL) return fms_fail("qkv_rope_store_bf16_tc: %ld rows of w", rows);
  Epilogue ep = {};
  ep.out = q_out;
  ep.bias = bias;
  ep.qkv = 1;
  ep.sincos = (const float2*)sincos;
  ep.positions = positions;
  ep.token_seq = token_seq;
  ep.slots = slots;
  ep.k_cache = (__nv_bfloat16*)k_cache;
  ep.v_cache = (__nv_bfloat16*)v_cache;
  ep.table = table;
  ep.table_stride = table_stride;
  ep.block_tokens = block_tokens;
  ep.nheads = nheads;
  ep.kvheads = kvheads;
  ep.head_dim = head_dim;
  ep.write_cache = write_cache;
  ep.n_seqs = n_seqs;
  ep.table_rows = table_rows;
  ep.pool_blocks = pool_blocks;
  ep.error_flag = error_flag;
  if (ep.sincos != nullptr && ((uintptr_t)ep.sincos & 15)) return fms_fail("qkv_rope_store_bf16_tc: the table must be 16-byte aligned");
  return launch(x, w, (int)rows, ep, M, (int)rows, K, error_flag, stream);
}

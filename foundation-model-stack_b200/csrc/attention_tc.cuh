// bfloat16 prefill attention on the tcgen05 tensor cores, for head sizes 64 and 128; included by attention.cu
// inside its namespace after attention_mma.cuh.  One block of 6 warps owns 128 query rows of one kv head — P
// positions x GH query heads (row = position * GH + head), so that a key/value block serves all of them — and
// walks over the sequence's key blocks of 64 positions:
//
//   warp 0    one lane loads the keys and values of a block by TMA (boxes of 64 positions x 64 values of a head,
//             128-byte swizzle) into one of two stages
//   warp 1    one lane issues S = Q K^T (128 x 64, accumulator in tensor memory, two buffers: the scores of the
//             next block are computed while the rows of this one are exponentiated), waits for the probabilities
//             and issues O += P V (128 x head size, accumulator in tensor memory; P is read from tensor memory,
//             V as it lies in the cache, as an MN-major operand)
//   warps 2-5 a thread per query row: read its row of S from tensor memory, mask by position, running maximum
//             and sum in float32 (base 2), write the probabilities as bfloat16 back into tensor memory, over the
//             scores they came from, rescale its row of O only when the maximum has grown by more
//             than 2^8 over the reference the exponents are taken against (the quotient O / l does not depend on
//             that reference); at the end divide by the sum and store
//
// Rows of a cache block beyond the sequence's length may hold anything; before the tensor cores read the values of
// the last block, those rows are overwritten with zeros in shared memory (a masked probability is an exact zero,
// but zero times NaN is not).  Every wait is bounded; a time-out is reported as error 4.
#pragma once

#include "tcgen05.cuh"

constexpr int TC_ROWS = 128;                 // query rows of a block
constexpr int TC_STAGES = 2;
constexpr int TC_KV_TILE = BLK * HD * 2;     // bytes of a block's keys (or values) of one kv head
constexpr int TC_Q_BYTES = TC_ROWS * HD * 2;
constexpr size_t TC_SMEM = 1024 + TC_Q_BYTES + (size_t)TC_STAGES * 2 * TC_KV_TILE + 256;  // two blocks fit an SM
constexpr int TC_TMEM_COLS = HD + 2 * BLK <= 128 ? 128 : 256;  // O: HD columns, S: two buffers of 64 columns

// 2^x in one special-function instruction (relative error about 2^-22; 0 for -inf)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

__host__ __device__ inline int tc_heads_per_block(int group) { return group < TC_ROWS ? group : TC_ROWS; }
__host__ __device__ inline int tc_positions_per_block(int group) { return TC_ROWS / tc_heads_per_block(group); }

__global__ void __launch_bounds__(192, 2) attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k,
                                                                 const __grid_constant__ CUtensorMap map_v, AttnArgs a,
                                                                 const int* __restrict__ tiles, int n_tiles,
                                                                 int* __restrict__ error_flag) {
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
  unsigned char* q_tile = smem;                            // HD / 64 tiles of [128 rows][128 bytes], swizzled
  unsigned char* kv = q_tile + TC_Q_BYTES;                 // per stage: keys (HD / 64 tiles of [64][128 B]), then values
  // keys and values have barriers of their own: the keys of block i + 2 may come once the scores of block i are
  // computed, the values only after its product
  uint64_t* k_full = reinterpret_cast<uint64_t*>(kv + (size_t)TC_STAGES * 2 * TC_KV_TILE);
  uint64_t* k_empty = k_full + TC_STAGES;
  uint64_t* v_full = k_empty + TC_STAGES;
  uint64_t* v_empty = v_full + TC_STAGES;
  uint64_t* s_full = v_empty + TC_STAGES;  // [2], as p_ready and o_done: block i uses entry i & 1, phase (i / 2) & 1
  uint64_t* p_ready = s_full + 2;
  uint64_t* o_done = p_ready + 2;
  uint64_t* q_ready = o_done + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_ready + 1);
  __shared__ int failed_flag;
  volatile int* failed = &failed_flag;
  pdl_launch_dependents();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = a.nheads / a.kvheads;
  const int gh = tc_heads_per_block(group), pp = TC_ROWS / gh;
  const int chunks = (group + gh - 1) / gh;
  // heads vary fastest and the tiles run from the last to the first: later positions have more keys, and the long
  // blocks of every head start before any short one
  const int hc = blockIdx.x % (a.kvheads * chunks);
  const int tile = n_tiles - 1 - blockIdx.x / (a.kvheads * chunks);
  const int kvh = hc / chunks, g0 = (hc - kvh * chunks) * gh;
  const int ng = min(gh, group - g0);
  const int seq = tiles[2 * tile], r0 = tiles[2 * tile + 1];
  const int row_begin = a.first_row[seq];
  const int n_new = a.first_row[seq + 1] - row_begin;
  const int len = a.len_after[seq];
  const int len_before = len - n_new;
  const int slot = a.slots[seq];
  const int pos_here = min(pp, n_new - r0);
  const int p_first = len_before + r0, p_last = p_first + pos_here - 1;
  const int kb_lo = a.window > 0 ? max(0, p_first - a.window + 1) / BLK : 0;
  const int kb_hi = p_last / BLK;
  const int nblocks = kb_hi - kb_lo + 1;

  if (threadIdx.x == 0) {
    failed_flag = 0;
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&p_ready[b], 4);  // one arrival a warp
      mbar_init(&o_done[b], 1);
    }
    mbar_init(q_ready, 128);
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, TC_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_o = tmem, tmem_s = tmem + HD;  // S buffer b at tmem_s + 64 b
  pdl_wait();

  if (warp == 0) {
    if (elect_one()) {
      for (int i = 0; i < nblocks && !*failed; ++i) {
        const int s = i % TC_STAGES;
        const int blk = block_of(a, slot, kb_lo + i);
        unsigned char* kdst = kv + (size_t)s * 2 * TC_KV_TILE;
        unsigned char* vdst = kdst + TC_KV_TILE;
        const int row = (max(blk, 0) * a.kvheads + kvh) * BLK;  // first row of the block in the [positions, HD] view
        if (!wait_or_abort(&k_empty[s], ((i / TC_STAGES) & 1) ^ 1, failed)) break;
        mbar_arrive_expect_tx(&k_full[s], TC_KV_TILE);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c) tma_load_2d(kdst + c * (BLK * 128), &map_k, c * 64, row, &k_full[s]);
        if (!wait_or_abort(&v_empty[s], ((i / TC_STAGES) & 1) ^ 1, failed)) break;
        mbar_arrive_expect_tx(&v_full[s], TC_KV_TILE);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c) tma_load_2d(vdst + c * (BLK * 128), &map_v, c * 64, row, &v_full[s]);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t IDESC_S = umma_idesc(TC_ROWS, BLK);
      constexpr uint32_t IDESC_O = umma_idesc(TC_ROWS, HD, true);
      const uint32_t qaddr = smem_u32(q_tile);
      // S(i) = Q K(i)^T into buffer i & 1: both operands K-major; k-step kk lies in tile kk / 4 at byte 32 (kk % 4)
      auto issue_scores = [&](int i) -> bool {
        const int s = i % TC_STAGES;
        if (!wait_or_abort(&k_full[s], (i / TC_STAGES) & 1, failed)) return false;
        tc_fence_after();
        const uint32_t kaddr = smem_u32(kv + (size_t)s * 2 * TC_KV_TILE);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
          umma(tmem_s + (i & 1) * BLK, umma_desc(qaddr + (kk / 4) * (TC_ROWS * 128) + (kk % 4) * 32),
               umma_desc(kaddr + (kk / 4) * (BLK * 128) + (kk % 4) * 32), IDESC_S, kk > 0);
        tc_commit(&s_full[i & 1]);
        tc_commit(&k_empty[s]);
        return true;
      };
      bool go = wait_or_abort(q_ready, 0, failed) && issue_scores(0);  // the query tile is in shared memory
      for (int i = 0; i < nblocks && go && !*failed; ++i) {
        // the scores of the next block, while the rows of this one are exponentiated (its buffer was read two
        // blocks ago: p_ready of that block has been seen)
        if (i + 1 < nblocks && !issue_scores(i + 1)) break;
        const int s = i % TC_STAGES;
        if (!wait_or_abort(&v_full[s], (i / TC_STAGES) & 1, failed)) break;
        if (!wait_or_abort(&p_ready[i & 1], (i >> 1) & 1, failed)) break;  // probabilities written, O rescaled
        tc_fence_after();
        const uint32_t vaddr = smem_u32(kv + (size_t)s * 2 * TC_KV_TILE) + TC_KV_TILE;
        // O += P V: P from tensor memory, where it lies over the scores it came from (16 keys = 8 columns);
        // V MN-major: 16 keys of a step are 16 rows of 128 bytes, the head's second 64 values lie one tile
        // (BLK * 128 bytes) further.  The scores of block i + 2 are issued after this product and overwrite P then.
#pragma unroll
        for (int kk = 0; kk < BLK / 16; ++kk)
          umma_a_tmem(tmem_o, tmem_s + (i & 1) * BLK + kk * 8, umma_desc_offsets(vaddr + kk * 16 * 128, BLK * 128, 1024),
                      IDESC_O, i > 0 || kk > 0);
        tc_commit(&v_empty[s]);
        tc_commit(&o_done[i & 1]);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;       // this thread's query row
    const int pi = r / gh, gi = r - pi * gh;
    const bool row_ok = pi < pos_here && gi < ng;
    const int my_pos = p_first + pi;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    // the query tile: row r, 16-byte piece c of 64-value chunk t at t * 16 KB + r * 128 + ((c ^ (r & 7)) << 4)
    {
      const __nv_bfloat16* q = (const __nv_bfloat16*)a.q +
                               ((size_t)(row_begin + r0 + (row_ok ? pi : 0)) * a.nheads + kvh * group + g0 + (row_ok ? gi : 0)) * HD;
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) {
        const uint4 v = row_ok ? *reinterpret_cast<const uint4*>(q + 8 * c) : make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(q_tile + (c / 8) * (TC_ROWS * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
      }
      fence_proxy_async();
      mbar_arrive(q_ready);
    }
    const float scale2 = a.scale * LOG2E;
    float m_ref = -INFINITY, l = 0.f;  // the exponents are taken against m_ref (base 2); l is the sum of them
    bool ok = true;
    for (int i = 0; i < nblocks && ok; ++i) {
      const int kb = kb_lo + i, s = i % TC_STAGES;
      ok = __all_sync(0xffffffffu, wait_or_abort(&s_full[i & 1], (i >> 1) & 1, failed));  // the same decision in
      if (!ok) break;                                                    // every lane: tensor-memory loads are warp-wide
      tc_fence_after();
      float sc[BLK];
      static_assert(BLK == 64, "a row of scores is read as 64 columns");
      tmem_load_2x32(tmem_s + (i & 1) * BLK + lane_base, tmem_s + (i & 1) * BLK + lane_base + 32, sc, sc + 32);
      // raw scores; the scale (positive) goes into the exponent's multiply-add.  A block that every row of the tile
      // sees whole needs no mask; rows without a query hold zeros there and are never stored.
      const bool whole = kb * BLK + BLK - 1 <= p_first && (a.window <= 0 || kb * BLK > p_last - a.window);
      if (!whole) {
#pragma unroll
        for (int j = 0; j < BLK; ++j) {
          const int kpos = kb * BLK + j;
          const bool visible = row_ok && kpos <= my_pos && (a.window <= 0 || kpos > my_pos - a.window);
          sc[j] = visible ? sc[j] : -INFINITY;
        }
      }
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < BLK; j += 4) {
#pragma unroll
        for (int e = 0; e < 4; ++e) mx[e] = fmaxf(mx[e], sc[j + e]);
      }
      const float tile_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale2;
      // a new reference only when the maximum has outgrown the old one by more than 2^8
      float alpha = 1.f;
      if (tile_max > m_ref + 8.f) {
        alpha = m_ref == -INFINITY ? 0.f : exp2f(m_ref - tile_max);
        m_ref = tile_max;
        l *= alpha;
      }
      if (i > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {  // warp-wide loads and stores: all lanes or none
        ok = __all_sync(0xffffffffu, wait_or_abort(&o_done[(i - 1) & 1], ((i - 1) >> 1) & 1, failed));
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          float o[32];
          tmem_load_32(tmem_o + lane_base + c0, o);
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] *= alpha;
          tmem_store_32(tmem_o + lane_base + c0, o);
        }
      }
      const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
      float ps[4] = {0.f, 0.f, 0.f, 0.f};
      float pk[BLK / 2];  // probabilities as bfloat16, two keys a word, into the columns their scores came from
#pragma unroll
      for (int j = 0; j < BLK / 2; ++j) {
        const float p0 = fast_exp2(fmaf(sc[2 * j], scale2, neg_m));  // 2^-inf = 0 for a masked key
        const float p1 = fast_exp2(fmaf(sc[2 * j + 1], scale2, neg_m));
        ps[j & 3] += p0 + p1;
        pk[j] = __uint_as_float(pack_bf16(p0, p1));
      }
      tmem_store_32(tmem_s + (i & 1) * BLK + lane_base, pk);
      const float psum = (ps[0] + ps[1]) + (ps[2] + ps[3]);
      l += psum;
      // the values of a block that the sequence fills only partly: rows beyond its length become zeros
      const int blk = block_of(a, slot, kb);
      if (kb * BLK + BLK > len || blk < 0) {
        ok = __all_sync(0xffffffffu, wait_or_abort(&v_full[s], (i / TC_STAGES) & 1, failed));
        if (!ok) break;
        unsigned char* vdst = kv + (size_t)s * 2 * TC_KV_TILE + TC_KV_TILE;
        const int first_bad = blk < 0 ? 0 : len - kb * BLK;  // a block that has left the window holds nothing
        for (int idx = r; idx < (BLK - first_bad) * (HD / 8); idx += 128) {
          const int row = first_bad + idx / (HD / 8), c = idx % (HD / 8);
          *reinterpret_cast<uint4*>(vdst + (c / 8) * (BLK * 128) + row * 128 + ((c & 7) << 4)) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[i & 1]);
    }
    if (ok && __all_sync(0xffffffffu, wait_or_abort(&o_done[(nblocks - 1) & 1], ((nblocks - 1) >> 1) & 1, failed))) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* o_row = (__nv_bfloat16*)a.out +
                             ((size_t)(row_begin + r0 + (row_ok ? pi : 0)) * a.nheads + kvh * group + g0 + (row_ok ? gi : 0)) * HD;
#pragma unroll
      for (int c0 = 0; c0 < HD; c0 += 32) {
        float o[32];
        tmem_load_32(tmem_o + lane_base + c0, o);  // warp-wide: every lane loads, only valid rows store
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) w[e] = pack_bf16(o[j + 2 * e] * inv, o[j + 2 * e + 1] * inv);
            *reinterpret_cast<uint4*>(o_row + c0 + j) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (threadIdx.x == 0 && *failed && error_flag) atomicExch(error_flag, 4);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TC_TMEM_COLS);
  }
}

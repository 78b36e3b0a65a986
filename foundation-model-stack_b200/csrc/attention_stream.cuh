// Decode attention for many sequences: persistent warps that stream the cache through shared memory with TMA.
// Included by attention.cu inside its namespace after attention_mma.cuh and tcgen05.cuh (head sizes 64 and 128).
//
// With hundreds of (sequence, kv head, split) units the launch is bound by bytes, and a block of threads per unit
// spends a third of its life without a request in flight (lengths, table, first keys, merge, exit).  Here a
// multiprocessor runs one block of SR_WARPS consumer warps and one producer warp.  Each consumer owns a ring of
// SR_STAGES stages in shared memory; a stage holds the 64 keys and 64 values of one cache block (TMA boxes of
// 64 x 64, 128-byte swizzle) and, for a unit's first block, its queries.  Lane w of the producer warp feeds
// consumer w: it takes the next unit from a counter in global memory (so that sequences of unequal lengths spread
// evenly), reads its length, slot and table entries, and issues the copies for its blocks as stages come free, so
// requests for the next block are in flight, across unit boundaries, while a consumer works on one.  The
// arithmetic is that of attn_decode_mma_kernel (products transposed, 8 query heads as the columns of the mma
// tile), with keys read from shared memory by ldmatrix.  A unit's result (m, l, o) goes to the same scratch, for
// attn_combine_kernel, which also puts the counter back to zero.
#pragma once

constexpr int SR_WARPS = HD >= 128 ? 3 : 6;  // consumers; measured against 2 (4) with three stages: 1-3% quicker
constexpr int SR_STAGES = 2;
constexpr int SR_KV_BYTES = BLK * HD * 2;                       // keys (or values) of a block
constexpr int SR_Q_BYTES = GROWS * HD * 2;                      // queries of a unit
constexpr int SR_STAGE_BYTES = 2 * SR_KV_BYTES + ((SR_Q_BYTES + 1023) / 1024) * 1024;
constexpr int SR_DESC_INTS = 8;                                 // a stage's description, written by the producer: live (0: no
                                                                // more work), sequence, kv head and chunk, split, key block,
                                                                // the split's first and last + 1 position, first block of a unit
constexpr size_t SR_SMEM = 1024 + (size_t)SR_WARPS * SR_STAGES * SR_STAGE_BYTES + SR_WARPS * SR_STAGES * (16 + SR_DESC_INTS * 4);

// byte offset, inside a [64 rows x HD] tile made of TMA boxes of 64 x 64 with the 128-byte swizzle, of the 16-byte
// piece `piece` (of HD / 8) of row `row`
__device__ __forceinline__ int sr_offset(int row, int piece) {
  return (piece >> 3) * (BLK * 128) + row * 128 + (((piece & 7) ^ (row & 7)) << 4);
}

__global__ void __launch_bounds__((SR_WARPS + 1) * 32, 1)
    attn_decode_stream_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, AttnArgs a,
                              float* __restrict__ part_o, float* __restrict__ part_ml, int n_seqs, int n_splits,
                              int* __restrict__ work_counter, int* __restrict__ error_flag) {
  extern __shared__ unsigned char sr_smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)sr_smem_unaligned + 1023) & ~(uintptr_t)1023);
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
  unsigned char* tail = smem + (size_t)SR_WARPS * SR_STAGES * SR_STAGE_BYTES;
  uint64_t* full_all = reinterpret_cast<uint64_t*>(tail);
  uint64_t* empty_all = full_all + SR_WARPS * SR_STAGES;
  int* descs_all = reinterpret_cast<int*>(empty_all + SR_WARPS * SR_STAGES);
  if (threadIdx.x == 0) {
    for (int s = 0; s < SR_WARPS * SR_STAGES; ++s) {
      mbar_init(full_all + s, 1);
      mbar_init(empty_all + s, 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  const int group = a.nheads / a.kvheads;
  const int chunks = (group + GROWS - 1) / GROWS;
  const int ny = a.kvheads * chunks;
  const long n_units = (long)n_seqs * ny * n_splits;
  pdl_wait();

  if (warp == SR_WARPS) {
    // ---- producer: lane w feeds consumer w ---------------------------------------------------------------
    if (lane >= SR_WARPS) return;
    unsigned char* ring = smem + (size_t)lane * SR_STAGES * SR_STAGE_BYTES;
    uint64_t* full = full_all + lane * SR_STAGES;
    uint64_t* empty = empty_all + lane * SR_STAGES;
    int* descs = descs_all + lane * SR_STAGES * SR_DESC_INTS;
    int seq = 0, y = 0, split = 0, slot = 0, k_lo = 0, k_hi = 0, kb = 0;
    bool open = false, first = false;
    for (int i = 0;; ++i) {
      const int s = i % SR_STAGES;
      if (i >= SR_STAGES && !mbar_wait(empty + s, (uint32_t)(i / SR_STAGES - 1) & 1u)) {
        if (error_flag) atomicExch(error_flag, 4);
        return;
      }
      int blk = -1, kb_here = 0;
      bool first_here = false;
      while (true) {
        if (open && kb * BLK < k_hi) {
          kb_here = kb++;
          blk = block_of(a, slot, kb_here);
          if (blk < 0) continue;  // given back behind a window
          first_here = first;
          first = false;
          break;
        }
        open = false;
        const long u = atomicAdd(work_counter, 1);
        if (u >= n_units) break;
        seq = (int)(u % n_seqs);
        const long rest = u / n_seqs;
        y = (int)(rest % ny);
        split = (int)(rest / ny);
        const int len = a.len_after[seq];
        const int kstart = a.window > 0 ? max(0, len - a.window) : 0;
        k_lo = max(kstart, split * SPLIT);
        k_hi = min(len, (split + 1) * SPLIT);
        if (k_lo >= k_hi) continue;
        slot = a.slots[seq];
        kb = k_lo / BLK;
        open = first = true;
      }
      int* d = descs + s * SR_DESC_INTS;
      d[0] = blk >= 0 ? 1 : 0;
      d[1] = seq; d[2] = y; d[3] = split; d[4] = kb_here; d[5] = k_lo; d[6] = k_hi; d[7] = first_here ? 1 : 0;
      if (blk < 0) {  // no more units: the consumer wakes, reads the end mark and leaves
        mbar_arrive(full + s);
        return;
      }
      unsigned char* st = ring + (size_t)s * SR_STAGE_BYTES;
      const int kvh = y / chunks, g0 = (y - kvh * chunks) * GROWS;
      const int ng = min(GROWS, group - g0);
      const int row = (blk * a.kvheads + kvh) * BLK;
      mbar_arrive_expect_tx(full + s, 2 * SR_KV_BYTES + (first_here ? ng * HD * 2 : 0));
#pragma unroll
      for (int h = 0; h < HD / 64; ++h) {
        tma_load_2d(st + h * (BLK * 128), &map_k, 64 * h, row, full + s);
        tma_load_2d(st + SR_KV_BYTES + h * (BLK * 128), &map_v, 64 * h, row, full + s);
      }
      if (first_here)
        bulk_copy_g2s(st + 2 * SR_KV_BYTES,
                      (const __nv_bfloat16*)a.q + ((size_t)a.first_row[seq] * a.nheads + kvh * group + g0) * HD, ng * HD * 2,
                      full + s);
    }
  }

  // ---- consumers --------------------------------------------------------------------------------------------
  unsigned char* ring = smem + (size_t)warp * SR_STAGES * SR_STAGE_BYTES;
  uint64_t* full = full_all + warp * SR_STAGES;
  uint64_t* empty = empty_all + warp * SR_STAGES;
  const int* descs = descs_all + warp * SR_STAGES * SR_DESC_INTS;
  uint32_t qf[HD / 16][2];
  float o[HD / 16][4];
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const float scale2 = a.scale * LOG2E;
  for (int i = 0;; ++i) {
    const int s = i % SR_STAGES;
    if (!mbar_wait(full + s, (uint32_t)(i / SR_STAGES) & 1u)) {
      if (lane == 0 && error_flag) atomicExch(error_flag, 4);
      // copies that may still be on their way into this warp's other stages: wait for them, again with a limit,
      // so that none lands in shared memory that has been given to another block
      for (int k = 1; k < SR_STAGES; ++k) mbar_wait(full + (i + k) % SR_STAGES, (uint32_t)((i + k) / SR_STAGES) & 1u);
      return;
    }
    const int* d = descs + s * SR_DESC_INTS;
    if (d[0] == 0) break;
    const int seq = d[1], y = d[2], split = d[3], kb = d[4], k_lo = d[5], k_hi = d[6];
    const bool first = d[7] != 0;
    const int kvh = y / chunks, g0 = (y - kvh * chunks) * GROWS;
    const int ng = min(GROWS, group - g0);
    const unsigned char* kbuf = ring + (size_t)s * SR_STAGE_BYTES;
    unsigned char* vbuf = ring + (size_t)s * SR_STAGE_BYTES + SR_KV_BYTES;
    if (first) {
      const unsigned char* qrow = kbuf + 2 * SR_KV_BYTES + (size_t)g * HD * 2;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        qf[ks][0] = g < ng ? *reinterpret_cast<const uint32_t*>(qrow + (16 * ks + 2 * c) * 2) : 0u;
        qf[ks][1] = g < ng ? *reinterpret_cast<const uint32_t*>(qrow + (16 * ks + 2 * c + 8) * 2) : 0u;
      }
#pragma unroll
      for (int j = 0; j < HD / 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
      m[0] = m[1] = -INFINITY;
      l[0] = l[1] = 0.f;
    }
    const bool whole = kb * BLK >= k_lo && kb * BLK + BLK <= k_hi;
    if (!whole) {  // rows of the block that are not this sequence's keys: their values must not meet a zero weight as NaN
      for (int pce = lane; pce < BLK * PIECES; pce += 32) {
        const int row = pce / PIECES, piece = pce - row * PIECES;
        const int pos = kb * BLK + row;
        if (pos < k_lo || pos >= k_hi) *reinterpret_cast<uint4*>(vbuf + sr_offset(row, piece)) = make_uint4(0, 0, 0, 0);
      }
      fence_proxy_async();  // these stores before the copies that will overwrite the stage
      __syncwarp();
    }
    // scores, 16 keys a tile: element e of tile t is (key 16 t + g + 8 (e / 2), head 2 c + (e % 2))
    float st[4][4];
#pragma unroll
    for (int t = 0; t < 4; ++t) st[t][0] = st[t][1] = st[t][2] = st[t][3] = 0.f;
    {
      const int krow = (lane & 7) + 8 * ((lane >> 3) & 1);  // row of the 16-key tile whose address this lane gives
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          uint32_t ka[4];
          ldmatrix_x4(ka, kbuf + sr_offset(16 * t + krow, 2 * ks + (lane >> 4)));
          mma16816(st[t], ka, qf[ks][0], qf[ks][1]);
        }
      }
    }
    if (!whole) {
#pragma unroll
      for (int t = 0; t < 4; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int kpos = kb * BLK + 16 * t + g + 8 * (e >> 1);
          if (kpos < k_lo || kpos >= k_hi) st[t][e] = -INFINITY;
        }
    }
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
      for (int e = 0; e < 4; ++e) tile_max[e & 1] = fmaxf(tile_max[e & 1], st[t][e]);
    float alpha[2], psum[2] = {0.f, 0.f}, neg_m[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 4));
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 8));
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 16));
      const float m_new = fmaxf(m[h], tile_max[h] * scale2);
      neg_m[h] = m_new == -INFINITY ? 0.f : -m_new;
      alpha[h] = ex2_approx(m[h] + neg_m[h]);
      m[h] = m_new;
    }
    uint32_t pb[4][2];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      float pr[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        pr[e] = ex2_approx(fmaf(st[t][e], scale2, neg_m[e & 1]));
        psum[e & 1] += pr[e];
      }
      pb[t][0] = movmatrix_trans(pack_bf16(pr[0], pr[1]));
      pb[t][1] = movmatrix_trans(pack_bf16(pr[2], pr[3]));
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 4);
      psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 8);
      psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 16);
      l[h] = l[h] * alpha[h] + psum[h];
    }
    if (!first) {
#pragma unroll
      for (int j = 0; j < HD / 16; ++j) {
        o[j][0] *= alpha[0]; o[j][1] *= alpha[1]; o[j][2] *= alpha[0]; o[j][3] *= alpha[1];
      }
    }
    // V^T tiles of 16 values x 16 keys: matrix (lane >> 3) of the four is (values + 8 ((lane >> 3) & 1), keys + 8 (lane >> 4))
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int vrow = 16 * t + (lane & 7) + (lane >> 4) * 8;
#pragma unroll
      for (int j = 0; j < HD / 16; ++j) {
        uint32_t av[4];
        ldmatrix_x4_trans(av, vbuf + sr_offset(vrow, 2 * j + ((lane >> 3) & 1)));
        mma16816(o[j], av, pb[t][0], pb[t][1]);
      }
    }
    if (kb == (k_hi - 1) / BLK) {  // the unit's last block: its result, unnormalised, for the merge over splits
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int r = 2 * c + e;  // head within the chunk
        if (r < ng) {
          const size_t at = ((size_t)seq * a.nheads + kvh * group + g0 + r) * n_splits + split;
          if (!FMS_IN(at, (size_t)n_seqs * a.nheads * n_splits)) continue;
#pragma unroll
          for (int j = 0; j < HD / 16; ++j) {
            part_o[at * HD + 16 * j + g] = o[j][e];
            part_o[at * HD + 16 * j + g + 8] = o[j][2 + e];
          }
          if (g == 0) {
            part_ml[at * 2] = m[e] * (1.f / LOG2E);  // natural units, which attn_combine_kernel expects
            part_ml[at * 2 + 1] = l[e];
          }
        }
      }
    }
    __syncwarp();  // every lane is past the stage
    if (lane == 0) mbar_arrive(empty + s);
  }
}

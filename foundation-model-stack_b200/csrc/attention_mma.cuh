// bfloat16 attention on the tensor cores (mma.sync m16n8k16, float32 accumulation), included by attention.cu
// inside its namespace after HD, BLK, SPLIT, AttnArgs.  Scores, softmax and the output accumulator are float32;
// the probabilities are rounded to bfloat16 for the second product, as in every flash-attention kernel.
#pragma once

constexpr int ROWB = HD * 2 + 16;  // bytes of a key/value row in shared memory: padded, so that the eight rows
                                   // of an 8x8 matrix (and of a fragment load) fall into different banks
constexpr int PIECES = HD / 8;     // 16-byte pieces of a row

__device__ __forceinline__ void mma16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, const void* smem_row) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
// Four 8x8 matrices, not transposed: lane l gives the address of row (l & 7) of matrix (l >> 3).
__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const void* smem_row) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
// Scores of a warp's 16 query rows against the 64 keys of a block in shared memory: s[j] is the 16 x 8 tile of
// keys 8 j .. 8 j + 7.  Consecutive mma go to different tiles, so that none waits for the one before.
__device__ __forceinline__ void scores_16x64(float (*s)[4], const uint32_t (*qf)[4], const unsigned char* kbuf, int lane) {
#pragma unroll
  for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
  const unsigned char* base = kbuf + (lane & 7) * ROWB + (lane >> 3) * 16;
#pragma unroll
  for (int ks = 0; ks < HD / 16; ks += 2) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint32_t b[4];  // keys 8 j .. 8 j + 7: (b[0], b[1]) for k-step ks, (b[2], b[3]) for k-step ks + 1
      if (ks + 1 < HD / 16) {
        ldmatrix_x4(b, base + 8 * j * ROWB + 32 * ks);
        mma16816(s[j], qf[ks], b[0], b[1]);
        mma16816(s[j], qf[ks + 1 < HD / 16 ? ks + 1 : ks], b[2], b[3]);
      } else {  // an odd number of k-steps: the last one alone
        const unsigned char* krow = kbuf + (8 * j + (lane >> 2)) * ROWB + 4 * (lane & 3) + 32 * ks;
        mma16816(s[j], qf[ks], *reinterpret_cast<const uint32_t*>(krow), *reinterpret_cast<const uint32_t*>(krow + 16));
      }
    }
  }
}
constexpr float LOG2E = 1.4426950408889634f;

// 2^x in one special-function instruction (relative error about 2^-22; 0 for -inf)
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0: the destination is filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait_group() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// asks for `bytes` (a multiple of 16) of global memory to be brought into L2
__device__ __forceinline__ void prefetch_l2(const void* gmem, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(gmem), "r"(bytes) : "memory");
}

// A warp copies the 64 rows of one cache block (keys or values of one kv head), or the first `rows` of them, into
// its padded buffer.  Rows outside [lo, hi) of the sequence are filled with zeros instead of being read.
__device__ __forceinline__ void copy_block_async(unsigned char* dst, const __nv_bfloat16* src, int first_pos, int lo,
                                                 int hi, int lane, int rows = BLK) {
  for (int p = lane; p < rows * PIECES; p += 32) {
    const int row = p / PIECES, piece = p - row * PIECES;
    const int pos = first_pos + row;
    cp_async_16(dst + row * ROWB + piece * 16, src + (size_t)row * HD + piece * 8, pos >= lo && pos < hi);
  }
}

// ---------------------------------------------------------------------------------------------------
// decode: grid (sequences, kv heads * head chunks, splits of 256 keys), NW warps.  With one query per sequence the
// products are taken transposed, so that the 8 columns of the mma tile are up to 8 query heads that share the kv
// head and nothing of the 16 rows is wasted:
//   S^T [64 keys x 8 heads]   = K [keys x HD] . Q^T      A = keys, read from global memory straight into
//                                                          registers (16 contiguous bytes a lane; the k index of
//                                                          the instruction is permuted alike for both operands)
//   O^T [HD x 8 heads]       += V^T [HD x keys] . P^T     A = values, copied to shared memory while the scores are
//                                                          taken and read transposed (ldmatrix.trans); B = the
//                                                          probabilities, turned from accumulator to operand
//                                                          layout by movmatrix
// Warp w takes the pieces of WK keys w, w + NW, ... of the split (WK = 64: a cache block; WK = 32: half of one, with
// 8 warps a split of 256 keys is then one piece a warp, all of a warp's keys are on their way at once and nothing
// is rescaled: the shortest chain, for launches of few blocks), each warp with a running softmax of its own; the
// warps' results are merged in shared memory and written as one unnormalised partial result (m, l, o) per head,
// which attn_combine_kernel merges over splits.
// ---------------------------------------------------------------------------------------------------
constexpr int GROWS = 8;  // query heads per block (columns of the mma tile)

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
  return y;
}

template <int NW, int WK>
__global__ void __launch_bounds__(NW * 32, WK == 32 ? 16 / NW : 12 / NW)
    attn_decode_mma_kernel(AttnArgs a, float* __restrict__ part_o, float* __restrict__ part_ml, int n_splits,
                           int pool_blocks) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
  const int seq = blockIdx.x, split = blockIdx.z;
  const int group = a.nheads / a.kvheads;
  const int chunks = (group + GROWS - 1) / GROWS;
  const int kvh = blockIdx.y / chunks, chunk = blockIdx.y - kvh * chunks;
  // While the kernels before this one are still running: ask for this block's keys and values to be brought into
  // L2.  Nothing orders these reads of the lengths and the table after the kernels that write them, so they may
  // be a step old; they only choose the addresses of a hint, and a block number outside the pool is left alone.
  // (Loads that bypass L1, so that no stale line is found again after the wait.)
  if (pool_blocks > 0 && lane == 0) {
    const int len0 = __ldcg(a.len_after + seq), slot0 = __ldcg(a.slots + seq);
    const int start0 = a.window > 0 ? max(0, len0 - a.window) : 0;
    const int lo0 = max(start0, split * SPLIT), hi0 = min(len0, (split + 1) * SPLIT);
    if (slot0 >= 0) {
      for (int piece = lo0 / WK + warp; piece * WK < hi0 && piece * WK / BLK < a.table_stride; piece += NW) {
        const int blk = __ldcg(a.table + (size_t)slot0 * a.table_stride + piece * WK / BLK);
        if (blk < 0 || blk >= pool_blocks) continue;
        const size_t at = (((size_t)blk * a.kvheads + kvh) * BLK + piece * WK % BLK) * HD;
        prefetch_l2((const __nv_bfloat16*)a.keys + at, WK * HD * 2);
        prefetch_l2((const __nv_bfloat16*)a.values + at, WK * HD * 2);
      }
    }
  }
  pdl_wait();
  const int g0 = chunk * GROWS;
  const int ng = min(GROWS, group - g0);
  // the three values every block needs, asked for together: none of them waits for another
  const int len = a.len_after[seq];
  const int slot = a.slots[seq];
  const int first_row = a.first_row[seq];
  const int pos = len - 1;
  const int kstart = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  const int k_lo = max(kstart, split * SPLIT), k_hi = min(len, (split + 1) * SPLIT);
  if (k_lo >= k_hi) return;
  const __nv_bfloat16* q = (const __nv_bfloat16*)a.q + (size_t)first_row * a.nheads * HD +
                           (size_t)(kvh * group + g0) * HD;
  const __nv_bfloat16* kc = (const __nv_bfloat16*)a.keys;
  const __nv_bfloat16* vc = (const __nv_bfloat16*)a.values;
  unsigned char* vbuf = smem_raw + (size_t)warp * WK * ROWB;  // one buffer of values per warp

  // A lane's part of the k index: of every 32 values of a row it holds the 8 from 8 c on (k-steps 2 s and
  // 2 s + 1 take two pairs each); of a last 16 alone, the instruction's own pairs 2 c and 2 c + 8.
  constexpr int G32 = HD / 32;
  constexpr bool TAIL = HD % 32 != 0;
  uint32_t qf[G32 + 1][4];  // B operand: head g0 + g (zeros beyond the group)
  {
    const __nv_bfloat16* qrow = q + (size_t)g * HD;
#pragma unroll
    for (int s = 0; s < G32; ++s) {
      const uint4 v = g < ng ? *reinterpret_cast<const uint4*>(qrow + 32 * s + 8 * c) : make_uint4(0, 0, 0, 0);
      qf[s][0] = v.x; qf[s][1] = v.y; qf[s][2] = v.z; qf[s][3] = v.w;
    }
    if (TAIL) {
      const uint32_t* t = reinterpret_cast<const uint32_t*>(qrow + 32 * G32 + 2 * c);
      qf[G32][0] = g < ng ? t[0] : 0u;
      qf[G32][1] = g < ng ? t[4] : 0u;
      qf[G32][2] = qf[G32][3] = 0u;
    }
  }
  float o[HD / 16][4];  // O^T: element e of tile j is (value 16 j + g + 8 (e / 2), head 2 c + (e % 2))
#pragma unroll
  for (int j = 0; j < HD / 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};  // of heads 2 c and 2 c + 1; maximum in units of log2
  const float scale2 = a.scale * LOG2E;  // scores are kept times log2(e): exp(x) = exp2(x log2 e)

  bool first_block = true;
  constexpr int WT = WK / 16;  // mma tiles of 16 keys a piece
  for (int piece = k_lo / WK + warp; piece * WK < k_hi; piece += NW) {
    const int first = piece * WK;  // position of the piece's first key
    const int blk = block_of(a, slot, first / BLK);
    if (blk < 0) continue;
    const size_t at = (((size_t)blk * a.kvheads + kvh) * BLK + first % BLK) * HD;
    const __nv_bfloat16* ksrc = kc + at;
    __syncwarp();  // the buffer is free: every lane is past the previous piece
    const bool whole = first >= k_lo && first + WK <= k_hi;  // every key of the piece counts: no masks
    const __nv_bfloat16* vsrc = vc + at;
    if (whole) {  // a lane copies piece (lane % PIECES) of the rows (lane / PIECES) + i (32 / PIECES): constant offsets
      if (32 % PIECES == 0) {  // the lanes of a warp cover whole rows
        constexpr int RSTEP = 32 % PIECES == 0 ? 32 / PIECES : 1;
        const int row0 = lane / PIECES, part = lane % PIECES;
        unsigned char* dst = vbuf + row0 * ROWB + part * 16;
        const __nv_bfloat16* src = vsrc + (size_t)row0 * HD + part * 8;
#pragma unroll
        for (int i = 0; i < WK / RSTEP; ++i) cp_async_16(dst + i * RSTEP * ROWB, src + (size_t)i * RSTEP * HD, true);
      } else {
        copy_block_async(vbuf, vsrc, first, k_lo, k_hi, lane, WK);
      }
    } else {
      copy_block_async(vbuf, vsrc, first, k_lo, k_hi, lane, WK);
    }
    cp_async_commit_group();
    // scores, 16 keys at a time: element e of tile t is (key 16 t + g + 8 (e / 2), head 2 c + (e % 2)).  Rows of
    // the block beyond the sequence are read too (they exist) and masked below.
    float st[WT][4];
    uint4 ka[2][G32 > 0 ? G32 : 1][2];
    uint32_t kt[2][2][2];
    auto load_keys = [&](int t) {
      const __nv_bfloat16* r0 = ksrc + (size_t)(16 * t + g) * HD;
      const __nv_bfloat16* r1 = r0 + 8 * HD;
#pragma unroll
      for (int s = 0; s < G32; ++s) {
        ka[t & 1][s][0] = *reinterpret_cast<const uint4*>(r0 + 32 * s + 8 * c);
        ka[t & 1][s][1] = *reinterpret_cast<const uint4*>(r1 + 32 * s + 8 * c);
      }
      if (TAIL) {
        const uint32_t* t0 = reinterpret_cast<const uint32_t*>(r0 + 32 * G32 + 2 * c);
        const uint32_t* t1 = reinterpret_cast<const uint32_t*>(r1 + 32 * G32 + 2 * c);
        kt[t & 1][0][0] = t0[0]; kt[t & 1][0][1] = t0[4];
        kt[t & 1][1][0] = t1[0]; kt[t & 1][1][1] = t1[4];
      }
    };
    load_keys(0);
#pragma unroll
    for (int t = 0; t < WT; ++t) {
      if (t + 1 < WT) load_keys(t + 1);
      st[t][0] = st[t][1] = st[t][2] = st[t][3] = 0.f;
#pragma unroll
      for (int s = 0; s < G32; ++s) {
        const uint4 k0 = ka[t & 1][s][0], k1 = ka[t & 1][s][1];
        const uint32_t a0[4] = {k0.x, k1.x, k0.y, k1.y}, a1[4] = {k0.z, k1.z, k0.w, k1.w};
        mma16816(st[t], a0, qf[s][0], qf[s][1]);
        mma16816(st[t], a1, qf[s][2], qf[s][3]);
      }
      if (TAIL) {
        const uint32_t a0[4] = {kt[t & 1][0][0], kt[t & 1][1][0], kt[t & 1][0][1], kt[t & 1][1][1]};
        mma16816(st[t], a0, qf[G32][0], qf[G32][1]);
      }
    }
    // raw scores; the scale (positive) goes into the exponent's multiply-add
    if (!whole) {
#pragma unroll
      for (int t = 0; t < WT; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int kpos = first + 16 * t + g + 8 * (e >> 1);
          if (kpos < k_lo || kpos >= k_hi) st[t][e] = -INFINITY;
        }
    }
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int t = 0; t < WT; ++t)
#pragma unroll
      for (int e = 0; e < 4; ++e) tile_max[e & 1] = fmaxf(tile_max[e & 1], st[t][e]);
    float alpha[2], psum[2] = {0.f, 0.f}, neg_m[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {  // over the keys: the lanes that differ in g
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 4));
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 8));
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 16));
      const float m_new = fmaxf(m[h], tile_max[h] * scale2);
      neg_m[h] = m_new == -INFINITY ? 0.f : -m_new;
      alpha[h] = ex2_approx(m[h] + neg_m[h]);  // 2^-inf = 0 while nothing has been seen
      m[h] = m_new;
    }
    uint32_t pb[WT][2];  // P^T as B operand of k-step t (keys 16 t ..): (keys 2 c, 2 c + 1 (+ 8); head g)
#pragma unroll
    for (int t = 0; t < WT; ++t) {
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        p[e] = ex2_approx(fmaf(st[t][e], scale2, neg_m[e & 1]));  // 2^-inf = 0 for a masked key
        psum[e & 1] += p[e];
      }
      pb[t][0] = movmatrix_trans(pack_bf16(p[0], p[1]));
      pb[t][1] = movmatrix_trans(pack_bf16(p[2], p[3]));
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 4);
      psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 8);
      psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 16);
      l[h] = l[h] * alpha[h] + psum[h];
    }
    if (!first_block) {  // nothing is accumulated yet in a warp's first block
#pragma unroll
      for (int j = 0; j < HD / 16; ++j) {
        o[j][0] *= alpha[0]; o[j][1] *= alpha[1]; o[j][2] *= alpha[0]; o[j][3] *= alpha[1];
      }
    }
    first_block = false;
    cp_async_wait_group<0>();
    __syncwarp();
    // V^T tiles of 16 values x 16 keys: matrix (lane >> 3) of the four is (values + 8 ((lane >> 3) & 1),
    // keys + 8 (lane >> 4)), its rows in shared memory are keys
#pragma unroll
    for (int t = 0; t < WT; ++t) {
      const unsigned char* vrow = vbuf + (16 * t + (lane & 7) + (lane >> 4) * 8) * ROWB + ((lane >> 3) & 1) * 16;
#pragma unroll
      for (int j = 0; j < HD / 16; ++j) {
        uint32_t av[4];
        ldmatrix_x4_trans(av, vrow + j * 32);
        mma16816(o[j], av, pb[t][0], pb[t][1]);
      }
    }
  }

  // merge the warps: each writes (m, l, o) of its 8 heads over its own buffer
  __syncwarp();
  float* wo = reinterpret_cast<float*>(vbuf);          // [8][HD]
  float* wml = wo + GROWS * HD;                        // [8][2]
#pragma unroll
  for (int j = 0; j < HD / 16; ++j) {
    wo[(2 * c) * HD + 16 * j + g] = o[j][0];
    wo[(2 * c + 1) * HD + 16 * j + g] = o[j][1];
    wo[(2 * c) * HD + 16 * j + g + 8] = o[j][2];
    wo[(2 * c + 1) * HD + 16 * j + g + 8] = o[j][3];
  }
  if (g == 0) {
    wml[2 * (2 * c)] = m[0]; wml[2 * (2 * c) + 1] = l[0];
    wml[2 * (2 * c + 1)] = m[1]; wml[2 * (2 * c + 1) + 1] = l[1];
  }
  __syncthreads();
  // a head's weights of the warps are taken once by each of the threads that share its values
  constexpr int TPH = NW * 32 / GROWS;  // threads per head
  const int r = tid / TPH;
  if (r < ng) {
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w)
      mm = fmaxf(mm, (reinterpret_cast<const float*>(smem_raw + (size_t)w * WK * ROWB) + GROWS * HD)[2 * r]);
    float f[NW], lsum = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float* wm = reinterpret_cast<const float*>(smem_raw + (size_t)w * WK * ROWB) + GROWS * HD;
      f[w] = wm[2 * r] == -INFINITY ? 0.f : ex2_approx(wm[2 * r] - mm);
      lsum += wm[2 * r + 1] * f[w];
    }
    const int head = kvh * group + g0 + r;
    const size_t at = ((size_t)seq * a.nheads + head) * n_splits + split;
    if (n_splits == 1) {  // nothing to merge with: this is the result (no second kernel is launched)
      __nv_bfloat16* out = (__nv_bfloat16*)a.out + (size_t)a.first_row[seq] * a.nheads * HD + (size_t)head * HD;
      const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
      for (int d = tid % TPH; d < HD; d += TPH) {
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w)
          sum += reinterpret_cast<const float*>(smem_raw + (size_t)w * WK * ROWB)[r * HD + d] * f[w];
        out[d] = __float2bfloat16_rn(sum * inv);
      }
    } else {
      for (int d = tid % TPH; d < HD; d += TPH) {
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w)
          sum += reinterpret_cast<const float*>(smem_raw + (size_t)w * WK * ROWB)[r * HD + d] * f[w];
        if (FMS_IN(at, (size_t)gridDim.x * a.nheads * n_splits)) part_o[at * HD + d] = sum;
      }
      if (tid % TPH == 0 && FMS_IN(at, (size_t)gridDim.x * a.nheads * n_splits)) {
        part_ml[at * 2] = mm * (1.f / LOG2E);  // back to natural units, which attn_combine_kernel expects
        part_ml[at * 2 + 1] = lsum;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// prefill: grid (query tiles, kv heads * head chunks), 4 warps.  The 64 rows of a block are P positions x GH
// query heads that share the kv head (row = position * GH + head; GH = min(group, 64), P = 64 / GH), so a key
// or value block is loaded once for all of them.  Each warp owns 16 rows; the warps share the key and value
// blocks, which are copied into shared memory two blocks ahead of use (cp.async, two stages).
// ---------------------------------------------------------------------------------------------------
constexpr int PF_WARPS = 4;
constexpr int PF_ROWS = 16 * PF_WARPS;

__host__ __device__ inline int prefill_heads_per_block(int group) { return group < PF_ROWS ? group : PF_ROWS; }
__host__ __device__ inline int prefill_positions_per_block(int group) { return PF_ROWS / prefill_heads_per_block(group); }

__global__ void __launch_bounds__(PF_WARPS * 32, HD <= 128 ? 3 : 1) attn_prefill_mma_kernel(AttnArgs a, const int* __restrict__ tiles) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
  const int group = a.nheads / a.kvheads;
  const int gh = prefill_heads_per_block(group), pp = PF_ROWS / gh;
  const int chunks = (group + gh - 1) / gh;
  const int kvh = blockIdx.y / chunks, g0 = (blockIdx.y - kvh * chunks) * gh;
  const int ng = min(gh, group - g0);
  const int seq = tiles[2 * blockIdx.x], r0 = tiles[2 * blockIdx.x + 1];
  const int row_begin = a.first_row[seq];
  const int n_new = a.first_row[seq + 1] - row_begin;
  const int len = a.len_after[seq];
  const int len_before = len - n_new;
  const int slot = a.slots[seq];
  const int pos_here = min(pp, n_new - r0);       // positions of this tile
  const int p_first = len_before + r0, p_last = p_first + pos_here - 1;
  const __nv_bfloat16* q = (const __nv_bfloat16*)a.q;
  const __nv_bfloat16* kc = (const __nv_bfloat16*)a.keys;
  const __nv_bfloat16* vc = (const __nv_bfloat16*)a.values;

  // the two rows of this lane: tile row -> (position index, head index)
  int row_pos[2];
  bool row_ok[2];
  const __nv_bfloat16* qrow[2];
  __nv_bfloat16* orow[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + g + 8 * h;
    const int pi = r / gh, gi = r - pi * gh;
    row_ok[h] = pi < pos_here && gi < ng;
    row_pos[h] = p_first + pi;
    const size_t at = ((size_t)(row_begin + r0 + (row_ok[h] ? pi : 0)) * a.nheads + kvh * group + g0 + (row_ok[h] ? gi : 0)) * HD;
    qrow[h] = q + at;
    orow[h] = (__nv_bfloat16*)a.out + at;
  }
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int s = 0; s < HD / 16; ++s) {
    const uint32_t* q0 = reinterpret_cast<const uint32_t*>(qrow[0] + 16 * s + 2 * c);
    const uint32_t* q1 = reinterpret_cast<const uint32_t*>(qrow[1] + 16 * s + 2 * c);
    qf[s][0] = row_ok[0] ? q0[0] : 0u;
    qf[s][1] = row_ok[1] ? q1[0] : 0u;
    qf[s][2] = row_ok[0] ? q0[4] : 0u;
    qf[s][3] = row_ok[1] ? q1[4] : 0u;
  }
  float o[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};  // running maximum in units of log2, and sum
  const float scale2 = a.scale * LOG2E;  // scores are kept times log2(e): exp(x) = exp2(x log2 e)

  const int kb_lo = a.window > 0 ? max(0, p_first - a.window + 1) / BLK : 0;
  const int kb_hi = p_last / BLK;
  const int nblocks = kb_hi - kb_lo + 1;
  constexpr int STAGE = 2 * BLK * ROWB;
  auto issue = [&](int i) {  // copies block kb_lo + i into stage i % 2 (all threads take part)
    if (i < nblocks) {
      const int kb = kb_lo + i;
      const int blk = block_of(a, slot, kb);
      unsigned char* kbuf = smem_raw + (size_t)(i & 1) * STAGE;
      unsigned char* vbuf = kbuf + BLK * ROWB;
      const __nv_bfloat16* ksrc = kc + ((size_t)max(blk, 0) * a.kvheads + kvh) * BLK * HD;
      const __nv_bfloat16* vsrc = vc + ((size_t)max(blk, 0) * a.kvheads + kvh) * BLK * HD;
      for (int p = tid; p < BLK * PIECES; p += PF_WARPS * 32) {
        const int row = p / PIECES, piece = p - row * PIECES;
        const bool valid = blk >= 0 && kb * BLK + row < len;
        cp_async_16(kbuf + row * ROWB + piece * 16, ksrc + (size_t)row * HD + piece * 8, valid);
        cp_async_16(vbuf + row * ROWB + piece * 16, vsrc + (size_t)row * HD + piece * 8, valid);
      }
    }
    cp_async_commit_group();
  };
  issue(0);
  issue(1);
  for (int i = 0; i < nblocks; ++i) {
    const int kb = kb_lo + i;
    cp_async_wait_group<1>();
    __syncthreads();
    const unsigned char* kbuf = smem_raw + (size_t)(i & 1) * STAGE;
    const unsigned char* vbuf = kbuf + BLK * ROWB;
    float s[8][4];
    scores_16x64(s, qf, kbuf, lane);
    // a block that every row of the tile sees whole needs no mask
    const bool whole = kb * BLK + BLK - 1 <= p_first && (a.window <= 0 || kb * BLK > p_last - a.window);
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        const int kpos = kb * BLK + 8 * j + 2 * c + (e & 1);
        const bool visible = whole || (kpos <= row_pos[h] && (a.window <= 0 || kpos > row_pos[h] - a.window));
        s[j][e] = (visible && row_ok[h]) ? s[j][e] * scale2 : -INFINITY;
        tile_max[h] = fmaxf(tile_max[h], s[j][e]);
      }
    float alpha[2], psum[2] = {0.f, 0.f}, m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
      const float m_new = fmaxf(m[r], tile_max[r]);
      m_use[r] = m_new == -INFINITY ? 0.f : m_new;
      alpha[r] = m[r] == -INFINITY ? 0.f : exp2f(m[r] - m_use[r]);
      m[r] = m_new;
    }
    uint32_t pf[4][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        p[e] = s[j][e] == -INFINITY ? 0.f : exp2f(s[j][e] - m_use[e >> 1]);
        psum[e >> 1] += p[e];
      }
      pf[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p[0], p[1]);
      pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 1);
      psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 2);
      l[r] = l[r] * alpha[r] + psum[r];
    }
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) {
      o[j][0] *= alpha[0]; o[j][1] *= alpha[0]; o[j][2] *= alpha[1]; o[j][3] *= alpha[1];
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const unsigned char* vrow = vbuf + (16 * t + (lane & 7) + ((lane >> 3) & 1) * 8) * ROWB + (lane >> 4) * 16;
#pragma unroll
      for (int jd = 0; jd < HD / 8; jd += 2) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vrow + jd * 16);
        mma16816(o[jd], pf[t], b[0], b[1]);
        mma16816(o[jd + 1], pf[t], b[2], b[3]);
      }
    }
    __syncthreads();  // every warp is done with this stage
    issue(i + 2);
  }
  cp_async_wait_group<0>();
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (!row_ok[h]) continue;
    const float inv = l[h] > 0.f ? 1.f / l[h] : 0.f;
#pragma unroll
    for (int j = 0; j < HD / 8; ++j)
      *reinterpret_cast<uint32_t*>(orow[h] + 8 * j + 2 * c) = pack_bf16(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
  }
}

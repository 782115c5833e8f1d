// Causal grouped-query prefill attention on the 5th-generation tensor cores (tcgen05).
// Included by attention_mma.cu (one head size per library; this form needs D == 128 or 64,
// 128 % heads-per-kv-head == 0 and a page size that divides 64).
//
// Upstream computes prefill attention with eager torch ops - scores, 32-bit softmax, value
// product (src/forge_engine/qwen3.py:187-206) - and has a Triton lab kernel with an online
// softmax (src/forge_engine/_triton_kernels.py:89-158).  This is the same math as a
// flash-attention tile loop, with both products on tcgen05:
//
//   block = 128 query rows (row = token * G + head in group) of one (entry, kv head)
//   warp 0   TMA producer: the query tile once (3-D box: 64 columns x G heads x 128/G tokens),
//            then per 64-key tile one box per page and 64-column block for K and for V
//   warp 1   MMA issuer: S[128 x 64] = Q K^T into tensor memory; after the softmax warps
//            have stored P (bfloat16, in tensor memory) O[128 x D] += P V, V read MN-major
//   warps 2-5  softmax: thread = row.  Loads its row of S, masks, keeps a running maximum
//            and sum in 32-bit, writes P; rescales O only when the maximum has grown by
//            more than 2^8 (the final division by the sum makes this exact); at the end
//            normalises O and stores it
//   Scores and probabilities are double-buffered in tensor memory: the scores of tile t+1
//   (and t+2) are computed while the softmax warps still work on tile t, so the tensor
//   core never waits for the softmax and the softmax only for its own arithmetic.
#pragma once

namespace {

constexpr int TC5_ROWS = 128;       // query rows per block
constexpr int TC5_KEYS = 64;        // keys per tile
constexpr int TC5_THREADS = 192;
constexpr int TC5_KV_STAGES = 4;
constexpr int TC5_TMEM_COLS = 512;
constexpr int TC5_COL_S = 0;        // 2 x 64 columns of 32-bit scores
constexpr int TC5_COL_P = 128;      // 2 x 32 columns holding 64 bfloat16 probabilities each
constexpr int TC5_COL_O = 256;      // D columns of 32-bit output accumulators (D <= 128)
constexpr float TC5_RESCALE_STEP = 8.f;   // in log2 units

constexpr int TC5_Q_BYTES = TC5_ROWS * D * 2;
constexpr int TC5_KV_BYTES = TC5_KEYS * D * 2;   // one matrix of one stage
constexpr size_t TC5_SMEM = (size_t)TC5_Q_BYTES + (size_t)2 * TC5_KV_STAGES * TC5_KV_BYTES + 24 * 8 + 64 + 1024;

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_addr(dst)), "l"(map), "r"(smem_addr(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

// K-major operand tile: rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t tc5_desc_kmajor(const void* tile) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr(tile) & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// MN-major operand tile (the N index runs along a 128-byte row): blocks of 64 N-elements
// `block_bytes` apart, 8-row (k) groups 1024 bytes apart.
__device__ __forceinline__ uint64_t tc5_desc_mnmajor(const void* tile, unsigned block_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr(tile) & 0x3FFFFu) >> 4);
  d |= (uint64_t)(block_bytes >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ unsigned tc5_idesc(int m, int n, bool b_mn_major) {
  unsigned d = 0;
  d |= 1u << 4;                    // f32 accumulate
  d |= 1u << 7;                    // A bf16
  d |= 1u << 10;                   // B bf16
  if (b_mn_major) d |= 1u << 16;
  d |= (unsigned)(n >> 3) << 17;
  d |= (unsigned)(m >> 4) << 24;
  return d;
}
__device__ __forceinline__ void tc5_mma_ss(unsigned tmem_d, uint64_t da, uint64_t db, unsigned idesc, unsigned acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void tc5_mma_ts(unsigned tmem_d, unsigned tmem_a, uint64_t db, unsigned idesc, unsigned acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
// 2^x by the special-function unit's single instruction (the bfloat16 path rounds the
// result to 8 bits anyway); exp2f() costs several times as many instructions.
__device__ __forceinline__ float tc5_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tc5_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tc5_ld32(unsigned taddr, float (&v)[32]) {
  unsigned r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tc5_st32(unsigned taddr, const unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__global__ void __launch_bounds__(TC5_THREADS)
attn_prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, AttnParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* q_tile = smem;                                   // [D/64][128 rows][128 B]
  unsigned char* k_tiles = q_tile + TC5_Q_BYTES;                  // [stages][D/64][64 keys][128 B]
  unsigned char* v_tiles = k_tiles + TC5_KV_STAGES * TC5_KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_tiles + TC5_KV_STAGES * TC5_KV_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;                 // [stages]
  uint64_t* kv_empty = kv_full + TC5_KV_STAGES; // [stages]
  uint64_t* s_full = kv_empty + TC5_KV_STAGES;   // [2]
  uint64_t* p_full = s_full + 2;                 // [2]
  uint64_t* pv_done = p_full + 2;                // completes once per value product
  uint64_t* o_full = pv_done + 1;
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(o_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  pdl_trigger();
  const int entry = blockIdx.y, kvh = blockIdx.z;
  const int tok0 = p.cu_tokens[entry];
  const int n_new = p.cu_tokens[entry + 1] - tok0;
  const int rows_total = n_new * p.groups;
  if (rows_total <= p.row_lo || rows_total > p.row_hi) return;
  const int row0 = (gridDim.x - 1 - blockIdx.x) * TC5_ROWS;      // long tiles first
  if (row0 >= rows_total) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int start = p.starts[entry];
  const int* table = p.block_table + (size_t)entry * p.max_pages;

  const int last_row = min(rows_total, row0 + TC5_ROWS) - 1;
  const int pos_first = start + row0 / p.groups;
  const int pos_last = start + last_row / p.groups;
  const int key_lo = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
  const int key_end = pos_last + 1;
  const int tile_begin = key_lo / TC5_KEYS, tile_end = (key_end + TC5_KEYS - 1) / TC5_KEYS;
  const int my_tiles = tile_end - tile_begin;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < TC5_KV_STAGES; ++s) { mbar_init(kv_full + s, 1); mbar_init(kv_empty + s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(s_full + b, 1); mbar_init(p_full + b, 4); }
    mbar_init(pv_done, 1);
    mbar_init(o_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)),
                 "r"(TC5_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- producer ----
    pdl_wait();
    if (lane == 0) {
      mbar_expect_tx(q_full, TC5_Q_BYTES);
#pragma unroll
      for (int blk = 0; blk < D / 64; ++blk)
        tma_load_3d(q_tile + blk * (TC5_ROWS * 128), &map_q, blk * 64 + kvh * p.groups * D, 0, tok0 + row0 / p.groups, q_full);
    }
    const int pages_per_tile = TC5_KEYS / p.page_size;
    const int rows_in_cache = p.num_pages * p.nkv * p.page_size;
    const int first_logical = tile_begin * pages_per_tile;
    const int total_pages = my_tiles * pages_per_tile;
    bool dead = false;
    for (int base = 0; base < total_pages; base += 32) {
      const int logical = first_logical + base + lane;
      const int key = logical * p.page_size;
      int my_row = rows_in_cache;            // outside the tensor: zeros
      if (base + lane < total_pages && key < key_end) {
        const int page = logical < p.max_pages ? table[logical] : -1;
        if (page >= 0 && page < p.num_pages) my_row = (page * p.nkv + kvh) * p.page_size;
        else if (key + p.page_size > key_lo) atomicOr(p.status, FE_STATUS_BAD_PAGE);
      }
      const int count = min(32, total_pages - base);
      for (int j = 0; j < count; ++j) {
        const int row = __shfl_sync(0xffffffffu, my_row, j);
        if (lane == 0 && !dead) {
          const int index = base + j;
          const int i = index / pages_per_tile, pg = index - i * pages_per_tile;
          const int s = i % TC5_KV_STAGES;
          if (pg == 0) {
            if (i >= TC5_KV_STAGES && !mbar_wait(kv_empty + s, ((i / TC5_KV_STAGES) & 1) ^ 1, abort_flag)) dead = true;
            if (!dead) mbar_expect_tx(kv_full + s, 2 * TC5_KV_BYTES);
          }
          if (!dead) {
#pragma unroll
            for (int blk = 0; blk < D / 64; ++blk) {
              const int offset = blk * (TC5_KEYS * 128) + pg * p.page_size * 128;
              tma_load_2d(k_tiles + s * TC5_KV_BYTES + offset, &map_k, blk * 64, row, kv_full + s);
              tma_load_2d(v_tiles + s * TC5_KV_BYTES + offset, &map_v, blk * 64, row, kv_full + s);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (lane == 0) {
      const unsigned idesc_qk = tc5_idesc(TC5_ROWS, TC5_KEYS, false);
      const unsigned idesc_pv = tc5_idesc(TC5_ROWS, D, true);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      // scores of tile t into buffer t % 2
      auto issue_scores = [&](int t) -> bool {
        const int s = t % TC5_KV_STAGES;
        if (!mbar_wait(kv_full + s, (t / TC5_KV_STAGES) & 1, abort_flag)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          // k = 16 is 32 bytes along the swizzled row, 4 steps per 64-column block
          const uint64_t da = tc5_desc_kmajor(q_tile + (kk >> 2) * (TC5_ROWS * 128)) + (uint64_t)((kk & 3) * 2);
          const uint64_t db = tc5_desc_kmajor(k_tiles + s * TC5_KV_BYTES + (kk >> 2) * (TC5_KEYS * 128)) + (uint64_t)((kk & 3) * 2);
          tc5_mma_ss(tmem_base + TC5_COL_S + (t & 1) * TC5_KEYS, da, db, idesc_qk, kk != 0 ? 1u : 0u);
        }
        tc5_commit(s_full + (t & 1));
        return true;
      };
      if (ok) ok = issue_scores(0);
      if (ok && my_tiles > 1) ok = issue_scores(1);
      for (int i = 0; i < my_tiles && ok; ++i) {
        const int s = i % TC5_KV_STAGES;
        ok = mbar_wait(p_full + (i & 1), (i >> 1) & 1, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // O += P V : 4 steps of 16 keys; V is MN-major, 16 keys = 2048 bytes further down
#pragma unroll
        for (int kk = 0; kk < TC5_KEYS / 16; ++kk) {
          const uint64_t db = tc5_desc_mnmajor(v_tiles + s * TC5_KV_BYTES + kk * 2048, TC5_KEYS * 128);
          tc5_mma_ts(tmem_base + TC5_COL_O, tmem_base + TC5_COL_P + (i & 1) * (TC5_KEYS / 2) + kk * 8, db, idesc_pv,
                     (i | kk) != 0 ? 1u : 0u);
        }
        tc5_commit(kv_empty + s);     // the stage may be refilled when these products are done
        tc5_commit(pv_done);
        if (i + 2 < my_tiles) ok = issue_scores(i + 2);
      }
      tc5_commit(o_full);
    }
  } else {
    // ---- softmax: thread = row ----
    pdl_wait();
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;                 // row inside the block = tensor-memory lane
    const int row = row0 + r;
    const bool row_valid = row < rows_total;
    const int pos = row_valid ? start + row / p.groups : -1;
    const unsigned lane_addr = tmem_base + ((unsigned)(quarter * 32) << 16);
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int i = 0; i < my_tiles && ok; ++i) {
      ok = mbar_wait(s_full + (i & 1), (i >> 1) & 1, abort_flag);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int key0 = (tile_begin + i) * TC5_KEYS;
      float s0[32], s1[32];
      tc5_ld32(lane_addr + TC5_COL_S + (i & 1) * TC5_KEYS, s0);
      tc5_ld32(lane_addr + TC5_COL_S + (i & 1) * TC5_KEYS + 32, s1);
      // every key of the tile visible to every row of the block?
      const bool clear = key0 + TC5_KEYS - 1 <= pos_first && key0 + TC5_KEYS <= key_end && row0 + TC5_ROWS <= rows_total &&
                         (p.window <= 0 || pos_last - key0 < p.window);
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        float a = s0[j] * p.scale_log2, b = s1[j] * p.scale_log2;
        if (!clear) {
          const int ka = key0 + j, kb = key0 + 32 + j;
          if (!(ka <= pos && ka < key_end && (p.window <= 0 || pos - ka < p.window))) a = -INFINITY;
          if (!(kb <= pos && kb < key_end && (p.window <= 0 || pos - kb < p.window))) b = -INFINITY;
        }
        s0[j] = a; s1[j] = b;
        mx = fmaxf(mx, fmaxf(a, b));
      }
      // the running maximum only moves when it has to grow by more than the step
      float corr = 1.f;
      if (mx > m_used + TC5_RESCALE_STEP || m_used == -INFINITY) {
        if (mx != -INFINITY) {
          corr = (m_used == -INFINITY) ? 0.f : exp2f(m_used - mx);
          m_used = mx;
        }
      }
      const float base = (m_used == -INFINITY) ? 0.f : m_used;
      float sum = 0.f;
      unsigned packed[32];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float a0 = tc5_exp2(s0[2 * j] - base), a1 = tc5_exp2(s0[2 * j + 1] - base);
        const float b0 = tc5_exp2(s1[2 * j] - base), b1 = tc5_exp2(s1[2 * j + 1] - base);
        sum += (a0 + a1) + (b0 + b1);
        packed[j] = pack_bf16(a0, a1);
        packed[16 + j] = pack_bf16(b0, b1);
      }
      l = l * corr + sum;
      // the scores of this tile were issued after the value product of tile i - 2, which
      // read this P buffer: it is free.  O is only touched once product i - 1 has finished.
      tc5_st32(lane_addr + TC5_COL_P + (i & 1) * (TC5_KEYS / 2), packed);
      if (i > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
        if (!mbar_wait(pv_done, (i - 1) & 1, abort_flag)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          float o[32];
          tc5_ld32(lane_addr + TC5_COL_O + c, o);
          unsigned bits[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) bits[j] = __float_as_uint(o[j] * corr);
          tc5_st32(lane_addr + TC5_COL_O + c, bits);
        }
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full + (i & 1));
    }
    // final: normalise and store this row
    if (ok) ok = mbar_wait(o_full, 0, abort_flag);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const int num_q_heads = p.nkv * p.groups;
      const int token = row / p.groups, g = row - token * p.groups;
      bf16* dst = p.out + ((size_t)(tok0 + token) * num_q_heads + kvh * p.groups + g) * D;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        float o[32];
        tc5_ld32(lane_addr + TC5_COL_O + c, o);
        if (row_valid) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            float v8[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v8[e] = o[j + e] * inv;
            store8(dst + c + j, v8);
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TC5_TMEM_COLS) : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag) atomicOr(p.status, FE_STATUS_WAIT_TIMEOUT);
}

// Tensor map of the step's queries of one kv head's group: [tokens][G heads][D], the token
// stride being the fused projection's row.  Box: 64 columns x G heads x 128/G tokens.
int make_query_map(CUtensorMap* map, const void* q, int q_stride, int tokens, int num_q_heads, int groups) {
  if (g_encode_tiled == nullptr) return FE_ERR_BAD_SHAPE;
  cuuint64_t dims[3] = {(cuuint64_t)num_q_heads * D, (cuuint64_t)groups, (cuuint64_t)tokens};
  // dimension 1 steps over the heads of a group: D elements; dimension 2 over tokens
  cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)q_stride * 2};
  cuuint32_t box[3] = {64u, (cuuint32_t)groups, (cuuint32_t)(TC5_ROWS / groups)};
  cuuint32_t elem[3] = {1, 1, 1};
  const CUresult r = g_encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box,
                                    elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 20000 + (int)r;
}

}  // namespace

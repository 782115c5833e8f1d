// Causal grouped-query prefill attention on the 5th-generation tensor cores (tcgen05).
// Included by attention_mma.cu (one head size per library; this form needs D == 128 or 64,
// 128 % heads-per-kv-head == 0 and a page size of 4..128 that divides 128).
//
// Upstream computes prefill attention with eager torch ops - scores, 32-bit softmax, value
// product (src/forge_engine/qwen3.py:187-206) - and has a Triton lab kernel with an online
// softmax (src/forge_engine/_triton_kernels.py:89-158).  This is the same math as a
// flash-attention tile loop, with both products on tcgen05:
//
//   block = two query tiles of 128 rows (row = token * G + head in group) of one (entry,
//           kv head); both tiles use the same key and value tiles of 128 keys
//   warp 0   TMA producer: the query tiles once (3-D boxes: 64 columns x G heads x 128/G
//            tokens), then per key tile one box per page and 64-column block, K and V in
//            rings of their own (a lane per page)
//   warp 1   MMA issuer: S_x[128 x 128] = Q_x K^T into tensor memory; after tile x's softmax
//            warps have stored P_x (bfloat16, over the first half of S_x's columns)
//            O_x[128 x D] += P_x V, V read MN-major; then at once the scores of the next
//            key tile for x, so that they are ready when the other tile's products end
//   warps 2-5, 6-9  softmax of tile 0 and of tile 1: thread = row.  Loads its row of S,
//            masks, keeps a running maximum and sum in 32-bit, writes P; rescales O only
//            when the maximum has grown by more than 2^8 (the final division by the sum
//            makes this exact); at the end normalises O and stores it
//   While one tile's rows are in the softmax the tensor core works on the other tile.
#pragma once

namespace {

constexpr int TC5_ROWS = 128;        // rows of one query tile
constexpr int TC5_BLOCK_ROWS = 256;  // two query tiles per block
constexpr int TC5_KEYS = 128;        // keys per tile
constexpr int TC5_THREADS = 320;
constexpr int TC5_K_STAGES = 2;      // key tiles in flight
constexpr int TC5_V_STAGES = 3;      // value tiles in flight: a value tile is needed a whole step after its keys
constexpr int TC5_TMEM_COLS = 512;
constexpr int TC5_COL_S = 0;         // + 128 x: 128 columns of 32-bit scores; P over the first 64
constexpr int TC5_COL_O = 256;       // + 128 x: D columns of 32-bit output accumulators
constexpr float TC5_RESCALE_STEP = 8.f;   // in log2 units

constexpr int TC5_Q_BYTES = TC5_ROWS * D * 2;    // one query tile
constexpr int TC5_KV_BYTES = TC5_KEYS * D * 2;   // one matrix of one stage
constexpr size_t TC5_SMEM_USED = (size_t)2 * TC5_Q_BYTES + (size_t)(TC5_K_STAGES + TC5_V_STAGES) * TC5_KV_BYTES + 24 * 8 + 64 + 1024;
// one block per SM whatever the head size: a block takes all of the SM's tensor memory
constexpr size_t TC5_SMEM = TC5_SMEM_USED > 120 * 1024 ? TC5_SMEM_USED : 120 * 1024;

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
__device__ __forceinline__ void tc5_mma_ts(unsigned tmem_d, unsigned tmem_a, uint64_t db, unsigned idesc, unsigned acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void tc5_mma_ss_first(unsigned tmem_d, uint64_t da, uint64_t db, unsigned idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc) : "memory");
}
__device__ __forceinline__ void tc5_mma_ss_acc(unsigned tmem_d, uint64_t da, uint64_t db, unsigned idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.eq.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc) : "memory");
}
__device__ __forceinline__ void tc5_mma_ts_acc(unsigned tmem_d, unsigned tmem_a, uint64_t db, unsigned idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.eq.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc) : "memory");
}
// 2^x by the special-function unit's single instruction (the bfloat16 path rounds the
// result to 8 bits anyway); exp2f() costs several times as many instructions.
__device__ __forceinline__ float tc5_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float tc5_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// two 32-bit floats in one 64-bit register pair, for the packed 32-bit instructions
__device__ __forceinline__ uint64_t tc5_pair(float lo, float hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ void tc5_unpair(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t tc5_fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t tc5_add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
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

__device__ __forceinline__ void tc5_ld32_issue(unsigned taddr, unsigned* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tc5_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc5_st16(unsigned taddr, const unsigned (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// The key range of one query tile, in key tiles of the block's own numbering.
struct Tc5Tile {
  bool valid;
  int row0, pos_first, pos_last, key_end, tile_begin, tile_end;
};
__device__ __forceinline__ Tc5Tile tc5_tile(int row0, int rows_total, int start, int groups, int window) {
  Tc5Tile t;
  t.row0 = row0;
  t.valid = row0 < rows_total;
  const int last_row = min(rows_total, row0 + TC5_ROWS) - 1;
  t.pos_first = start + row0 / groups;
  t.pos_last = start + last_row / groups;
  const int key_lo = window > 0 ? max(0, t.pos_first - window + 1) : 0;
  t.key_end = t.pos_last + 1;
  t.tile_begin = key_lo / TC5_KEYS;
  t.tile_end = (t.key_end + TC5_KEYS - 1) / TC5_KEYS;
  return t;
}

__global__ void __launch_bounds__(TC5_THREADS, 1)
attn_prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, AttnParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* q_tiles = smem;                                  // [2][D/64][128 rows][128 B]
  unsigned char* k_tiles = q_tiles + 2 * TC5_Q_BYTES;             // [stages][D/64][128 keys][128 B]
  unsigned char* v_tiles = k_tiles + TC5_K_STAGES * TC5_KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_tiles + TC5_V_STAGES * TC5_KV_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;                   // [key stages]
  uint64_t* v_full = k_full + TC5_K_STAGES;      // [value stages]
  // freed[n & 3], event n: the tensor core has finished everything issued up to the end of key
  // tile n - 1 (event 0: the first scores).  Then the stage of value tile n - 1 and the stage of
  // key tile n may be filled again.  One commit a key tile instead of one per ring: every
  // commit and every wait is time the issuing thread does not issue in.
  uint64_t* freed = v_full + TC5_V_STAGES;       // [4]
  uint64_t* s_full = freed + 4;                  // [2 query tiles]
  uint64_t* p_full = s_full + 2;                 // [2]
  uint64_t* o_full = p_full + 2;
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(o_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  pdl_trigger();
  const int entry = blockIdx.y, kvh = blockIdx.x;
  const int tok0 = p.cu_tokens[entry];
  const int n_new = p.cu_tokens[entry + 1] - tok0;
  const int rows_total = n_new * p.groups;
  if (rows_total <= p.row_lo || rows_total > p.row_hi) return;
  // blocks start in the order of blockIdx.x, y, z: the long query blocks of every head first
  const int row0 = (gridDim.z - 1 - blockIdx.z) * TC5_BLOCK_ROWS;
  if (row0 >= rows_total) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int start = p.starts[entry];
  const int* table = p.block_table + (size_t)entry * p.max_pages;

  // tile 1 holds later tokens: its keys start no earlier and end no earlier than tile 0's
  const Tc5Tile t0 = tc5_tile(row0, rows_total, start, p.groups, p.window);
  const Tc5Tile t1 = tc5_tile(row0 + TC5_ROWS, rows_total, start, p.groups, p.window);
  const int tile_begin = t0.tile_begin;
  const int tile_end = t1.valid ? t1.tile_end : t0.tile_end;
  const int n_tiles = tile_end - tile_begin;
  const int key_end = t1.valid ? t1.key_end : t0.key_end;
  const int key_lo = p.window > 0 ? max(0, t0.pos_first - p.window + 1) : 0;
  // does query tile x take part in key tile i (counted from tile_begin)?
  auto active = [&](int x, int i) -> bool {
    return x == 0 ? (tile_begin + i < t0.tile_end) : (t1.valid && tile_begin + i >= t1.tile_begin);
  };

  if (threadIdx.x == 0) {
    tma_prefetch_map(&map_q);
    tma_prefetch_map(&map_k);
    tma_prefetch_map(&map_v);
    mbar_init(q_full, 1);
    for (int s = 0; s < TC5_K_STAGES; ++s) mbar_init(k_full + s, 1);
    for (int s = 0; s < TC5_V_STAGES; ++s) mbar_init(v_full + s, 1);
    for (int s = 0; s < 4; ++s) mbar_init(freed + s, 1);
    for (int x = 0; x < 2; ++x) { mbar_init(s_full + x, 1); mbar_init(p_full + x, 4); }
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
      mbar_expect_tx(q_full, t1.valid ? 2 * TC5_Q_BYTES : TC5_Q_BYTES);
      for (int x = 0; x < (t1.valid ? 2 : 1); ++x)
#pragma unroll
        for (int blk = 0; blk < D / 64; ++blk)
          tma_load_3d(q_tiles + x * TC5_Q_BYTES + blk * (TC5_ROWS * 128), &map_q, blk * 64 + kvh * p.groups * D, 0,
                      tok0 + (row0 + x * TC5_ROWS) / p.groups, q_full);
    }
    const int pages_per_tile = TC5_KEYS / p.page_size;          // <= 32: a lane per page
    const int rows_in_cache = p.num_pages * p.nkv * p.page_size;
    bool ok = true;
    for (int i = 0; i < n_tiles && ok; ++i) {
      const int ks = i % TC5_K_STAGES, vs = i % TC5_V_STAGES;
      const int logical = (tile_begin + i) * pages_per_tile + lane;
      const int key = logical * p.page_size;
      int row = rows_in_cache;            // outside the tensor: zeros
      if (lane < pages_per_tile && key < key_end) {
        const int page = logical < p.max_pages ? table[logical] : -1;
        if (page >= 0 && page < p.num_pages) row = (page * p.nkv + kvh) * p.page_size;
        else if (key + p.page_size > key_lo) atomicOr(p.status, FE_STATUS_BAD_PAGE);
      }
      const int offset = lane * p.page_size * 128;
      // keys; from the third tile on both stages were in use before: key tile i - 2 and value
      // tile i - 3 are free after event i - 2
      if (lane == 0) {
        if (i >= 2) ok = mbar_wait(freed + ((i - 2) & 3), ((i - 2) >> 2) & 1, abort_flag);
        if (ok) mbar_expect_tx(k_full + ks, TC5_KV_BYTES);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane < pages_per_tile) {
#pragma unroll
        for (int blk = 0; blk < D / 64; ++blk)
          tma_load_2d(k_tiles + ks * TC5_KV_BYTES + blk * (TC5_KEYS * 128) + offset, &map_k, blk * 64, row, k_full + ks);
      }
      // values
      if (lane == 0) mbar_expect_tx(v_full + vs, TC5_KV_BYTES);
      if (lane < pages_per_tile) {
#pragma unroll
        for (int blk = 0; blk < D / 64; ++blk)
          tma_load_2d(v_tiles + vs * TC5_KV_BYTES + blk * (TC5_KEYS * 128) + offset, &map_v, blk * 64, row, v_full + vs);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (lane == 0) {
      const unsigned idesc_qk = tc5_idesc(TC5_ROWS, TC5_KEYS, false);
      const unsigned idesc_pv = tc5_idesc(TC5_ROWS, D, true);
      // descriptors differ in their low word only (the address in 16-byte units): tiles of
      // 64 columns lie rows x 128 bytes apart, 16 columns of a swizzled row 32 bytes
      const uint64_t q_desc = tc5_desc_kmajor(q_tiles), k_desc = tc5_desc_kmajor(k_tiles);
      const uint64_t v_desc = tc5_desc_mnmajor(v_tiles, TC5_KEYS * 128);
      // S_x = Q_x K(t)^T; the keys' stage must be full
      auto issue_scores = [&](int x, int t) {
        const uint64_t qa = q_desc + (uint64_t)(x * (TC5_Q_BYTES >> 4));
        const uint64_t kb = k_desc + (uint64_t)((t % TC5_K_STAGES) * (TC5_KV_BYTES >> 4));
        const unsigned dst = tmem_base + TC5_COL_S + x * TC5_KEYS;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t step_q = (uint64_t)(((kk >> 2) * (TC5_ROWS * 128) >> 4) + (kk & 3) * 2);
          const uint64_t step_k = (uint64_t)(((kk >> 2) * (TC5_KEYS * 128) >> 4) + (kk & 3) * 2);
          if (kk == 0) tc5_mma_ss_first(dst, qa, kb, idesc_qk);
          else tc5_mma_ss_acc(dst, qa + step_q, kb + step_k, idesc_qk);
        }
        tc5_commit(s_full + x);
      };
      unsigned done[2] = {0u, 0u};      // value products issued per query tile
      bool ok = mbar_wait(q_full, 0, abort_flag);
      if (ok) ok = mbar_wait(k_full, 0, abort_flag);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (active(0, 0)) issue_scores(0, 0);
        if (active(1, 0)) issue_scores(1, 0);
        tc5_commit(freed);
      }
      for (int i = 0; i < n_tiles && ok; ++i) {
        const int s = i % TC5_V_STAGES, next_k = (i + 1) % TC5_K_STAGES;
        const unsigned next_k_parity = ((i + 1) / TC5_K_STAGES) & 1;
        const bool more = i + 1 < n_tiles;
        // this tile's values and the next tile's keys: both were asked for long ago, and waiting
        // for them here keeps the waits out of the stretch between a tile's P and its next scores
        ok = mbar_wait(v_full + s, (i / TC5_V_STAGES) & 1, abort_flag);
        if (ok && more) ok = mbar_wait(k_full + next_k, next_k_parity, abort_flag);
#pragma unroll
        for (int x = 0; x < 2 && ok; ++x) {
          if (active(x, i)) {
            ok = mbar_wait(p_full + x, done[x] & 1, abort_flag);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // O_x += P_x V : 8 steps of 16 keys; V is MN-major, 16 keys = 2048 bytes further down
            const uint64_t vb = v_desc + (uint64_t)(s * (TC5_KV_BYTES >> 4));
            const unsigned o_dst = tmem_base + TC5_COL_O + x * 128, p_src = tmem_base + TC5_COL_S + x * TC5_KEYS;
            tc5_mma_ts(o_dst, p_src, vb, idesc_pv, done[x] != 0 ? 1u : 0u);
#pragma unroll
            for (int kk = 1; kk < TC5_KEYS / 16; ++kk)
              tc5_mma_ts_acc(o_dst, p_src + kk * 8, vb + (uint64_t)(kk * (2048 >> 4)), idesc_pv);
            ++done[x];
          }
          if (more && active(x, i + 1)) {
            // these scores overwrite P_x: the tensor core runs them after the product above
            issue_scores(x, i + 1);
          }
        }
        if (!ok) break;
        // event i + 1: value tile i and key tile i + 1 have been used by all that was issued
        if (more) tc5_commit(freed + ((i + 1) & 3));
      }
      tc5_commit(o_full);
    }
  } else {
    // ---- softmax: thread = row of query tile x ----
    pdl_wait();
    const int x = (warp - 2) >> 2;
    const Tc5Tile& mine = x == 0 ? t0 : t1;
    const int quarter = warp & 3;                      // the quarter of tensor memory this warp may touch
    const int r = quarter * 32 + lane;                 // row inside the tile = tensor-memory lane
    const int row = mine.row0 + r;
    const bool row_valid = row < rows_total;
    const int pos = row_valid ? start + row / p.groups : -1;
    const unsigned lane_addr = tmem_base + ((unsigned)(quarter * 32) << 16);
    const unsigned s_addr = lane_addr + TC5_COL_S + x * TC5_KEYS;
    const unsigned o_addr = lane_addr + TC5_COL_O + x * 128;
    float m_used = -INFINITY, l = 0.f;
    bool ok = mine.valid;
    unsigned count = 0;                                // key tiles this query tile has taken
    for (int i = 0; i < n_tiles && ok; ++i) {
      if (!active(x, i)) continue;
      ok = mbar_wait(s_full + x, count & 1, abort_flag);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int key0 = (tile_begin + i) * TC5_KEYS;
      unsigned raw[TC5_KEYS];
#pragma unroll
      for (int c = 0; c < TC5_KEYS / 32; ++c) tc5_ld32_issue(s_addr + c * 32, raw + c * 32);
      tc5_ld_wait();
      // every key of the tile visible to every row of the tile?
      const bool clear = key0 + TC5_KEYS - 1 <= mine.pos_first && key0 + TC5_KEYS <= mine.key_end &&
                         mine.row0 + TC5_ROWS <= rows_total && (p.window <= 0 || mine.pos_last - key0 < p.window);
      if (!clear) {
        // this row sees the keys j_lo..j_hi of the tile (none when the row is past the end)
        const int j_hi = min(pos, mine.key_end - 1) - key0;
        if (p.window > 0) {
          const int j_lo = pos - p.window + 1 - key0;
#pragma unroll
          for (int j = 0; j < TC5_KEYS; ++j) raw[j] = (j <= j_hi && j >= j_lo) ? raw[j] : 0xff800000u;   // -inf
        } else {
#pragma unroll
          for (int j = 0; j < TC5_KEYS; ++j) raw[j] = j <= j_hi ? raw[j] : 0xff800000u;
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int j = 0; j < TC5_KEYS; j += 8) {
        mx0 = tc5_max3(mx0, __uint_as_float(raw[j]), __uint_as_float(raw[j + 1]));
        mx1 = tc5_max3(mx1, __uint_as_float(raw[j + 2]), __uint_as_float(raw[j + 3]));
        mx2 = tc5_max3(mx2, __uint_as_float(raw[j + 4]), __uint_as_float(raw[j + 5]));
        mx3 = tc5_max3(mx3, __uint_as_float(raw[j + 6]), __uint_as_float(raw[j + 7]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;   // the scale is positive
      // the running maximum only moves when it has to grow by more than the step
      float corr = 1.f;
      if (mx > m_used + TC5_RESCALE_STEP || m_used == -INFINITY) {
        if (mx != -INFINITY) {
          corr = (m_used == -INFINITY) ? 0.f : exp2f(m_used - mx);
          m_used = mx;
        }
      }
      const float neg_base = (m_used == -INFINITY) ? 0.f : -m_used;
      // two scores at a time through the packed 32-bit multiply-add and add
      const uint64_t scale2 = tc5_pair(p.scale_log2, p.scale_log2), base2 = tc5_pair(neg_base, neg_base);
      uint64_t sum_a = tc5_pair(0.f, 0.f), sum_b = sum_a;
#pragma unroll
      for (int c = 0; c < TC5_KEYS / 32; ++c) {
        unsigned packed[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float e0, e1;
          tc5_unpair(tc5_fma2(tc5_pair(__uint_as_float(raw[c * 32 + 2 * j]), __uint_as_float(raw[c * 32 + 2 * j + 1])), scale2, base2), e0, e1);
          e0 = tc5_exp2(e0); e1 = tc5_exp2(e1);
          if (j & 1) sum_b = tc5_add2(sum_b, tc5_pair(e0, e1));
          else sum_a = tc5_add2(sum_a, tc5_pair(e0, e1));
          packed[j] = pack_bf16(e0, e1);
        }
        // P over the scores' own columns: this row's scores are all in registers by now
        tc5_st16(s_addr + c * 16, packed);
      }
      float sum0, sum1;
      tc5_unpair(tc5_add2(sum_a, sum_b), sum0, sum1);
      l = l * corr + (sum0 + sum1);
      // O_x is only touched once the previous value product of this tile has finished: the
      // scores of this key tile were issued after it and the tensor core finishes in order, so
      // it had when s_full completed.  The next one is not issued before this warp has arrived
      // below.
      if (count > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          float o[32];
          tc5_ld32(o_addr + c, o);
          unsigned bits[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) bits[j] = __float_as_uint(o[j] * corr);
          tc5_st32(o_addr + c, bits);
        }
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full + x);
      ++count;
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
        tc5_ld32(o_addr + c, o);
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

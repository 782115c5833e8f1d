// Tensor-core causal grouped-query attention over cache pages (bfloat16), compiled for
// one head size: -DFE_HEAD_DIM=<multiple of 16, 16..256>.
//
// Two kernels share the tile code.  Both treat the G query heads of one kv head as extra
// query rows (row = token * G + head_in_group), so a key/value tile is loaded once per
// kv head and used by all its query heads.
//
//  * prefill: block = (64-row tile, entry, kv head); 4 warps x 16 rows; all warps walk
//    the same 64-key tiles (double-buffered cp.async from the pages); online softmax in
//    32-bit; handles portions that start anywhere (start > 0) and windows.
//  * decode:  for entries with at most 16 rows (one new token, or a few): block =
//    (split, entry, kv head); the key range is cut into `num_splits` contiguous runs of
//    64-key tiles; inside a block each warp takes 16 keys of every tile; the four
//    partial results are merged in shared memory and either stored (one split) or written
//    as unnormalised (max, sum, acc) to a workspace that fe_attn_merge combines.
//
// Upstream's counterparts: the eager attention of src/forge_engine/qwen3.py:187-206
// (scores, 32-bit softmax, value product) and the single-request decode kernel of
// src/forge_engine/kernels/cuda_paged.py:276-347 (online softmax over pages).
//
// Rounding: scores and softmax statistics are 32-bit; probabilities are rounded to
// bfloat16 for the value product (as upstream rounds them, qwen3.py:200); the row sum
// uses the unrounded values.
#include <cuda.h>
#include <stdio.h>

#include <map>
#include <tuple>

#include "attention_common.cuh"

#ifndef FE_HEAD_DIM
#error "compile with -DFE_HEAD_DIM=<head size>"
#endif
#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)
#define SYM(name) CAT(name, FE_HEAD_DIM)

namespace {

constexpr int D = FE_HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size must be a multiple of 16 up to 256");
constexpr int LD = D + 8;          // padded row length in shared memory (elements)
constexpr int CHUNKS = D / 8;      // 16-byte chunks per row
constexpr int BN = 64;             // keys per tile
constexpr int BM = 64;             // rows per prefill block
constexpr int THREADS = 128;
constexpr int DEC_ROWS = 16;

struct AttnParams {
  const bf16* q;
  int q_stride;
  bf16* out;           // [tokens, num_q_heads * D]
  const bf16* k;
  const bf16* v;
  const int* block_table;
  int max_pages, page_size, num_pages, nkv, groups;
  const int* cu_tokens;  // [entries + 1]
  const int* starts;     // [entries] tokens already cached before this step
  int window;
  float scale_log2;      // scale * log2(e)
  int* status;
  int row_lo, row_hi;    // the kernel handles entries with row_lo < rows <= row_hi
  int num_splits;
  float* ws_acc;         // [entries, nkv, splits, 16, D]
  float* ws_ml;          // [entries, nkv, splits, 16, 2]
  unsigned* ws_count;    // [entries, nkv] zeroed arrival counters, or null: a merge kernel follows
  int cluster_merge;     // 1: the splits of a pair form one cluster and combine through shared memory;
                         // 2: clusters of 8 splits do, and the clusters' results go through the workspace
};

__device__ __forceinline__ unsigned smem_addr(const void* p) {
  return (unsigned)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int size = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(dst)), "l"(src), "r"(size));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&h);
}

// Stage keys [key0, key0 + BN) of (entry, kv head) into kdst[BN][LD] and their values into
// vdst[BN][LD].  Rows at or beyond key_end, and rows whose page is missing, are zero-filled.
// A thread looks its row's page up once and then issues that row's 16-byte copies for
// both matrices, so the address arithmetic is paid per row, not per copy.
__device__ __forceinline__ void load_kv_tile(bf16* kdst, bf16* vdst, const AttnParams& p, const int* table,
                                             int kvh, int key0, int key_lo, int key_end, int tid) {
  constexpr int PARTS = THREADS / BN;              // threads per row
  constexpr int PER = (CHUNKS + PARTS - 1) / PARTS;  // chunks per thread and matrix
  const int row = tid / PARTS, part = tid - row * PARTS;
  const int key = key0 + row;
  size_t offset = 0;
  bool valid = key < key_end && key >= 0;
  if (valid) {
    const int logical = key / p.page_size;
    const int page = logical < p.max_pages ? table[logical] : -1;
    if (page < 0 || page >= p.num_pages) {
      valid = false;
      if (key >= key_lo) atomicOr(p.status, FE_STATUS_BAD_PAGE);  // a key some row must see
    } else {
      offset = (((size_t)page * p.nkv + kvh) * p.page_size + (key - logical * p.page_size)) * D;
    }
  }
  const bf16* ksrc = p.k + offset;
  const bf16* vsrc = p.v + offset;
  bf16* kd = kdst + row * LD;
  bf16* vd = vdst + row * LD;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int chunk = part + i * PARTS;     // neighbouring threads take neighbouring chunks
    if (chunk < CHUNKS) {
      cp_async16(kd + chunk * 8, ksrc + chunk * 8, valid);
      cp_async16(vd + chunk * 8, vsrc + chunk * 8, valid);
    }
  }
}

// One 16-row x NKEYS slice: S = Q K^T, masked online softmax, O += P V.
//   qf    - Q fragments of this warp's 16 rows (D/16 k-steps)
//   ks,vs - shared tiles; this warp uses keys [koff, koff + NKEYS) of them
//   key0  - absolute position of the first of those keys
// Where element (key, col) of a staged tile lives.  Padded: rows of LD elements (cp.async
// path).  Swizzled: what TMA writes with 128-byte swizzle - two-dimensional boxes of 64
// columns, so a tile is D/64 column blocks of [64 keys][128 bytes], and inside a row the
// 16-byte chunk c sits at chunk c ^ (row & 7).
struct PaddedTile {
  static __device__ __forceinline__ const bf16* at(const bf16* base, int key, int col) { return base + key * LD + col; }
};

// A key's D elements lie together as D/64 lines of 128 bytes; the 128-byte swizzle goes by
// the line (what one TMA box of a whole page chunk, seen as lines, leaves in shared memory).
struct LineSwizzledTile {
  static __device__ __forceinline__ const bf16* at(const bf16* base, int key, int col) {
    const int line = key * (D / 64) + (col >> 6), chunk = (col >> 3) & 7;
    return base + line * 64 + ((chunk ^ (line & 7)) << 3);
  }
};

template <int NKEYS, typename Tile = PaddedTile>
__device__ __forceinline__ void tile_step(const unsigned (&qf)[D / 16][4], const bf16* ks, const bf16* vs,
                                          int koff, int key0, int key_end, int pos_a, int pos_b,
                                          int window, float scale_log2, bool need_mask, float (&m)[2],
                                          float (&l)[2], float (&o)[D / 8][4], int lane) {
  constexpr int NT = NKEYS / 8;
  float s[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
    for (int j2 = 0; j2 < NT / 2; ++j2) {
      unsigned b[4];
      const int key = koff + j2 * 16 + (lane & 7) + ((lane >> 4) << 3);
      const int col = kk * 16 + ((lane >> 3) & 1) * 8;
      ldmatrix_x4(b, Tile::at(ks, key, col));
      mma_bf16(s[2 * j2], qf[kk], b[0], b[1]);
      mma_bf16(s[2 * j2 + 1], qf[kk], b[2], b[3]);
    }
  }
  const int t = lane & 3;
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float val = s[j][e] * scale_log2;
      if (need_mask) {
        const int key = key0 + j * 8 + 2 * t + (e & 1);
        const int pos = (e < 2) ? pos_a : pos_b;
        const bool seen = key <= pos && key < key_end && (window <= 0 || pos - key < window);
        if (!seen) val = -INFINITY;
      }
      s[j][e] = val;
      mx[e >> 1] = fmaxf(mx[e >> 1], val);
    }
  }
  float corr[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    const float m_new = fmaxf(m[r], mx[r]);
    corr[r] = (m[r] == -INFINITY) ? 0.f : exp2f(m[r] - m_new);
    m[r] = m_new;
  }
  float sum[2] = {0.f, 0.f};
  const float base_a = (m[0] == -INFINITY) ? 0.f : m[0];
  const float base_b = (m[1] == -INFINITY) ? 0.f : m[1];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    s[j][0] = exp2f(s[j][0] - base_a);
    s[j][1] = exp2f(s[j][1] - base_a);
    s[j][2] = exp2f(s[j][2] - base_b);
    s[j][3] = exp2f(s[j][3] - base_b);
    sum[0] += s[j][0] + s[j][1];
    sum[1] += s[j][2] + s[j][3];
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
    sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
    l[r] = l[r] * corr[r] + sum[r];
  }
#pragma unroll
  for (int n = 0; n < D / 8; ++n) {
    o[n][0] *= corr[0]; o[n][1] *= corr[0];
    o[n][2] *= corr[1]; o[n][3] *= corr[1];
  }
#pragma unroll
  for (int kk = 0; kk < NKEYS / 16; ++kk) {
    unsigned a[4];
    a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int n2 = 0; n2 < D / 16; ++n2) {
      unsigned b[4];
      const int key = koff + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
      const int col = n2 * 16 + (lane >> 4) * 8;
      ldmatrix_x4_trans(b, Tile::at(vs, key, col));
      mma_bf16(o[2 * n2], a, b[0], b[1]);
      mma_bf16(o[2 * n2 + 1], a, b[2], b[3]);
    }
  }
}

// Stage `rows` query rows (row = token * G + head in group) starting at row0 into qs[rows][LD].
__device__ __forceinline__ void load_q_rows(bf16* qs, const AttnParams& p, int tok0, int kvh, int row0,
                                            int rows_total, int rows, int tid, int nthreads) {
  for (int idx = tid; idx < rows * CHUNKS; idx += nthreads) {
    const int r = idx / CHUNKS, chunk = idx - r * CHUNKS;
    const int row = row0 + r;
    const bool valid = row < rows_total;
    const bf16* src = p.q;
    if (valid) {
      const int token = row / p.groups, g = row - token * p.groups;
      src = p.q + (size_t)(tok0 + token) * p.q_stride + (size_t)(kvh * p.groups + g) * D + chunk * 8;
    }
    cp_async16(qs + r * LD + chunk * 8, src, valid);
  }
}

__global__ void __launch_bounds__(THREADS) attn_prefill_kernel(AttnParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // Two key/value stages.  The query tile is staged in the second stage's buffers, read
  // into registers once, and the space is then used for keys and values: three blocks
  // fit on an SM instead of two.
  bf16* kbuf = reinterpret_cast<bf16*>(smem_raw);   // [2][BN][LD]
  bf16* vbuf = kbuf + 2 * BN * LD;                  // [2][BN][LD]
  bf16* qs = kbuf + BN * LD;                        // [BM][LD] over stage 1 (BM == BN)

  pdl_trigger();
  pdl_wait();
  const int entry = blockIdx.y, kvh = blockIdx.z;
  const int tok0 = p.cu_tokens[entry];
  const int n_new = p.cu_tokens[entry + 1] - tok0;
  const int rows_total = n_new * p.groups;
  if (rows_total <= p.row_lo || rows_total > p.row_hi) return;
  // Later row tiles see more keys and run longer: start them first so that the last
  // round of blocks is made of short ones.
  const int row0 = (gridDim.x - 1 - blockIdx.x) * BM;
  if (row0 >= rows_total) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int start = p.starts[entry];
  const int* table = p.block_table + (size_t)entry * p.max_pages;

  const int last_row = min(rows_total, row0 + BM) - 1;
  const int pos_first = start + row0 / p.groups;
  const int pos_last = start + last_row / p.groups;
  const int key_lo = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
  const int key_end = pos_last + 1;
  const int tile_begin = key_lo / BN, tile_end = (key_end + BN - 1) / BN;

  load_q_rows(qs, p, tok0, kvh, row0, rows_total, BM, tid, THREADS);
  load_kv_tile(kbuf, vbuf, p, table, kvh, tile_begin * BN, key_lo, key_end, tid);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  unsigned qf[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk)
    ldmatrix_x4(qf[kk], qs + (warp * 16 + (lane & 15)) * LD + kk * 16 + (lane >> 4) * 8);
  __syncthreads();   // the query tile's space may now take keys

  const int ra = row0 + warp * 16 + (lane >> 2), rb = ra + 8;
  const int pos_a = ra < rows_total ? start + ra / p.groups : -1;
  const int pos_b = rb < rows_total ? start + rb / p.groups : -1;
  // positions of this warp's 16 rows, for the decision whether a tile needs masking
  const int wrow0 = row0 + warp * 16;
  const int wpos_min = start + min(wrow0, rows_total - 1) / p.groups;
  const bool warp_has_padding = wrow0 + 16 > rows_total;
  const int wpos_max = start + min(wrow0 + 15, rows_total - 1) / p.groups;

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }

  for (int tile = tile_begin; tile < tile_end; ++tile) {
    const int buf = (tile - tile_begin) & 1;
    if (tile + 1 < tile_end) {
      load_kv_tile(kbuf + (buf ^ 1) * BN * LD, vbuf + (buf ^ 1) * BN * LD, p, table, kvh, (tile + 1) * BN, key_lo,
                   key_end, tid);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int key0 = tile * BN;
    // keys of this tile that no row of the warp can see are skipped altogether
    if (wrow0 < rows_total && key0 <= wpos_max) {
      const bool full = !warp_has_padding && key0 + BN - 1 <= wpos_min && key0 + BN <= key_end &&
                        (p.window <= 0 || wpos_max - key0 < p.window);
      tile_step<BN>(qf, kbuf + buf * BN * LD, vbuf + buf * BN * LD, 0, key0, key_end, pos_a, pos_b, p.window,
                    p.scale_log2, !full, m, l, o, lane);
    }
    __syncthreads();
  }

  const int num_q_heads = p.nkv * p.groups;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = half ? rb : ra;
    if (row >= rows_total) continue;
    const int token = row / p.groups, g = row - token * p.groups;
    const float inv = l[half] > 0.f ? 1.f / l[half] : 0.f;
    bf16* dst = p.out + ((size_t)(tok0 + token) * num_q_heads + kvh * p.groups + g) * D + 2 * (lane & 3);
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      const __nv_bfloat162 v2 = __floats2bfloat162_rn(o[n][2 * half] * inv, o[n][2 * half + 1] * inv);
      *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) = v2;
    }
  }
}

constexpr int DEC_STAGES = 3;       // key/value tiles in flight per block (ring)
constexpr int MERGE_MAX_SPLITS = 64;

__global__ void __launch_bounds__(THREADS) attn_decode_kernel(AttnParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);   // [16][LD]
  bf16* kbuf = qs + DEC_ROWS * LD;                // [DEC_STAGES][BN][LD]
  bf16* vbuf = kbuf + DEC_STAGES * BN * LD;       // [DEC_STAGES][BN][LD]
  __shared__ int last_block;

  pdl_trigger();
  pdl_wait();
  const int split = blockIdx.x, entry = blockIdx.y, kvh = blockIdx.z;
  const int tok0 = p.cu_tokens[entry];
  const int n_new = p.cu_tokens[entry + 1] - tok0;
  const int rows_total = n_new * p.groups;
  if (rows_total <= p.row_lo || rows_total > p.row_hi) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int start = p.starts[entry];
  const int* table = p.block_table + (size_t)entry * p.max_pages;

  const int pos_last = start + n_new - 1;
  const int key_lo = p.window > 0 ? max(0, start - p.window + 1) : 0;
  const int key_end = pos_last + 1;
  const int tile_first = key_lo / BN, tile_stop = (key_end + BN - 1) / BN;
  const int tiles = tile_stop - tile_first;
  const int per_split = (tiles + p.num_splits - 1) / p.num_splits;
  const int tile_begin = tile_first + split * per_split;
  const int tile_end = min(tile_stop, tile_begin + per_split);
  const int my_tiles = max(0, tile_end - tile_begin);

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }

  const int ra = lane >> 2, rb = ra + 8;
  const int pos_a = ra < rows_total ? start + ra / p.groups : -1;
  const int pos_b = rb < rows_total ? start + rb / p.groups : -1;

  if (my_tiles > 0) {
    // ring of DEC_STAGES tiles: tiles i+1 .. i+DEC_STAGES-1 are in flight while tile i is used
    load_q_rows(qs, p, tok0, kvh, 0, rows_total, DEC_ROWS, tid, THREADS);
#pragma unroll
    for (int i = 0; i < DEC_STAGES - 1; ++i) {
      if (i < my_tiles)
        load_kv_tile(kbuf + i * BN * LD, vbuf + i * BN * LD, p, table, kvh, (tile_begin + i) * BN, key_lo, key_end, tid);
      cp_async_commit();
    }
    unsigned qf[D / 16][4];
    for (int i = 0; i < my_tiles; ++i) {
      const int ahead = i + DEC_STAGES - 1;
      if (ahead < my_tiles) {
        const int sa = ahead % DEC_STAGES;
        load_kv_tile(kbuf + sa * BN * LD, vbuf + sa * BN * LD, p, table, kvh, (tile_begin + ahead) * BN, key_lo,
                     key_end, tid);
      }
      cp_async_commit();
      cp_async_wait<DEC_STAGES - 1>();
      __syncthreads();
      if (i == 0) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          ldmatrix_x4(qf[kk], qs + (lane & 15) * LD + kk * 16 + (lane >> 4) * 8);
      }
      const int stage = i % DEC_STAGES;
      const int key0 = (tile_begin + i) * BN + warp * 16;   // this warp's 16 keys of the tile
      if (key0 < key_end)
        tile_step<16>(qf, kbuf + stage * BN * LD, vbuf + stage * BN * LD, warp * 16, key0, key_end, pos_a, pos_b,
                      p.window, p.scale_log2, true, m, l, o, lane);
      __syncthreads();
    }
    cp_async_wait<0>();
  }

  // merge the four warps: reuse the (now idle) key/value buffers
  float* acc_s = reinterpret_cast<float*>(kbuf);          // [4][16][D]
  float* ml_s = acc_s + 4 * DEC_ROWS * D;                 // [4][16][2]
  __syncthreads();
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = half ? rb : ra;
    float* dst = acc_s + ((size_t)warp * DEC_ROWS + row) * D + 2 * (lane & 3);
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      dst[n * 8] = o[n][2 * half];
      dst[n * 8 + 1] = o[n][2 * half + 1];
    }
    if ((lane & 3) == 0) {
      ml_s[(warp * DEC_ROWS + row) * 2] = m[half];
      ml_s[(warp * DEC_ROWS + row) * 2 + 1] = l[half];
    }
  }
  __syncthreads();
  const int num_q_heads = p.nkv * p.groups;
  const size_t pair = (size_t)entry * p.nkv + kvh;
  for (int idx = tid; idx < rows_total * D; idx += THREADS) {
    const int row = idx / D, d = idx - row * D;
    float big = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) big = fmaxf(big, ml_s[(w * DEC_ROWS + row) * 2]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = ml_s[(w * DEC_ROWS + row) * 2];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - big);
      num += acc_s[((size_t)w * DEC_ROWS + row) * D + d] * f;
      den += ml_s[(w * DEC_ROWS + row) * 2 + 1] * f;
    }
    if (p.num_splits == 1) {
      const int token = row / p.groups, g = row - token * p.groups;
      p.out[((size_t)(tok0 + token) * num_q_heads + kvh * p.groups + g) * D + d] =
          __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
    } else {
      const size_t slot = pair * p.num_splits + split;
      p.ws_acc[(slot * DEC_ROWS + row) * D + d] = num;
      if (d == 0) {
        p.ws_ml[(slot * DEC_ROWS + row) * 2] = big;
        p.ws_ml[(slot * DEC_ROWS + row) * 2 + 1] = den;
      }
    }
  }
  if (p.num_splits == 1 || p.ws_count == nullptr) return;   // one split, or a separate merge kernel follows

  // The block that publishes its partial result last combines all of them, in split
  // order, so that no second kernel is needed and the sum does not depend on timing.
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned arrived = atomicAdd(p.ws_count + pair, 1u);
    last_block = arrived == (unsigned)p.num_splits - 1u;
    if (last_block) p.ws_count[pair] = 0u;
  }
  __syncthreads();
  if (!last_block) return;
  __threadfence();
  float* weight_s = reinterpret_cast<float*>(kbuf);       // [16][MERGE_MAX_SPLITS]
  const int splits = p.num_splits;
  const size_t slot0 = pair * splits;
  for (int row = warp; row < rows_total; row += THREADS / 32) {
    float mv[MERGE_MAX_SPLITS / 32], lv[MERGE_MAX_SPLITS / 32];
    float big = -INFINITY;
#pragma unroll
    for (int i = 0; i < MERGE_MAX_SPLITS / 32; ++i) {
      const int sp = lane + i * 32;
      mv[i] = -INFINITY; lv[i] = 0.f;
      if (sp < splits) {
        mv[i] = __ldcg(p.ws_ml + ((slot0 + sp) * DEC_ROWS + row) * 2);
        lv[i] = __ldcg(p.ws_ml + ((slot0 + sp) * DEC_ROWS + row) * 2 + 1);
      }
      big = fmaxf(big, mv[i]);
    }
    big = warp_max(big);
    float den = 0.f;
#pragma unroll
    for (int i = 0; i < MERGE_MAX_SPLITS / 32; ++i) {
      mv[i] = (mv[i] == -INFINITY) ? 0.f : exp2f(mv[i] - big);
      den += lv[i] * mv[i];
    }
    den = warp_sum(den);
    const float inv = den > 0.f ? 1.f / den : 0.f;
#pragma unroll
    for (int i = 0; i < MERGE_MAX_SPLITS / 32; ++i) {
      const int sp = lane + i * 32;
      if (sp < splits) weight_s[row * MERGE_MAX_SPLITS + sp] = mv[i] * inv;
    }
  }
  __syncthreads();
  for (int idx = tid; idx < rows_total * D; idx += THREADS) {
    const int row = idx / D, d = idx - row * D;
    const float* src = p.ws_acc + (slot0 * DEC_ROWS + row) * D + d;
    float num = 0.f;
#pragma unroll 4
    for (int sp = 0; sp < splits; ++sp) num += __ldcg(src + (size_t)sp * DEC_ROWS * D) * weight_s[row * MERGE_MAX_SPLITS + sp];
    const int token = row / p.groups, g = row - token * p.groups;
    p.out[((size_t)(tok0 + token) * num_q_heads + kvh * p.groups + g) * D + d] = __float2bfloat16_rn(num);
  }
}

// ---------------------------------------------------------------------------
// Split decode attention with the key/value tiles staged by TMA (head sizes that are
// multiples of 64, page sizes that divide 64).  One extra warp is the producer: for every
// 64-key tile it looks the pages up and issues one tensor copy per page and 64-column block
// (128-byte swizzle) into a ring of stages, signalled by mbarriers; the four consumer warps
// never issue a load and never meet at a block-wide barrier while keys stream.  Tiles that
// only hold keys of earlier steps are requested before the wait on the previous kernel.
// ---------------------------------------------------------------------------
constexpr int TMA_STAGES = 3;
constexpr int TMA_THREADS = THREADS + 32;
constexpr unsigned TMA_WAIT_LIMIT = 20000000u;

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// Bounded wait on a phase; false (and the flag set) when the bound is hit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity, volatile int* abort_flag) {
  for (unsigned i = 0; i < TMA_WAIT_LIMIT; ++i) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    if (ok) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
// Asks for a tensor map ahead of the first copy that uses it.
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_addr(dst)), "l"(map), "r"(smem_addr(bar)), "r"(c0), "r"(c1) : "memory");
}

__global__ void __launch_bounds__(TMA_THREADS)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       AttnParams p) {
  extern __shared__ unsigned char smem_raw[];
  constexpr int TILE_BYTES = BN * D * 2;    // one matrix of one stage
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  bf16* kbuf = reinterpret_cast<bf16*>(smem);                                   // [TMA_STAGES][D/64][BN][64]
  bf16* vbuf = reinterpret_cast<bf16*>(smem + TMA_STAGES * TILE_BYTES);
  bf16* qs = reinterpret_cast<bf16*>(smem + 2 * TMA_STAGES * TILE_BYTES);         // [16][LD]
  uint64_t* full = reinterpret_cast<uint64_t*>(qs + DEC_ROWS * LD);
  uint64_t* empty = full + TMA_STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + TMA_STAGES);
  __shared__ int last_block;

  pdl_trigger();
  const int split = blockIdx.x, entry = blockIdx.y, kvh = blockIdx.z;
  const int tok0 = p.cu_tokens[entry];
  const int n_new = p.cu_tokens[entry + 1] - tok0;
  const int rows_total = n_new * p.groups;
  if (rows_total <= p.row_lo || rows_total > p.row_hi) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int start = p.starts[entry];
  const int* table = p.block_table + (size_t)entry * p.max_pages;

  const int pos_last = start + n_new - 1;
  const int key_lo = p.window > 0 ? max(0, start - p.window + 1) : 0;
  const int key_end = pos_last + 1;
  const int tile_first = key_lo / BN, tile_stop = (key_end + BN - 1) / BN;
  const int tiles = tile_stop - tile_first;
  const int per_split = (tiles + p.num_splits - 1) / p.num_splits;
  const int tile_begin = tile_first + split * per_split;
  const int tile_end = min(tile_stop, tile_begin + per_split);
  const int my_tiles = max(0, tile_end - tile_begin);

  if (tid == 0) {
    tma_prefetch_map(&map_k);
    tma_prefetch_map(&map_v);
    for (int s = 0; s < TMA_STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  const int ra = lane >> 2, rb = ra + 8;

  if (warp == 4) {
    // ---- producer ----
    // The lanes fetch the block-table entries of up to 32 pages at once (one coalesced
    // load instead of a chain of dependent ones); lane 0 then issues the copies.
    if (my_tiles > 0) {
      const int pages_per_tile = BN / p.page_size;
      const int rows_in_cache = p.num_pages * p.nkv * p.page_size;
      const int first_logical = tile_begin * pages_per_tile;
      const int total_pages = my_tiles * pages_per_tile;
      bool waited = false, dead = false;
      for (int base = 0; base < total_pages; base += 32) {
        const int logical = first_logical + base + lane;
        const int key = logical * p.page_size;
        int my_row = rows_in_cache;          // outside the tensor: the copy fills zeros
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
            const int s = i % TMA_STAGES;
            if (pg == 0) {
              const int key0 = (tile_begin + i) * BN;
              // keys of this step are written by the kernel before this one
              if (!waited && (key0 + BN > start || i >= TMA_STAGES)) { pdl_wait(); waited = true; }
              if (i >= TMA_STAGES && !mbar_wait(empty + s, ((i / TMA_STAGES) & 1) ^ 1, abort_flag)) dead = true;
              if (!dead) mbar_expect_tx(full + s, 2 * TILE_BYTES);
            }
            if (!dead) {
              // one box per page and matrix: the page's keys of this head are contiguous
              const int offset = pg * p.page_size * D;
              tma_load_2d(kbuf + s * (BN * D) + offset, &map_k, 0, row * (D / 64), full + s);
              tma_load_2d(vbuf + s * (BN * D) + offset, &map_v, 0, row * (D / 64), full + s);
            }
          }
        }
      }
      if (lane == 0 && !waited) pdl_wait();
    }
  } else {
    // ---- consumers: warp w takes keys [16 w, 16 w + 16) of every tile ----
    pdl_wait();
    const int pos_a = ra < rows_total ? start + ra / p.groups : -1;
    const int pos_b = rb < rows_total ? start + rb / p.groups : -1;
    if (my_tiles > 0) {
      // the four warps stage the query rows themselves (named barrier of 128 threads)
      load_q_rows(qs, p, tok0, kvh, 0, rows_total, DEC_ROWS, tid, THREADS);
      cp_async_commit();
      cp_async_wait<0>();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      unsigned qf[D / 16][4];
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk)
        ldmatrix_x4(qf[kk], qs + (lane & 15) * LD + kk * 16 + (lane >> 4) * 8);
      for (int i = 0; i < my_tiles; ++i) {
        const int s = i % TMA_STAGES;
        if (!mbar_wait(full + s, (i / TMA_STAGES) & 1, abort_flag)) break;
        const int key0 = (tile_begin + i) * BN + warp * 16;
        if (key0 < key_end)
          tile_step<16, LineSwizzledTile>(qf, kbuf + s * (BN * D), vbuf + s * (BN * D), warp * 16, key0, key_end, pos_a,
                                      pos_b, p.window, p.scale_log2, true, m, l, o, lane);
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);
      }
    }
  }
  __syncthreads();   // every load has landed and every warp is done with the stages

  // merge the four consumer warps: reuse the key stages
  float* acc_s = reinterpret_cast<float*>(kbuf);          // [4][16][D]
  float* ml_s = acc_s + 4 * DEC_ROWS * D;                 // [4][16][2]
  float* part_s = reinterpret_cast<float*>(vbuf);         // [16][D] this block's partial result (cluster merge)
  float* part_ml_s = part_s + DEC_ROWS * D;               // [16][2]
  if (warp < 4) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = half ? rb : ra;
      if (row >= rows_total) continue;          // rows without a query are not read below
      float2* dst = reinterpret_cast<float2*>(acc_s + ((size_t)warp * DEC_ROWS + row) * D + 2 * (lane & 3));
#pragma unroll
      for (int n = 0; n < D / 8; ++n) dst[n * 4] = make_float2(o[n][2 * half], o[n][2 * half + 1]);
      if ((lane & 3) == 0) {
        ml_s[(warp * DEC_ROWS + row) * 2] = m[half];
        ml_s[(warp * DEC_ROWS + row) * 2 + 1] = l[half];
      }
    }
  }
  __syncthreads();
  const int num_q_heads = p.nkv * p.groups;
  const size_t pair = (size_t)entry * p.nkv + kvh;
  for (int idx = tid; idx < rows_total * D; idx += TMA_THREADS) {
    const int row = idx / D, d = idx - row * D;
    float big = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) big = fmaxf(big, ml_s[(w * DEC_ROWS + row) * 2]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = ml_s[(w * DEC_ROWS + row) * 2];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - big);
      num += acc_s[((size_t)w * DEC_ROWS + row) * D + d] * f;
      den += ml_s[(w * DEC_ROWS + row) * 2 + 1] * f;
    }
    if (p.num_splits == 1) {
      const int token = row / p.groups, g = row - token * p.groups;
      p.out[((size_t)(tok0 + token) * num_q_heads + kvh * p.groups + g) * D + d] =
          __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
    } else if (p.cluster_merge) {
      part_s[row * D + d] = num;
      if (d == 0) {
        part_ml_s[row * 2] = big;
        part_ml_s[row * 2 + 1] = den;
      }
    } else {
      const size_t slot = pair * p.num_splits + split;
      p.ws_acc[(slot * DEC_ROWS + row) * D + d] = num;
      if (d == 0) {
        p.ws_ml[(slot * DEC_ROWS + row) * 2] = big;
        p.ws_ml[(slot * DEC_ROWS + row) * 2 + 1] = den;
      }
    }
  }
  if (tid == 0 && *abort_flag) atomicOr(p.status, FE_STATUS_WAIT_TIMEOUT);
  if (p.num_splits == 1) return;

  if (p.cluster_merge) {
    // The splits of this (entry, kv head) are the blocks of one cluster.  Every block
    // finishes a share of the rows: it reads the blocks' partial results of those rows
    // from their shared memory and combines them in block order.
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    // cluster_merge 2: clusters of 8; what a cluster combines is one partial result of several
    const int splits = p.cluster_merge == 2 ? 8 : p.num_splits;
    const int rank = split % splits;
    const int share = (rows_total + splits - 1) / splits;
    const int row_begin = rank * share, row_end = min(rows_total, row_begin + share);
    const unsigned local_part = smem_addr(part_s), local_ml = smem_addr(part_ml_s);
    for (int idx = tid; idx < (row_end - row_begin) * D; idx += TMA_THREADS) {
      const int row = row_begin + idx / D, d = idx % D;
      float mv[8], lv[8], av[8];
#pragma unroll
      for (int peer = 0; peer < 8; ++peer) {
        mv[peer] = -INFINITY; lv[peer] = 0.f; av[peer] = 0.f;
        if (peer < splits) {
          unsigned remote_ml, remote_part;
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_ml) : "r"(local_ml), "r"(peer));
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_part) : "r"(local_part), "r"(peer));
          asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(mv[peer]) : "r"(remote_ml + (unsigned)(row * 8)) : "memory");
          asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(lv[peer]) : "r"(remote_ml + (unsigned)(row * 8 + 4)) : "memory");
          asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(av[peer]) : "r"(remote_part + (unsigned)((row * D + d) * 4)) : "memory");
        }
      }
      float big = -INFINITY;
#pragma unroll
      for (int peer = 0; peer < 8; ++peer) big = fmaxf(big, mv[peer]);
      float num = 0.f, den = 0.f;
#pragma unroll
      for (int peer = 0; peer < 8; ++peer) {
        const float f = (mv[peer] == -INFINITY) ? 0.f : exp2f(mv[peer] - big);
        num += av[peer] * f;
        den += lv[peer] * f;
      }
      if (p.cluster_merge == 2) {
        const size_t slot = pair * (p.num_splits / 8) + split / 8;
        p.ws_acc[(slot * DEC_ROWS + row) * D + d] = num;
        if (d == 0) {
          p.ws_ml[(slot * DEC_ROWS + row) * 2] = big;
          p.ws_ml[(slot * DEC_ROWS + row) * 2 + 1] = den;
        }
      } else {
        const int token = row / p.groups, g = row - token * p.groups;
        p.out[((size_t)(tok0 + token) * num_q_heads + kvh * p.groups + g) * D + d] =
            __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
      }
    }
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");   // partial results stay alive until read
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (p.cluster_merge != 2) return;
  }

  // the block that publishes its (or its cluster's) partial result last combines all of
  // them, in split order
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned arrived = atomicAdd(p.ws_count + pair, 1u);
    last_block = arrived == (unsigned)p.num_splits - 1u;
    if (last_block) p.ws_count[pair] = 0u;
  }
  __syncthreads();
  if (!last_block) return;
  __threadfence();
  float* weight_s = reinterpret_cast<float*>(kbuf);       // [16][MERGE_MAX_SPLITS]
  const int splits = p.cluster_merge == 2 ? p.num_splits / 8 : p.num_splits;
  const size_t slot0 = pair * splits;
  for (int row = warp; row < rows_total; row += TMA_THREADS / 32) {
    float mv[MERGE_MAX_SPLITS / 32], lv[MERGE_MAX_SPLITS / 32];
    float big = -INFINITY;
#pragma unroll
    for (int i = 0; i < MERGE_MAX_SPLITS / 32; ++i) {
      const int sp = lane + i * 32;
      mv[i] = -INFINITY; lv[i] = 0.f;
      if (sp < splits) {
        mv[i] = __ldcg(p.ws_ml + ((slot0 + sp) * DEC_ROWS + row) * 2);
        lv[i] = __ldcg(p.ws_ml + ((slot0 + sp) * DEC_ROWS + row) * 2 + 1);
      }
      big = fmaxf(big, mv[i]);
    }
    big = warp_max(big);
    float den = 0.f;
#pragma unroll
    for (int i = 0; i < MERGE_MAX_SPLITS / 32; ++i) {
      mv[i] = (mv[i] == -INFINITY) ? 0.f : exp2f(mv[i] - big);
      den += lv[i] * mv[i];
    }
    den = warp_sum(den);
    const float inv = den > 0.f ? 1.f / den : 0.f;
#pragma unroll
    for (int i = 0; i < MERGE_MAX_SPLITS / 32; ++i) {
      const int sp = lane + i * 32;
      if (sp < splits) weight_s[row * MERGE_MAX_SPLITS + sp] = mv[i] * inv;
    }
  }
  __syncthreads();
  for (int idx = tid; idx < rows_total * D; idx += TMA_THREADS) {
    const int row = idx / D, d = idx - row * D;
    const float* src = p.ws_acc + (slot0 * DEC_ROWS + row) * D + d;
    float num = 0.f;
#pragma unroll 4
    for (int sp = 0; sp < splits; ++sp) num += __ldcg(src + (size_t)sp * DEC_ROWS * D) * weight_s[row * MERGE_MAX_SPLITS + sp];
    const int token = row / p.groups, g = row - token * p.groups;
    p.out[((size_t)(tok0 + token) * num_q_heads + kvh * p.groups + g) * D + d] = __float2bfloat16_rn(num);
  }
}

// Combine the splits' (max, sum, acc) of every row: block = (entry, kv head).  The splits'
// weights exp2(m_s - max) / sum are worked out once per row in shared memory; then every
// thread owns one or more columns and sums over the splits with independent loads.
__global__ void __launch_bounds__(THREADS) attn_merge_kernel(AttnParams p) {
  __shared__ float weight_s[DEC_ROWS][MERGE_MAX_SPLITS];
  pdl_trigger();
  pdl_wait();
  const int entry = blockIdx.x, kvh = blockIdx.y;
  const int tok0 = p.cu_tokens[entry];
  const int n_new = p.cu_tokens[entry + 1] - tok0;
  const int rows_total = n_new * p.groups;
  if (rows_total <= p.row_lo || rows_total > p.row_hi) return;
  const int num_q_heads = p.nkv * p.groups;
  const int splits = p.num_splits;
  const size_t slot0 = ((size_t)entry * p.nkv + kvh) * splits;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = warp; row < rows_total; row += THREADS / 32) {
    float mv[MERGE_MAX_SPLITS / 32], lv[MERGE_MAX_SPLITS / 32];
    float big = -INFINITY;
#pragma unroll
    for (int i = 0; i < MERGE_MAX_SPLITS / 32; ++i) {
      const int s = lane + i * 32;
      mv[i] = -INFINITY; lv[i] = 0.f;
      if (s < splits) {
        const float2 ml = *reinterpret_cast<const float2*>(p.ws_ml + ((slot0 + s) * DEC_ROWS + row) * 2);
        mv[i] = ml.x; lv[i] = ml.y;
      }
      big = fmaxf(big, mv[i]);
    }
    big = warp_max(big);
    float den = 0.f;
#pragma unroll
    for (int i = 0; i < MERGE_MAX_SPLITS / 32; ++i) {
      mv[i] = (mv[i] == -INFINITY) ? 0.f : exp2f(mv[i] - big);
      den += lv[i] * mv[i];
    }
    den = warp_sum(den);
    const float inv = den > 0.f ? 1.f / den : 0.f;
#pragma unroll
    for (int i = 0; i < MERGE_MAX_SPLITS / 32; ++i) {
      const int s = lane + i * 32;
      if (s < splits) weight_s[row][s] = mv[i] * inv;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < rows_total * D; idx += THREADS) {
    const int row = idx / D, d = idx - row * D;
    const float* src = p.ws_acc + (slot0 * DEC_ROWS + row) * D + d;
    float num = 0.f;
#pragma unroll 4
    for (int s = 0; s < splits; ++s) num += src[(size_t)s * DEC_ROWS * D] * weight_s[row][s];
    const int token = row / p.groups, g = row - token * p.groups;
    p.out[((size_t)(tok0 + token) * num_q_heads + kvh * p.groups + g) * D + d] = __float2bfloat16_rn(num);
  }
}

static_assert(BM == BN, "the query tile is staged in one key stage");
constexpr size_t PREFILL_SMEM = (size_t)(4 * BN) * LD * sizeof(bf16);
constexpr size_t DECODE_KV_SMEM = (size_t)(DEC_ROWS + 2 * DEC_STAGES * BN) * LD * sizeof(bf16);
constexpr size_t DECODE_MERGE_SMEM =
    (size_t)DEC_ROWS * LD * sizeof(bf16) + (size_t)4 * DEC_ROWS * (D + 2) * sizeof(float) +
    (size_t)DEC_ROWS * MERGE_MAX_SPLITS * sizeof(float);
constexpr size_t DECODE_SMEM = DECODE_KV_SMEM > DECODE_MERGE_SMEM ? DECODE_KV_SMEM : DECODE_MERGE_SMEM;

}  // namespace

namespace {

constexpr size_t DECODE_TMA_SMEM = (size_t)2 * TMA_STAGES * BN * D * sizeof(bf16) + (size_t)DEC_ROWS * LD * sizeof(bf16) +
                                   (size_t)2 * TMA_STAGES * 8 + 16 + 1024;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Tensor map of one cache matrix seen as [pages * kv heads * page_size rows, D columns]:
// boxes of page_size rows x 64 columns, 128-byte swizzle, zeros outside.  Maps are kept
// per (pointer, rows, page size): a model has two per attention layer.
EncodeTiledFn g_encode_tiled = nullptr;

bool ensure_encode() {
  if (g_encode_tiled == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      g_encode_tiled = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return g_encode_tiled != nullptr;
}

// The map is copied into *out: the table below may drop its entries when it grows large,
// so no caller keeps a pointer into it.
bool cache_map(CUtensorMap* out, const void* base, int rows, int page_size, bool lines = false) {
  // lines: the matrix seen as [rows * D/64 lines, 64 columns]; a box is a whole page chunk
  // (page_size * D/64 lines, contiguous in memory)
  static std::map<std::tuple<const void*, int, int, bool>, CUtensorMap> maps;
  const auto key = std::make_tuple(base, rows, page_size, lines);
  auto found = maps.find(key);
  if (found != maps.end()) {
    *out = found->second;
    return true;
  }
  if (!ensure_encode()) return false;
  EncodeTiledFn encode = g_encode_tiled;
  CUtensorMap map;
  const int per_row = lines ? D / 64 : 1;
  if (page_size * per_row > 256) return false;
  cuuint64_t dims[2] = {(cuuint64_t)(lines ? 64 : D), (cuuint64_t)rows * per_row};
  cuuint64_t strides[1] = {(cuuint64_t)(lines ? 64 : D) * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)(page_size * per_row)};
  cuuint32_t elem[2] = {1, 1};
  if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (maps.size() > 4096) maps.clear();
  maps.emplace(key, map);
  *out = map;
  return true;
}

}  // namespace

#include "attention_noalloc.h"
#include "attention_tc5.cuh"
#include "attention_balanced.cuh"

// Workspace sizes (in floats) the decode path needs for `entries` and `num_splits`.
FE_EXPORT long long SYM(fe_attn_workspace_floats_d)(int entries, int num_kv_heads, int num_splits) {
  return (long long)entries * num_kv_heads * num_splits * DEC_ROWS * (D + 2);
}

// Blocks of the balanced decode kernel: as many as the GPU holds at once (0: it cannot run).
// Its workspace holds 2 * blocks * 16 * (D + 2) floats.
FE_EXPORT int SYM(fe_attn_balanced_blocks_d)() {
  static int blocks = -1;
  if (blocks < 0) {
    blocks = 0;
    int device = 0, sms = 0, per_sm = 0;
    if ((D % 64) == 0 && ensure_encode() && cudaGetDevice(&device) == cudaSuccess &&
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) == cudaSuccess &&
        cudaFuncSetAttribute(attn_decode_balanced_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)DECODE_BALANCED_SMEM) == cudaSuccess &&
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_decode_balanced_kernel, TMA_THREADS,
                                                      DECODE_BALANCED_SMEM) == cudaSuccess)
      blocks = sms * per_sm < BAL_MAX_BLOCKS ? sms * per_sm : BAL_MAX_BLOCKS;
  }
  return blocks;
}

// `counters` (one zeroed unsigned per entry and kv head, left zeroed) lets the decode
// kernel combine its splits itself; without it a merge kernel is launched.
// mode bit 0: run the prefill kernel for entries with more than `decode_rows` rows;
// mode bit 1: run the decode kernel (and the merge, if num_splits > 1) for the others.
// decode_rows is 16 when the decode kernel may be used, 0 to send everything to prefill.
FE_EXPORT int SYM(fe_attention_mma_d)(const void* q, int q_stride, void* out, const void* k_cache,
                                      const void* v_cache, const int* block_table, int max_pages,
                                      int page_size, int num_pages, int num_kv_heads, int groups,
                                      const int* cu_tokens, const int* starts, int entries, int max_new,
                                      int total_tokens, int window, float scale, int mode, int num_splits,
                                      float* workspace, unsigned* counters, int* status, cudaStream_t stream) {
  if (entries <= 0) return 0;
  if (groups < 1 || groups > DEC_ROWS || num_splits < 0 || num_splits > MERGE_MAX_SPLITS) return FE_ERR_BAD_SHAPE;
  if (entries > 65535 || num_kv_heads > 65535) return FE_ERR_TOO_LARGE;
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) return FE_ERR_BAD_ALIGN;
  if ((q_stride % 8) != 0) return FE_ERR_BAD_ALIGN;
  AttnParams p;
  p.q = (const bf16*)q; p.q_stride = q_stride; p.out = (bf16*)out;
  p.k = (const bf16*)k_cache; p.v = (const bf16*)v_cache;
  p.block_table = block_table; p.max_pages = max_pages; p.page_size = page_size; p.num_pages = num_pages;
  p.nkv = num_kv_heads; p.groups = groups; p.cu_tokens = cu_tokens; p.starts = starts;
  p.window = window; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  p.num_splits = num_splits;
  p.ws_acc = workspace;
  p.ws_ml = workspace ? workspace + (size_t)entries * num_kv_heads * num_splits * DEC_ROWS * D : nullptr;
  p.ws_count = counters;
  p.cluster_merge = 0;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)PREFILL_SMEM);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DECODE_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const bool use_decode = (mode & 2) != 0;
  const int decode_rows = use_decode ? DEC_ROWS : 0;
  if (mode & 1) {
    const int max_rows = max_new * groups;
    if (max_rows > decode_rows) {
      p.row_lo = decode_rows; p.row_hi = 0x7fffffff;
      // tcgen05 form where its shapes hold; FORGE_ENGINE_PREFILL_MMA=1 keeps the mma.sync kernel
      static const bool force_mma = getenv("FORGE_ENGINE_PREFILL_MMA") != nullptr && getenv("FORGE_ENGINE_PREFILL_MMA")[0] == '1';
      const bool tc5_ok = !force_mma && (D == 128 || D == 64) && (TC5_ROWS % groups) == 0 && page_size <= TC5_KEYS &&
                          page_size * 32 >= TC5_KEYS && (TC5_KEYS % page_size) == 0 && scale > 0.f && ensure_encode();
      CUtensorMap mk_copy, mv_copy;
      const CUtensorMap* mk = tc5_ok && cache_map(&mk_copy, k_cache, num_pages * num_kv_heads * page_size, page_size) ? &mk_copy : nullptr;
      const CUtensorMap* mv = mk && cache_map(&mv_copy, v_cache, num_pages * num_kv_heads * page_size, page_size) ? &mv_copy : nullptr;
      CUtensorMap mq;
      if (mk && mv && make_query_map(&mq, q, q_stride, total_tokens, num_kv_heads * groups, groups) == 0) {
        static bool tc5_configured = false;
        if (!tc5_configured) {
          const cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     (int)TC5_SMEM);
          if (e != cudaSuccess) return (int)e;
          tc5_configured = true;
        }
        const int query_blocks = (max_rows + TC5_BLOCK_ROWS - 1) / TC5_BLOCK_ROWS;
        if (query_blocks > 65535) return FE_ERR_TOO_LARGE;
        dim3 grid(num_kv_heads, entries, query_blocks);
        const int rc = fe_launch_dependent(attn_prefill_tc5_kernel, grid, dim3(TC5_THREADS), TC5_SMEM, stream, mq, *mk,
                                           *mv, p);
        if (rc) return rc;
      } else {
        dim3 grid((max_rows + BM - 1) / BM, entries, num_kv_heads);
        const int rc = fe_launch_dependent(attn_prefill_kernel, grid, dim3(THREADS), PREFILL_SMEM, stream, p);
        if (rc) return rc;
      }
    }
  }
  if (use_decode && num_splits == 0) {
    // the step's tiles spread evenly over as many blocks as the GPU holds at once
    if (workspace == nullptr || entries > BAL_MAX_ENTRIES) return FE_ERR_BAD_SHAPE;
    if ((D % 64) != 0 || page_size > BN || (BN % page_size) != 0) return FE_ERR_BAD_SHAPE;
    CUtensorMap mk_copy, mv_copy;
    const CUtensorMap* mk = cache_map(&mk_copy, k_cache, num_pages * num_kv_heads * page_size, page_size, true) ? &mk_copy : nullptr;
    const CUtensorMap* mv = mk && cache_map(&mv_copy, v_cache, num_pages * num_kv_heads * page_size, page_size, true) ? &mv_copy : nullptr;
    if (!mk || !mv) return FE_ERR_BAD_SHAPE;
    const int blocks = SYM(fe_attn_balanced_blocks_d)();
    if (blocks <= 0) return FE_ERR_BAD_SHAPE;
    p.row_lo = 0; p.row_hi = DEC_ROWS;
    p.ws_ml = workspace + (size_t)2 * blocks * DEC_ROWS * D;
    int rc = fe_launch_dependent(attn_decode_balanced_kernel, dim3(blocks), dim3(TMA_THREADS), DECODE_BALANCED_SMEM,
                                 stream, *mk, *mv, p, entries);
    if (rc) return rc;
    rc = fe_launch_dependent(attn_merge_balanced_kernel, dim3(entries, num_kv_heads), dim3(THREADS), 0, stream, p,
                             entries, blocks);
    if (rc) return rc;
    return fe_last_error();
  }
  if (use_decode) {
    if (num_splits > 1 && workspace == nullptr) return FE_ERR_BAD_SHAPE;
    p.row_lo = 0; p.row_hi = DEC_ROWS;
    dim3 grid(num_splits, entries, num_kv_heads);
    int rc = 0;
    const bool tma_ok = (D % 64) == 0 && page_size <= BN && (BN % page_size) == 0 && (num_splits == 1 || counters != nullptr);
    CUtensorMap mk_copy, mv_copy;
    const CUtensorMap* mk = tma_ok && cache_map(&mk_copy, k_cache, num_pages * num_kv_heads * page_size, page_size, true) ? &mk_copy : nullptr;
    const CUtensorMap* mv = mk && cache_map(&mv_copy, v_cache, num_pages * num_kv_heads * page_size, page_size, true) ? &mv_copy : nullptr;
    if (mk && mv) {
      static bool tma_configured = false;
      if (!tma_configured) {
        const cudaError_t e = cudaFuncSetAttribute(attn_decode_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   (int)DECODE_TMA_SMEM);
        if (e != cudaSuccess) return (int)e;
        tma_configured = true;
      }
      // up to 8 splits: one cluster per (entry, kv head), partial results never leave the SMs;
      // a multiple of 8: clusters of 8 combine theirs first, the last block to arrive the clusters'
      p.cluster_merge = (num_splits > 1 && num_splits <= 8) ? 1 : ((num_splits > 8 && num_splits % 8 == 0) ? 2 : 0);
      rc = fe_launch_dependent_shaped(attn_decode_tma_kernel, grid, dim3(TMA_THREADS), DECODE_TMA_SMEM, stream,
                                      dim3(p.cluster_merge == 1 ? num_splits : (p.cluster_merge == 2 ? 8 : 1), 1, 1), *mk, *mv, p);
      p.cluster_merge = 0;
    } else {
      rc = fe_launch_dependent(attn_decode_kernel, grid, dim3(THREADS), DECODE_SMEM, stream, p);
    }
    if (rc) return rc;
    if (num_splits > 1 && counters == nullptr) {
      dim3 mgrid(entries, num_kv_heads);
      rc = fe_launch_dependent(attn_merge_kernel, mgrid, dim3(THREADS), 0, stream, p);
      if (rc) return rc;
    }
  }
  return fe_last_error();
}

// ---------------------------------------------------------------------------
// Split decode attention for callers that must not allocate (see attention_noalloc.h).
// No counterpart upstream.
// ---------------------------------------------------------------------------

// Scratch for the splits' partial results, held by every GPU that loads this library
// until the process exits: 1,048,576 floats = 4 MiB (the size and the error code are the
// header's, so that declaration and definition cannot drift apart).
#define FE_NOALLOC_SCRATCH_FLOATS FE_ATTENTION_NOALLOC_SCRATCH_FLOATS
static __device__ __align__(256) float fe_noalloc_scratch[FE_NOALLOC_SCRATCH_FLOATS];

#define FE_NOALLOC_MAX_DEVICES 64

FE_EXPORT int SYM(fe_attention_decode_noalloc_d)(const void* q, int q_stride, void* out,
                                                 const void* k_cache, const void* v_cache,
                                                 const int* block_table, int max_pages, int page_size,
                                                 int num_pages, int num_kv_heads, int groups,
                                                 const int* cu_tokens, const int* starts, int entries,
                                                 int max_new, int window, float scale, int num_splits,
                                                 int* status, cudaStream_t stream) {
  // Device address of the scratch array, looked up once per device.  In host code the
  // array's name is only a handle for the runtime, not a pointer a kernel could use.
  static float* scratch_of_device[FE_NOALLOC_MAX_DEVICES] = {nullptr};
  if (entries <= 0) return 0;
  if (groups < 1 || num_splits < 1 || num_splits > MERGE_MAX_SPLITS || max_new < 1 || max_new * groups > DEC_ROWS)
    return FE_ERR_BAD_SHAPE;
  if (entries > 65535 || num_kv_heads > 65535) return FE_ERR_TOO_LARGE;
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) return FE_ERR_BAD_ALIGN;
  if ((q_stride % 8) != 0) return FE_ERR_BAD_ALIGN;
  // with one split a block writes its result straight to `out` and the array is not touched
  const long long needed = num_splits == 1 ? 0 : (long long)entries * num_kv_heads * num_splits * DEC_ROWS * (D + 2);
  if (needed > FE_NOALLOC_SCRATCH_FLOATS) {
    fprintf(stderr,
            "fe_attention_decode_noalloc: entries=%d x kv_heads=%d x splits=%d needs %lld floats of scratch, "
            "the built-in array holds %d; use fewer splits or fewer entries per call\n",
            entries, num_kv_heads, num_splits, needed, FE_NOALLOC_SCRATCH_FLOATS);
    return FE_ERR_SCRATCH_TOO_SMALL;
  }
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= FE_NOALLOC_MAX_DEVICES) return FE_ERR_TOO_LARGE;
  if (scratch_of_device[device] == nullptr) {
    float* address = nullptr;
    e = cudaGetSymbolAddress((void**)&address, fe_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DECODE_SMEM);
    if (e != cudaSuccess) return (int)e;
    scratch_of_device[device] = address;
  }
  float* scratch = scratch_of_device[device];
  AttnParams p;
  p.q = (const bf16*)q; p.q_stride = q_stride; p.out = (bf16*)out;
  p.k = (const bf16*)k_cache; p.v = (const bf16*)v_cache;
  p.block_table = block_table; p.max_pages = max_pages; p.page_size = page_size; p.num_pages = num_pages;
  p.nkv = num_kv_heads; p.groups = groups; p.cu_tokens = cu_tokens; p.starts = starts;
  p.window = window; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  p.num_splits = num_splits;
  p.ws_acc = scratch;
  p.ws_ml = scratch + (size_t)entries * num_kv_heads * num_splits * DEC_ROWS * D;
  p.ws_count = nullptr;
  p.cluster_merge = 0;
  p.row_lo = 0; p.row_hi = DEC_ROWS;
  dim3 grid(num_splits, entries, num_kv_heads);
  attn_decode_kernel<<<grid, THREADS, DECODE_SMEM, stream>>>(p);
  if (num_splits > 1) {
    dim3 mgrid(entries, num_kv_heads);
    attn_merge_kernel<<<mgrid, THREADS, 0, stream>>>(p);
  }
  return fe_last_error();
}

// y[n, o] = sum_k x[n, k] * w[o, k]  on the 5th-generation tensor cores (tcgen05), bfloat16
// operands, 32-bit accumulators in tensor memory, operands staged by TMA.
//
// Orientation: the 128-row side of the MMA is the *weight* ([out, in] rows, K-major, as
// nn.Linear stores them: src/forge_engine/qwen3.py:113-122), the N side is the tokens.
// With few tokens (decode) a block still streams a full 128 x 64 weight tile per stage, so
// the kernel is bound by reading the weights once; with many tokens N grows to 256.
//
//   block (6 warps):  warp 0  TMA producer: per 64-wide k-block one weight tile
//                             [128 x 64] and one token tile [N x 64], 128-byte swizzle
//                     warp 1  allocates tensor memory, issues tcgen05.mma (one lane),
//                             commits to the stage's "empty" barrier
//                     warps 2-5  epilogue: tcgen05.ld of their 32 accumulator lanes
//                             (lane = output feature, column = token), bias / SiLU*mul /
//                             residual add, coalesced stores along the feature dimension
//   grid (feature tiles, token tiles, k-splits).  With k-splits > 1 the blocks of one tile
//   add their partial tiles in split order, so results do not depend on timing: up to 8
//   splits form a thread-block cluster whose blocks each finish a share of the tile's
//   tokens, reading the others' partial tiles from their shared memory; beyond that (or for
//   wide token tiles) partial tiles go through a workspace and the block that arrives last
//   adds them.
//
// Every wait on an mbarrier is bounded; when a bound is hit the block sets a bit in the
// status word, stops issuing work, frees its tensor memory and returns.  The bound is far
// longer than any copy takes, so by the time it is hit the block's own copies in flight have
// landed.  fe_gemm_tc5_set_test_fault makes one wait run out on purpose (a short bound and a
// producer that leaves out one load), so that a test can see the status word and that the
// device is usable afterwards; nothing traps, faults or spins on.
#include "tcgen05.cuh"

namespace {

using namespace tc5;

constexpr int THREADS = 192;
// Widest token tile whose k-splits add up inside a cluster: the 32-bit partial tile of a
// block (tokens x 128 features) must fit in its ring of stages (128 tokens: 64 of 96 KB).
constexpr int CLUSTER_REDUCE_TOKENS = 128;

enum Epilogue { EPI_STORE_BF16 = 0, EPI_STORE_F32 = 1, EPI_ADD_F32 = 2, EPI_SILU_MUL_BF16 = 3, EPI_QKV_ROPE = 4 };

// What the fused q/k/v projection needs beyond the product (EPI_QKV_ROPE; head size 128, so
// that a 128-feature tile is one head): per-head RMS norm of q and k with one [128] weight
// each (src/forge_engine/qwen3.py:141-150), the half-split rotation (qwen3.py:345-381) and
// the write of k and v into their cache pages (src/forge_engine/cache.py:385-416).  q is
// stored rotated into y; k and v go to the pages only.
struct QkvRope {
  const float* q_weight;   // [128] or null: no norm
  const float* k_weight;
  float eps;
  const float2* table;     // [n, 64] (cos, sin) of every token's angles, or null: no rotation
  const int* positions;    // [n] position of every token in its request
  const int* token_entry;  // [n] row of the block table
  bf16* k_cache;           // [pages, kv heads, page_size, 128]
  bf16* v_cache;
  const int* block_table;  // [entries, max_pages]
  int max_pages, page_size, num_pages, num_q_heads, num_kv_heads, write_kv;
};

struct GemmParams {
  void* y;
  const float* bias;
  int n, o, k;
  int epilogue;
  int ksplit;
  int cluster_reduce;    // k-splits of a tile form a cluster and add their partial tiles through shared memory
  int atomic_add;        // EPI_ADD_F32 with k-splits: every block adds its partial tile into y itself (32-bit atomics)
  float* ws_part;        // [feature tiles, token tiles, ksplit, BN, BM] floats
  unsigned* ws_count;    // [feature tiles * token tiles], zero before and after a launch
  int* status;
  unsigned wait_limit;   // polls a wait may take before the block gives up
  int skip_kblock;       // test fault: the producer leaves out the load of this k-block (-1: none)
  QkvRope rope;          // EPI_QKV_ROPE only
};

template <int BN, int EPI = 0> __host__ __device__ constexpr int stages_for() {
  // stage = weight tile (16 KB) + token tile (BN * 128 B).  Narrow token tiles keep the ring
  // at about 100 KB (108, 100 and 96 KB for 16, 32 and 64 tokens), two blocks per SM, so that
  // one block's epilogue and set-up overlap another's streaming and a product's 150-190
  // blocks all run at once; the widest tile takes the SM alone.
  // (The gate/up product has about one block per SM; eight stages and the SM to itself for its
  // 64-token form measured worse, 6.44 against 5.81 ms per step at batch 64: the next product's
  // blocks then find no room to become resident and fill their rings meanwhile.  Shallower
  // rings with more blocks per SM for 16 tokens, -DFE_TC5_STAGES_16=5, 4, 3: 2.14, 2.20 and
  // 2.36 ms per decode step at batch 1 against 2.11 ms with 6; 4 stages at batch 8: 2.52
  // against 2.46 ms.  The gate/up product alone with 5, 8 or 12 stages at batch 8: 2.47, 2.94
  // and 2.96 ms: from 7 stages on no second block fits on the SM.)
#ifndef FE_TC5_STAGES_16
#define FE_TC5_STAGES_16 6
#endif
  return BN <= 16 ? FE_TC5_STAGES_16 : (BN <= 32 ? 5 : (BN <= 64 ? 4 : (BN == 128 ? 3 : 4)));
}

// Finished values of one accumulator row (feature) for 16 consecutive tokens.
template <int EPI>
__device__ __forceinline__ void store16(const GemmParams& p, float (&v)[16], int feature, int token0, int lane) {
  if (EPI == EPI_SILU_MUL_BF16) {
    // weight rows alternate 16 gate features, 16 up features: lanes 0-15 hold gate,
    // lanes 16-31 the matching up.  The lower half-warp finishes even tokens, the upper
    // half odd ones, so both halves store.
    const int half_o = p.o >> 1;
    const int out_feature = (feature >> 5) * 16 + (lane & 15);
    bf16* y = reinterpret_cast<bf16*>(p.y);
#pragma unroll
    for (int j = 0; j < 16; j += 2) {
      const float send = lane < 16 ? v[j + 1] : v[j];
      const float recv = __shfl_xor_sync(0xffffffffu, send, 16);
      const int token = token0 + j + (lane < 16 ? 0 : 1);
      const float r = lane < 16 ? silu_f(v[j]) * recv : silu_f(recv) * v[j + 1];
      if (token < p.n && out_feature < half_o) y[(size_t)token * half_o + out_feature] = __float2bfloat16_rn(r);
    }
    return;
  }
  if (feature >= p.o) return;
  const float b = p.bias ? p.bias[feature] : 0.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int token = token0 + j;
    if (token >= p.n) break;
    const size_t at = (size_t)token * p.o + feature;
    const float r = v[j] + b;
    if (EPI == EPI_STORE_BF16) reinterpret_cast<bf16*>(p.y)[at] = __float2bfloat16_rn(r);
    else if (EPI == EPI_STORE_F32) reinterpret_cast<float*>(p.y)[at] = r;
    else reinterpret_cast<float*>(p.y)[at] = __ldcg(reinterpret_cast<const float*>(p.y) + at) + r;
  }
}

// EPI_QKV_ROPE: the 128 epilogue threads hold one head's 128 values of one token.  `turn`
// alternates between two sets of exchange buffers so that one named barrier per step is
// enough.  Same arithmetic as qk_rope_cache.cu, on the 32-bit sums instead of their
// bfloat16 roundings.
__device__ __forceinline__ void rope_token(const GemmParams& p, float v, int head, int d, int token, float* exchange,
                                           int turn, int quarter, int lane) {
  const QkvRope& r = p.rope;
  const bool live = token < p.n;
  const bool is_q = head < r.num_q_heads, is_k = !is_q && head < r.num_q_heads + r.num_kv_heads;
  float* sums = exchange + turn * 136;      // [4] warps' sums of squares, then [128] normalised values
  float* values = sums + 8;
  float out = v + (p.bias ? p.bias[head * 128 + d] : 0.f);
  const int pos = live ? r.positions[token] : 0;
  if (is_q || is_k) {
    const float* w = is_q ? r.q_weight : r.k_weight;
    if (w) {
      float ss = out * out;
#pragma unroll
      for (int offset = 16; offset > 0; offset >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, offset);
      if (lane == 0) sums[quarter] = ss;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      ss = ((sums[0] + sums[1]) + sums[2]) + sums[3];
      out = out * rsqrtf(ss / 128.f + r.eps) * w[d];
    }
    if (r.table) {
      values[d] = out;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const float partner = values[d ^ 64];
      const float2 cs = live ? r.table[(size_t)token * 64 + (d & 63)] : make_float2(1.f, 0.f);
      out = d < 64 ? out * cs.x - partner * cs.y : out * cs.x + partner * cs.y;
    }
  }
  if (!live) return;
  if (is_q) {
    reinterpret_cast<bf16*>(p.y)[(size_t)token * p.o + head * 128 + d] = __float2bfloat16_rn(out);
    return;
  }
  if (!r.write_kv) return;
  const int logical = pos / r.page_size, slot = pos - logical * r.page_size;
  if (pos < 0 || logical >= r.max_pages) {
    if (d == 0 && p.status) atomicOr(p.status, FE_STATUS_BAD_POSITION);
    return;
  }
  const int page = r.block_table[(size_t)r.token_entry[token] * r.max_pages + logical];
  if (page < 0 || page >= r.num_pages) {
    if (d == 0 && p.status) atomicOr(p.status, FE_STATUS_BAD_PAGE);
    return;
  }
  const int kvh = is_k ? head - r.num_q_heads : head - r.num_q_heads - r.num_kv_heads;
  bf16* cache = is_k ? r.k_cache : r.v_cache;
  cache[(((size_t)page * r.num_kv_heads + kvh) * r.page_size + slot) * 128 + d] = __float2bfloat16_rn(out);
}

// One finished value: feature `feature` (this lane's accumulator row) of token `token`.  All
// lanes of the warp call it for the same token.
template <int EPI>
__device__ __forceinline__ void store_one(const GemmParams& p, float v, int feature, int token, int lane) {
  if (EPI == EPI_SILU_MUL_BF16) {
    // lanes 0-15 hold 16 gate features, lanes 16-31 the matching up features
    const float up = __shfl_xor_sync(0xffffffffu, v, 16);
    const int half_o = p.o >> 1;
    const int out_feature = (feature >> 5) * 16 + (lane & 15);
    if (lane < 16 && token < p.n && out_feature < half_o)
      reinterpret_cast<bf16*>(p.y)[(size_t)token * half_o + out_feature] = __float2bfloat16_rn(silu_f(v) * up);
    return;
  }
  if (feature >= p.o || token >= p.n) return;
  const size_t at = (size_t)token * p.o + feature;
  const float r = v + (p.bias ? p.bias[feature] : 0.f);
  if (EPI == EPI_STORE_BF16) reinterpret_cast<bf16*>(p.y)[at] = __float2bfloat16_rn(r);
  else if (EPI == EPI_STORE_F32) reinterpret_cast<float*>(p.y)[at] = r;
  else reinterpret_cast<float*>(p.y)[at] = __ldcg(reinterpret_cast<const float*>(p.y) + at) + r;
}

template <int BN, int EPI>
__global__ void __launch_bounds__(THREADS)
gemm_tc5_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GemmParams p) {
  constexpr int STAGES = stages_for<BN, EPI>();
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  static_assert(BN > CLUSTER_REDUCE_TOKENS || BN * BM * 4 <= STAGES * (A_BYTES + B_BYTES),
                "a block's partial tile is stashed over its ring of stages");
  extern __shared__ unsigned char smem_raw[];
  // 1024-byte alignment: the swizzle pattern repeats every 8 rows of 128 bytes
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* a_tiles = smem;
  unsigned char* b_tiles = smem + STAGES * A_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(b_tiles + STAGES * B_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_done = empty + STAGES;
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* last_flag = const_cast<int*>(abort_flag) + 1;
  float* exchange = reinterpret_cast<float*>(last_flag + 2);     // EPI_QKV_ROPE: 2 x 136 floats

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int kblocks = (p.k + BK - 1) / BK;
  const int per_split = (kblocks + p.ksplit - 1) / p.ksplit;
  const int kb_begin = blockIdx.z * per_split;
  const int kb_end = min(kblocks, kb_begin + per_split);
  const int my_blocks = max(0, kb_end - kb_begin);

  if (threadIdx.x == 0) {
    tma_prefetch_map(&map_w);
    tma_prefetch_map(&map_x);
    for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    mbar_init(acc_done, 1);
    *abort_flag = 0;
    *last_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_slot;

  pdl_trigger();   // the kernel after this one may begin its own weight prefetch
  if (warp == 0) {
    if (lane == 0) {
      // Weights do not depend on the kernel before this one: fill the ring with weight
      // tiles first, then wait for that kernel, then fetch the token tiles.
      const int ahead = min(STAGES, my_blocks);
      for (int i = 0; i < ahead; ++i) {
        if (kb_begin + i == p.skip_kblock) continue;      // test fault: this stage never fills
        mbar_expect_tx(full + i, A_BYTES + B_BYTES);
        tma_load_2d(a_tiles + i * A_BYTES, &map_w, (kb_begin + i) * BK, m0, full + i);
      }
      pdl_wait();
      for (int i = 0; i < ahead; ++i)
        if (kb_begin + i != p.skip_kblock) tma_load_2d(b_tiles + i * B_BYTES, &map_x, (kb_begin + i) * BK, n0, full + i);
      for (int i = ahead; i < my_blocks; ++i) {
        const int s = i % STAGES;
        const unsigned parity = ((i / STAGES) & 1) ^ 1;
        if (!mbar_wait(empty + s, parity, abort_flag, p.wait_limit)) break;
        if (kb_begin + i == p.skip_kblock) continue;      // test fault: this stage never fills
        mbar_expect_tx(full + s, A_BYTES + B_BYTES);
        const int kcoord = (kb_begin + i) * BK;
        tma_load_2d(a_tiles + s * A_BYTES, &map_w, kcoord, m0, full + s);
        tma_load_2d(b_tiles + s * B_BYTES, &map_x, kcoord, n0, full + s);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const unsigned idesc = umma_idesc(BN);
      bool ok = true;
      for (int i = 0; i < my_blocks && ok; ++i) {
        const int s = i % STAGES;
        const unsigned parity = (i / STAGES) & 1;
        ok = mbar_wait(full + s, parity, abort_flag, p.wait_limit);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t da = umma_desc(a_tiles + s * A_BYTES);
        const uint64_t db = umma_desc(b_tiles + s * B_BYTES);
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk) {
          // 16 k = 32 bytes further along the swizzled row: +2 in units of 16 bytes
          umma_f16(tmem_base, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (i | kk) != 0 ? 1u : 0u);
        }
        umma_commit(empty + s);      // the stage may be refilled once these MMAs have read it
      }
      umma_commit(acc_done);         // arrives when every MMA issued above has finished
    }
  } else {
    // epilogue warps 2..5 own accumulator lanes 32 * (warp % 4) .. +31
    const int quarter = warp & 3;
    const int feature = m0 + quarter * 32 + lane;
    mbar_wait(acc_done, 0, abort_flag, p.wait_limit);
    pdl_wait();   // returns at once after the producer's wait; orders this warp's own global accesses
    // all four epilogue warps take the same path: agree on the outcome of the wait
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const bool ok = *abort_flag == 0;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned lane_base = tmem_base + ((unsigned)(quarter * 32) << 16);
    const bool split = p.ksplit > 1;
    if (ok && split && p.atomic_add) {
      // "+=" commutes: no block waits for another, the partial sums meet in memory
      float* y = reinterpret_cast<float*>(p.y);
#pragma unroll 1
      for (int c = 0; c < BN && my_blocks > 0; c += 16) {
        float v[16];
        tmem_ld16(lane_base + c, v);
        if (feature < p.o) {
          const float b = (p.bias && blockIdx.z == 0) ? p.bias[feature] : 0.f;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int token = n0 + c + j;
            if (token < p.n)
              asm volatile("red.relaxed.gpu.global.add.f32 [%0], %1;" ::"l"(y + (size_t)token * p.o + feature), "f"(v[j] + b) : "memory");
          }
        }
      }
    } else if (ok && !split) {
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        float v[16];
        if (my_blocks > 0) tmem_ld16(lane_base + c, v);
        else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
        }
        if (EPI == EPI_QKV_ROPE) {
#pragma unroll 1
          for (int j = 0; j < 16; ++j) rope_token(p, v[j], blockIdx.x, quarter * 32 + lane, n0 + c + j, exchange, j & 1, quarter, lane);
        } else {
          store16<EPI>(p, v, feature, n0 + c, lane);
        }
      }
    } else if (ok && p.cluster_reduce) {
      // stash the partial tile in this block's shared memory ([token][feature], over the
      // first weight stages, which nobody reads any more); the cluster's blocks add the
      // stashes below
      float* stash = reinterpret_cast<float*>(a_tiles);
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        float v[16];
        if (my_blocks > 0) tmem_ld16(lane_base + c, v);
        else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) stash[(c + j) * BM + quarter * 32 + lane] = v[j];
      }
    } else if (ok) {
      // publish the partial tile: ws[tile][split][token][feature]
      const size_t tile = (size_t)blockIdx.x * gridDim.y + blockIdx.y;
      float* mine = p.ws_part + (tile * p.ksplit + blockIdx.z) * (size_t)(BN * BM);
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        float v[16];
        if (my_blocks > 0) tmem_ld16(lane_base + c, v);
        else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) mine[(size_t)(c + j) * BM + quarter * 32 + lane] = v[j];
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) {
        const unsigned arrived = atomicAdd(p.ws_count + tile, 1u);
        const int last = arrived == (unsigned)p.ksplit - 1u;
        if (last) p.ws_count[tile] = 0u;
        *last_flag = last;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*last_flag) {
        __threadfence();
        const float* all = p.ws_part + tile * p.ksplit * (size_t)(BN * BM);
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
          for (int sp = 0; sp < p.ksplit; ++sp) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              v[j] += __ldcg(all + (size_t)sp * (BN * BM) + (size_t)(c + j) * BM + quarter * 32 + lane);
          }
          if (EPI == EPI_QKV_ROPE) {
#pragma unroll 1
            for (int j = 0; j < 16; ++j) rope_token(p, v[j], blockIdx.x, quarter * 32 + lane, n0 + c + j, exchange, j & 1, quarter, lane);
          } else {
            store16<EPI>(p, v, feature, n0 + c, lane);
          }
        }
      }
    }
  }

  if (p.cluster_reduce) {
    // every thread of every block of the cluster takes part in both barriers
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    unsigned rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    if (warp >= 2 && *abort_flag == 0) {
      // every block of the cluster finishes a share of the tile's live tokens: it adds the
      // blocks' partial values of those tokens in block order (the sum does not depend on
      // timing, on the number of tokens or on which block does it) and stores them
      const int quarter = warp & 3;
      const int row = quarter * 32 + lane;
      const int live = min(BN, p.n - n0);
      const int share = (live + p.ksplit - 1) / p.ksplit;
      const int t_begin = (int)rank * share, t_end = min(live, t_begin + share);
      const unsigned local = smem_u32(a_tiles);
      unsigned remote[8];
#pragma unroll
      for (int peer = 0; peer < 8; ++peer)
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote[peer]) : "r"(local), "r"(peer < p.ksplit ? peer : 0));
      constexpr bool PLAIN_STORE = EPI == EPI_STORE_BF16 || EPI == EPI_STORE_F32 || EPI == EPI_ADD_F32;
      if (PLAIN_STORE && (p.o & 3) == 0 && (reinterpret_cast<uintptr_t>(p.y) & 15) == 0) {
        // A warp takes a token and a lane four neighbouring features: one 16-byte load per
        // block of the cluster instead of four 4-byte ones (the loads between SMs are what
        // this phase waits for), two tokens in flight, and the residual row fetched first.
        const int f4 = m0 + lane * 4;
        const bool inside = f4 < p.o;
        for (int t = t_begin + quarter; t < t_end; t += 8) {
          float4 prior[2], part[2][8];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int tok = t + 4 * u;
            prior[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (EPI == EPI_ADD_F32 && inside && tok < t_end)
              prior[u] = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.y) +
                                                                (size_t)(n0 + tok) * p.o + f4));
          }
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int tok = t + 4 * u;
#pragma unroll
            for (int peer = 0; peer < 8; ++peer) {
              part[u][peer] = make_float4(0.f, 0.f, 0.f, 0.f);
              if (peer < p.ksplit && tok < t_end)
                asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];"
                             : "=f"(part[u][peer].x), "=f"(part[u][peer].y), "=f"(part[u][peer].z), "=f"(part[u][peer].w)
                             : "r"(remote[peer] + (unsigned)((tok * BM + lane * 4) * 4)) : "memory");
            }
          }
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int tok = t + 4 * u;
            if (tok >= t_end || !inside) continue;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int peer = 0; peer < 8; ++peer) {
              v.x += part[u][peer].x; v.y += part[u][peer].y; v.z += part[u][peer].z; v.w += part[u][peer].w;
            }
            if (p.bias) {
              v.x += p.bias[f4]; v.y += p.bias[f4 + 1]; v.z += p.bias[f4 + 2]; v.w += p.bias[f4 + 3];
            }
            const size_t at = (size_t)(n0 + tok) * p.o + f4;
            if (EPI == EPI_STORE_BF16) {
              __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
              uint2 packed;
              packed.x = *reinterpret_cast<unsigned*>(&lo);
              packed.y = *reinterpret_cast<unsigned*>(&hi);
              *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(p.y) + at) = packed;
            } else if (EPI == EPI_STORE_F32) {
              *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.y) + at) = v;
            } else {
              *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.y) + at) =
                  make_float4(prior[u].x + v.x, prior[u].y + v.y, prior[u].z + v.z, prior[u].w + v.w);
            }
          }
        }
      } else
      // four tokens at a time, so that their loads from the other blocks are in flight together
      for (int t = t_begin; t < t_end; t += 4) {
        float part[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int peer = 0; peer < 8; ++peer) {
            part[u][peer] = 0.f;
            if (peer < p.ksplit && t + u < t_end)
              asm volatile("ld.shared::cluster.f32 %0, [%1];"
                           : "=f"(part[u][peer]) : "r"(remote[peer] + (unsigned)(((t + u) * BM + row) * 4)) : "memory");
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (t + u < t_end) {        // the same for the whole block
            float v = 0.f;
#pragma unroll
            for (int peer = 0; peer < 8; ++peer) v += part[u][peer];
            if (EPI == EPI_QKV_ROPE) rope_token(p, v, blockIdx.x, row, n0 + t + u, exchange, (t + u) & 1, quarter, lane);
            else store_one<EPI>(p, v, m0 + row, n0 + t + u, lane);
          }
        }
      }
    }
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");   // stashes stay alive until read
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicOr(p.status, FE_STATUS_WAIT_TIMEOUT);
}

template <int BN, int EPI> constexpr size_t smem_bytes() {
  return (size_t)stages_for<BN, EPI>() * (BM * BK * 2 + BN * BK * 2) + (2 * stages_for<BN, EPI>() + 1) * 8 + 16 +
         (EPI == EPI_QKV_ROPE ? 2 * 136 * 4 : 0) + 1024;
}

template <int BN, int EPI>
int launch_one(const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, dim3 grid, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    const cudaError_t e = cudaFuncSetAttribute(gemm_tc5_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)smem_bytes<BN, EPI>());
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int rc = fe_launch_dependent_cluster(gemm_tc5_kernel<BN, EPI>, grid, dim3(THREADS), smem_bytes<BN, EPI>(), stream,
                                             p.cluster_reduce ? p.ksplit : 1, mw, mx, p);
  if (rc) return rc;
  return fe_last_error();
}

template <int BN>
int launch_bn(const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, dim3 grid, cudaStream_t stream) {
  switch (p.epilogue) {
    case EPI_STORE_BF16: return launch_one<BN, EPI_STORE_BF16>(mw, mx, p, grid, stream);
    case EPI_STORE_F32: return launch_one<BN, EPI_STORE_F32>(mw, mx, p, grid, stream);
    case EPI_ADD_F32: return launch_one<BN, EPI_ADD_F32>(mw, mx, p, grid, stream);
    case EPI_SILU_MUL_BF16: return launch_one<BN, EPI_SILU_MUL_BF16>(mw, mx, p, grid, stream);
    case EPI_QKV_ROPE:
      if (BN <= 64) return launch_one<(BN <= 64 ? BN : 16), EPI_QKV_ROPE>(mw, mx, p, grid, stream);
      return FE_ERR_BAD_SHAPE;
  }
  return FE_ERR_BAD_DTYPE;
}

// Test fault (see the head of this file); 0 / -1: none.
unsigned g_test_wait_limit = 0;
int g_test_skip_kblock = -1;

}  // namespace

// For tests of the bounded waits only: launches after this call poll at most `wait_limit`
// times per wait (0: the usual bound) and their producers leave out the load of k-block
// `skip_kblock` (-1: none), so that the block waiting for it gives up, sets
// FE_STATUS_WAIT_TIMEOUT and returns.  Call with (0, -1) to go back to normal.
FE_EXPORT void fe_gemm_tc5_set_test_fault(unsigned wait_limit, int skip_kblock) {
  g_test_wait_limit = wait_limit;
  g_test_skip_kblock = skip_kblock;
}

// Token-tile width the kernel uses for n tokens.
FE_EXPORT int fe_gemm_tc5_tile(int n) { return n <= 16 ? 16 : (n <= 32 ? 32 : (n <= 64 ? 64 : (n <= 128 ? 128 : 256))); }

static int run_gemm(const void* x, const void* w, const float* bias, void* y, int n, int o, int k, int epilogue, int ksplit,
                    float* ws_part, unsigned* ws_count, int* status, const QkvRope* rope, cudaStream_t stream) {
  if (n <= 0 || o <= 0) return 0;
  if (k <= 0 || (k % 8) != 0) return FE_ERR_BAD_SHAPE;
  if (epilogue == EPI_SILU_MUL_BF16 && ((o % 32) != 0 || bias != nullptr)) return FE_ERR_BAD_SHAPE;
  if ((((uintptr_t)x) | ((uintptr_t)w)) & 15) return FE_ERR_BAD_ALIGN;
  if (ksplit < 1) ksplit = 1;
  const int kblocks = (k + BK - 1) / BK;
  if (ksplit > kblocks) ksplit = kblocks;
  const int bn = fe_gemm_tc5_tile(n);

  CUtensorMap mw, mx;
  int rc = make_map(&mw, w, o, k, BM);
  if (rc) return rc;
  rc = make_map(&mx, x, n, k, bn);
  if (rc) return rc;
  // Partial sums of a "+=" product may meet in memory through 32-bit atomic adds instead of
  // being added in split order by the blocks of a cluster: no block then waits for the
  // slowest of its cluster, at the price of a sum whose rounding depends on the order of
  // arrival (FORGE_ENGINE_ATOMIC_SPLITK=0 keeps the ordered sum).
  static int atomic_wish = -1;
  if (atomic_wish < 0) {
    const char* text = getenv("FORGE_ENGINE_ATOMIC_SPLITK");
    atomic_wish = (text != nullptr && text[0] == '0') ? 0 : 1;
  }
  const int atomic_add = (epilogue == EPI_ADD_F32 && ksplit > 1 && atomic_wish) ? 1 : 0;
  if (ksplit > 1 && !atomic_add && !(ksplit <= 8 && bn <= CLUSTER_REDUCE_TOKENS) && (ws_part == nullptr || ws_count == nullptr))
    return FE_ERR_BAD_SHAPE;
  const int cluster_reduce = (!atomic_add && ksplit > 1 && ksplit <= 8 && bn <= CLUSTER_REDUCE_TOKENS) ? 1 : 0;
  GemmParams p{y, bias, n, o, k, epilogue, ksplit, cluster_reduce, atomic_add, ws_part, ws_count, status,
               g_test_wait_limit ? g_test_wait_limit : WAIT_LIMIT, g_test_skip_kblock, rope ? *rope : QkvRope{}};
  dim3 grid((o + BM - 1) / BM, (n + bn - 1) / bn, ksplit);
  if (grid.y > 65535 || grid.z > 65535) return FE_ERR_TOO_LARGE;
  switch (bn) {
    case 16: return launch_bn<16>(mw, mx, p, grid, stream);
    case 32: return launch_bn<32>(mw, mx, p, grid, stream);
    case 64: return launch_bn<64>(mw, mx, p, grid, stream);
    case 128: return launch_bn<128>(mw, mx, p, grid, stream);
    default: return launch_bn<256>(mw, mx, p, grid, stream);
  }
}

// epilogue: 0 store bf16 [n, o]; 1 store f32 [n, o]; 2 add into f32 [n, o];
// 3 y[n, o/2] = silu(gate) * up (bf16) for w whose rows alternate 16 gate, 16 up features.
// ksplit > 1 needs ws_part (floats: feature tiles * token tiles * ksplit * tile * 128) and
// ws_count (one zeroed unsigned per output tile; left zeroed).
FE_EXPORT int fe_gemm_tc5(const void* x, const void* w, const float* bias, void* y, int n, int o, int k,
                          int epilogue, int ksplit, float* ws_part, unsigned* ws_count, int* status,
                          cudaStream_t stream) {
  if (epilogue < EPI_STORE_BF16 || epilogue > EPI_SILU_MUL_BF16) return FE_ERR_BAD_DTYPE;
  return run_gemm(x, w, bias, y, n, o, k, epilogue, ksplit, ws_part, ws_count, status, nullptr, stream);
}

// The fused q/k/v projection of up to 64 tokens with 128-wide heads: y [n, (nq + 2 nkv) * 128]
// receives the normalised, rotated queries; keys (normalised, rotated) and values go straight
// into their cache pages [pages, nkv, page_size, 128].  q_weight / k_weight may be null (no
// norm); table is the (cos, sin) table of fe_rope_table for these tokens, or null (no rotation).
FE_EXPORT int fe_gemm_tc5_qkv_rope(const void* x, const void* w, const float* bias, void* y, int n, int k, int ksplit,
                                   const float* q_weight, const float* k_weight, float eps, const void* table,
                                   const int* positions, const int* token_entry, void* k_cache, void* v_cache,
                                   const int* block_table, int max_pages, int page_size, int num_pages,
                                   int num_q_heads, int num_kv_heads, int write_kv, int* status,
                                   cudaStream_t stream) {
  if (n > 64 || num_q_heads < 1 || num_kv_heads < 1 || page_size < 1) return FE_ERR_BAD_SHAPE;
  static_assert(BM == 128, "a feature tile is one head of 128");
  const int o = (num_q_heads + 2 * num_kv_heads) * 128;
  const int ks = ksplit < 1 ? 1 : (ksplit > 8 ? 8 : ksplit);     // splits beyond a cluster would need the workspace
  QkvRope rope{q_weight, k_weight, eps, (const float2*)table, positions, token_entry, (bf16*)k_cache, (bf16*)v_cache,
               block_table, max_pages, page_size, num_pages, num_q_heads, num_kv_heads, write_kv};
  return run_gemm(x, w, bias, y, n, o, k, EPI_QKV_ROPE, ks, nullptr, nullptr, status, &rope, stream);
}

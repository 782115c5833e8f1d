// Several dependent projections of a decode step in ONE persistent kernel (bfloat16, up to
// 16 tokens): for instance  o-projection (+= residual)  ->  RMSNorm + gate/up with SiLU*mul
// ->  down-projection (+= residual).
//
// Why: at few tokens every projection is a stream of weights that takes 5-15 us; as kernels
// of their own each pays a launch, a first round trip to memory, a split-k reduction and a
// drain, during which nothing streams.  Upstream runs them as separate nn.Linear calls
// (src/forge_engine/qwen3.py:207, 225-227, 254-260).  Here one block per SM stays resident
// for the whole chain and its TMA producer warp walks straight through the weights of all
// projections - they depend on nothing - while the hand-over of activations between
// projections (a few KB through L2, announced by counters) happens beside the stream.
//
//   block (6 warps, one block per SM, `gridDim.x` = number of SMs):
//     warp 0     TMA producer: weight tiles [128 x 64] of all its units of all projections,
//                in order, through a ring of 7 stages
//     warp 1     allocates tensor memory; waits for a projection's input, fetches its token
//                tiles (TMA) where the input is bfloat16 activations, issues tcgen05.mma into
//                one of two accumulators
//     warps 2-5  (a) where the input is the RMS norm of the 32-bit residual stream: compute it
//                for all tokens and write the bfloat16 operand tiles into shared memory
//                (every block does this for itself: 16 x 2560 values from L2);
//                (b) epilogue: tcgen05.ld, then add into the residual (red.global.add.f32)
//                or SiLU(gate) * up -> bfloat16
//
// Units: a projection's weight is cut into tiles of 128 output features x 64-wide k-blocks.
// As many whole tiles as there are blocks go one to each block; the k-blocks of the tiles
// left over (all tiles, if there are fewer tiles than blocks) are dealt to the blocks in
// equal contiguous shares, so every block streams the same number of bytes.  A share of a
// tile is a partial sum: for "+= residual" it is simply added (32-bit atomic adds commute up
// to rounding); for SiLU*mul the shares are added into a staging tile and the block whose
// share completes the tile applies the activation.
//
// Hand-over: `op_done[j]` counts finished k-blocks of projection j (release after the stores,
// acquire by the pollers); projection j+1 starts when it reaches tiles x k-blocks.  All
// counters and the staging tiles are zero when the kernel starts and are left zero.
//
// Every wait (mbarrier, counter) is bounded; when a bound is hit the block sets
// FE_STATUS_WAIT_TIMEOUT, stops issuing work, frees its tensor memory and returns.  The
// blocks wait for one another, so all of them must be resident at once: the launcher uses
// one block per SM and never more blocks than SMs.
#include "tcgen05.cuh"

namespace {

using namespace tc5;

constexpr int CH_THREADS = 320;              // producer, MMA, 4 epilogue warps, 4 more for norm operands
constexpr int CH_BN = 16;                       // token tile
constexpr int CH_STAGES = 7;
constexpr int CH_A_BYTES = BM * BK * 2;         // 16 KB weight tile
constexpr int CH_B_TILE = CH_BN * BK * 2;       // 2 KB token tile of one k-block
constexpr int CH_B_TILES = 44;                  // token tiles a block keeps for one projection
constexpr int CH_NORM_PIECES = CH_B_TILES * 8 / 32;   // 16-byte pieces of a normalised row per lane
constexpr int CH_MAX_OPS = 3;
constexpr int CH_MAX_LEFT = 160;                // leftover tiles of one projection (fewer than blocks)
constexpr int CH_COUNTERS = 8 + CH_MAX_OPS * CH_MAX_LEFT;
constexpr size_t CH_SMEM = (size_t)CH_STAGES * CH_A_BYTES + (size_t)CH_B_TILES * CH_B_TILE + (size_t)CH_B_TILES * BK * 4 + 256 + 1024;

enum { SRC_TMA = 0, SRC_NORM = 1 };
enum { EPI_ADD = 0, EPI_SILU = 1 };

struct ChainOp {
  int m, k;              // output features, reduction length
  int src;               // SRC_TMA: bfloat16 activations [n, k] (tensor map); SRC_NORM: RMS norm of resid
  int epi;               // EPI_ADD: out float [n, m] += ; EPI_SILU: out bf16 [n, m / 2]
  void* out;
  const float* resid;    // SRC_NORM: float [n, k]
  const float* norm_w;   // SRC_NORM: [k]
  float eps;
};

struct ChainParams {
  ChainOp op[CH_MAX_OPS];
  int n_ops, n;
  unsigned* counters;    // [CH_COUNTERS]: op_done[0..2], exit at [3], tile counters from [8]
  float* staging;        // [CH_MAX_LEFT][16][128], zero at entry and exit
  int* status;
  unsigned wait_limit;
  unsigned long long* trace;   // optional [blocks][16] nanosecond stamps (see fe_decode_chain_trace)
};

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define CH_STAMP(slot) do { if (p.trace) p.trace[(size_t)me * 16 + (slot)] = now_ns(); } while (0)

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_add_f32(float* p, float v) {
  asm volatile("red.relaxed.gpu.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
// Bounded wait for a counter to reach `target`.
__device__ __forceinline__ bool wait_counter(const unsigned* counter, unsigned target, volatile int* abort_flag,
                                             unsigned limit) {
  for (unsigned i = 0; i < limit; ++i) {
    if (ld_acquire(counter) >= target) return true;
    if ((i & 63u) == 63u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

__device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Unit `idx` of block `c` (of `blocks`) in a projection of `tiles` x `kblocks`: first the
// block's share of the left-over tiles (one or two pieces), then its whole tiles.  Shares come
// first so that a left-over tile is complete - and finished by the block that completes it -
// early in the projection, not at its end.
__device__ __forceinline__ bool unit_of(int tiles, int kblocks, int blocks, int c, int idx, int& tile, int& kb0,
                                        int& kbn) {
  const int full = tiles / blocks;
  const int left = tiles - full * blocks;
  int shares = 0;
  if (left > 0) {
    const long long all = (long long)left * kblocks;
    const long long lo = all * c / blocks, hi = all * (c + 1) / blocks;
    if (lo < hi) {
      const int t0 = (int)(lo / kblocks);
      const long long first_end = hi < (long long)(t0 + 1) * kblocks ? hi : (long long)(t0 + 1) * kblocks;
      shares = first_end < hi ? 2 : 1;
      if (idx == 0) {
        tile = full * blocks + t0;
        kb0 = (int)(lo - (long long)t0 * kblocks);
        kbn = (int)(first_end - lo);
        return true;
      }
      if (idx == 1 && shares == 2) {
        tile = full * blocks + t0 + 1;
        kb0 = 0;
        kbn = (int)(hi - first_end);
        return true;
      }
    }
  }
  if (idx - shares < full) {
    tile = (idx - shares) * blocks + c;
    kb0 = 0;
    kbn = kblocks;
    return true;
  }
  return false;
}

__device__ __forceinline__ const CUtensorMap* pick(int j, const CUtensorMap* a, const CUtensorMap* b,
                                                   const CUtensorMap* c) {
  return j == 0 ? a : (j == 1 ? b : c);
}

// Walks a block's weight tiles of all projections in the order they are used.
struct TileCursor {
  int j, idx, kb, tile, kb0, kbn;
  bool valid;
};
__device__ __forceinline__ void cursor_seek(TileCursor& c, const ChainParams& p, int blocks, int me) {
  // from (j, idx) on: the first unit that exists
  while (c.j < p.n_ops) {
    if (unit_of(ceil_div(p.op[c.j].m, BM), ceil_div(p.op[c.j].k, BK), blocks, me, c.idx, c.tile, c.kb0, c.kbn)) {
      c.kb = c.kb0;
      c.valid = true;
      return;
    }
    ++c.j;
    c.idx = 0;
  }
  c.valid = false;
}
__device__ __forceinline__ void cursor_step(TileCursor& c, const ChainParams& p, int blocks, int me) {
  if (++c.kb < c.kb0 + c.kbn) return;
  ++c.idx;
  cursor_seek(c, p, blocks, me);
}

__device__ __forceinline__ void red_release_u32(unsigned* p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned atom_add_acq_rel_u32(unsigned* p, unsigned v) {
  unsigned old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}

__global__ void __launch_bounds__(CH_THREADS, 1)
decode_chain_kernel(const __grid_constant__ CUtensorMap mw0, const __grid_constant__ CUtensorMap mw1,
                    const __grid_constant__ CUtensorMap mw2, const __grid_constant__ CUtensorMap mb0,
                    const __grid_constant__ CUtensorMap mb1, const __grid_constant__ CUtensorMap mb2, ChainParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* a_tiles = smem;
  unsigned char* b_tiles = smem + CH_STAGES * CH_A_BYTES;
  float* norm_w_s = reinterpret_cast<float*>(b_tiles + CH_B_TILES * CH_B_TILE);     // [CH_B_TILES * 64]
  uint64_t* full = reinterpret_cast<uint64_t*>(norm_w_s + CH_B_TILES * BK);
  uint64_t* empty = full + CH_STAGES;
  uint64_t* acc_full = empty + CH_STAGES;      // [2]
  uint64_t* acc_empty = acc_full + 2;          // [2]
  uint64_t* b_ready = acc_empty + 2;           // [1]
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(b_ready + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* agree = abort_flag + 1;        // [2] what the epilogue warps agreed on, alternating
  volatile int* last_flag = agree + 2;
  volatile int* prep_go = last_flag + 1;       // whether the warps that prepare a norm operand go on

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int blocks = gridDim.x, me = blockIdx.x;
  unsigned* op_done = p.counters;
  unsigned* exit_count = p.counters + 3;
  unsigned* tile_count = p.counters + 8;
  const unsigned poll_limit = p.wait_limit >> 4 ? p.wait_limit >> 4 : 1u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < CH_STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(acc_full + a, 1); mbar_init(acc_empty + a, 1); }
    mbar_init(b_ready, 1);
    *abort_flag = 0;
    agree[0] = agree[1] = 1;
    *last_flag = 0;
    *prep_go = 1;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(32)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (warp >= 2) {
    // rows of tokens that do not exist stay zero in every token tile
    uint4* b16 = reinterpret_cast<uint4*>(b_tiles);
    for (int i = threadIdx.x - 64; i < CH_B_TILES * CH_B_TILE / 16; i += CH_THREADS - 64) b16[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_slot;
  pdl_trigger();
  if (threadIdx.x == 0) CH_STAMP(0);

  if (warp == 0) {
    // ---------------- producer: the weights of every unit of every projection, in order.
    // (Asking for tiles beyond the ring to be brought into L2 - cp.async.bulk.prefetch.tensor,
    // 16 tiles ahead - kept memory busy while the products waited for a hand-over, but slowed
    // the stream itself, gate/up from 14.6 to 19.2 us, and read 20 % more from DRAM: taken out.)
    if (lane == 0) {
      TileCursor load = {0, 0, 0, 0, 0, 0, false};
      cursor_seek(load, p, blocks, me);
      unsigned it = 0;
      int last_j = 0;
      while (load.valid) {
        const int s = it % CH_STAGES;
        if (it >= CH_STAGES && !mbar_wait(empty + s, ((it / CH_STAGES) - 1) & 1, abort_flag, p.wait_limit)) break;
        if (load.j != last_j) {
          CH_STAMP(1 + 5 * last_j + 4);     // the last weight tile of projection last_j is on its way
          last_j = load.j;
        }
        mbar_expect_tx(full + s, CH_A_BYTES);
        tma_load_2d(a_tiles + s * CH_A_BYTES, pick(load.j, &mw0, &mw1, &mw2), load.kb * BK, load.tile * BM, full + s);
        cursor_step(load, p, blocks, me);
        ++it;
      }
      CH_STAMP(1 + 5 * last_j + 4);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (and fetcher of bfloat16 token tiles)
    if (lane == 0) {
      const unsigned idesc = umma_idesc(CH_BN);
      unsigned it = 0, units_done = 0, b_phase = 0;
      bool ok = true;
      for (int j = 0; j < p.n_ops && ok; ++j) {
        const ChainOp& op = p.op[j];
        const int tiles = ceil_div(op.m, BM), kblocks = ceil_div(op.k, BK);
        int tile, kb0, kbn;
        if (!unit_of(tiles, kblocks, blocks, me, 0, tile, kb0, kbn)) continue;     // nothing of this projection is mine
        if (op.src == SRC_TMA) {
          if (j == 0) pdl_wait();
          else ok = wait_counter(op_done + j - 1, (unsigned)ceil_div(p.op[j - 1].m, BM) * (unsigned)ceil_div(p.op[j - 1].k, BK),
                                 abort_flag, poll_limit);
          if (!ok) break;
          CH_STAMP(1 + 5 * j + 0);                             // input of projection j is complete
          asm volatile("fence.proxy.async;" ::: "memory");     // others' stores, seen above, before the TMA reads them
          const CUtensorMap* mb = pick(j, &mb0, &mb1, &mb2);
          int mine = 0;
          for (int idx = 0; unit_of(tiles, kblocks, blocks, me, idx, tile, kb0, kbn); ++idx) mine += kbn;
          mbar_expect_tx(b_ready, (unsigned)mine * CH_B_TILE);
          int base = 0;
          for (int idx = 0; unit_of(tiles, kblocks, blocks, me, idx, tile, kb0, kbn); ++idx) {
            for (int kb = kb0; kb < kb0 + kbn; ++kb)
              tma_load_2d(b_tiles + (base + kb - kb0) * CH_B_TILE, mb, kb * BK, 0, b_ready);
            base += kbn;
          }
        }
        if (!mbar_wait(b_ready, b_phase, abort_flag, p.wait_limit)) break;
        b_phase ^= 1u;
        CH_STAMP(1 + 5 * j + 1);                               // token tiles in shared memory
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        int base = 0;
        for (int idx = 0; ok && unit_of(tiles, kblocks, blocks, me, idx, tile, kb0, kbn); ++idx) {
          const unsigned acc = units_done & 1u;
          if (units_done >= 2 && !mbar_wait(acc_empty + acc, ((units_done >> 1) - 1) & 1, abort_flag, p.wait_limit)) {
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          for (int kb = kb0; kb < kb0 + kbn; ++kb, ++it) {
            const int s = it % CH_STAGES;
            if (!mbar_wait(full + s, (it / CH_STAGES) & 1, abort_flag, p.wait_limit)) {
              ok = false;
              break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int b_index = op.src == SRC_NORM ? kb : base + kb - kb0;
            const uint64_t da = umma_desc(a_tiles + s * CH_A_BYTES);
            const uint64_t db = umma_desc(b_tiles + b_index * CH_B_TILE);
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk)
              umma_f16(tmem_base + acc * CH_BN, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc,
                       (kb > kb0 || kk > 0) ? 1u : 0u);
            umma_commit(empty + s);
          }
          if (!ok) break;
          umma_commit(acc_full + acc);
          ++units_done;
          base += kbn;
        }
        CH_STAMP(1 + 5 * j + 2);                               // last product of projection j issued
      }
    }
  } else {
    // ---------------- warps 2-5: every epilogue; warps 2-9: the operand of a norm projection
    const int te = threadIdx.x - 64;           // 0..255; the epilogue warps are 0..127
    const int we = te >> 5;                    // 0..7
    const bool helper = warp >= 6;             // takes part in norm operands only
    const int quarter = warp & 3;              // tensor-memory lanes 32 * quarter ..
    unsigned units_done = 0, round = 0;
    bool dead = false;                         // a wait ran out: only keep the other warps from hanging
    // One thread looks at the abort flag, all take what it saw: the warps never part ways.
    auto all_agree = [&]() -> bool {
      if (te == 0) agree[round & 1u] = *abort_flag == 0;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const bool go = agree[round & 1u] != 0;
      ++round;
      return go;
    };
    // the norm weights of the first projection that needs them: fetched while the weights stream
    auto preload_norm_weights = [&](int from) {
      for (int j = from; j < p.n_ops; ++j) {
        if (p.op[j].src != SRC_NORM) continue;
        for (int i = te - 128; i < p.op[j].k; i += 128) norm_w_s[i] = __ldg(p.op[j].norm_w + i);
        return;
      }
    };
    if (helper) preload_norm_weights(0);
    pdl_wait();     // orders this thread's accesses after the kernels before this one
    for (int j = 0; j < p.n_ops; ++j) {
      const ChainOp& op = p.op[j];
      const int tiles = ceil_div(op.m, BM), kblocks = ceil_div(op.k, BK);
      const int full_rounds = tiles / blocks;
      int tile, kb0, kbn;
      if (!unit_of(tiles, kblocks, blocks, me, 0, tile, kb0, kbn)) continue;
      if (op.src == SRC_NORM) {
        if (te == 0) {
          if (!dead && j > 0)
            wait_counter(op_done + j - 1, (unsigned)ceil_div(p.op[j - 1].m, BM) * (unsigned)ceil_div(p.op[j - 1].k, BK),
                         abort_flag, poll_limit);
          *prep_go = (!dead && *abort_flag == 0) ? 1 : 0;
          CH_STAMP(1 + 5 * j + 0);                             // input of projection j is complete
        }
        asm volatile("bar.sync 2, 256;" ::: "memory");
        if (*prep_go == 0) break;                              // every warp of this group leaves together
        // x * rsqrt(mean(x^2) + eps) * w in 32-bit, rounded once (as fe_add_rmsnorm does).  A warp
        // takes a token; a lane takes every 32nd group of 8 neighbouring values (one 16-byte
        // piece of a tile row) and asks for all of its groups at once - the row comes from L2,
        // and only many loads in flight hide that latency - then keeps them in registers
        // between the sum of squares and the scaling.
        const int k = op.k;
        const int pieces = k >> 3;                        // k is a multiple of 8
        const float4* w = reinterpret_cast<const float4*>(norm_w_s);
        for (int row = we; row < p.n; row += 8) {
          const float4* x = reinterpret_cast<const float4*>(op.resid + (size_t)row * k);
          float4 xa[CH_NORM_PIECES], xb[CH_NORM_PIECES];
#pragma unroll
          for (int i = 0; i < CH_NORM_PIECES; ++i) {
            const int c = lane + 32 * i;
            xa[i] = xb[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < pieces) {
              xa[i] = __ldcg(x + 2 * c);
              xb[i] = __ldcg(x + 2 * c + 1);
            }
          }
          float ss = 0.f;
#pragma unroll
          for (int i = 0; i < CH_NORM_PIECES; ++i)
            ss += (xa[i].x * xa[i].x + xa[i].y * xa[i].y + xa[i].z * xa[i].z + xa[i].w * xa[i].w) +
                  (xb[i].x * xb[i].x + xb[i].y * xb[i].y + xb[i].z * xb[i].z + xb[i].w * xb[i].w);
          ss = warp_sum(ss);
          const float inv = rsqrtf(ss / (float)k + op.eps);
#pragma unroll
          for (int i = 0; i < CH_NORM_PIECES; ++i) {
            const int c = lane + 32 * i;
            if (c >= kblocks * 8) continue;
            uint4 packed = make_uint4(0u, 0u, 0u, 0u);     // beyond k: zeros
            if (c < pieces) {
              const float4 wa = w[2 * c], wb = w[2 * c + 1];
              const __nv_bfloat162 h0 = __floats2bfloat162_rn(xa[i].x * inv * wa.x, xa[i].y * inv * wa.y);
              const __nv_bfloat162 h1 = __floats2bfloat162_rn(xa[i].z * inv * wa.z, xa[i].w * inv * wa.w);
              const __nv_bfloat162 h2 = __floats2bfloat162_rn(xb[i].x * inv * wb.x, xb[i].y * inv * wb.y);
              const __nv_bfloat162 h3 = __floats2bfloat162_rn(xb[i].z * inv * wb.z, xb[i].w * inv * wb.w);
              packed.x = *reinterpret_cast<const unsigned*>(&h0);
              packed.y = *reinterpret_cast<const unsigned*>(&h1);
              packed.z = *reinterpret_cast<const unsigned*>(&h2);
              packed.w = *reinterpret_cast<const unsigned*>(&h3);
            }
            // 128-byte swizzle: 16-byte piece (c & 7) of row `row` sits at piece (c & 7) ^ (row & 7)
            unsigned char* at = b_tiles + (c >> 3) * CH_B_TILE + (row >> 3) * 1024 + (row & 7) * 128 +
                                (((c & 7) ^ (row & 7)) << 4);
            *reinterpret_cast<uint4*>(at) = packed;
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("bar.sync 2, 256;" ::: "memory");
        if (te == 0) mbar_arrive(b_ready);
        if (helper) preload_norm_weights(j + 1);
      }
      if (helper || dead) continue;
      for (int idx = 0; unit_of(tiles, kblocks, blocks, me, idx, tile, kb0, kbn); ++idx) {
        const unsigned acc = units_done & 1u;
        mbar_wait(acc_full + acc, (units_done >> 1) & 1, abort_flag, p.wait_limit);
        if (!all_agree()) { dead = true; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        float v[16];
        tmem_ld16(tmem_base + ((unsigned)(quarter * 32) << 16) + acc * CH_BN, v);
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (te == 0) mbar_arrive(acc_empty + acc);
        ++units_done;
        const int row = quarter * 32 + lane;
        const int feature = tile * BM + row;
        if (op.epi == EPI_ADD) {
          float* y = reinterpret_cast<float*>(op.out);
          if (feature < op.m) {
#pragma unroll
            for (int t = 0; t < 16; ++t)
              if (t < p.n) red_add_f32(y + (size_t)t * op.m + feature, v[t]);
          }
          // the barrier orders the warps' adds before thread 0, whose release publishes them
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (te == 0) red_release_u32(op_done + j, (unsigned)kbn);
          continue;
        }
        // EPI_SILU: weight rows alternate 16 gate and 16 up features; lanes 0-15 hold gate,
        // lanes 16-31 the matching up values
        const bool whole = kbn == kblocks;
        bool finish = whole;
        float* stage = p.staging + (size_t)(tile - full_rounds * blocks) * (16 * BM);
        if (!whole) {
#pragma unroll
          for (int t = 0; t < 16; ++t)
            if (t < p.n) red_add_f32(stage + t * BM + row, v[t]);
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (te == 0) {
            const unsigned before = atom_add_acq_rel_u32(tile_count + j * CH_MAX_LEFT + (tile - full_rounds * blocks), (unsigned)kbn);
            *last_flag = before + (unsigned)kbn == (unsigned)kblocks;
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          finish = *last_flag != 0;
          if (finish) {
#pragma unroll
            for (int t = 0; t < 16; ++t) {
              v[t] = 0.f;
              if (t < p.n) {
                v[t] = __ldcg(stage + t * BM + row);
                stage[t * BM + row] = 0.f;
              }
            }
          }
        }
        if (finish) {
          const int half_m = op.m >> 1;
          const int out_feature = (feature >> 5) * 16 + (lane & 15);
          bf16* y = reinterpret_cast<bf16*>(op.out);
#pragma unroll
          for (int t = 0; t < 16; t += 2) {
            const float send = lane < 16 ? v[t + 1] : v[t];
            const float recv = __shfl_xor_sync(0xffffffffu, send, 16);
            const int token = t + (lane < 16 ? 0 : 1);
            const float r = lane < 16 ? silu_f(v[t]) * recv : silu_f(recv) * v[t + 1];
            if (token < p.n && out_feature < half_m) y[(size_t)token * half_m + out_feature] = __float2bfloat16_rn(r);
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (te == 0) {
            if (!whole) tile_count[j * CH_MAX_LEFT + (tile - full_rounds * blocks)] = 0u;
            red_release_u32(op_done + j, (unsigned)kblocks);
          }
        }
      }
      if (te == 0) CH_STAMP(1 + 5 * j + 3);                    // this block's share of projection j is published
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(32) : "memory");
  }
  if (threadIdx.x == 0) {
    if (*abort_flag && p.status) atomicOr(p.status, FE_STATUS_WAIT_TIMEOUT);
    __threadfence();
    // the block that leaves last puts the counters back to zero for the next launch
    if (atomicAdd(exit_count, 1u) == (unsigned)blocks - 1u) {
      for (int i = 0; i < CH_COUNTERS; ++i) p.counters[i] = 0u;
    }
  }
}

unsigned long long* g_chain_trace = nullptr;

int sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
      sms = 0;
  }
  return sms;
}

}  // namespace

// What the caller must provide beside the tensors: `counters` (unsigned[fe_decode_chain_counters()],
// zeroed once; every launch leaves them zero) and `staging` (float[fe_decode_chain_staging()],
// likewise).
FE_EXPORT int fe_decode_chain_counters() { return CH_COUNTERS; }
FE_EXPORT int fe_decode_chain_staging() { return CH_MAX_LEFT * 16 * BM; }

// Timeline for profiling: with a buffer of fe_decode_chain_blocks() x 16 64-bit words, later
// launches write nanosecond stamps (%globaltimer) per block: [0] start; for projection j at
// [1 + 5 j ..]: input complete, token tiles in shared memory, last product issued, share
// published, last weight tile requested.  nullptr switches it off.
FE_EXPORT void fe_decode_chain_trace(unsigned long long* buffer) { g_chain_trace = buffer; }
FE_EXPORT int fe_decode_chain_blocks() { return sm_count(); }

// One projection of the chain, as the caller describes it.
struct FeChainOp {
  const void* w;          // bfloat16 [m, k]
  const void* x;          // src 0: bfloat16 [n, k] activations; src 1: float [n, k] residual stream
  const float* norm_w;    // src 1: float [k]
  void* out;              // epi 0: float [n, m], added to; epi 1: bfloat16 [n, m / 2]
  int m, k, src, epi;
  float eps;
};

// Whether the chain kernel takes these projections (sizes only); 0 = yes, else an FE_ERR code.
FE_EXPORT int fe_decode_chain_check(const FeChainOp* ops, int n_ops, int n) {
  const int blocks = sm_count();
  if (blocks < 1 || blocks > CH_MAX_LEFT) return FE_ERR_BAD_SHAPE;
  if (n_ops < 1 || n_ops > CH_MAX_OPS || n < 1 || n > CH_BN) return FE_ERR_BAD_SHAPE;
  for (int j = 0; j < n_ops; ++j) {
    const FeChainOp& op = ops[j];
    if (op.m < 1 || op.k < 8 || (op.k % 8) != 0) return FE_ERR_BAD_SHAPE;
    const int tiles = (op.m + BM - 1) / BM, kblocks = (op.k + BK - 1) / BK;
    if (op.src == SRC_NORM) {
      if (kblocks > CH_B_TILES) return FE_ERR_BAD_SHAPE;
    } else if (op.src == SRC_TMA) {
      const long long left = tiles % blocks;
      const long long share = (left * kblocks + blocks - 1) / blocks;
      if ((long long)(tiles / blocks) * kblocks + share > CH_B_TILES) return FE_ERR_BAD_SHAPE;
    } else {
      return FE_ERR_BAD_SHAPE;
    }
    if (op.epi == EPI_SILU) {
      if ((op.m % 32) != 0) return FE_ERR_BAD_SHAPE;
    } else if (op.epi != EPI_ADD) {
      return FE_ERR_BAD_SHAPE;
    }
  }
  return 0;
}

FE_EXPORT int fe_decode_chain(const FeChainOp* ops, int n_ops, int n, unsigned* counters, float* staging, int* status,
                              cudaStream_t stream) {
  int rc = fe_decode_chain_check(ops, n_ops, n);
  if (rc) return rc;
  if (counters == nullptr || staging == nullptr) return FE_ERR_BAD_SHAPE;
  CUtensorMap mw[CH_MAX_OPS], mb[CH_MAX_OPS];
  ChainParams p = {};
  p.n_ops = n_ops;
  p.n = n;
  p.counters = counters;
  p.staging = staging;
  p.status = status;
  p.wait_limit = WAIT_LIMIT;
  p.trace = g_chain_trace;
  for (int j = 0; j < CH_MAX_OPS; ++j) {
    const FeChainOp& op = ops[j < n_ops ? j : 0];
    if ((((uintptr_t)op.w) | ((uintptr_t)op.x) | ((uintptr_t)op.out)) & 15) return FE_ERR_BAD_ALIGN;
    rc = make_map(&mw[j], op.w, op.m, op.k, BM);
    if (rc) return rc;
    if (op.src == SRC_TMA) {
      rc = make_map(&mb[j], op.x, n, op.k, CH_BN);
      if (rc) return rc;
    } else {
      if (op.norm_w == nullptr || (((uintptr_t)op.norm_w) & 15)) return FE_ERR_BAD_ALIGN;
      mb[j] = mw[j];    // not used
    }
    if (j < n_ops) {
      ChainOp& d = p.op[j];
      d.m = op.m; d.k = op.k; d.src = op.src; d.epi = op.epi;
      d.out = op.out;
      d.resid = op.src == SRC_NORM ? reinterpret_cast<const float*>(op.x) : nullptr;
      d.norm_w = op.norm_w;
      d.eps = op.eps;
    }
  }
  static bool configured = false;
  if (!configured) {
    const cudaError_t e = cudaFuncSetAttribute(decode_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CH_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  rc = fe_launch_dependent(decode_chain_kernel, dim3(sm_count()), dim3(CH_THREADS), CH_SMEM, stream, mw[0], mw[1], mw[2],
                           mb[0], mb[1], mb[2], p);
  if (rc) return rc;
  return fe_last_error();
}

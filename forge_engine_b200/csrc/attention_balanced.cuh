// Decode attention with the step's key tiles spread evenly over a fixed number of blocks
// (included by attention_mma.cu; same tile code, same TMA staging as attn_decode_tma_kernel).
//
// The decode entries' (entry, kv head) pairs, one after the other, form one line.  A pair
// takes as many units of the line as it has 64-key tiles, and BAL_PAIR_UNITS more before
// them for what a block spends on a pair beside its tiles (query rows, combining the four
// warps, writing out), so that many short requests weigh what they cost.  Block c of G takes
// units [c U / G, (c + 1) U / G): it walks through the pairs that its stretch touches, and
// its producer warp keeps the ring of stages full across the borders between them, so that
// a block loads without a pause from its first tile to its last and all blocks finish at
// about the same time whatever the requests' lengths are.  A pair whose tiles lie inside one
// block is finished there.  A pair that a block's border cuts leaves unnormalised
// (max, sum, acc) of its pieces in a workspace, at most two per block (slot 2c: the first
// piece the block works on, slot 2c + 1: a later one, which is then its last), and
// attn_merge_balanced_kernel combines them in block order.  Every block works the same cut
// out from the entries' lengths, so no plan is made on the host and a replayed CUDA graph
// follows the lengths of the step it runs for.
//
// Upstream walks one request's pages in one block (src/forge_engine/kernels/cuda_paged.py:276-347).

constexpr int BAL_MAX_ENTRIES = 256;    // the entries' tile counts, first tokens and lengths live in shared memory
constexpr int BAL_MAX_BLOCKS = 304;     // pieces a pair can have = blocks of the grid

// 64-key tiles that entry `entry` needs, and its first tile; 0 for entries of the other kernels.
__device__ __forceinline__ int bal_entry_tiles(const AttnParams& p, int entry, int* tile_first) {
  const int tok0 = p.cu_tokens[entry];
  const int n_new = p.cu_tokens[entry + 1] - tok0;
  const int rows_total = n_new * p.groups;
  *tile_first = 0;
  if (rows_total <= p.row_lo || rows_total > p.row_hi) return 0;
  const int start = p.starts[entry];
  const int key_lo = p.window > 0 ? max(0, start - p.window + 1) : 0;
  const int key_end = start + n_new;
  *tile_first = key_lo / BN;
  return (key_end + BN - 1) / BN - *tile_first;
}

// What a pair costs beside its tiles, in tiles.  Measured with 1 / 2 / 3: 64 requests of 16 to
// 4,096 keys 101 / 95 / 96 us, 24 requests of 3,000 keys beside 8 of one key 72 / 59 / 60 us,
// 64 requests of 2,048 keys 93 / 94 / 95 us.
constexpr int BAL_PAIR_UNITS = 2;

// Units of the line that one (entry, kv head) pair with `tiles` tiles takes.
__device__ __forceinline__ int bal_pair_units(int tiles) { return tiles > 0 ? tiles + BAL_PAIR_UNITS : 0; }

// Where the line is cut: block c begins at unit floor(c U / G).
__device__ __forceinline__ long long bal_begin(long long c, long long total, int blocks) { return c * total / blocks; }
// The block that unit u belongs to.
__device__ __forceinline__ int bal_block_of(long long u, long long total, int blocks) {
  return (int)(((u + 1) * blocks - 1) / total);
}

// The entries' numbers that every segment needs, copied to shared memory once per block.
struct BalEntries {
  int* prefix;     // [entries + 1] units of one kv head of the entries before e
  int* cu;         // [entries + 1] first token of e
  int* start;      // [entries] tokens cached before this step
};

// One stretch of a block's walk: tiles [tile_begin, tile_begin + count) of (entry, kvh).
struct BalSegment {
  int entry, kvh, tile_begin, count;   // count 0: the walk is over
  int tok0, n_new, start;
  long long next;  // the unit behind the segment
  bool whole;      // the pair's every tile: the result is final
};

// The first segment with tiles at or behind unit `tau` and before `end`.  An entry's pairs
// lie together, kv head by kv head; a pair's first BAL_PAIR_UNITS units carry no tile.
__device__ __forceinline__ BalSegment bal_locate(const AttnParams& p, const BalEntries& in, int entries, long long tau,
                                                 long long end) {
  BalSegment s;
  s.count = 0;
  s.next = end;
  while (tau < end) {
    int lo = 0, hi = entries - 1;           // the last entry with nkv * prefix[e] <= tau: it has tiles
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if ((long long)p.nkv * in.prefix[mid] <= tau) lo = mid; else hi = mid - 1;
    }
    const int u_e = in.prefix[lo + 1] - in.prefix[lo];
    const int t_e = u_e - BAL_PAIR_UNITS;
    const long long r = tau - (long long)p.nkv * in.prefix[lo];
    const int kvh = (int)(r / u_e);
    const int local = (int)(r - (long long)kvh * u_e);                    // unit inside the pair
    const int stop = (int)min((long long)u_e, local + (end - tau));       // the stretch ends here inside the pair
    const int first = max(0, local - BAL_PAIR_UNITS);
    const int count = stop - BAL_PAIR_UNITS - first;
    tau += stop - local;
    if (count <= 0) continue;               // the stretch ends before the pair's first tile
    s.entry = lo;
    s.kvh = kvh;
    s.count = count;
    s.next = tau;
    s.whole = first == 0 && count == t_e;
    s.tok0 = in.cu[lo];
    s.n_new = in.cu[lo + 1] - s.tok0;
    s.start = in.start[lo];
    const int key_lo = p.window > 0 ? max(0, s.start - p.window + 1) : 0;
    s.tile_begin = key_lo / BN + first;
    return s;
  }
  return s;
}

// Fill `in`: exclusive prefix sums of the units of one kv head of every entry, their first tokens and their
// lengths (all threads of the block call it; the first warp scans).
__device__ __forceinline__ void bal_prefix(const AttnParams& p, int entries, const BalEntries& in, int tid, int nthreads) {
  for (int e = tid; e < entries; e += nthreads) {
    int unused;
    in.prefix[e + 1] = bal_pair_units(bal_entry_tiles(p, e, &unused));
    in.cu[e] = p.cu_tokens[e];
    in.start[e] = p.starts[e];
  }
  if (tid == 0) { in.prefix[0] = 0; in.cu[entries] = p.cu_tokens[entries]; }
  __syncthreads();
  if (tid < 32) {
    int carry = 0;
    for (int base = 0; base < entries; base += 32) {
      const int e = base + tid;
      int v = e < entries ? in.prefix[e + 1] : 0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, v, d);
        if (tid >= d) v += up;
      }
      if (e < entries) in.prefix[e + 1] = carry + v;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(TMA_THREADS, D <= 128 ? 2 : 1)
attn_decode_balanced_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            AttnParams p, int entries) {
  extern __shared__ unsigned char smem_raw[];
  constexpr int TILE_BYTES = BN * D * 2;    // one matrix of one stage
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  bf16* kbuf = reinterpret_cast<bf16*>(smem);                                   // [TMA_STAGES] tiles of 64 keys
  bf16* vbuf = reinterpret_cast<bf16*>(smem + TMA_STAGES * TILE_BYTES);
  bf16* qs = reinterpret_cast<bf16*>(smem + 2 * TMA_STAGES * TILE_BYTES);         // [2][16][LD]: this segment's rows and the next one's
  uint64_t* full = reinterpret_cast<uint64_t*>(qs + 2 * DEC_ROWS * LD);
  uint64_t* empty = full + TMA_STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + TMA_STAGES);
  float* ml_s = reinterpret_cast<float*>(const_cast<int*>(abort_flag) + 4);       // [4][16][2]
  BalEntries in;
  in.prefix = reinterpret_cast<int*>(ml_s + 4 * DEC_ROWS * 2);
  in.cu = in.prefix + BAL_MAX_ENTRIES + 1;
  in.start = in.cu + BAL_MAX_ENTRIES + 1;

  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    tma_prefetch_map(&map_k);
    tma_prefetch_map(&map_v);
    for (int s = 0; s < TMA_STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  // the entries' lengths are the step's inputs, not the work of the kernel before this one
  bal_prefix(p, entries, in, tid, TMA_THREADS);
  const long long total = (long long)p.nkv * in.prefix[entries];
  // with fewer units than blocks the first `total` blocks take one unit each: no block in
  // the middle of a pair may be without a piece, the merge counts on one from each
  const int blocks = (int)min((long long)gridDim.x, total);
  const bool idle = (int)blockIdx.x >= blocks;
  const long long begin = idle ? 0 : bal_begin(blockIdx.x, total, blocks);
  const long long end = idle ? 0 : bal_begin(blockIdx.x + 1, total, blocks);
  const int num_q_heads = p.nkv * p.groups;

  if (warp == 4) {
    // ---- producer: one walk over the block's stretch, the ring never drains at a border ----
    const int pages_per_tile = BN / p.page_size;
    const int rows_in_cache = p.num_pages * p.nkv * p.page_size;
    bool waited = false, dead = false;
    int it = 0;                             // tiles issued so far: ring position
    for (long long tau = begin; tau < end && !dead;) {
      const BalSegment seg = bal_locate(p, in, entries, tau, end);
      if (seg.count == 0) break;
      const int* table = p.block_table + (size_t)seg.entry * p.max_pages;
      const int start = seg.start;
      const int key_lo = p.window > 0 ? max(0, start - p.window + 1) : 0;
      const int key_end = start + seg.n_new;
      const int first_logical = seg.tile_begin * pages_per_tile;
      const int total_pages = seg.count * pages_per_tile;
      for (int base = 0; base < total_pages; base += 32) {
        const int logical = first_logical + base + lane;
        const int key = logical * p.page_size;
        int my_row = rows_in_cache;          // outside the tensor: the copy fills zeros
        if (base + lane < total_pages && key < key_end) {
          const int page = logical < p.max_pages ? table[logical] : -1;
          if (page >= 0 && page < p.num_pages) my_row = (page * p.nkv + seg.kvh) * p.page_size;
          else if (key + p.page_size > key_lo) atomicOr(p.status, FE_STATUS_BAD_PAGE);
        }
        const int count = min(32, total_pages - base);
        for (int j = 0; j < count; ++j) {
          const int row = __shfl_sync(0xffffffffu, my_row, j);
          if (lane == 0 && !dead) {
            const int index = base + j;
            const int i = index / pages_per_tile, pg = index - i * pages_per_tile;
            const int n = it + i;
            const int s = n % TMA_STAGES;
            if (pg == 0) {
              const int key0 = (seg.tile_begin + i) * BN;
              // keys of this step are written by the kernel before this one
              if (!waited && (key0 + BN > start || n >= TMA_STAGES)) { pdl_wait(); waited = true; }
              if (n >= TMA_STAGES && !mbar_wait(empty + s, ((n / TMA_STAGES) & 1) ^ 1, abort_flag)) dead = true;
              if (!dead) mbar_expect_tx(full + s, 2 * TILE_BYTES);
            }
            if (!dead) {
              const int offset = pg * p.page_size * D;
              tma_load_2d(kbuf + s * (BN * D) + offset, &map_k, 0, row * (D / 64), full + s);
              tma_load_2d(vbuf + s * (BN * D) + offset, &map_v, 0, row * (D / 64), full + s);
            }
          }
        }
      }
      dead = __shfl_sync(0xffffffffu, dead ? 1 : 0, 0) != 0;
      it += seg.count;
      tau = seg.next;
    }
    if (lane == 0 && !waited) pdl_wait();
  } else {
    // ---- consumers: warp w takes keys [16 w, 16 w + 16) of every tile ----
    pdl_wait();
    const int ra = lane >> 2, rb = ra + 8;
    int it = 0, buf = 0;
    bool alive = true;
    BalSegment seg = bal_locate(p, in, entries, begin, end);
    if (seg.count > 0) {
      load_q_rows(qs, p, seg.tok0, seg.kvh, 0, seg.n_new * p.groups, DEC_ROWS, tid, THREADS);
      cp_async_commit();
    }
    bool first_piece = true;                // the block's first segment goes to slot 2c
    while (seg.count > 0 && alive) {
      const int tok0 = seg.tok0;
      const int rows_total = seg.n_new * p.groups;
      const int start = seg.start;
      const int key_end = start + seg.n_new;
      const int pos_a = ra < rows_total ? start + ra / p.groups : -1;
      const int pos_b = rb < rows_total ? start + rb / p.groups : -1;

      // the pair's query rows were requested a segment ago; the segment before has been written out
      cp_async_wait<0>();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      unsigned qf[D / 16][4];
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk)
        ldmatrix_x4(qf[kk], qs + (buf * DEC_ROWS + (lane & 15)) * LD + kk * 16 + (lane >> 4) * 8);
      // request the next pair's rows now: they arrive while this segment's keys are worked on
      const BalSegment next = bal_locate(p, in, entries, seg.next, end);
      if (next.count > 0) {
        load_q_rows(qs + (buf ^ 1) * DEC_ROWS * LD, p, next.tok0, next.kvh, 0, next.n_new * p.groups, DEC_ROWS, tid, THREADS);
        cp_async_commit();
      }

      float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
      float o[D / 8][4];
#pragma unroll
      for (int n = 0; n < D / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
      int s = 0;
      for (int i = 0; i < seg.count; ++i) {
        const int n = it + i;
        s = n % TMA_STAGES;
        if (!mbar_wait(full + s, (n / TMA_STAGES) & 1, abort_flag)) { alive = false; break; }
        const int key0 = (seg.tile_begin + i) * BN + warp * 16;
        if (key0 < key_end)
          tile_step<16, LineSwizzledTile>(qf, kbuf + s * (BN * D), vbuf + s * (BN * D), warp * 16, key0, key_end, pos_a,
                                          pos_b, p.window, p.scale_log2, true, m, l, o, lane);
        __syncwarp();
        // the segment's last stage stays with the consumers: the warps combine their results in it
        if (lane == 0 && i + 1 < seg.count) mbar_arrive(empty + s);
      }
      // all four warps leave the loop the same way: a wait that gave up has set the flag
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*abort_flag) { alive = false; break; }

      // warps 0 and 1 write their accumulators over the stage's keys, warps 2 and 3 over its values
      float* acc_k = reinterpret_cast<float*>(kbuf + s * (BN * D));      // [2][16][D]
      float* acc_v = reinterpret_cast<float*>(vbuf + s * (BN * D));
      float* mine = (warp < 2 ? acc_k : acc_v) + (size_t)(warp & 1) * DEC_ROWS * D;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int row = half ? rb : ra;
        if (row >= rows_total) continue;
        float2* dst = reinterpret_cast<float2*>(mine + (size_t)row * D + 2 * (lane & 3));
#pragma unroll
        for (int n = 0; n < D / 8; ++n) dst[n * 4] = make_float2(o[n][2 * half], o[n][2 * half + 1]);
        if ((lane & 3) == 0) {
          ml_s[(warp * DEC_ROWS + row) * 2] = m[half];
          ml_s[(warp * DEC_ROWS + row) * 2 + 1] = l[half];
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      // the block's first segment goes to slot 2c, a later one that a border cuts to 2c + 1
      const size_t slot = (size_t)blockIdx.x * 2 + (first_piece ? 0 : 1);
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
          num += ((w < 2 ? acc_k : acc_v)[((size_t)(w & 1) * DEC_ROWS + row) * D + d]) * f;
          den += ml_s[(w * DEC_ROWS + row) * 2 + 1] * f;
        }
        if (seg.whole) {
          const int token = row / p.groups, g = row - token * p.groups;
          p.out[((size_t)(tok0 + token) * num_q_heads + seg.kvh * p.groups + g) * D + d] =
              __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
        } else {
          p.ws_acc[(slot * DEC_ROWS + row) * D + d] = num;
          if (d == 0) {
            p.ws_ml[(slot * DEC_ROWS + row) * 2] = big;
            p.ws_ml[(slot * DEC_ROWS + row) * 2 + 1] = den;
          }
        }
      }
      // hand the stage back: ordinary stores to it come before the copies that refill it
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(empty + s);
      it += seg.count;
      seg = next;
      buf ^= 1;
      first_piece = false;
    }
  }
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicOr(p.status, FE_STATUS_WAIT_TIMEOUT);
}

// Combine the pieces of every pair that a block border cut: block = (entry, kv head).  It
// works the same cut out as the kernel above (`blocks` = that kernel's grid), so it knows
// which blocks hold the pair's pieces and in which of their two slots; pieces are added in
// block order.  Pairs that lay inside one block were finished there.
__global__ void __launch_bounds__(THREADS) attn_merge_balanced_kernel(AttnParams p, int entries, int blocks) {
  __shared__ float weight_s[DEC_ROWS * BAL_MAX_BLOCKS];
  __shared__ int sums_s[2][THREADS / 32];
  pdl_trigger();
  const int entry = blockIdx.x, kvh = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // tiles before this entry and of all entries (the step's inputs: read before the wait)
  int before = 0, all = 0;
  for (int e = threadIdx.x; e < entries; e += THREADS) {
    int unused;
    const int u = bal_pair_units(bal_entry_tiles(p, e, &unused));
    all += u;
    if (e < entry) before += u;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    before += __shfl_xor_sync(0xffffffffu, before, d);
    all += __shfl_xor_sync(0xffffffffu, all, d);
  }
  if (lane == 0) { sums_s[0][warp] = before; sums_s[1][warp] = all; }
  __syncthreads();
  before = 0; all = 0;
#pragma unroll
  for (int w = 0; w < THREADS / 32; ++w) { before += sums_s[0][w]; all += sums_s[1][w]; }
  int tile_first;
  const int t_e = bal_entry_tiles(p, entry, &tile_first);
  const long long total = (long long)p.nkv * all;
  blocks = (int)min((long long)blocks, total);
  // the pair's units begin at `pair_begin`, its tiles BAL_PAIR_UNITS later
  const long long pair_begin = (long long)p.nkv * before + (long long)kvh * bal_pair_units(t_e);
  const long long tiles_begin = pair_begin + BAL_PAIR_UNITS;
  const int c_first = t_e > 0 ? bal_block_of(tiles_begin, total, blocks) : 0;
  const int c_last = t_e > 0 ? bal_block_of(tiles_begin + t_e - 1, total, blocks) : 0;
  const int parts = c_last - c_first + 1;
  // the first block worked on another pair before this one when its stretch begins before the pair
  const int first_slot = 2 * c_first + (t_e > 0 && pair_begin > bal_begin(c_first, total, blocks) ? 1 : 0);
  // slot of piece i: the first block's, then slot 2c of every later block
  auto slot_of = [&](int i) -> size_t { return i == 0 ? (size_t)first_slot : (size_t)2 * (c_first + i); };

  // every block waits, also those without work: the kernel after this one may begin only
  // when the kernel before it has finished
  pdl_wait();
  if (parts == 1) return;
  const int tok0 = p.cu_tokens[entry];
  const int rows_total = (p.cu_tokens[entry + 1] - tok0) * p.groups;
  const int num_q_heads = p.nkv * p.groups;
  for (int row = warp; row < rows_total; row += THREADS / 32) {
    float big = -INFINITY;
    for (int i = lane; i < parts; i += 32) big = fmaxf(big, __ldcg(p.ws_ml + (slot_of(i) * DEC_ROWS + row) * 2));
    big = warp_max(big);
    float den = 0.f;
    for (int i = lane; i < parts; i += 32) {
      const float mv = __ldcg(p.ws_ml + (slot_of(i) * DEC_ROWS + row) * 2);
      const float f = (mv == -INFINITY) ? 0.f : exp2f(mv - big);
      weight_s[row * BAL_MAX_BLOCKS + i] = f;
      den += __ldcg(p.ws_ml + (slot_of(i) * DEC_ROWS + row) * 2 + 1) * f;
    }
    den = warp_sum(den);
    const float inv = den > 0.f ? 1.f / den : 0.f;
    for (int i = lane; i < parts; i += 32) weight_s[row * BAL_MAX_BLOCKS + i] *= inv;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < rows_total * D; idx += THREADS) {
    const int row = idx / D, d = idx - row * D;
    float num = 0.f;
#pragma unroll 8
    for (int i = 0; i < parts; ++i)
      num += __ldcg(p.ws_acc + (slot_of(i) * DEC_ROWS + row) * D + d) * weight_s[row * BAL_MAX_BLOCKS + i];
    const int token = row / p.groups, g = row - token * p.groups;
    p.out[((size_t)(tok0 + token) * num_q_heads + kvh * p.groups + g) * D + d] = __float2bfloat16_rn(num);
  }
}

constexpr size_t DECODE_BALANCED_SMEM = DECODE_TMA_SMEM + (size_t)DEC_ROWS * LD * sizeof(bf16) + 16 +
                                        (size_t)4 * DEC_ROWS * 2 * sizeof(float) +
                                        (size_t)3 * (BAL_MAX_ENTRIES + 1) * sizeof(int);

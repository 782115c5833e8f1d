// Next-token choice from rows of 32-bit logits: argmax, or temperature -> top-k ->
// top-p -> min-p -> softmax -> one draw, in the order of upstream's filter
// (src/forge_engine/sampling.py:49-140).  One block per row; nothing is sorted:
// the k-th largest value and the nucleus boundary are found by a 4-pass radix
// search over an order-preserving integer image of the shifted logits, with counts
// and fixed-point probability mass per digit, so that the result does not depend on
// the order in which threads arrive.  Groups of warps count into histograms of their own
// in shared memory (a vocabulary's keys fall into a handful of digits in the first pass: one
// shared histogram would serialise 150,000 atomic adds on five addresses), and the
// histograms are added up after each pass.
//
// Ties: among values equal to the k-th largest, the lowest indices are kept (exactly
// k survive).  Values equal to the nucleus boundary are all kept.
// The draw: u = uniform(seed, counter) from a counter hash (see fe_uniform below and
// its Python twin), target = u * sum(weights of survivors), first index whose running
// sum in index order exceeds target.
#include "common.cuh"

#define FE_STATUS_BAD_LOGITS 16
#define SMP_THREADS 1024
#define MASS_SCALE 1099511627776.0f  // 2^40
#define SMP_GROUPS 8                 // histogram copies; warp w counts into copy w % 8

__host__ __device__ inline unsigned long long splitmix64(unsigned long long z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// 24 random bits -> [0, 1).  The same two lines in Python give the same number.
__host__ __device__ inline float fe_uniform(unsigned long long seed, unsigned long long counter) {
  const unsigned long long h = splitmix64(splitmix64(seed) ^ (counter * 0xD1342543DE82EF95ull));
  return (float)(h >> 40) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ unsigned int float_key(float x) {
  const unsigned int u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct Survive {
  unsigned int thr_key;  // keep key > thr_key
  int tie_cut;           // keep key == thr_key only for index <= tie_cut
  float min_w;           // keep exp(x) >= min_w
};

__device__ __forceinline__ bool survives(const Survive& s, unsigned int key, int index, float w) {
  if (w < s.min_w) return false;
  return key > s.thr_key || (key == s.thr_key && index <= s.tie_cut);
}

// Exclusive scan of one value per thread in thread order; total returned to everyone.
template <typename V>
__device__ V block_exclusive_scan(V v, V* scratch /* 33 */, V* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  V inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const V t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  __syncthreads();
  if (lane == 31) scratch[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    V w = scratch[lane];
    V winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const V t = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += t;
    }
    scratch[lane] = winc - w;
    if (lane == 31) scratch[32] = winc;
  }
  __syncthreads();
  *total = scratch[32];
  return scratch[warp] + inc - v;
}

// ---- the blocks of a row's cluster ----
// A row is cut into `parts` contiguous slices of the vocabulary, one per block of a
// thread-block cluster (1 block: no cluster).  What the blocks have to agree on - the
// maximum, histograms, counts, sums - every block leaves in its own shared memory, and after
// one cluster barrier every block reads all of them in block order, so that all reach the
// same decision.  Buffers alternate between two copies: a block can be at most one
// exchange ahead of the slowest reader.
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned int peer_address(const void* mine, int rank) {
  unsigned int remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
               : "=r"(remote) : "r"((unsigned int)__cvta_generic_to_shared(mine)), "r"(rank));
  return remote;
}
__device__ __forceinline__ unsigned int peer_u32(const void* mine, int rank) {
  unsigned int v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(peer_address(mine, rank)) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long peer_u64(const void* mine, int rank) {
  unsigned long long v;
  asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(peer_address(mine, rank)) : "memory");
  return v;
}

__global__ void __launch_bounds__(SMP_THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ min_p, const unsigned long long* __restrict__ seeds,
              const unsigned long long* __restrict__ counters, int* __restrict__ out, int* status) {
  __shared__ float red_v[32];
  __shared__ int red_i[32];
  __shared__ unsigned int hist_n[2][256];            // this block's counts per digit (two copies, see above)
  __shared__ unsigned long long hist_m[2][256];      // ... and masses
  __shared__ unsigned int all_n[256];                // the row's counts per digit
  __shared__ unsigned long long all_m[256];
  __shared__ unsigned long long group_m[SMP_GROUPS * 256];
  __shared__ unsigned int group_n[SMP_GROUPS * 256];
  __shared__ unsigned long long share[2][2];         // scalars handed to the other blocks
  __shared__ unsigned long long scan_u[33];
  __shared__ float scan_f[33];
  __shared__ int scan_i[33];
  __shared__ unsigned int sh_prefix;
  __shared__ unsigned long long sh_mass_above;
  __shared__ int sh_remaining;
  __shared__ int sh_pick;

  const int parts = gridDim.x, part = blockIdx.x, row = blockIdx.y;
  const float* x = logits + (size_t)row * vocab;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = warp % SMP_GROUPS;
  const int chunk = (vocab + parts - 1) / parts;
  const int lo = min(vocab, part * chunk), hi = min(vocab, lo + chunk);   // this block's slice
  int turn = 0;                                                            // which copy the next exchange uses

  // ---- argmax, lowest index on ties; NaN and +inf are reported ----
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  bool bad = false;
  for (int i = lo + tid; i < hi; i += SMP_THREADS) {
    const float v = x[i];
    if (v != v || v == INFINITY) bad = true;
    if (v > best) { best = v; best_i = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if (lane == 0) { red_v[warp] = best; red_i[warp] = best_i; }
  if (bad) atomicOr(status, FE_STATUS_BAD_LOGITS);
  __syncthreads();
  if (warp == 0) {
    best = red_v[lane];
    best_i = red_i[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { share[turn][0] = __float_as_uint(best); share[turn][1] = (unsigned long long)(unsigned int)best_i; }
  }
  cluster_sync();
  float row_max = -INFINITY;
  int arg = 0x7fffffff;
  for (int r = 0; r < parts; ++r) {       // slices are in index order: the first of equal maxima wins
    const float v = __uint_as_float((unsigned int)peer_u64(&share[turn][0], r));
    const int at = (int)(unsigned int)peer_u64(&share[turn][1], r);
    if (v > row_max || (v == row_max && at < arg)) { row_max = v; arg = at; }
  }
  turn ^= 1;
  if (arg == 0x7fffffff) arg = 0;
  const float temp = temperature ? temperature[row] : 0.f;
  if (temp <= 0.f || row_max == -INFINITY) {
    if (tid == 0 && part == 0) out[row] = arg;
    cluster_sync();        // nobody leaves while another block may still read its shared memory
    return;
  }
  const float inv_t = 1.f / temp;
  Survive keep{0u, 0x7fffffff, 0.f};
#define SHIFTED(i) ((x[i] - row_max) * inv_t)
  // after the blocks' histograms are complete: add them up over the cluster, in block order
#define GATHER_HISTOGRAMS(WITH_MASS)                                                                  \
  do {                                                                                                \
    if (tid < 256) {                                                                                  \
      unsigned int n = 0u;                                                                            \
      unsigned long long m = 0ull;                                                                    \
      for (int w = 0; w < SMP_GROUPS; ++w) {                                                          \
        n += group_n[w * 256 + tid];                                                                  \
        if (WITH_MASS) m += group_m[w * 256 + tid];                                                   \
      }                                                                                               \
      hist_n[turn][tid] = n;                                                                          \
      if (WITH_MASS) hist_m[turn][tid] = m;                                                           \
    }                                                                                                 \
    cluster_sync();                                                                                   \
    if (tid < 256) {                                                                                  \
      unsigned int n = 0u;                                                                            \
      unsigned long long m = 0ull;                                                                    \
      for (int r = 0; r < parts; ++r) {                                                               \
        n += peer_u32(&hist_n[turn][tid], r);                                                         \
        if (WITH_MASS) m += peer_u64(&hist_m[turn][tid], r);                                          \
      }                                                                                               \
      all_n[tid] = n;                                                                                 \
      if (WITH_MASS) all_m[tid] = m;                                                                  \
    }                                                                                                 \
    turn ^= 1;                                                                                        \
    __syncthreads();                                                                                  \
  } while (0)

  // ---- top-k: radix search for the k-th largest key ----
  const int k = top_k ? top_k[row] : 0;
  if (k > 0 && k < vocab) {
    if (tid == 0) { sh_prefix = 0u; sh_remaining = k; }
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int b = tid; b < SMP_GROUPS * 256; b += SMP_THREADS) group_n[b] = 0u;
      __syncthreads();
      const unsigned int prefix = sh_prefix;
      const unsigned int mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
      if (shift == 24) {
        // first pass: every key takes part and they fall into a handful of digits; lanes of
        // a warp that hit the same digit add together, one atomic per digit and warp step
        for (int base = lo; base < hi; base += SMP_THREADS) {
          const int i = base + tid;
          const unsigned int digit = i < hi ? (float_key(SHIFTED(i)) >> 24) : 0xffffffffu;
          const unsigned int peers = __match_any_sync(0xffffffffu, digit);
          if (digit != 0xffffffffu && lane == __ffs(peers) - 1) atomicAdd(&group_n[group * 256 + digit], (unsigned int)__popc(peers));
        }
      } else {
        for (int i = lo + tid; i < hi; i += SMP_THREADS) {
          const unsigned int key = float_key(SHIFTED(i));
          if ((key & mask) == prefix) atomicAdd(&group_n[group * 256 + ((key >> shift) & 255u)], 1u);
        }
      }
      __syncthreads();
      GATHER_HISTOGRAMS(false);
      if (tid == 0) {
        int remaining = sh_remaining;
        int b = 255;
        for (; b > 0; --b) {
          if ((int)all_n[b] >= remaining) break;
          remaining -= (int)all_n[b];
        }
        sh_prefix = prefix | ((unsigned int)b << shift);
        sh_remaining = remaining;  // how many of the chosen digit are still wanted
      }
      __syncthreads();
    }
    keep.thr_key = sh_prefix;
    const int want_ties = sh_remaining;
    // the want_ties lowest indices among keys equal to the threshold survive
    const int seg = (hi - lo + SMP_THREADS - 1) / SMP_THREADS;
    const int begin = min(hi, lo + tid * seg), end = min(hi, begin + seg);
    int mine = 0;
    for (int i = begin; i < end; ++i) mine += float_key(SHIFTED(i)) == keep.thr_key;
    int total;
    int before = block_exclusive_scan<int>(mine, scan_i, &total);
    if (tid == 0) { share[turn][0] = (unsigned long long)(unsigned int)total; sh_pick = 0x7fffffff; }
    cluster_sync();
    int all_total = 0;
    for (int r = 0; r < parts; ++r) {
      const int theirs = (int)(unsigned int)peer_u64(&share[turn][0], r);
      if (r < part) before += theirs;
      all_total += theirs;
    }
    turn ^= 1;
    if (all_total > want_ties && before < want_ties && before + mine >= want_ties) {
      int seen = before;
      for (int i = begin; i < end; ++i) {
        if (float_key(SHIFTED(i)) == keep.thr_key && ++seen == want_ties) { sh_pick = i; break; }
      }
    }
    __syncthreads();
    if (tid == 0) share[turn][0] = (unsigned long long)(unsigned int)sh_pick;
    cluster_sync();
    int cut = 0x7fffffff;
    for (int r = 0; r < parts; ++r) cut = min(cut, (int)(unsigned int)peer_u64(&share[turn][0], r));
    turn ^= 1;
    keep.tie_cut = cut;
    __syncthreads();
  }

  // ---- top-p: smallest key whose mass of strictly larger survivors is <= top_p * Z ----
  const float p = top_p ? top_p[row] : 1.f;
  if (p < 1.f) {
    if (tid == 0) { sh_prefix = 0u; sh_mass_above = 0ull; }
    unsigned long long limit = 0ull;
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int b = tid; b < SMP_GROUPS * 256; b += SMP_THREADS) { group_n[b] = 0u; group_m[b] = 0ull; }
      __syncthreads();
      const unsigned int prefix = sh_prefix;
      const unsigned int mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
      unsigned long long local_total = 0ull;
      if (shift == 24) {
        // first pass: the survivors fall into a handful of digits.  Lanes that hit the same
        // digit add their masses together (in two 20-bit halves, so that 32 of them fit the
        // 32-bit warp reduction) and one of them does the atomics
        for (int base = lo; base < hi; base += SMP_THREADS) {
          const int i = base + tid;
          unsigned int digit = 0xffffffffu;
          unsigned long long mass = 0ull;
          if (i < hi) {
            const float s = SHIFTED(i);
            const unsigned int key = float_key(s);
            const float w = expf(s);
            if (survives(keep, key, i, w)) {
              mass = (unsigned long long)(w * MASS_SCALE);      // at most 2^40
              local_total += mass;
              digit = key >> 24;
            }
          }
          const unsigned int peers = __match_any_sync(0xffffffffu, digit);
          const unsigned int low = __reduce_add_sync(peers, (unsigned int)(mass & 0xfffffull));
          const unsigned int high = __reduce_add_sync(peers, (unsigned int)(mass >> 20));
          if (digit != 0xffffffffu && lane == __ffs(peers) - 1) {
            atomicAdd(&group_n[group * 256 + digit], (unsigned int)__popc(peers));
            atomicAdd(&group_m[group * 256 + digit], ((unsigned long long)high << 20) + low);
          }
        }
      } else {
        for (int i = lo + tid; i < hi; i += SMP_THREADS) {
          const float s = SHIFTED(i);
          const unsigned int key = float_key(s);
          if ((key & mask) != prefix) continue;
          const float w = expf(s);
          if (!survives(keep, key, i, w)) continue;
          atomicAdd(&group_n[group * 256 + ((key >> shift) & 255u)], 1u);
          atomicAdd(&group_m[group * 256 + ((key >> shift) & 255u)], (unsigned long long)(w * MASS_SCALE));
        }
      }
      if (shift == 24) {
        unsigned long long total;
        block_exclusive_scan<unsigned long long>(local_total, scan_u, &total);
        if (tid == 0) share[turn][1] = total;     // read after the barrier inside the gather below
      }
      __syncthreads();
      const int shared_turn = turn;
      GATHER_HISTOGRAMS(true);
      if (shift == 24) {
        unsigned long long total = 0ull;
        for (int r = 0; r < parts; ++r) total += peer_u64(&share[shared_turn][1], r);
        limit = (unsigned long long)((double)p * (double)total);
      }
      if (tid == 0) {
        unsigned long long above = sh_mass_above;
        int chosen = -1;
        unsigned long long chosen_above = above;
        for (int b = 255; b >= 0; --b) {
          if (all_n[b] == 0u) continue;
          if (above <= limit) { chosen = b; chosen_above = above; }
          else break;
          above += all_m[b];
        }
        if (chosen < 0) {  // cannot happen: the largest survivor has nothing above it
          for (int b = 255; b >= 0; --b) if (all_n[b]) { chosen = b; break; }
        }
        sh_prefix = prefix | ((unsigned int)chosen << shift);
        sh_mass_above = chosen_above;
      }
      __syncthreads();
    }
    const unsigned int boundary = sh_prefix;
    if (boundary > keep.thr_key) { keep.thr_key = boundary; keep.tie_cut = 0x7fffffff; }
    __syncthreads();
  }

  // ---- min-p: drop p_i < min_p * p_max  <=>  exp(x_i) < min_p (the largest has exp 1) ----
  const float mp = min_p ? min_p[row] : 0.f;
  if (mp > 0.f) keep.min_w = mp;

  // ---- draw in index order ----
  const int seg = (hi - lo + SMP_THREADS - 1) / SMP_THREADS;
  const int begin = min(hi, lo + tid * seg), end = min(hi, begin + seg);
  float mine = 0.f;
  int last_survivor = -1;
  for (int i = begin; i < end; ++i) {
    const float s = SHIFTED(i);
    const float w = expf(s);
    if (survives(keep, float_key(s), i, w)) { mine += w; last_survivor = i; }
  }
  float block_total;
  float before = block_exclusive_scan<float>(mine, scan_f, &block_total);
  if (tid == 0) share[turn][0] = __float_as_uint(block_total);
  cluster_sync();
  float total = 0.f, earlier = 0.f;
  for (int r = 0; r < parts; ++r) {
    const float theirs = __uint_as_float((unsigned int)peer_u64(&share[turn][0], r));
    if (r == part) earlier = total;         // the sum of the slices before this one, in block order
    total += theirs;
  }
  turn ^= 1;
  before += earlier;
  const float u = fe_uniform(seeds ? seeds[row] : 0ull, counters ? counters[row] : 0ull);
  const float target = u * total;
  // the last thread (in index order over the whole row) that has survivors and starts at or below target
  int cand = (last_survivor >= 0 && before <= target) ? part * SMP_THREADS + tid : -1;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cand = max(cand, __shfl_xor_sync(0xffffffffu, cand, o));
  __syncthreads();
  if (lane == 0) red_i[warp] = cand;
  __syncthreads();
  if (warp == 0) {
    cand = red_i[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = max(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    if (lane == 0) share[turn][0] = (unsigned long long)(unsigned int)cand;
  }
  cluster_sync();
  int owner = -1;
  for (int r = 0; r < parts; ++r) owner = max(owner, (int)(unsigned int)peer_u64(&share[turn][0], r));
  turn ^= 1;
  if (owner < 0) {
    if (tid == 0 && part == 0) out[row] = arg;
  } else if (part * SMP_THREADS + tid == owner) {
    float c = before;
    int pick = last_survivor;
    for (int i = begin; i < end; ++i) {
      const float s = SHIFTED(i);
      const float w = expf(s);
      if (!survives(keep, float_key(s), i, w)) continue;
      c += w;
      if (target < c) { pick = i; break; }
    }
    out[row] = pick;
  }
  cluster_sync();          // nobody leaves while another block may still read its shared memory
#undef GATHER_HISTOGRAMS
#undef SHIFTED
}

FE_EXPORT int fe_sample(const float* logits, int rows, int vocab, const float* temperature,
                        const int* top_k, const float* top_p, const float* min_p,
                        const unsigned long long* seeds, const unsigned long long* counters,
                        int* out, int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return FE_ERR_BAD_SHAPE;
  if (rows > 65535) return FE_ERR_TOO_LARGE;
  // a row's vocabulary over up to 8 blocks (one cluster) while the blocks of all rows still
  // run at once (two fit on each of the 148 SMs) and a block keeps at least 4,096 logits
  int parts = 1;
  while (parts < 8 && rows * parts * 2 <= 296 && vocab >= parts * 2 * 4096) parts *= 2;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(parts, rows);
  config.blockDim = dim3(SMP_THREADS);
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = parts;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  config.attrs = attribute;
  config.numAttrs = parts > 1 ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&config, sample_kernel, logits, vocab, temperature, top_k, top_p, min_p,
                                           seeds, counters, out, status);
  if (e != cudaSuccess) return (int)e;
  return fe_last_error();
}

// Host copy of the uniform, for the Python twin's self-check.
FE_EXPORT float fe_uniform_host(unsigned long long seed, unsigned long long counter) {
  return fe_uniform(seed, counter);
}

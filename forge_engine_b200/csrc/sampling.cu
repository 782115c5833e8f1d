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

__global__ void __launch_bounds__(SMP_THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ min_p, const unsigned long long* __restrict__ seeds,
              const unsigned long long* __restrict__ counters, int* __restrict__ out, int* status) {
  __shared__ float red_v[32];
  __shared__ int red_i[32];
  __shared__ unsigned int hist_n[256];
  __shared__ unsigned long long hist_m[256];
  __shared__ unsigned long long group_m[SMP_GROUPS * 256];
  __shared__ unsigned int group_n[SMP_GROUPS * 256];
  const int group = (threadIdx.x >> 5) % SMP_GROUPS;
  __shared__ unsigned long long scan_u[33];
  __shared__ float scan_f[33];
  __shared__ int scan_i[33];
  __shared__ unsigned int sh_prefix;
  __shared__ unsigned long long sh_mass_above;
  __shared__ int sh_remaining;
  __shared__ int sh_pick;

  const int row = blockIdx.x;
  const float* x = logits + (size_t)row * vocab;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // ---- argmax, lowest index on ties; NaN and +inf are reported ----
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  bool bad = false;
  for (int i = tid; i < vocab; i += SMP_THREADS) {
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
    if (lane == 0) { red_v[0] = best; red_i[0] = best_i; }
  }
  __syncthreads();
  const float row_max = red_v[0];
  const int arg = red_i[0] == 0x7fffffff ? 0 : red_i[0];
  const float temp = temperature ? temperature[row] : 0.f;
  if (temp <= 0.f || row_max == -INFINITY) {
    if (tid == 0) out[row] = arg;
    return;
  }
  const float inv_t = 1.f / temp;
  Survive keep{0u, 0x7fffffff, 0.f};
#define SHIFTED(i) ((x[i] - row_max) * inv_t)

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
        for (int base = 0; base < vocab; base += SMP_THREADS) {
          const int i = base + tid;
          const unsigned int digit = i < vocab ? (float_key(SHIFTED(i)) >> 24) : 0xffffffffu;
          const unsigned int peers = __match_any_sync(0xffffffffu, digit);
          if (digit != 0xffffffffu && lane == __ffs(peers) - 1) atomicAdd(&group_n[group * 256 + digit], (unsigned int)__popc(peers));
        }
      } else {
        for (int i = tid; i < vocab; i += SMP_THREADS) {
          const unsigned int key = float_key(SHIFTED(i));
          if ((key & mask) == prefix) atomicAdd(&group_n[group * 256 + ((key >> shift) & 255u)], 1u);
        }
      }
      __syncthreads();
      if (tid < 256) {
        unsigned int total_n = 0u;
        for (int w = 0; w < SMP_GROUPS; ++w) total_n += group_n[w * 256 + tid];
        hist_n[tid] = total_n;
      }
      __syncthreads();
      if (tid == 0) {
        int remaining = sh_remaining;
        int b = 255;
        for (; b > 0; --b) {
          if ((int)hist_n[b] >= remaining) break;
          remaining -= (int)hist_n[b];
        }
        sh_prefix = prefix | ((unsigned int)b << shift);
        sh_remaining = remaining;  // how many of the chosen digit are still wanted
      }
      __syncthreads();
    }
    keep.thr_key = sh_prefix;
    const int want_ties = sh_remaining;
    // the want_ties lowest indices among keys equal to the threshold survive
    const int seg = (vocab + SMP_THREADS - 1) / SMP_THREADS;
    const int begin = tid * seg, end = min(vocab, begin + seg);
    int mine = 0;
    for (int i = begin; i < end; ++i) mine += float_key(SHIFTED(i)) == keep.thr_key;
    int total;
    const int before = block_exclusive_scan<int>(mine, scan_i, &total);
    if (tid == 0) sh_pick = 0x7fffffff;
    __syncthreads();
    if (total > want_ties && before < want_ties && before + mine >= want_ties) {
      int seen = before;
      for (int i = begin; i < end; ++i) {
        if (float_key(SHIFTED(i)) == keep.thr_key && ++seen == want_ties) { sh_pick = i; break; }
      }
    }
    __syncthreads();
    keep.tie_cut = sh_pick;
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
        for (int base = 0; base < vocab; base += SMP_THREADS) {
          const int i = base + tid;
          unsigned int digit = 0xffffffffu;
          unsigned long long mass = 0ull;
          if (i < vocab) {
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
        for (int i = tid; i < vocab; i += SMP_THREADS) {
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
        limit = (unsigned long long)((double)p * (double)total);
      }
      __syncthreads();
      if (tid < 256) {
        unsigned int total_n = 0u;
        unsigned long long total_m = 0ull;
        for (int w = 0; w < SMP_GROUPS; ++w) { total_n += group_n[w * 256 + tid]; total_m += group_m[w * 256 + tid]; }
        hist_n[tid] = total_n;
        hist_m[tid] = total_m;
      }
      __syncthreads();
      if (tid == 0) {
        unsigned long long above = sh_mass_above;
        int chosen = -1;
        unsigned long long chosen_above = above;
        for (int b = 255; b >= 0; --b) {
          if (hist_n[b] == 0u) continue;
          if (above <= limit) { chosen = b; chosen_above = above; }
          else break;
          above += hist_m[b];
        }
        if (chosen < 0) {  // cannot happen: the largest survivor has nothing above it
          for (int b = 255; b >= 0; --b) if (hist_n[b]) { chosen = b; break; }
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
  const int seg = (vocab + SMP_THREADS - 1) / SMP_THREADS;
  const int begin = tid * seg, end = min(vocab, begin + seg);
  float mine = 0.f;
  int last_survivor = -1;
  for (int i = begin; i < end; ++i) {
    const float s = SHIFTED(i);
    const float w = expf(s);
    if (survives(keep, float_key(s), i, w)) { mine += w; last_survivor = i; }
  }
  float total;
  const float before = block_exclusive_scan<float>(mine, scan_f, &total);
  const float u = fe_uniform(seeds ? seeds[row] : 0ull, counters ? counters[row] : 0ull);
  const float target = u * total;
  // the last thread (in thread order) that has survivors and starts at or below target
  int cand = (last_survivor >= 0 && before <= target) ? tid : -1;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cand = max(cand, __shfl_xor_sync(0xffffffffu, cand, o));
  __syncthreads();
  if (lane == 0) red_i[warp] = cand;
  __syncthreads();
  if (warp == 0) {
    cand = red_i[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = max(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    if (lane == 0) red_i[0] = cand;
  }
  __syncthreads();
  const int owner = red_i[0];
  if (owner < 0) {
    if (tid == 0) out[row] = arg;
    return;
  }
  if (tid == owner) {
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
#undef SHIFTED
}

FE_EXPORT int fe_sample(const float* logits, int rows, int vocab, const float* temperature,
                        const int* top_k, const float* top_p, const float* min_p,
                        const unsigned long long* seeds, const unsigned long long* counters,
                        int* out, int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return FE_ERR_BAD_SHAPE;
  sample_kernel<<<rows, SMP_THREADS, 0, stream>>>(logits, vocab, temperature, top_k, top_p, min_p,
                                                  seeds, counters, out, status);
  return fe_last_error();
}

// Host copy of the uniform, for the Python twin's self-check.
FE_EXPORT float fe_uniform_host(unsigned long long seed, unsigned long long counter) {
  return fe_uniform(seed, counter);
}

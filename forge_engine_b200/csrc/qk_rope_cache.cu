// Per-head q/k RMSNorm + rotary position encoding + write of K and V into cache pages.
//
// Upstream does these as separate torch ops: q_norm/k_norm over head_dim with one
// weight shared by all heads (src/forge_engine/qwen3.py:141-150), the rotation
// x*cos + rotate_half(x)*sin with half-split pairing (src/forge_engine/qwen3.py:345-381)
// and a copy of the new K/V into pages after the forward (src/forge_engine/cache.py:385-416).
// Here one kernel reads the fused projection output [N, (nq + 2 nkv) * D] once,
// rewrites q in place and stores k, v straight into their pages.
//
// The angle is float(position) * inv_freq[j] with inv_freq computed by the caller
// in 32-bit; cos and sin are taken in 32-bit and not rounded.
#include "attention_common.cuh"

template <typename T>
__global__ void qk_rope_cache_kernel(T* __restrict__ qkv, const float* __restrict__ q_weight,
                                     const float* __restrict__ k_weight, float eps,
                                     const float* __restrict__ inv_freq, const float2* __restrict__ table,
                                     int rotary_dim, const int* __restrict__ positions,
                                     const int* __restrict__ token_entry, PagedKV cache,
                                     int num_q_heads, int write_kv, int* status) {
  pdl_trigger();
  pdl_wait();
  const int token = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int warps = (blockDim.x >> 5) * gridDim.y;             // warps working on this token
  const int warp = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int D = cache.head_dim, nkv = cache.num_kv_heads;
  const int heads_total = num_q_heads + 2 * nkv;
  const int pos = positions[token];
  const int entry = token_entry[token];
  const int half = rotary_dim >> 1;

  int page = -1, slot = 0;
  if (write_kv) {
    const int logical = pos / cache.page_size;
    slot = pos - logical * cache.page_size;
    if (pos < 0 || logical >= cache.max_pages) {
      if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, FE_STATUS_BAD_POSITION);
    } else {
      page = cache.block_table[(size_t)entry * cache.max_pages + logical];
      if (page < 0 || page >= cache.num_pages) {
        if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, FE_STATUS_BAD_PAGE);
        page = -1;
      }
    }
  }

  for (int head = warp; head < heads_total; head += warps) {
    T* x = qkv + (size_t)token * heads_total * D + (size_t)head * D;
    const bool is_q = head < num_q_heads;
    const bool is_k = !is_q && head < num_q_heads + nkv;
    if (!is_q && !write_kv) continue;
    T* dst = x;  // q is rewritten in place
    if (!is_q) {
      if (page < 0) continue;
      const int kvh = is_k ? head - num_q_heads : head - num_q_heads - nkv;
      T* base = (T*)(is_k ? cache.k : cache.v);
      dst = base + kv_offset(cache, page, kvh, slot);
    }
    if (!is_q && !is_k) {  // value: plain copy
      for (int i = lane; i < D; i += 32) dst[i] = x[i];
      continue;
    }
    const float* w = is_q ? q_weight : k_weight;
    float inv = 1.f;
    if (w) {
      float ss = 0.f;
      for (int i = lane; i < D; i += 32) {
        const float v = to_float(x[i]);
        ss += v * v;
      }
      ss = warp_sum(ss);
      inv = rsqrtf(ss / (float)D + eps);
    }
    // rotated part: pairs (j, j + half), j < half
    for (int j = lane; j < half; j += 32) {
      float a = to_float(x[j]) * inv, b = to_float(x[j + half]) * inv;
      if (w) { a *= w[j]; b *= w[j + half]; }
      float c = 1.f, s = 0.f;
      if (table) {
        const float2 cs = table[(size_t)token * half + j];
        c = cs.x;
        s = cs.y;
      } else if (inv_freq) {
        const float angle = (float)pos * inv_freq[j];
        c = cosf(angle);
        s = sinf(angle);
      }
      const float ra = a * c - b * s, rb = b * c + a * s;
      dst[j] = from_float<T>(ra);
      dst[j + half] = from_float<T>(rb);
    }
    // tail that is not rotated
    for (int i = rotary_dim + lane; i < D; i += 32) {
      float a = to_float(x[i]) * inv;
      if (w) a *= w[i];
      dst[i] = from_float<T>(a);
    }
  }
}

// bfloat16, the whole head rotated, D a multiple of 64 up to 256: a group of D/8 lanes takes
// one head, every lane four neighbouring elements of the first half and their partners in
// the second half (two 8-byte loads, kept in registers between the norm and the rotation).
// Cosine and sine depend on the token and the pair only: a lane computes its four once and
// uses them for every head it meets.  Same arithmetic, element by element, as the kernel
// above.
template <int D>
__global__ void qk_rope_cache_vec_kernel(bf16* __restrict__ qkv, const float* __restrict__ q_weight,
                                         const float* __restrict__ k_weight, float eps,
                                         const float* __restrict__ inv_freq, const float2* __restrict__ table,
                                         const int* __restrict__ positions,
                                         const int* __restrict__ token_entry, PagedKV cache, int num_q_heads,
                                         int write_kv, int* status) {
  constexpr int LANES = D / 8;            // lanes per head
  constexpr int HEADS = 32 / LANES;       // heads a warp takes at a time
  constexpr int HALF = D / 2;
  pdl_trigger();
  pdl_wait();
  const int token = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int sub = lane / LANES, l = lane - sub * LANES;
  const int warps = (blockDim.x >> 5) * gridDim.y;
  const int warp = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int nkv = cache.num_kv_heads;
  const int heads_total = num_q_heads + 2 * nkv;
  const int pos = positions[token];
  const int entry = token_entry[token];

  int page = -1, slot = 0;
  if (write_kv) {
    const int logical = pos / cache.page_size;
    slot = pos - logical * cache.page_size;
    if (pos < 0 || logical >= cache.max_pages) {
      if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, FE_STATUS_BAD_POSITION);
    } else {
      page = cache.block_table[(size_t)entry * cache.max_pages + logical];
      if (page < 0 || page >= cache.num_pages) {
        if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, FE_STATUS_BAD_PAGE);
        page = -1;
      }
    }
  }

  const int j0 = 4 * l;                   // this lane's pairs: (j0 + e, j0 + e + HALF)
  float cs[4], sn[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    cs[e] = 1.f; sn[e] = 0.f;
    if (table) {
      const float2 both = table[(size_t)token * HALF + j0 + e];
      cs[e] = both.x;
      sn[e] = both.y;
    } else if (inv_freq) {
      const float angle = (float)pos * inv_freq[j0 + e];
      cs[e] = cosf(angle);
      sn[e] = sinf(angle);
    }
  }
  unsigned group_mask = 0xffffffffu;
  if constexpr (LANES < 32) group_mask = ((1u << LANES) - 1u) << (sub * LANES);

  for (int head = warp * HEADS + sub; head < heads_total; head += warps * HEADS) {
    bf16* x = qkv + (size_t)token * heads_total * D + (size_t)head * D;
    const bool is_q = head < num_q_heads;
    const bool is_k = !is_q && head < num_q_heads + nkv;
    if (!is_q && (!write_kv || page < 0)) continue;
    bf16* dst = x;  // q is rewritten in place
    if (!is_q) {
      const int kvh = is_k ? head - num_q_heads : head - num_q_heads - nkv;
      dst = (bf16*)(is_k ? cache.k : cache.v) + kv_offset(cache, page, kvh, slot);
    }
    float a[4], b[4];
    load4(x + j0, a);
    load4(x + HALF + j0, b);
    if (is_q || is_k) {
      const float* w = is_q ? q_weight : k_weight;
      float inv = 1.f;
      if (w) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) ss += a[e] * a[e] + b[e] * b[e];
#pragma unroll
        for (int offset = LANES / 2; offset > 0; offset >>= 1) ss += __shfl_xor_sync(group_mask, ss, offset);
        inv = rsqrtf(ss / (float)D + eps);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float u = a[e] * inv, v = b[e] * inv;
        if (w) { u *= w[j0 + e]; v *= w[j0 + e + HALF]; }
        a[e] = u * cs[e] - v * sn[e];
        b[e] = v * cs[e] + u * sn[e];
      }
    }
    store4(dst + j0, a);
    store4(dst + HALF + j0, b);
  }
}

// The same for a projection whose k-splits met in a 32-bit buffer through atomic adds
// (`sums` [n, (nq + 2 nkv) * D], bias already added): reads the sums, puts zeros back - the
// buffer is then ready for the next projection that adds into it -, norms and rotates in
// 32-bit and stores q as bfloat16 into `q_out` (same row layout; only the q columns are
// written) and k, v into their pages.  Same arithmetic as above, on the unrounded sums.
template <int D>
__global__ void qk_rope_cache_sums_kernel(float* __restrict__ sums, bf16* __restrict__ q_out,
                                          const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                                          float eps, const float* __restrict__ inv_freq,
                                          const float2* __restrict__ table, const int* __restrict__ positions,
                                          const int* __restrict__ token_entry, PagedKV cache, int num_q_heads,
                                          int write_kv, int* status) {
  constexpr int LANES = D / 8;
  constexpr int HEADS = 32 / LANES;
  constexpr int HALF = D / 2;
  pdl_trigger();
  const int token = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int sub = lane / LANES, l = lane - sub * LANES;
  const int warps = (blockDim.x >> 5) * gridDim.y;
  const int warp = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int nkv = cache.num_kv_heads;
  const int heads_total = num_q_heads + 2 * nkv;
  // the step's own integers and the rotation table do not depend on the projection
  const int pos = positions[token];
  const int entry = token_entry[token];
  int page = -1, slot = 0;
  if (write_kv) {
    const int logical = pos / cache.page_size;
    slot = pos - logical * cache.page_size;
    if (pos < 0 || logical >= cache.max_pages) {
      if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, FE_STATUS_BAD_POSITION);
    } else {
      page = cache.block_table[(size_t)entry * cache.max_pages + logical];
      if (page < 0 || page >= cache.num_pages) {
        if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, FE_STATUS_BAD_PAGE);
        page = -1;
      }
    }
  }
  const int j0 = 4 * l;
  pdl_wait();
  float cs[4], sn[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    cs[e] = 1.f; sn[e] = 0.f;
    if (table) {
      const float2 both = table[(size_t)token * HALF + j0 + e];
      cs[e] = both.x;
      sn[e] = both.y;
    } else if (inv_freq) {
      const float angle = (float)pos * inv_freq[j0 + e];
      cs[e] = cosf(angle);
      sn[e] = sinf(angle);
    }
  }
  unsigned group_mask = 0xffffffffu;
  if constexpr (LANES < 32) group_mask = ((1u << LANES) - 1u) << (sub * LANES);
  const float zero[4] = {0.f, 0.f, 0.f, 0.f};
  for (int head = warp * HEADS + sub; head < heads_total; head += warps * HEADS) {
    float* x = sums + (size_t)token * heads_total * D + (size_t)head * D;
    const bool is_q = head < num_q_heads;
    const bool is_k = !is_q && head < num_q_heads + nkv;
    float a[4], b[4];
    load4(x + j0, a);
    load4(x + HALF + j0, b);
    store4(x + j0, zero);
    store4(x + HALF + j0, zero);
    if (!is_q && (!write_kv || page < 0)) continue;
    bf16* dst = q_out + (size_t)token * heads_total * D + (size_t)head * D;
    if (!is_q) {
      const int kvh = is_k ? head - num_q_heads : head - num_q_heads - nkv;
      dst = (bf16*)(is_k ? cache.k : cache.v) + kv_offset(cache, page, kvh, slot);
    }
    if (is_q || is_k) {
      const float* w = is_q ? q_weight : k_weight;
      float inv = 1.f;
      if (w) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) ss += a[e] * a[e] + b[e] * b[e];
#pragma unroll
        for (int offset = LANES / 2; offset > 0; offset >>= 1) ss += __shfl_xor_sync(group_mask, ss, offset);
        inv = rsqrtf(ss / (float)D + eps);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float u = a[e] * inv, v = b[e] * inv;
        if (w) { u *= w[j0 + e]; v *= w[j0 + e + HALF]; }
        a[e] = u * cs[e] - v * sn[e];
        b[e] = v * cs[e] + u * sn[e];
      }
    }
    store4(dst + j0, a);
    store4(dst + HALF + j0, b);
  }
}

// cos and sin of float(position) * inv_freq[j] for every token and pair j, taken once per
// step: table [n, half] of (cos, sin).  The angles are the same in every layer.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, int half, int n,
                                  float2* __restrict__ table) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n * half) return;
  const int token = i / half, j = i - token * half;
  const float angle = (float)positions[token] * inv_freq[j];
  table[i] = make_float2(cosf(angle), sinf(angle));
}

FE_EXPORT int fe_rope_table(const int* positions, const float* inv_freq, int half, int n, void* table, cudaStream_t stream) {
  if (n <= 0 || half <= 0) return 0;
  const int threads = 128;
  return fe_launch_dependent(rope_table_kernel, dim3((n * half + threads - 1) / threads), dim3(threads), 0, stream, positions,
                             inv_freq, half, n, (float2*)table);
}

// `table` (optional): the output of fe_rope_table for these tokens and inv_freq; without it
// the kernel takes cosine and sine itself.
FE_EXPORT int fe_qk_rope_cache(void* qkv, int dtype, const float* q_weight, const float* k_weight,
                               float eps, const float* inv_freq, const void* table, int rotary_dim,
                               const int* positions, const int* token_entry, void* k_cache,
                               void* v_cache, const int* block_table, int max_pages,
                               int page_size, int num_pages, int num_q_heads, int num_kv_heads,
                               int head_dim, int n_tokens, int write_kv, int* status,
                               cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1)) return FE_ERR_BAD_SHAPE;
  PagedKV cache{k_cache, v_cache, block_table, max_pages, page_size, num_pages, num_kv_heads, head_dim};
  const int heads_total = num_q_heads + 2 * num_kv_heads;
  // one warp per head while the batch is small (latency matters), up to 8 heads per warp
  // when there are many tokens
  int per_warp = n_tokens >= 512 ? 8 : (n_tokens >= 64 ? 2 : 1);
  const int warps_needed = (heads_total + per_warp - 1) / per_warp;
  const int warps = warps_needed < 4 ? warps_needed : 4;
  const int blocks_y = (warps_needed + warps - 1) / warps;
  if (blocks_y > 65535) return FE_ERR_TOO_LARGE;
  dim3 grid(n_tokens, blocks_y);
  const bool vec = dtype == FE_DTYPE_BF16 && rotary_dim == head_dim && (head_dim == 64 || head_dim == 128 || head_dim == 256) &&
                   (((uintptr_t)qkv | (uintptr_t)k_cache | (uintptr_t)v_cache) & 7) == 0;
  if (vec) {
    // a warp takes 32 / (D / 8) heads at a time
    const int at_a_time = 256 / head_dim;
    const int slots = (heads_total + at_a_time - 1) / at_a_time;
    per_warp = n_tokens >= 512 ? 4 : 1;
    const int need = (slots + per_warp - 1) / per_warp;
    const int w = need < 4 ? need : 4;
    dim3 vgrid(n_tokens, (need + w - 1) / w);
#define LAUNCH_VEC(DIM)                                                                                         \
    return fe_launch_dependent(qk_rope_cache_vec_kernel<DIM>, vgrid, dim3(w * 32), 0, stream, (bf16*)qkv, q_weight, \
                               k_weight, eps, inv_freq, (const float2*)table, positions, token_entry, cache, num_q_heads,  \
                               write_kv, status)
    if (head_dim == 64) LAUNCH_VEC(64);
    if (head_dim == 128) LAUNCH_VEC(128);
    LAUNCH_VEC(256);
#undef LAUNCH_VEC
  }
  if (dtype == FE_DTYPE_F32)
    return fe_launch_dependent(qk_rope_cache_kernel<float>, grid, dim3(warps * 32), 0, stream, (float*)qkv, q_weight, k_weight,
        eps, inv_freq, (const float2*)table, rotary_dim, positions, token_entry, cache, num_q_heads, write_kv, status);
  else if (dtype == FE_DTYPE_BF16)
    return fe_launch_dependent(qk_rope_cache_kernel<bf16>, grid, dim3(warps * 32), 0, stream, (bf16*)qkv, q_weight, k_weight,
        eps, inv_freq, (const float2*)table, rotary_dim, positions, token_entry, cache, num_q_heads, write_kv, status);
  else
    return FE_ERR_BAD_DTYPE;
  return fe_last_error();
}

// The form for 32-bit sums of a projection's atomic k-splits (see qk_rope_cache_sums_kernel):
// head sizes 64, 128 and 256, the whole head rotated (or no rotation: inv_freq and table null).
FE_EXPORT int fe_qk_rope_cache_sums(float* sums, void* q_out, const float* q_weight, const float* k_weight, float eps,
                                    const float* inv_freq, const void* table, const int* positions,
                                    const int* token_entry, void* k_cache, void* v_cache, const int* block_table,
                                    int max_pages, int page_size, int num_pages, int num_q_heads, int num_kv_heads,
                                    int head_dim, int n_tokens, int write_kv, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (head_dim != 64 && head_dim != 128 && head_dim != 256) return FE_ERR_BAD_SHAPE;
  if ((((uintptr_t)sums) & 15) || (((uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 7)) return FE_ERR_BAD_ALIGN;
  PagedKV cache{k_cache, v_cache, block_table, max_pages, page_size, num_pages, num_kv_heads, head_dim};
  const int heads_total = num_q_heads + 2 * num_kv_heads;
  const int at_a_time = 256 / head_dim;
  const int slots = (heads_total + at_a_time - 1) / at_a_time;
  const int per_warp = n_tokens >= 512 ? 4 : 1;
  const int need = (slots + per_warp - 1) / per_warp;
  const int w = need < 4 ? need : 4;
  dim3 grid(n_tokens, (need + w - 1) / w);
#define LAUNCH_SUMS(DIM)                                                                                          \
  return fe_launch_dependent(qk_rope_cache_sums_kernel<DIM>, grid, dim3(w * 32), 0, stream, sums, (bf16*)q_out, q_weight, \
                             k_weight, eps, inv_freq, (const float2*)table, positions, token_entry, cache, num_q_heads,    \
                             write_kv, status)
  if (head_dim == 64) LAUNCH_SUMS(64);
  if (head_dim == 128) LAUNCH_SUMS(128);
  LAUNCH_SUMS(256);
#undef LAUNCH_SUMS
}

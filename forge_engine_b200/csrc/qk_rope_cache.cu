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
                                     const float* __restrict__ inv_freq, int rotary_dim,
                                     const int* __restrict__ positions,
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
      if (inv_freq) {
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

FE_EXPORT int fe_qk_rope_cache(void* qkv, int dtype, const float* q_weight, const float* k_weight,
                               float eps, const float* inv_freq, int rotary_dim,
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
  if (dtype == FE_DTYPE_F32)
    return fe_launch_dependent(qk_rope_cache_kernel<float>, grid, dim3(warps * 32), 0, stream, (float*)qkv, q_weight, k_weight,
        eps, inv_freq, rotary_dim, positions, token_entry, cache, num_q_heads, write_kv, status);
  else if (dtype == FE_DTYPE_BF16)
    return fe_launch_dependent(qk_rope_cache_kernel<bf16>, grid, dim3(warps * 32), 0, stream, (bf16*)qkv, q_weight, k_weight,
        eps, inv_freq, rotary_dim, positions, token_entry, cache, num_q_heads, write_kv, status);
  else
    return FE_ERR_BAD_DTYPE;
  return fe_last_error();
}

// Causal grouped-query attention over cache pages, one query token per block.
//
// The plain form upstream uses for prefill is softmax(q k^T * scale + mask) v with the
// softmax in 32-bit (src/forge_engine/qwen3.py:187-206); its decode kernel walks the
// pages position by position with an online softmax in 32-bit
// (src/forge_engine/kernels/cuda_paged.py:276-347).  This kernel is the general form
// of both: any number of new tokens per request, keys read from pages (the new
// tokens' keys have been written before it runs), optional window.  It is the true
// 32-bit attention and the fallback for shapes the tensor-core kernels refuse.
//
// Work split: block = (token, q head), 4 warps.  Keys [lo, pos] are cut into chunks
// of 32 starting at lo; warp w takes chunks w, w+4, ...; inside a chunk a lane owns
// one key for the score and D/32 output elements for the value sum.  The four
// partial (max, sum, acc) are merged in a fixed order.  Nothing depends on what else
// is in the batch.
#include "attention_common.cuh"

#define ATT_WARPS 4
#define ATT_MAX_D 256

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_simt_kernel(const T* __restrict__ q, int q_stride, PagedKV cache,
                      const int* __restrict__ positions, const int* __restrict__ token_entry,
                      int window, float scale, T* __restrict__ out, int num_q_heads, int* status) {
  extern __shared__ float smem[];
  const int D = cache.head_dim;
  float* qs = smem;                        // [D]
  float* part_acc = smem + D;              // [ATT_WARPS][D]
  float* part_m = part_acc + ATT_WARPS * D;  // [ATT_WARPS]
  float* part_l = part_m + ATT_WARPS;      // [ATT_WARPS]

  const int token = blockIdx.x, head = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = head / (num_q_heads / cache.num_kv_heads);
  const int pos = positions[token];
  const int entry = token_entry[token];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const T* kbase = (const T*)cache.k;
  const T* vbase = (const T*)cache.v;
  const int* table = cache.block_table + (size_t)entry * cache.max_pages;

  const T* qrow = q + (size_t)token * q_stride + (size_t)head * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) qs[i] = to_float(qrow[i]);
  __syncthreads();

  const int nd = (D + 31) >> 5;
  float acc[ATT_MAX_D / 32];
#pragma unroll
  for (int i = 0; i < ATT_MAX_D / 32; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  const int n_keys = pos - lo + 1;
  const int n_chunks = (n_keys + 31) >> 5;
  for (int c = warp; c < n_chunks; c += ATT_WARPS) {
    const int key = lo + (c << 5) + lane;
    bool valid = key <= pos;
    long long off = -1;
    if (valid) {
      const int logical = key / cache.page_size;
      int page = -1;
      if (logical < cache.max_pages) page = table[logical];
      if (page < 0 || page >= cache.num_pages) {
        atomicOr(status, FE_STATUS_BAD_PAGE);
        valid = false;
      } else {
        off = (long long)kv_offset(cache, page, kvh, key - logical * cache.page_size);
      }
    }
    float s = -INFINITY;
    if (valid) {
      const T* kp = kbase + off;
      float dot = 0.f;
      for (int d = 0; d < D; d += 8) {
        float kk[8];
        load8(kp + d, kk);
#pragma unroll
        for (int e = 0; e < 8; ++e) dot += qs[d + e] * kk[e];
      }
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = valid ? expf(s - m_new) : 0.f;
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < ATT_MAX_D / 32; ++i) acc[i] *= corr;
    const int in_chunk = min(32, n_keys - (c << 5));
    for (int j = 0; j < in_chunk; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const long long oj = __shfl_sync(0xffffffffu, off, j);
      if (oj < 0) continue;
      const T* vp = vbase + oj;
#pragma unroll
      for (int i = 0; i < ATT_MAX_D / 32; ++i) {
        const int d = lane + (i << 5);
        if (i < nd && d < D) acc[i] += pj * to_float(vp[d]);
      }
    }
  }

  if (lane == 0) { part_m[warp] = m; part_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < ATT_MAX_D / 32; ++i) {
    const int d = lane + (i << 5);
    if (i < nd && d < D) part_acc[warp * D + d] = acc[i];
  }
  __syncthreads();
  float big = -INFINITY;
#pragma unroll
  for (int w = 0; w < ATT_WARPS; ++w) big = fmaxf(big, part_m[w]);
  T* orow = out + (size_t)token * num_q_heads * D + (size_t)head * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
      const float f = (part_m[w] == -INFINITY) ? 0.f : expf(part_m[w] - big);
      num += part_acc[w * D + d] * f;
      den += part_l[w] * f;
    }
    orow[d] = from_float<T>(den > 0.f ? num / den : 0.f);
  }
}

FE_EXPORT int fe_attention_simt(const void* q, int q_stride, int dtype, const void* k_cache,
                                const void* v_cache, const int* block_table, int max_pages,
                                int page_size, int num_pages, const int* positions,
                                const int* token_entry, int window, float scale, void* out,
                                int num_q_heads, int num_kv_heads, int head_dim, int n_tokens,
                                int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (head_dim % 8 || head_dim > ATT_MAX_D || head_dim < 8) return FE_ERR_BAD_SHAPE;
  if (num_q_heads % num_kv_heads || num_q_heads > 65535) return FE_ERR_BAD_SHAPE;
  PagedKV cache{k_cache, v_cache, block_table, max_pages, page_size, num_pages, num_kv_heads, head_dim};
  dim3 grid(n_tokens, num_q_heads);
  const size_t smem = sizeof(float) * (head_dim * (1 + ATT_WARPS) + 2 * ATT_WARPS);
  if (dtype == FE_DTYPE_F32)
    attention_simt_kernel<float><<<grid, ATT_WARPS * 32, smem, stream>>>((const float*)q, q_stride,
        cache, positions, token_entry, window, scale, (float*)out, num_q_heads, status);
  else if (dtype == FE_DTYPE_BF16)
    attention_simt_kernel<bf16><<<grid, ATT_WARPS * 32, smem, stream>>>((const bf16*)q, q_stride,
        cache, positions, token_entry, window, scale, (bf16*)out, num_q_heads, status);
  else
    return FE_ERR_BAD_DTYPE;
  return fe_last_error();
}

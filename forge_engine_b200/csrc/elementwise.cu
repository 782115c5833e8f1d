// Embedding gather, fused residual-add + RMSNorm, SiLU*mul.
//
// Upstream counterparts: nn.Embedding (src/forge_engine/qwen3.py:325), the fused
// residual RMSNorm (src/forge_engine/_triton_kernels.py:32-58; plain form
// src/forge_engine/kernels/__init__.py:12-26) and F.silu(gate) * up
// (src/forge_engine/qwen3.py:227).  The residual stream is kept in 32-bit.
#include "common.cuh"

// ---------------------------------------------------------------------------
// embedding: residual[n, :] = float(table[ids[n], :])
// ---------------------------------------------------------------------------
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int hidden, int vocab, int* status) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const int id = ids[row];
  float* dst = out + (size_t)row * hidden;
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(status, FE_STATUS_BAD_TOKEN);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.f;
    return;
  }
  const T* src = table + (size_t)id * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_float(src[i]);
}

FE_EXPORT int fe_embedding(const int* ids, const void* table, int table_dtype, float* out,
                           int n, int hidden, int vocab, int* status, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (table_dtype == FE_DTYPE_F32)
    return fe_launch_dependent(embedding_kernel<float>, dim3(n), dim3(threads), 0, stream, ids, (const float*)table, out, hidden, vocab, status);
  else if (table_dtype == FE_DTYPE_BF16)
    return fe_launch_dependent(embedding_kernel<bf16>, dim3(n), dim3(threads), 0, stream, ids, (const bf16*)table, out, hidden, vocab, status);
  else
    return FE_ERR_BAD_DTYPE;
  return fe_last_error();
}

// ---------------------------------------------------------------------------
// x = residual[src] + update[src];  residual[src] = x (optional);
// out[r] = x * rsqrt(mean(x^2) + eps) * weight       -- all in 32-bit, one rounding
// src = row_map ? row_map[r] : r
// ---------------------------------------------------------------------------
template <typename TU, typename TO, int PER>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const TU* __restrict__ update,
                                   const float* __restrict__ weight, TO* __restrict__ out,
                                   const int* __restrict__ row_map, int size, float eps,
                                   int write_residual) {
  // PER > 0: every thread keeps its PER elements (strided by blockDim) in registers between
  // the two passes; PER == 0: rows too long for that are read twice.
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = row_map ? row_map[r] : r;
  float* res = residual + (size_t)src * size;
  const TU* upd = update ? update + (size_t)src * size : nullptr;
  TO* dst = out + (size_t)r * size;
  float ss = 0.f;
  if constexpr (PER > 0) {
    float x[PER > 0 ? PER : 1];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      x[j] = 0.f;
      if (i < size) {
        x[j] = res[i];
        if (upd) x[j] += to_float(upd[i]);
        if (write_residual) res[i] = x[j];
        ss += x[j] * x[j];
      }
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)size + eps);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < size) dst[i] = from_float<TO>(x[j] * inv * weight[i]);
    }
  } else {
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
      float x = res[i];
      if (upd) x += to_float(upd[i]);
      if (write_residual) res[i] = x;
      ss += x * x;
    }
    const float total = block_sum(ss, scratch);
    const float inv = rsqrtf(total / (float)size + eps);
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
      float x = res[i];
      if (upd && !write_residual) x += to_float(upd[i]);
      dst[i] = from_float<TO>(x * inv * weight[i]);
    }
  }
}

// Rows whose length is a multiple of 4 and at most 4 * 4 * 1024: a thread keeps up to PER
// groups of four neighbouring elements (16-byte loads of the residual), same arithmetic.
template <typename TU, typename TO, int PER>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ residual, const TU* __restrict__ update,
                                       const float* __restrict__ weight, TO* __restrict__ out,
                                       const int* __restrict__ row_map, int size, float eps,
                                       int write_residual) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = row_map ? row_map[r] : r;
  float* res = residual + (size_t)src * size;
  const TU* upd = update ? update + (size_t)src * size : nullptr;
  TO* dst = out + (size_t)r * size;
  const int groups = size >> 2;
  float x[PER][4];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int g = threadIdx.x + j * blockDim.x;
    if (g < groups) {
      load4(res + 4 * g, x[j]);
      if (upd) {
        float u[4];
        load4(upd + 4 * g, u);
#pragma unroll
        for (int e = 0; e < 4; ++e) x[j][e] += u[e];
      }
      if (write_residual) store4(res + 4 * g, x[j]);
#pragma unroll
      for (int e = 0; e < 4; ++e) ss += x[j][e] * x[j][e];
    }
  }
  const float inv = rsqrtf(block_sum(ss, scratch) / (float)size + eps);
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int g = threadIdx.x + j * blockDim.x;
    if (g < groups) {
      float w[4], y[4];
      load4(weight + 4 * g, w);
#pragma unroll
      for (int e = 0; e < 4; ++e) y[e] = x[j][e] * inv * w[e];
      store4(dst + 4 * g, y);
    }
  }
}

FE_EXPORT int fe_add_rmsnorm(float* residual, const void* update, int update_dtype,
                             const float* weight, void* out, int out_dtype, const int* row_map,
                             int rows, int size, float eps, int write_residual,
                             cudaStream_t stream) {
  if (rows <= 0) return 0;
  int rc = 0;
  const int update_bytes = update_dtype == FE_DTYPE_F32 ? 16 : 8, out_bytes = out_dtype == FE_DTYPE_F32 ? 16 : 8;
  if ((size % 4) == 0 && size <= 16384 && ((uintptr_t)residual % 16) == 0 && ((uintptr_t)weight % 16) == 0 &&
      ((uintptr_t)update % update_bytes) == 0 && ((uintptr_t)out % out_bytes) == 0) {
    const int groups = size / 4;
    const int per = groups <= 1024 ? 1 : groups <= 2048 ? 2 : 4;
    const int vthreads = (((groups + per - 1) / per) + 31) / 32 * 32;
#define LAUNCH_VEC(TU, TO)                                                                                        \
    do {                                                                                                          \
      if (per == 1)                                                                                               \
        rc = fe_launch_dependent(add_rmsnorm_vec_kernel<TU, TO, 1>, dim3(rows), dim3(vthreads), 0, stream, residual, \
            (const TU*)update, weight, (TO*)out, row_map, size, eps, write_residual);                             \
      else if (per == 2)                                                                                          \
        rc = fe_launch_dependent(add_rmsnorm_vec_kernel<TU, TO, 2>, dim3(rows), dim3(vthreads), 0, stream, residual, \
            (const TU*)update, weight, (TO*)out, row_map, size, eps, write_residual);                             \
      else                                                                                                        \
        rc = fe_launch_dependent(add_rmsnorm_vec_kernel<TU, TO, 4>, dim3(rows), dim3(vthreads), 0, stream, residual, \
            (const TU*)update, weight, (TO*)out, row_map, size, eps, write_residual);                             \
    } while (0)
    if (update_dtype == FE_DTYPE_F32 && out_dtype == FE_DTYPE_F32) LAUNCH_VEC(float, float);
    else if (update_dtype == FE_DTYPE_BF16 && out_dtype == FE_DTYPE_BF16) LAUNCH_VEC(bf16, bf16);
    else if (update_dtype == FE_DTYPE_F32 && out_dtype == FE_DTYPE_BF16) LAUNCH_VEC(float, bf16);
    else if (update_dtype == FE_DTYPE_BF16 && out_dtype == FE_DTYPE_F32) LAUNCH_VEC(bf16, float);
    else return FE_ERR_BAD_DTYPE;
#undef LAUNCH_VEC
    return rc ? rc : fe_last_error();
  }
  int threads = 32;
  while (threads < 512 && threads * 4 < size) threads <<= 1;
  const int per = (size + threads - 1) / threads;
#define LAUNCH(TU, TO)                                                                               \
  do {                                                                                               \
    if (per <= 4)                                                                                    \
      rc = fe_launch_dependent(add_rmsnorm_kernel<TU, TO, 4>, dim3(rows), dim3(threads), 0, stream, residual, (const TU*)update,      \
          weight, (TO*)out, row_map, size, eps, write_residual);                                     \
    else if (per <= 16)                                                                              \
      rc = fe_launch_dependent(add_rmsnorm_kernel<TU, TO, 16>, dim3(rows), dim3(threads), 0, stream, residual, (const TU*)update,     \
          weight, (TO*)out, row_map, size, eps, write_residual);                                     \
    else                                                                                             \
      rc = fe_launch_dependent(add_rmsnorm_kernel<TU, TO, 0>, dim3(rows), dim3(threads), 0, stream, residual, (const TU*)update,      \
          weight, (TO*)out, row_map, size, eps, write_residual);                                     \
  } while (0)
  if (update_dtype == FE_DTYPE_F32 && out_dtype == FE_DTYPE_F32) LAUNCH(float, float);
  else if (update_dtype == FE_DTYPE_BF16 && out_dtype == FE_DTYPE_BF16) LAUNCH(bf16, bf16);
  else if (update_dtype == FE_DTYPE_F32 && out_dtype == FE_DTYPE_BF16) LAUNCH(float, bf16);
  else if (update_dtype == FE_DTYPE_BF16 && out_dtype == FE_DTYPE_F32) LAUNCH(bf16, float);
  else return FE_ERR_BAD_DTYPE;
#undef LAUNCH
  return rc ? rc : fe_last_error();
}

// ---------------------------------------------------------------------------
// out[n, i] = silu(gate_up[n, i]) * gate_up[n, inter + i]
// ---------------------------------------------------------------------------
__device__ __forceinline__ float silu(float x) { return x / (1.f + expf(-x)); }

// block == 0: a row is [all gate | all up]; block == B > 0: a row alternates B gate
// features, B up features (the layout the fused projection kernels want).
__device__ __forceinline__ void silu_sources(int i, int inter, int block, int* gate_at, int* up_at) {
  if (block == 0) { *gate_at = i; *up_at = inter + i; }
  else { const int b = i / block; *gate_at = 2 * b * block + (i - b * block); *up_at = *gate_at + block; }
}

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, int block) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const T* g = gate_up + (size_t)row * 2 * inter;
  T* o = out + (size_t)row * inter;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= inter) return;
  int ga, ua;
  silu_sources(i, inter, block, &ga, &ua);
  o[i] = from_float<T>(silu(to_float(g[ga])) * to_float(g[ua]));
}

template <typename T>
__global__ void silu_mul_vec8_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, int block) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const T* g = gate_up + (size_t)row * 2 * inter;
  T* o = out + (size_t)row * inter;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (i >= inter) return;
  int ga, ua;
  silu_sources(i, inter, block, &ga, &ua);   // block is a multiple of 8, so 8 features stay together
  float a[8], b[8];
  load8_streaming(g + ga, a);      // gate and up are read once: they need not stay in the caches
  load8_streaming(g + ua, b);
#pragma unroll
  for (int k = 0; k < 8; ++k) a[k] = silu(a[k]) * b[k];
  store8(o + i, a);
}

FE_EXPORT int fe_silu_mul(const void* gate_up, void* out, int dtype, int rows, int inter, int block,
                          cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (block < 0 || (block > 0 && (inter % block) != 0)) return FE_ERR_BAD_SHAPE;
  const bool vec = (inter % 8) == 0 && (block % 8) == 0 && ((uintptr_t)gate_up % 32) == 0 && ((uintptr_t)out % 32) == 0;
  const int threads = 256;
  const int per = vec ? 8 : 1;
  dim3 grid(rows, (inter + threads * per - 1) / (threads * per));
  if (grid.y > 65535) return FE_ERR_TOO_LARGE;
  if (dtype == FE_DTYPE_F32) {
    if (vec) return fe_launch_dependent(silu_mul_vec8_kernel<float>, grid, dim3(threads), 0, stream, (const float*)gate_up, (float*)out, inter, block);
    else return fe_launch_dependent(silu_mul_kernel<float>, grid, dim3(threads), 0, stream, (const float*)gate_up, (float*)out, inter, block);
  } else if (dtype == FE_DTYPE_BF16) {
    if (vec) return fe_launch_dependent(silu_mul_vec8_kernel<bf16>, grid, dim3(threads), 0, stream, (const bf16*)gate_up, (bf16*)out, inter, block);
    else return fe_launch_dependent(silu_mul_kernel<bf16>, grid, dim3(threads), 0, stream, (const bf16*)gate_up, (bf16*)out, inter, block);
  } else {
    return FE_ERR_BAD_DTYPE;
  }
  return fe_last_error();
}

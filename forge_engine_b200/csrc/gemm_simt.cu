// y[n, o] = sum_k x[n, k] * w[o, k] (+ bias[o]) (+ y[n, o])   -- plain FFMA, no tensor cores.
//
// This is the matrix product of the true 32-bit path and of any tensor whose
// checkpoint dtype is float32.  Both operands are K-major, like nn.Linear's
// [out, in] weight (src/forge_engine/qwen3.py:113-122).  Each output element is
// summed over k in ascending order by one thread, so a row's result does not depend
// on how many other rows are in the call.
#include "common.cuh"

#define GS_BM 64
#define GS_BN 64
#define GS_BK 16

template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TX* __restrict__ x, const TW* __restrict__ w, const float* __restrict__ bias,
                 TY* __restrict__ y, int n, int o, int k, int accumulate) {
  __shared__ float xs[GS_BK][GS_BM + 4];
  __shared__ float ws[GS_BK][GS_BN + 4];
  const int tid = threadIdx.x;
  const int row0 = blockIdx.y * GS_BM, col0 = blockIdx.x * GS_BN;
  const int ty = tid >> 4, tx = tid & 15;
  const int lr = tid >> 2, lk = (tid & 3) << 2;  // this thread stages row lr, k offsets lk..lk+3
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < k; k0 += GS_BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int kk = k0 + lk + e;
      const int xr = row0 + lr, wr = col0 + lr;
      xs[lk + e][lr] = (xr < n && kk < k) ? to_float(x[(size_t)xr * k + kk]) : 0.f;
      ws[lk + e][lr] = (wr < o && kk < k) ? to_float(w[(size_t)wr * k + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GS_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = row0 + ty * 4 + i;
    if (r >= n) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tx * 4 + j;
      if (c >= o) continue;
      float v = acc[i][j];
      if (bias) v += bias[c];
      TY* dst = y + (size_t)r * o + c;
      if (accumulate) v += to_float(*dst);
      *dst = from_float<TY>(v);
    }
  }
}

template <typename TX, typename TW, typename TY>
static int launch_simt(const void* x, const void* w, const float* bias, void* y, int n, int o, int k,
                       int accumulate, cudaStream_t stream) {
  dim3 grid((o + GS_BN - 1) / GS_BN, (n + GS_BM - 1) / GS_BM);
  if (grid.y > 65535) return FE_ERR_TOO_LARGE;
  gemm_simt_kernel<TX, TW, TY><<<grid, 256, 0, stream>>>((const TX*)x, (const TW*)w, bias, (TY*)y, n, o,
                                                        k, accumulate);
  return fe_last_error();
}

FE_EXPORT int fe_gemm_simt(const void* x, int x_dtype, const void* w, int w_dtype, const float* bias,
                           void* y, int y_dtype, int n, int o, int k, int accumulate,
                           cudaStream_t stream) {
  if (n <= 0 || o <= 0) return 0;
  if (k <= 0) return FE_ERR_BAD_SHAPE;
  const int code = x_dtype * 4 + w_dtype * 2 + y_dtype;
  switch (code) {
    case 0: return launch_simt<float, float, float>(x, w, bias, y, n, o, k, accumulate, stream);
    case 1: return launch_simt<float, float, bf16>(x, w, bias, y, n, o, k, accumulate, stream);
    case 2: return launch_simt<float, bf16, float>(x, w, bias, y, n, o, k, accumulate, stream);
    case 3: return launch_simt<float, bf16, bf16>(x, w, bias, y, n, o, k, accumulate, stream);
    case 4: return launch_simt<bf16, float, float>(x, w, bias, y, n, o, k, accumulate, stream);
    case 5: return launch_simt<bf16, float, bf16>(x, w, bias, y, n, o, k, accumulate, stream);
    case 6: return launch_simt<bf16, bf16, float>(x, w, bias, y, n, o, k, accumulate, stream);
    case 7: return launch_simt<bf16, bf16, bf16>(x, w, bias, y, n, o, k, accumulate, stream);
  }
  return FE_ERR_BAD_DTYPE;
}

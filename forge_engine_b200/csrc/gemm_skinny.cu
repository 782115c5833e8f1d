// y[n, o] = sum_k x[n, k] * w[o, k] for a handful of rows n (decode steps): bfloat16 in,
// 32-bit accumulate, tensor-core mma with the weights streamed straight from global
// memory.  With few tokens the product is bound by reading w once; the library GEMM
// reaches about half of the memory bandwidth on these shapes, this kernel is built to
// keep many 16-byte loads in flight per SM instead.
//
// Upstream computes every projection with nn.Linear (src/forge_engine/qwen3.py:113-122,
// 210-227); this is the same product for [out, in] weights.
//
// Work split: block = 16 output features x all of K; its 8 warps take interleaved 32-wide
// blocks of k, and their partial sums are added in a fixed order in shared memory.  A
// thread's 16-byte load of a weight row (8 consecutive k) feeds the A operand of two
// mma k-steps; the activations are loaded with the same permutation of k, so no shared
// memory staging of the weights is needed.
//
// Epilogues: store (bf16 or f32), add into a 32-bit tensor (residual stream), or
// SiLU(gate) * up for a weight whose rows alternate 8 gate features, 8 up features.
#include "common.cuh"

namespace {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int ROWS = 16;
constexpr int KB = 32;   // k per block: 4 lanes x 8 elements per row

enum Epilogue { EPI_STORE_BF16 = 0, EPI_STORE_F32 = 1, EPI_ADD_F32 = 2, EPI_SILU_MUL_BF16 = 3 };

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_cached(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }

// NT: token tiles of 8 (n <= 8 * NT); U: k-blocks in flight per warp and iteration.
template <int NT, int U, int EPI>
__global__ void __launch_bounds__(THREADS)
gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const float* __restrict__ bias,
                   void* __restrict__ y, int n, int o, int k, float* __restrict__ ws_part,
                   unsigned* __restrict__ ws_count) {
  // gridDim.y blocks share one 16-feature tile, each taking every gridDim.y-th group of
  // 8 k-blocks.  Their partial tiles go to ws_part; the block that arrives last adds them
  // in block order (so the sum does not depend on timing) and runs the epilogue.
  __shared__ float part[WARPS][ROWS][NT * 8 + 1];
  __shared__ bool is_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * ROWS;
  const int ra = row0 + g, rb = ra + 8;
  const bool va = ra < o, vb = rb < o;
  const bf16* wa = w + (size_t)(va ? ra : 0) * k + t * 8;
  const bf16* wb = w + (size_t)(vb ? rb : 0) * k + t * 8;
  const bf16* xrow[NT];
  bool xv[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int token = j * 8 + g;
    xv[j] = token < n;
    xrow[j] = x + (size_t)(xv[j] ? token : 0) * k + t * 8;
  }
  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }

  const int blocks = (k + KB - 1) / KB;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  const int ksplit = gridDim.y;
  // this block's k-blocks: groups of WARPS * U consecutive blocks, every ksplit-th group
  for (int b0 = blockIdx.y * WARPS * U + warp; b0 < blocks; b0 += WARPS * U * ksplit) {
    uint4 fa[U], fb[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int kk = (b0 + u * WARPS) * KB;
      const bool in = kk + t * 8 < k;     // k is a multiple of 8, so a chunk is in or out as a whole
      fa[u] = (in && va) ? ld_stream(wa + kk) : zero;
      fb[u] = (in && vb) ? ld_stream(wb + kk) : zero;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int kk = (b0 + u * WARPS) * KB;
      const bool in = kk + t * 8 < k;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const uint4 fx = (in && xv[j]) ? ld_cached(xrow[j] + kk) : zero;
        mma16816(acc[j], fa[u].x, fb[u].x, fa[u].y, fb[u].y, fx.x, fx.y);
        mma16816(acc[j], fa[u].z, fb[u].z, fa[u].w, fb[u].w, fx.z, fx.w);
      }
    }
  }

#pragma unroll
  for (int j = 0; j < NT; ++j) {
    part[warp][g][j * 8 + 2 * t] = acc[j][0];
    part[warp][g][j * 8 + 2 * t + 1] = acc[j][1];
    part[warp][g + 8][j * 8 + 2 * t] = acc[j][2];
    part[warp][g + 8][j * 8 + 2 * t + 1] = acc[j][3];
  }
  __syncthreads();
  constexpr int NTOK = NT * 8;
  if (ksplit > 1) {
    // fold this block's eight warps and publish the tile
    float* mine = ws_part + ((size_t)blockIdx.x * ksplit + blockIdx.y) * ROWS * NTOK;
    for (int idx = threadIdx.x; idx < ROWS * NTOK; idx += THREADS) {
      const int r = idx / NTOK, token = idx - r * NTOK;
      float v = 0.f;
#pragma unroll
      for (int wi = 0; wi < WARPS; ++wi) v += part[wi][r][token];
      mine[idx] = v;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned arrived = atomicAdd(ws_count + blockIdx.x, 1u);
      is_last = arrived == (unsigned)ksplit - 1u;
      if (is_last) ws_count[blockIdx.x] = 0u;   // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const float* all = ws_part + (size_t)blockIdx.x * ksplit * ROWS * NTOK;
    for (int idx = threadIdx.x; idx < ROWS * NTOK; idx += THREADS) {
      const int r = idx / NTOK, token = idx - r * NTOK;
      float v = 0.f;
      for (int sp = 0; sp < ksplit; ++sp) v += __ldcg(all + (size_t)sp * ROWS * NTOK + idx);
      part[0][r][token] = v;
#pragma unroll
      for (int wi = 1; wi < WARPS; ++wi) part[wi][r][token] = 0.f;
    }
    __syncthreads();
  }
  if (EPI == EPI_SILU_MUL_BF16) {
    // rows 0..7 of the tile are gate features, rows 8..15 the matching up features
    const int half_o = o >> 1;
    for (int idx = threadIdx.x; idx < 8 * n; idx += THREADS) {
      const int token = idx >> 3, r = idx & 7;
      const int feature = blockIdx.x * 8 + r;
      if (feature >= half_o) continue;
      float gate = 0.f, up = 0.f;
#pragma unroll
      for (int wi = 0; wi < WARPS; ++wi) { gate += part[wi][r][token]; up += part[wi][r + 8][token]; }
      reinterpret_cast<bf16*>(y)[(size_t)token * half_o + feature] = __float2bfloat16_rn(silu_f(gate) * up);
    }
    return;
  }
  for (int idx = threadIdx.x; idx < ROWS * n; idx += THREADS) {
    const int token = idx >> 4, r = idx & 15;
    const int row = row0 + r;
    if (row >= o) continue;
    float v = 0.f;
#pragma unroll
    for (int wi = 0; wi < WARPS; ++wi) v += part[wi][r][token];
    if (bias) v += bias[row];
    const size_t at = (size_t)token * o + row;
    if (EPI == EPI_STORE_BF16) reinterpret_cast<bf16*>(y)[at] = __float2bfloat16_rn(v);
    else if (EPI == EPI_STORE_F32) reinterpret_cast<float*>(y)[at] = v;
    else reinterpret_cast<float*>(y)[at] += v;
  }
}

template <int NT, int U>
int launch(int epi, const bf16* x, const bf16* w, const float* bias, void* y, int n, int o, int k,
           int ksplit, float* ws_part, unsigned* ws_count, cudaStream_t stream) {
  const int tiles = (o + ROWS - 1) / ROWS;
  const int blocks = (k + KB - 1) / KB;
  const int groups = (blocks + WARPS * U - 1) / (WARPS * U);
  if (ksplit > groups) ksplit = groups;
  if (ksplit < 1) ksplit = 1;
  dim3 grid(tiles, ksplit);
  switch (epi) {
    case EPI_STORE_BF16: gemm_skinny_kernel<NT, U, EPI_STORE_BF16><<<grid, THREADS, 0, stream>>>(x, w, bias, y, n, o, k, ws_part, ws_count); break;
    case EPI_STORE_F32: gemm_skinny_kernel<NT, U, EPI_STORE_F32><<<grid, THREADS, 0, stream>>>(x, w, bias, y, n, o, k, ws_part, ws_count); break;
    case EPI_ADD_F32: gemm_skinny_kernel<NT, U, EPI_ADD_F32><<<grid, THREADS, 0, stream>>>(x, w, bias, y, n, o, k, ws_part, ws_count); break;
    case EPI_SILU_MUL_BF16: gemm_skinny_kernel<NT, U, EPI_SILU_MUL_BF16><<<grid, THREADS, 0, stream>>>(x, w, bias, y, n, o, k, ws_part, ws_count); break;
    default: return FE_ERR_BAD_DTYPE;
  }
  return fe_last_error();
}

}  // namespace

// epilogue: 0 store bf16 [n, o]; 1 store f32 [n, o]; 2 add into f32 [n, o];
// 3 y[n, o/2] = silu(gate) * up (bf16) for w whose rows alternate 8 gate, 8 up features.
// ksplit > 1 lets that many blocks share a 16-feature tile; it needs ws_part (floats:
// tiles * ksplit * 16 * 64 at most) and ws_count (one zeroed unsigned per tile, left zeroed).
FE_EXPORT int fe_gemm_skinny(const void* x, const void* w, const float* bias, void* y, int n, int o, int k,
                             int epilogue, int ksplit, float* ws_part, unsigned* ws_count,
                             cudaStream_t stream) {
  if (n <= 0 || o <= 0) return 0;
  if (n > 64 || k <= 0 || (k % 8) != 0) return FE_ERR_BAD_SHAPE;
  if (epilogue == EPI_SILU_MUL_BF16 && ((o % 16) != 0 || bias != nullptr)) return FE_ERR_BAD_SHAPE;
  if ((((uintptr_t)x) | ((uintptr_t)w)) & 15) return FE_ERR_BAD_ALIGN;
  const bf16* xp = (const bf16*)x;
  const bf16* wp = (const bf16*)w;
  if (ksplit > 1 && (ws_part == nullptr || ws_count == nullptr)) return FE_ERR_BAD_SHAPE;
  if (n <= 8) return launch<1, 8>(epilogue, xp, wp, bias, y, n, o, k, ksplit, ws_part, ws_count, stream);
  if (n <= 16) return launch<2, 8>(epilogue, xp, wp, bias, y, n, o, k, ksplit, ws_part, ws_count, stream);
  if (n <= 32) return launch<4, 4>(epilogue, xp, wp, bias, y, n, o, k, ksplit, ws_part, ws_count, stream);
  return launch<8, 2>(epilogue, xp, wp, bias, y, n, o, k, ksplit, ws_part, ws_count, stream);
}

// Shared device helpers for the sm_100a kernels of this engine.
//
// Element types: `float` and `__nv_bfloat16`.  Every kernel does its arithmetic in
// 32-bit and rounds once, on store.  Launchers have C linkage, take raw device
// pointers and the stream to launch on, and return a cudaError_t as int (or one of
// the FE_ERR_* codes below for an argument they refuse).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <utility>

#define FE_DTYPE_F32 0
#define FE_DTYPE_BF16 1

#define FE_ERR_BAD_DTYPE 10001
#define FE_ERR_BAD_SHAPE 10002
#define FE_ERR_BAD_ALIGN 10003
#define FE_ERR_TOO_LARGE 10004

// Bits of the device status word kernels set instead of trapping.
#define FE_STATUS_BAD_TOKEN 1      // token id outside the vocabulary
#define FE_STATUS_BAD_PAGE 2       // block table entry outside the pool or negative
#define FE_STATUS_BAD_POSITION 4   // position outside the block table
#define FE_STATUS_WAIT_TIMEOUT 8   // a bounded wait inside a kernel ran out

#define FE_EXPORT extern "C" __attribute__((visibility("default")))

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order
// of additions depends only on blockDim, never on the data or on other blocks.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < warps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Loads of 8 consecutive elements as floats (16 bytes of bf16, 32 bytes of float).
__device__ __forceinline__ void load8(const float* p, float* out) {
  const float4 a = reinterpret_cast<const float4*>(p)[0];
  const float4 b = reinterpret_cast<const float4*>(p)[1];
  out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
  out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float* out) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
// The same with the evict-first hint, for data that is read once.
__device__ __forceinline__ void load8_streaming(const float* p, float* out) {
  const float4 a = __ldcs(reinterpret_cast<const float4*>(p));
  const float4 b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
  out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
  out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
__device__ __forceinline__ void load8_streaming(const bf16* p, float* out) {
  const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(p));
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void store8(float* p, const float* v) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(bf16* p, const float* v) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// The same for 4 consecutive elements (8 bytes of bf16, 16 bytes of float).
__device__ __forceinline__ void load4(const float* p, float* out) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
}
__device__ __forceinline__ void load4(const bf16* p, float* out) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
}
__device__ __forceinline__ void store4(float* p, const float* v) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(bf16* p, const float* v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 raw;
  raw.x = *reinterpret_cast<const unsigned*>(&a);
  raw.y = *reinterpret_cast<const unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

static inline int fe_last_error() { return (int)cudaGetLastError(); }

// Programmatic dependent launch.  A kernel that is launched "dependent" may start while
// the kernel before it on the stream is still running; it must execute pdl_wait() before it
// reads or writes anything that kernel (or an earlier one) touches.  pdl_trigger() in a
// kernel lets the next kernel, if it was launched dependent, start early.  Both are no-ops
// for kernels launched the ordinary way.
// FORGE_ENGINE_PDL=0 in the environment launches every kernel the ordinary way.
static inline int fe_pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) {
    const char* text = getenv("FORGE_ENGINE_PDL");
    enabled = (text != nullptr && text[0] == '0') ? 0 : 1;
  }
  return enabled;
}

// Launch `kernel` as a dependent of the kernel before it on `stream`.  Only for kernels that
// call pdl_wait() before their first access to global memory another kernel may write.
// `cluster` with more than one block additionally groups that many consecutive blocks into
// one thread-block cluster (they can then read one another's shared memory).
template <typename... KArgs, typename... Args>
static inline int fe_launch_dependent_shaped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                             cudaStream_t stream, dim3 cluster, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = fe_pdl_enabled();
  config.attrs = attribute;
  config.numAttrs = 1;
  if (cluster.x * cluster.y * cluster.z > 1) {
    attribute[1].id = cudaLaunchAttributeClusterDimension;
    attribute[1].val.clusterDim.x = cluster.x;
    attribute[1].val.clusterDim.y = cluster.y;
    attribute[1].val.clusterDim.z = cluster.z;
    config.numAttrs = 2;
  }
  return (int)cudaLaunchKernelEx(&config, kernel, std::forward<Args>(args)...);
}

// Cluster of `cluster_z` blocks along the grid's z axis (1: no cluster).
template <typename... KArgs, typename... Args>
static inline int fe_launch_dependent_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                              cudaStream_t stream, int cluster_z, Args&&... args) {
  return fe_launch_dependent_shaped(kernel, grid, block, smem, stream, dim3(1, 1, (unsigned)(cluster_z > 1 ? cluster_z : 1)),
                                    std::forward<Args>(args)...);
}

template <typename... KArgs, typename... Args>
static inline int fe_launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t stream, Args&&... args) {
  return fe_launch_dependent_cluster(kernel, grid, block, smem, stream, 1, std::forward<Args>(args)...);
}

__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

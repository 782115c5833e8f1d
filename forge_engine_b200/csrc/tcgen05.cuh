// tcgen05 / TMA / mbarrier wrappers shared by the tensor-core product kernels of this engine
// (inline PTX for sm_100a), and the host-side tensor-map encoder.
//
// Every wait on an mbarrier is bounded: mbar_wait gives up after `limit` polls (or when another
// role of the block has given up), and the caller then stops issuing work, frees its tensor
// memory and returns with FE_STATUS_WAIT_TIMEOUT set.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace tc5 {

constexpr int BM = 128;        // weight rows (output features) per block
constexpr int BK = 64;         // k per stage: 128 bytes of bfloat16 = one swizzle row
constexpr int UMMA_K = 16;
constexpr unsigned WAIT_LIMIT = 20000000u;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Non-blocking test of a phase, so that the loop around it has a bound of its own.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: false when the limit was hit or another role has already given up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity, volatile int* abort_flag,
                                          unsigned limit = WAIT_LIMIT) {
  for (unsigned i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

// Asks for a tensor map ahead of the first copy that uses it (the map is a kernel parameter;
// the copy engine otherwise fetches its 128 bytes when that copy is issued).
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}

// Shared-memory matrix descriptor: K-major tile, rows of 128 bytes, 128-byte swizzle,
// 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(const void* tile) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_u32(tile) & 0x3FFFFu) >> 4);   // start address
  d |= (uint64_t)1 << 16;                              // leading byte offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset
  d |= (uint64_t)1 << 46;                              // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                              // 128-byte swizzle
  return d;
}

__device__ __forceinline__ unsigned umma_idesc(int n) {
  unsigned d = 0;
  d |= 1u << 4;                  // accumulator: f32
  d |= 1u << 7;                  // A: bf16
  d |= 1u << 10;                 // B: bf16
  d |= (unsigned)(n >> 3) << 17; // N
  d |= (unsigned)(BM >> 4) << 24;  // M
  return d;                      // both operands K-major, no negation, dense
}

__device__ __forceinline__ void umma_f16(unsigned tmem_d, uint64_t desc_a, uint64_t desc_b, unsigned idesc,
                                         unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld16(unsigned taddr, float (&v)[16]) {
  unsigned r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// [rows, k] bfloat16, row-major; box = box_rows x 64 elements, 128-byte swizzle; reads
// outside the tensor give zeros.
static inline int make_map(CUtensorMap* map, const void* base, int rows, int k, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return FE_ERR_BAD_SHAPE;
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)k * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 20000 + (int)r;
}

}  // namespace tc5

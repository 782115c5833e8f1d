/* Split decode attention over the paged cache for callers that must not allocate.
 *
 * This entry point has no counterpart in the upstream project (marcoharuni/forge-engine);
 * it exists for programs that embed these kernels without a tensor library.
 *
 * Who needs it.  The usual entry point (fe_attention_mma_d<HEAD>) takes a workspace
 * pointer for the partial results of its splits, and the Python binding gets that
 * workspace from torch's allocator on every call.  Some hosts cannot do either:
 *   - a service that hands all device memory to an arena of its own at start-up, so
 *     that a later cudaMalloc would fail or fragment what it manages;
 *   - a latency-critical loop, because cudaMalloc and cudaFree synchronise the whole
 *     device and stall every other stream while they run;
 *   - plain C or C++ programs that load the .so directly and have no allocator to ask.
 * For them the scratch lives inside the library, in a __device__ array of fixed size.
 * The caller still passes every input and the output buffer.
 *
 * One function per head size, in the library built for that head size
 * (libforge_engine_b200_attn_d<HEAD>.so, compiled with -DFE_HEAD_DIM=<HEAD>; HEAD is any
 * multiple of 16 from 16 to 256):
 *
 *   int fe_attention_decode_noalloc_d<HEAD>(...same leading arguments as below...);
 *
 * The prototypes for 64 and 128 are declared at the end of this file; for another head
 * size write FE_DECLARE_ATTENTION_DECODE_NOALLOC(<HEAD>); after including it.
 *
 * Arguments
 *   q, q_stride     bfloat16 queries; row n starts at q + n * q_stride elements and holds
 *                   num_kv_heads * groups heads of HEAD elements (already normalised and
 *                   rotated); q_stride must be a multiple of 8; q 16-byte aligned
 *   out             bfloat16 [tokens, num_kv_heads * groups * HEAD]
 *   k_cache,v_cache bfloat16 [num_pages, num_kv_heads, page_size, HEAD], 16-byte aligned;
 *                   the step's own keys and values must already be stored in them
 *   block_table     int32 [entries, max_pages]: page of tokens [i*page_size, (i+1)*page_size)
 *   cu_tokens       int32 [entries + 1]: where each entry's new tokens start
 *   starts          int32 [entries]: tokens each entry held before this step
 *   max_new         the most new tokens any entry brings; max_new * groups must be <= 16
 *                   (this is the decode kernel: one new token, or a few)
 *   window          0 for full attention, else how many most recent keys a query sees
 *   scale           factor on q.k before the softmax
 *   num_splits      how many blocks share one (entry, kv head)'s key range (>= 1)
 *   status          int32 device word; bit 2 is set if a needed page is missing
 *   stream          the CUDA stream to launch on
 * Returns 0 on success; 10002 for a shape it does not take; 10003 for misalignment;
 * 10005 when num_splits > 1 and entries * num_kv_heads * num_splits * 16 * (HEAD + 2)
 * exceeds the scratch (1,048,576 floats = 4 MiB; a line naming the sizes is also written to
 * stderr; with one split the array is not used and any number of entries is taken); any
 * other non-zero value is a cudaError_t.
 *
 * What to know
 *   - It calls no cudaMalloc, cudaFree or other allocating routine.  The 4 MiB array is
 *     part of the library image: every GPU whose context loads the library holds it
 *     until the process exits.
 *   - The first call on each device looks the array's device address up
 *     (cudaGetSymbolAddress) and raises the kernel's shared-memory limit, with that
 *     device current.  Make that first call outside of any stream capture, and from one
 *     host thread: the table of looked-up addresses is a plain static, so two threads
 *     making a device's first call at the same moment would race on it (later calls only
 *     read it and may come from any thread).
 *   - All calls on a device share the one array, and it keeps what the last call left.
 *     Nothing in it has to start at zero: every slot a call reads is written earlier in
 *     that same call.  Two calls that overlap on the GPU (different streams, or the same
 *     graph launched twice at once) would write the same slots and race: keep calls that
 *     use this entry point ordered on the device.
 */
#ifndef FORGE_ENGINE_B200_ATTENTION_NOALLOC_H
#define FORGE_ENGINE_B200_ATTENTION_NOALLOC_H

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FE_ATTENTION_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define FE_ERR_SCRATCH_TOO_SMALL 10005

#define FE_DECLARE_ATTENTION_DECODE_NOALLOC(HEAD)                                                     \
  int fe_attention_decode_noalloc_d##HEAD(                                                            \
      const void* q, int q_stride, void* out, const void* k_cache, const void* v_cache,               \
      const int* block_table, int max_pages, int page_size, int num_pages, int num_kv_heads,          \
      int groups, const int* cu_tokens, const int* starts, int entries, int max_new, int window,      \
      float scale, int num_splits, int* status, cudaStream_t stream)

FE_DECLARE_ATTENTION_DECODE_NOALLOC(64);
FE_DECLARE_ATTENTION_DECODE_NOALLOC(128);

#ifdef __cplusplus
}
#endif
#endif

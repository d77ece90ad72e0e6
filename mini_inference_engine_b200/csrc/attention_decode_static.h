/* A decode-attention entry point that allocates nothing.  It has no counterpart in the reference
 * (brave30/mini-inference-engine), whose decode attention always lets torch allocate its partial
 * results (inference_engine/kernels/decode_attention.py:146-148); it exists for this library's users.
 *
 * Who needs it: a host program that has handed all of the device's memory out at start-up (to the
 * cache pages, typically) and has no allocator left to ask for a few megabytes per call; a caller on
 * a latency-critical loop, for whom cudaMalloc is unusable because it synchronises the whole device;
 * and a caller that links this library from C or another runtime and has no torch allocator to pass
 * tensors from.  Such a caller passes inputs and outputs only.  The partial results and the split
 * counters of the kernel live in one array inside the library
 * (`static __device__ __align__(256)`, MIE_STATIC_SCRATCH_BYTES bytes), which every GPU that loads
 * the library holds until the process exits.
 *
 * Rules of use:
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress) with that
 *    device current; make that first call before any stream capture.  Later calls on the device
 *    reuse the address.
 *  - Sizes beyond the array are refused with MIE_ERR_TOO_LARGE (-2) and a message that
 *    mie_decode_attention_static_error() returns; nothing is launched.  The limits:
 *        rows * heads * splits * head_dim  <= MIE_STATIC_MAX_PART_O    (float32 partial outputs)
 *        rows * heads * splits             <= MIE_STATIC_MAX_PART_LSE
 *        rows * kv_heads * ceil(group/16)  <= MIE_STATIC_MAX_UNITS     (split counters)
 *    With splits == 1 the scratch is not used and only the kernel's own limits apply.
 *  - Every call uses the same array.  Calls that may overlap on the GPU (two streams, two threads)
 *    race on it: serialise them, e.g. by issuing them on one stream.  The counters are cleared on
 *    the stream at the start of every call, so a call does not depend on what the last one left.
 *  - No cudaMalloc, cudaFree or allocating library routine is called.
 *  - The kernel is launched with the programmatic-stream-serialization attribute, like every kernel
 *    of this library, and reads the lengths, the block tables and every cached row except the newest
 *    (position ctx - 1 of a row) BEFORE it waits for the kernel in front of it on the stream.  So the
 *    kernel directly in front may write only that newest position of each row's cache (and q); a
 *    caller whose preceding kernel writes older positions, the tables or the lengths must put a stream
 *    synchronisation, an event or any ordinary launch between the two, or set MIE_B200_PDL=0.
 */
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define MIE_STATIC_MAX_PART_O (1 << 20)     /* floats: 4 MiB */
#define MIE_STATIC_MAX_PART_LSE (1 << 14)   /* floats */
#define MIE_STATIC_MAX_UNITS (1 << 12)      /* ints */
#define MIE_STATIC_SCRATCH_BYTES (4 * (MIE_STATIC_MAX_PART_O + MIE_STATIC_MAX_PART_LSE + MIE_STATIC_MAX_UNITS))

#ifdef __cplusplus
extern "C" {
#endif

/* Same arguments and result as mie_decode_attention (attention_decode.cu) without the three scratch
 * pointers: q [tokens, ...] bfloat16 with q_stride elements between tokens, caches
 * [pages, kv_heads, page_size, head_dim] bfloat16, int32 block tables and row arrays, out
 * [tokens, heads, head_dim] bfloat16.  Returns 0, a cudaError_t (> 0), or a negative refusal. */
int mie_decode_attention_static(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                                const int* block_tables, int table_stride, const int* row_q_start,
                                const int* row_q_len, const int* row_ctx_len, int num_rows, void* out,
                                int num_heads, int num_kv_heads, int head_dim, int page_size, float scale,
                                int window, int splits, cudaStream_t stream);

/* The message of the calling thread's last refusal or set-up failure ("" if none). */
const char* mie_decode_attention_static_error(void);

#ifdef __cplusplus
}
#endif

// Paged decode attention for bfloat16: one new token per request against its cached context,
// grouped by kv head and split along the context (flash-decoding), with the merge of the splits
// inside the same launch -- one kernel per layer, no second one.
//
// What the reference does in two Triton kernels (inference_engine/kernels/decode_attention.py:20-103:
// a (batch, kv head, split) grid of tl.dot programs plus a log-sum-exp merge kernel) is here one
// CUDA kernel on the warp-level tensor-core path (mma.sync m16n8k16, bfloat16 in, float32
// accumulate); the work per byte of cache is too small for anything but the memory system and the
// chain of latencies around it to matter:
//
//   grid = (splits, kv heads x head chunks, rows).  A block owns one request row, one kv head, up
//   to 16 query heads of its group (the MMA's 16 rows) and one contiguous part of the context.
//   Keys and values arrive in tiles of 64 positions, two to four stages in flight, either 16 bytes
//   per thread through cp.async into padded shared memory or a page per TMA copy into swizzled
//   shared memory (the caller's choice, see ops.decode_uses_tma); warp w multiplies positions
//   16w..16w+15 of each tile, keeping its own running max / sum / output, and the four warps are
//   merged once at the end.  Scores, softmax and accumulators are float32; P is rounded to bfloat16
//   for the P.V product, as in the reference (decode_attention.py:69).
//   The row's lengths, its page table and every cached row but the newest token's are older than
//   the step, so a block reads them and starts its copies before it waits for the kernel in front
//   of it (programmatic dependent launch), and fetches the newest row again afterwards.
//
// Merging the splits, two ways.  (1) 2, 4 or 8 splits and no scratch given: the splits of a
// (row, kv head, chunk) are launched as one thread-block cluster; every block sends its normalised
// partial outputs to the blocks that own them (each owns a share of the (head, dimension) items) and
// its base-2 log-sum-exps to all of them, straight into their shared memory; after one cluster barrier
// each owner merges what it received (weights 2^(lse_s - max), in rank order).  No global round trip,
// no atomics.  (2) Any number of splits with scratch memory: each block writes
// its partial output and log-sum-exp to the scratch and bumps a counter of its unit; the block that
// sees the count complete merges all partials and resets the counter, so the scratch needs no
// clearing between launches.  Rows with q_len != 1 are left to the prefill
// kernel (their blocks exit at once).
#include "attention_decode.cuh"

// Scratch (optional; without it splits must be 1, 2, 4 or 8): part_o float32 [rows * heads * splits * head_dim], part_lse
// float32 [rows * heads * splits], counters int32 [rows * kv_heads * chunks], the counters zero
// before the first launch (the kernel leaves them zero).  `stages`: key/value tiles in flight per
// block (2, 3 or 4; 0 = 4).  `num_pages`: pages in each cache (rows of the TMA tensor map); 0 keeps the
// cp.async copies.  `check_pages`: pages in each cache for the range check of block-table entries (0: unchecked).
// `min_part_tiles` (scratch merge): a row is cut into at most (its 64-key tiles / this) parts, so that one launch
// laid out for long contexts leaves short rows whole; 0: every row into `splits` parts.  `cos_t` / `sin_t` (float32
// [max_pos, head_dim / 2], or both null): rotate q and the new key inside this kernel and write the new key and
// value into the cache -- the q|k|v activation then comes unrotated and nothing has written the cache row of
// position ctx - 1 yet; head_dim % 32 == 0, the whole head rotates.
extern "C" int mie_decode_attention(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                                    const int* block_tables, int table_stride, const int* row_q_start,
                                    const int* row_q_len, const int* row_ctx_len, int num_rows, void* out,
                                    int num_heads, int num_kv_heads, int head_dim, int page_size, float scale,
                                    int window, int splits, float* part_o, float* part_lse, int* counters,
                                    int stages, int64_t num_pages, int64_t check_pages, int min_part_tiles,
                                    const float* cos_t, const float* sin_t, int max_pos,
                                    cudaStream_t stream) {
    return decode_attention_launch(q, q_stride, k_cache, v_cache, block_tables, table_stride, row_q_start, row_q_len,
                                   row_ctx_len, num_rows, out, num_heads, num_kv_heads, head_dim, page_size, scale,
                                   window, splits, part_o, part_lse, counters, stream, stages, num_pages, check_pages,
                                   g_range_report, min_part_tiles, cos_t, sin_t, max_pos);
}

// Non-zero when a block of any launch so far gave up a bounded wait (TMA copies that did not arrive).
extern "C" int mie_decode_attention_error(void) { return g_error_host ? *g_error_host : 0; }
extern "C" void mie_decode_attention_clear_error(void) { if (g_error_host) *g_error_host = 0; }

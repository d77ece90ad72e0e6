// Paged causal prefill attention for bfloat16: rows with two or more new tokens (prompt portions,
// fresh or continued), reading earlier positions through the block table.
//
// The reference runs a library attention per portion, on the portion's own k/v when it is the
// first one and on k/v gathered back out of the pages plus an O(n x context) boolean mask when it is
// not (inference_engine/model.py:146-158, inference_engine/engine.py:169-178).  Here one kernel
// serves both: every key, old or new, comes from the cache pages, and causality is a comparison of
// positions.
//
//   grid.x = query tiles over all rows (64 queries each, longest-running tiles first),
//   grid.y = query heads.  4 warps, 16 query rows each (mma.sync m16n8k16, bfloat16 in, float32
//   accumulate).  Keys and values come in tiles of 64 positions through cp.async, two stages.
//   S = Q K^T for the warp's 16 rows x 64 keys, masked by position (j <= p, j > p - window),
//   online softmax in base 2 with float32 max / sum, P rounded to bfloat16, O += P V.
#include "mma_common.cuh"
#include "range_check.cuh"

#define PRE_WARPS 4
#define PRE_BM 64
#define PRE_BN 64
#define PRE_MAX_D 128
#define PRE_PAGE_SLOTS 1024

struct PrefillParams {
    const bf16* q; int64_t q_stride;
    const bf16* k_cache; const bf16* v_cache;
    const int* block_tables; int table_stride;
    const int* row_q_start; const int* row_q_len; const int* row_ctx_len; int num_rows;
    bf16* out;
    int num_heads, num_kv_heads, page_size, page_shift, window, min_q_len;
    float scale_log2e;
    int64_t check_pages;     // pages in each cache, for the range check of block-table entries
    int* report;             // range report (range_check.cuh)
};

template <int D>
__global__ void __launch_bounds__(PRE_WARPS * 32)
prefill_attention_kernel(const PrefillParams p) {
    constexpr int DP = D + 8;
    constexpr int KSTEPS = D / 16, NBLK = D / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* k_s = reinterpret_cast<bf16*>(smem_raw);                 // [2][PRE_BN][DP]
    bf16* v_s = k_s + 2 * PRE_BN * DP;                             // [2][PRE_BN][DP]
    __shared__ int s_row, s_q0;
    __shared__ int s_pages[PRE_PAGE_SLOTS];                        // this block's page ids, fetched once

    pdl_launch_dependents();
    if (threadIdx.x < 32) {
        // which row and query tile (a whole warp asks: warp_find_row); tiles are numbered from the end of each row
        // backwards so that the tiles with the longest key range start first
        int tile, tiles;
        const int r = warp_find_row(p.row_q_len, p.num_rows, (int)blockIdx.x,
                                    [&](int ql) { return ql >= p.min_q_len ? (ql + PRE_BM - 1) / PRE_BM : 0; }, tile, tiles);
        if (threadIdx.x == 0) { s_row = r; s_q0 = (tiles - 1 - tile) * PRE_BM; }
    }
    __syncthreads();
    const int row = s_row;
    if (row < 0) return;
    pdl_wait();
    const int q0 = s_q0;
    const int q_len = p.row_q_len[row], ctx = p.row_ctx_len[row], q_start = p.row_q_start[row];
    const int head = blockIdx.y;
    const int kvh = head / (p.num_heads / p.num_kv_heads);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int quad = lane >> 2, tq = lane & 3;

    const int pos0 = ctx - q_len + q0;                              // position of the tile's first query
    const int nq = min(PRE_BM, q_len - q0);                         // queries in this tile
    const int k_hi = pos0 + nq;                                     // one past the last key any query reads
    const int k_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int kbeg = k_lo & ~(PRE_BN - 1);
    const int ntiles = (k_hi - kbeg + PRE_BN - 1) / PRE_BN;

    // this warp's 16 queries; thread rows r0 = quad and r1 = quad + 8
    const int wq = warp * 16;
    unsigned qf[KSTEPS][4];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = wq + quad + (i & 1) * 8, c = ks * 16 + tq * 2 + (i >> 1) * 8;
            qf[ks][i] = r < nq ? *reinterpret_cast<const unsigned*>(
                                     p.q + (int64_t)(q_start + q0 + r) * p.q_stride + (int64_t)head * D + c) : 0u;
        }
    const int qpos[2] = {pos0 + wq + quad, pos0 + wq + quad + 8};
    const bool warp_has_rows = wq < nq;

    float o[NBLK][4];
#pragma unroll
    for (int n = 0; n < NBLK; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    // page ids go to shared memory first: a look-up in global memory inside the tile loop would put a
    // memory round trip in front of every tile's copies
    const int* table = p.block_tables + (int64_t)row * p.table_stride;
    const int first_page = kbeg >> p.page_shift;
    const int n_pages = ((k_hi - 1) >> p.page_shift) - first_page + 1;
    for (int i = threadIdx.x; i < min(n_pages, PRE_PAGE_SLOTS); i += PRE_WARPS * 32)
        s_pages[i] = checked_page(table[first_page + i], p.check_pages, p.report, MIE_K_ATTENTION_PREFILL, first_page + i);
    __syncthreads();
    constexpr int CHUNKS_PER_ROW = D / 8;
    auto load_tile = [&](int t, int stage) {
        const int k0 = kbeg + t * PRE_BN;
        bf16* kd = k_s + stage * PRE_BN * DP;
        bf16* vd = v_s + stage * PRE_BN * DP;
        for (int idx = threadIdx.x; idx < PRE_BN * CHUNKS_PER_ROW; idx += PRE_WARPS * 32) {
            const int r = idx / CHUNKS_PER_ROW, c = (idx - r * CHUNKS_PER_ROW) * 8;
            const int key = k0 + r;
            if (key >= k_lo && key < k_hi) {
                const int pi = (key >> p.page_shift) - first_page;
                const int page = pi < PRE_PAGE_SLOTS ? s_pages[pi] : checked_page(table[first_page + pi], p.check_pages, p.report, MIE_K_ATTENTION_PREFILL, first_page + pi);
                const int64_t src = (((int64_t)page * p.num_kv_heads + kvh) * p.page_size + (key & (p.page_size - 1))) * D + c;
                cp_async16(kd + r * DP + c, p.k_cache + src);
                cp_async16(vd + r * DP + c, p.v_cache + src);
            } else {
                *reinterpret_cast<uint4*>(kd + r * DP + c) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(vd + r * DP + c) = make_uint4(0, 0, 0, 0);
            }
        }
    };

    load_tile(0, 0);
    cp_async_commit();
    for (int t = 0; t < ntiles; ++t) {
        const int stage = t & 1;
        if (t + 1 < ntiles) load_tile(t + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const int key0 = kbeg + t * PRE_BN;
        // a warp whose last query sits before this tile has nothing to read in it
        if (warp_has_rows && key0 <= pos0 + min(wq + 15, nq - 1)) {
            const bf16* kt = k_s + stage * PRE_BN * DP;
            const bf16* vt = v_s + stage * PRE_BN * DP;
            float s[PRE_BN / 8][4];
#pragma unroll
            for (int n = 0; n < PRE_BN / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
                for (int n2 = 0; n2 < PRE_BN / 16; ++n2) {
                    unsigned b0, b1, b2, b3;
                    ldmatrix_x4(b0, b1, b2, b3,
                                kt + (n2 * 16 + (lane & 7) + (lane >> 4) * 8) * DP + ks * 16 + ((lane >> 3) & 1) * 8);
                    mma_bf16(s[2 * n2], qf[ks], b0, b1);
                    mma_bf16(s[2 * n2 + 1], qf[ks], b2, b3);
                }
            }
            // only tiles that touch the diagonal, the window's edge or the range's start need masking
            const bool need_mask = key0 + PRE_BN - 1 > pos0 + wq || key0 < k_lo ||
                                   (p.window > 0 && key0 <= pos0 + wq + 15 - p.window);
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < PRE_BN / 8; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float v = s[n][i] * p.scale_log2e;
                    if (need_mask) {
                        const int key = key0 + n * 8 + tq * 2 + (i & 1);
                        const int qp = qpos[i >> 1];
                        const bool ok = key <= qp && (p.window <= 0 || key > qp - p.window);
                        v = ok ? v : -INFINITY;
                    }
                    s[n][i] = v;
                    mx[i >> 1] = fmaxf(mx[i >> 1], v);
                }
            float alpha[2], sum[2] = {0.f, 0.f};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                const float mn = fmaxf(m[h], mx[h]);
                alpha[h] = mn == -INFINITY ? 1.f : exp2f(m[h] - mn);
                m[h] = mn;
            }
            unsigned pf[PRE_BN / 16][4];
#pragma unroll
            for (int n = 0; n < PRE_BN / 8; ++n) {
                float pv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float mm = m[i >> 1];
                    pv[i] = mm == -INFINITY ? 0.f : exp2f(s[n][i] - mm);
                    sum[i >> 1] += pv[i];
                }
                pf[n >> 1][(n & 1) * 2] = pack_bf16(pv[0], pv[1]);
                pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(pv[2], pv[3]);
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 1);
                sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 2);
                l[h] = l[h] * alpha[h] + sum[h];
            }
#pragma unroll
            for (int n = 0; n < NBLK; ++n) {
                o[n][0] *= alpha[0]; o[n][1] *= alpha[0]; o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
            }
#pragma unroll
            for (int kk = 0; kk < PRE_BN / 16; ++kk) {
#pragma unroll
                for (int n2 = 0; n2 < NBLK / 2; ++n2) {
                    unsigned b0, b1, b2, b3;
                    ldmatrix_x4_trans(b0, b1, b2, b3,
                                      vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * DP + n2 * 16 + (lane >> 4) * 8);
                    mma_bf16(o[2 * n2], pf[kk], b0, b1);
                    mma_bf16(o[2 * n2 + 1], pf[kk], b2, b3);
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

    if (!warp_has_rows) return;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = wq + quad + h * 8;
        if (r >= nq) continue;
        const float inv = l[h] > 0.f ? 1.0f / l[h] : 0.f;
        bf16* op = p.out + ((int64_t)(q_start + q0 + r) * p.num_heads + head) * D;
#pragma unroll
        for (int n = 0; n < NBLK; ++n) {
            *reinterpret_cast<unsigned*>(op + n * 8 + tq * 2) = pack_bf16(o[n][h * 2] * inv, o[n][h * 2 + 1] * inv);
        }
    }
}

template <int D>
static int launch_prefill(const PrefillParams& p, int work_tokens, int work_rows, cudaStream_t stream) {
    const size_t smem = (size_t)2 * 2 * PRE_BN * (D + 8) * sizeof(bf16);
    cudaError_t e = cudaFuncSetAttribute(prefill_attention_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const dim3 grid((work_tokens + PRE_BM - 1) / PRE_BM + work_rows, p.num_heads);     // tiles <= tokens / 64 + rows
    return launch_kernel(prefill_attention_kernel<D>, grid, dim3(PRE_WARPS * 32), smem, stream, p);
}

// Rows with fewer than `min_q_len` new tokens are skipped (the decode kernel serves single tokens).  work_rows /
// work_tokens: how many rows have min_q_len tokens or more, and their tokens in sum, where the caller knows (the grid
// is laid out for the tiles they can have); 0: every row may, num_rows / num_tokens.
extern "C" int mie_prefill_attention(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                                     const int* block_tables, int table_stride, const int* row_q_start,
                                     const int* row_q_len, const int* row_ctx_len, int num_rows, int num_tokens,
                                     void* out, int num_heads, int num_kv_heads, int head_dim, int page_size,
                                     float scale, int window, int min_q_len, long long num_pages, int work_rows,
                                     int work_tokens, cudaStream_t stream) {
    if (num_rows <= 0 || num_tokens <= 0) return 0;
    if (work_rows <= 0 || work_tokens <= 0 || work_rows > num_rows || work_tokens > num_tokens) { work_rows = num_rows; work_tokens = num_tokens; }
    if (head_dim < 16 || head_dim > PRE_MAX_D || head_dim % 16) return MIE_ERR_BAD_ARG;
    if (num_kv_heads <= 0 || num_heads % num_kv_heads || num_heads > 65535) return MIE_ERR_BAD_ARG;
    if (page_size < 1 || (page_size & (page_size - 1))) return MIE_ERR_BAD_ARG;
    PrefillParams p;
    p.q = (const bf16*)q; p.q_stride = q_stride;
    p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
    p.block_tables = block_tables; p.table_stride = table_stride;
    p.row_q_start = row_q_start; p.row_q_len = row_q_len; p.row_ctx_len = row_ctx_len; p.num_rows = num_rows;
    p.out = (bf16*)out;
    p.num_heads = num_heads; p.num_kv_heads = num_kv_heads; p.page_size = page_size;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.window = window; p.min_q_len = min_q_len;
    p.scale_log2e = scale * 1.4426950408889634f;
    p.check_pages = num_pages > 0 ? (int64_t)num_pages : ((int64_t)1 << 40); p.report = g_range_report;
    switch (head_dim) {
        case 16: return launch_prefill<16>(p, work_tokens, work_rows, stream);
        case 32: return launch_prefill<32>(p, work_tokens, work_rows, stream);
        case 48: return launch_prefill<48>(p, work_tokens, work_rows, stream);
        case 64: return launch_prefill<64>(p, work_tokens, work_rows, stream);
        case 80: return launch_prefill<80>(p, work_tokens, work_rows, stream);
        case 96: return launch_prefill<96>(p, work_tokens, work_rows, stream);
        case 112: return launch_prefill<112>(p, work_tokens, work_rows, stream);
        case 128: return launch_prefill<128>(p, work_tokens, work_rows, stream);
    }
    return MIE_ERR_BAD_ARG;
}

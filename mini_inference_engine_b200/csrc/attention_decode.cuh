// The decode attention kernel, its parameter block and its launch by head size, shared by the two
// entry points that differ only in where the scratch memory comes from (attention_decode.cu: the
// caller's; attention_decode_static.cu: a fixed array inside the library).
#pragma once
#include "mma_common.cuh"
#include "tcgen05_common.cuh"      // mbarrier, TMA copies, bounded waits, the tensor-map encoder
#include "range_check.cuh"
#include "rope_math.cuh"

#define DEC_WARPS 4
#define DEC_TILE 64
#define DEC_MAX_D 128
#define DEC_PAGE_SLOTS 1024

struct DecodeParams {
    const bf16* q; int64_t q_stride;
    const bf16* k_cache; const bf16* v_cache;
    const int* block_tables; int table_stride;
    const int* row_q_start; const int* row_q_len; const int* row_ctx_len;
    bf16* out;
    float* part_o; float* part_lse; int* counters;      // scratch (splits > 1)
    int num_heads, num_kv_heads, page_size, page_shift, window, splits, chunks;
    int stages;              // tiles in flight per block (2, 3 or 4)
    int min_part_tiles;      // scratch merge: a row is cut into no more parts than it has this many tiles for (0: always `splits`)
    int cluster;             // 1: the splits of a (row, kv head, chunk) are a thread-block cluster and merge through shared memory
    float scale_log2e;
    int* error;              // host-visible error word (TMA path: a bounded wait that ran out)
    uint32_t recv_offset;    // where the cluster merge's receive slots start in dynamic shared memory
    int64_t check_pages;     // pages in each cache, for the range check of block-table entries (0: unchecked)
    int* report;             // range report (range_check.cuh); null: nowhere
    // Rotation inside this kernel (null: q and the newest key arrive rotated, and the newest cache row is written):
    // q, the new key and the new value are read UNROTATED from the row's q|k|v activation (q_stride wide: the new
    // key head kvh sits (num_heads + kvh) heads in, the value num_kv_heads heads further), q and the key are
    // rotated by the token's position ctx - 1 with the whole head as rotary width (D % 32 == 0), and the block
    // whose part holds that position writes key and value into the cache (the block of the first chunk of heads).
    const float* cos_t; const float* sin_t; int max_pos;
};

// Where the 16-byte piece `chunk` of key row `row` lies inside a tile that TMA wrote with the
// 128-byte swizzle: rows of 64 elements (128 bytes), 64 rows (8 KB) per 64-column part of the head,
// the piece index XORed with the row's place in its group of eight.
// 2^x by the hardware approximation (two ulp; -inf gives 0): the library call costs several
// instructions where one does, in loops that issue instructions most of the time.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t swz_tile_off(int row, int chunk) {
    return (uint32_t)((chunk >> 3) * 8192 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}


// TMA = true (head sizes 64 and 128, pages of at least 8 positions): keys and values arrive a page per
// copy (cp.async.bulk.tensor through the block table, 128-byte swizzle, an mbarrier per stage) instead of
// 16 bytes per thread per cp.async: a thousand address computations a tile less, and the copies of a
// tile are in flight from one instruction each.  Measured on B200 (32 q / 4 kv heads of 64): with more
// blocks than fit beside one another it is the faster way (128 requests x 512 keys 20.6 -> 14.9 us,
// 256 x 512 34.4 -> 29.2 us, 256 x 2048 101 -> 96 us = 5.6 TB/s); where a block walks a long part
// alone it is not (64 x 2048: 40.0 -> 42.9 us), so the caller chooses (ops.decode_uses_tma).
template <int D, int NSTAGE, bool TMA>
__global__ void __launch_bounds__(DEC_WARPS * 32)
decode_attention_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const DecodeParams p) {
    constexpr int DP = D + 8;                    // padded row: ldmatrix rows fall into different banks
    constexpr int KSTEPS = D / 16, NBLK = D / 8;
    constexpr int PARTS = (D + 63) / 64;                           // 64-column parts of a head (TMA layout)
    constexpr uint32_t KV_TILE_BYTES = PARTS * 8192;               // one tile of keys (or values) as TMA lays it out
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* k_s = reinterpret_cast<bf16*>(smem_raw);                 // [NSTAGE][DEC_TILE][DP]
    bf16* v_s = k_s + NSTAGE * DEC_TILE * DP;                      // [NSTAGE][DEC_TILE][DP]
    // TMA layout: swizzled tiles on 1024-byte lines: stage s = keys | values, 2 * KV_TILE_BYTES each
    const uint32_t tma_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* tma_tiles = smem_raw + (tma_base - smem_u32(smem_raw));
    __shared__ __align__(8) uint64_t full_bar[4];
    __shared__ int abort_flag;
    // cluster merge: what the other splits send this block (its share of the outputs, and every split's
    // log-sum-exp), one slot per sender.  Behind the tiles in dynamic shared memory, and only there when the
    // launch is a cluster: without splits these 5 KB would cost the fourth block on an SM.
    float4* recv_o = reinterpret_cast<float4*>(smem_raw + p.recv_offset);               // [16 * (D / 4) + 8]
    float (*recv_lse)[16] = reinterpret_cast<float (*)[16]>(recv_o + 16 * (D / 4) + 8); // [8][16]
    __shared__ float m_s[DEC_WARPS][16], l_s[DEC_WARPS][16];
    __shared__ __align__(16) float c_lse[16];
    __shared__ int s_pages[DEC_PAGE_SLOTS];                        // this block's page ids, fetched once
    __shared__ int s_last;

    // The row's lengths, its page table and every cached key and value except the newest token's are
    // older than this step: nothing the kernel before this one writes.  So the block reads them and
    // starts its first copies before it waits for that kernel, and fetches the newest token's key and
    // value (and the queries) afterwards.
    pdl_launch_dependents();
    const int row = blockIdx.z;
    if (p.row_q_len[row] != 1) {                                   // another kernel's row
        pdl_wait();                                                // no block ends before the kernel in front has: later kernels rely on it
        return;
    }
    if (p.cluster) cluster_arrive_relaxed();                       // see the merge: a block is written to only once it runs
    const int G = p.num_heads / p.num_kv_heads;
    const int kvh = blockIdx.y / p.chunks, chunk = blockIdx.y - kvh * p.chunks;
    const int g0 = chunk * 16, gn = min(16, G - g0);               // query heads of this block within the group
    const int split = blockIdx.x;
    const int ctx = p.row_ctx_len[row];
    const int token = p.row_q_start[row];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int quad = lane >> 2, tq = lane & 3;

    // this block's part of the context: the range [lo, ctx) cut into `splits` parts of whole tiles
    const int lo = p.window > 0 ? (max(0, ctx - p.window) & ~(DEC_TILE - 1)) : 0;
    const int first_key = p.window > 0 ? max(0, ctx - p.window) : 0;
    const int tiles_total = (ctx - lo + DEC_TILE - 1) / DEC_TILE;
    // The grid is laid out for the longest context the launch may meet; a row is cut into as many parts as
    // its own length pays for (scratch merge only: the blocks of a cluster all take part in its barriers).
    // The parts beyond that leave at once, and a row that stays whole writes its output directly.
    const int eff = (!p.cluster && p.min_part_tiles > 0) ? min(p.splits, max(1, tiles_total / p.min_part_tiles)) : p.splits;
    if (split >= eff) {
        pdl_wait();
        return;
    }
    // tiles go round evenly: every part gets tiles_total / eff of them and the first (tiles_total % eff) parts one
    // more, so that no part waits at the merge for one that walked twice as many as it needed to
    const int tiles_base = tiles_total / eff, tiles_more = tiles_total - tiles_base * eff;
    const int tiles_mine = tiles_base + (split < tiles_more ? 1 : 0);
    const int kbeg = lo + (split * tiles_base + min(split, tiles_more)) * DEC_TILE;
    const int kend = min(ctx, kbeg + tiles_mine * DEC_TILE);
    const int ntiles = kend > kbeg ? (kend - kbeg + DEC_TILE - 1) / DEC_TILE : 0;

    float o[NBLK][4];
#pragma unroll
    for (int n = 0; n < NBLK; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    volatile int* abort_p = &abort_flag;
    if (TMA) {
        if (threadIdx.x == 0) {
            abort_flag = 0;
            for (int s = 0; s < NSTAGE; ++s) mbar_init(&full_bar[s], 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        // A copy brings whole pages; rows of a tile that no page of this part covers keep what the shared
        // memory held.  Their scores are masked, but 0 * NaN is NaN: they must be finite.
        if ((kend - kbeg) & (DEC_TILE - 1))
            for (uint32_t i = threadIdx.x * 16; i < (uint32_t)NSTAGE * 2 * KV_TILE_BYTES; i += DEC_WARPS * 32 * 16)
                *reinterpret_cast<uint4*>(tma_tiles + i) = make_uint4(0, 0, 0, 0);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // barriers and zeros before the TMA unit touches them
    }

    // The page ids of this block's part go to shared memory first: a lookup in global memory inside the
    // tile loop would put a memory round trip in front of every tile's copies.
    const int* table = p.block_tables + (int64_t)row * p.table_stride;
    const int first_page = kbeg >> p.page_shift;
    const int n_pages = ntiles > 0 ? ((kend - 1) >> p.page_shift) - first_page + 1 : 0;
    const int64_t page_limit = p.check_pages > 0 ? p.check_pages : ((int64_t)1 << 40);
    for (int i = threadIdx.x; i < min(n_pages, DEC_PAGE_SLOTS); i += DEC_WARPS * 32)
        s_pages[i] = checked_page(table[first_page + i], page_limit, p.report, MIE_K_ATTENTION_DECODE, first_page + i);
    __syncthreads();
    constexpr int CHUNKS_PER_ROW = D / 8;                          // 16-byte pieces per key
    const int rows_per_copy = min(p.page_size, DEC_TILE);          // TMA: one copy = one page (or a 64-row piece of it)
    auto load_tile = [&](int t, int stage) {
        const int k0 = kbeg + t * DEC_TILE;
        if (TMA) {
            if (warp == 0) {                                       // lane c copies page c of the tile, keys and values
                const int copies = (min(DEC_TILE, kend - k0) + rows_per_copy - 1) / rows_per_copy;
                if (lane == 0) mbar_expect_tx(&full_bar[stage], (uint32_t)copies * rows_per_copy * 128u * PARTS * 2u);
                __syncwarp();
                if (lane < copies) {
                    const int key = k0 + lane * rows_per_copy;
                    const int pi = (key >> p.page_shift) - first_page;
                    const int page = pi < DEC_PAGE_SLOTS ? s_pages[pi] : checked_page(table[first_page + pi], page_limit, p.report, MIE_K_ATTENTION_DECODE, first_page + pi);
                    const int src_row = (page * p.num_kv_heads + kvh) * p.page_size + (key & (p.page_size - 1));
                    unsigned char* kd = tma_tiles + (size_t)stage * 2 * KV_TILE_BYTES + (size_t)lane * rows_per_copy * 128;
#pragma unroll
                    for (int part = 0; part < PARTS; ++part) {
                        tma_load_2d(kd + part * 8192, &map_k, &full_bar[stage], part * 64, src_row);
                        tma_load_2d(kd + KV_TILE_BYTES + part * 8192, &map_v, &full_bar[stage], part * 64, src_row);
                    }
                }
            }
            return;
        }
        bf16* kd = k_s + stage * DEC_TILE * DP;
        bf16* vd = v_s + stage * DEC_TILE * DP;
        for (int idx = threadIdx.x; idx < DEC_TILE * CHUNKS_PER_ROW; idx += DEC_WARPS * 32) {
            const int r = idx / CHUNKS_PER_ROW, c = (idx - r * CHUNKS_PER_ROW) * 8;
            const int key = k0 + r;
            if (key < kend) {
                const int pi = (key >> p.page_shift) - first_page;
                const int page = pi < DEC_PAGE_SLOTS ? s_pages[pi] : checked_page(table[first_page + pi], page_limit, p.report, MIE_K_ATTENTION_DECODE, first_page + pi);
                const int64_t src = (((int64_t)page * p.num_kv_heads + kvh) * p.page_size + (key & (p.page_size - 1))) * D + c;
                cp_async16(kd + r * DP + c, p.k_cache + src);
                cp_async16(vd + r * DP + c, p.v_cache + src);
            } else {                                               // beyond the part: zeros, so that 0 * v stays 0
                *reinterpret_cast<uint4*>(kd + r * DP + c) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(vd + r * DP + c) = make_uint4(0, 0, 0, 0);
            }
        }
    };

#pragma unroll
    for (int t = 0; t < NSTAGE - 1; ++t) {
        if (t < ntiles) load_tile(t, t);
        cp_async_commit();
    }
    pdl_wait();                                                    // q and the newest key and value are the previous kernel's
    const int newest = ctx - 1;                                    // the only cached position written during this step
    if (p.cos_t && range_position(newest, p.max_pos) != MIE_RANGE_OK) {   // no row of the tables for this position
        // reported; the block goes on without rotating (it takes part in the merge's barriers and counters)
        if (threadIdx.x == 0 && split == 0 && blockIdx.y == 0) range_report(p.report, MIE_RANGE_POSITION, MIE_K_ATTENTION_DECODE, row, newest);
    }
    const bool rotate = p.cos_t && range_position(newest, p.max_pos) == MIE_RANGE_OK;
    // Q fragments (A operand), rows = query heads of the group, zero beyond gn
    unsigned qf[KSTEPS][4];
    {
        const bf16* qb = p.q + (int64_t)token * p.q_stride + (int64_t)(kvh * G + g0) * D;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = quad + (i & 1) * 8, c = ks * 16 + tq * 2 + (i >> 1) * 8;
                qf[ks][i] = r < gn ? *reinterpret_cast<const unsigned*>(qb + (int64_t)r * D + c) : 0u;
            }
        }
        if constexpr (KSTEPS % 2 == 0) {
            if (rotate) {
                // a thread holds dimension c of a head in k-step ks and its partner c + D / 2 in k-step ks + KSTEPS / 2
                const float* cs = p.cos_t + (int64_t)newest * (D / 2);
                const float* sn = p.sin_t + (int64_t)newest * (D / 2);
#pragma unroll
                for (int ks = 0; ks < KSTEPS / 2; ++ks) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int c = ks * 16 + tq * 2 + (i >> 1) * 8;
                        const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qf[ks][i]));
                        const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qf[ks + KSTEPS / 2][i]));
                        const float c0 = cs[c], c1 = cs[c + 1], s0 = sn[c], s1 = sn[c + 1];
                        const __nv_bfloat162 lo = __floats2bfloat162_rn(x.x * c0 - y.x * s0, x.y * c1 - y.y * s1);
                        const __nv_bfloat162 hi = __floats2bfloat162_rn(y.x * c0 + x.x * s0, y.y * c1 + x.y * s1);
                        qf[ks][i] = *reinterpret_cast<const unsigned*>(&lo);
                        qf[ks + KSTEPS / 2][i] = *reinterpret_cast<const unsigned*>(&hi);
                    }
                }
            }
        }
    }

    for (int t = 0; t < ntiles; ++t) {
        const int stage = t % NSTAGE;
        if (t + NSTAGE - 1 < ntiles) load_tile(t + NSTAGE - 1, (t + NSTAGE - 1) % NSTAGE);
        if (TMA) {
            // bounded; every thread sees the bytes itself, and the block goes on or gives up as one
            if (!__syncthreads_and(mbar_wait(&full_bar[stage], (t / NSTAGE) & 1, abort_p))) break;
        } else {
            cp_async_commit();
            cp_async_wait<NSTAGE - 1>();                           // tile t has landed; NSTAGE - 1 younger ones may be in flight
            __syncthreads();
        }
        if ((rotate || t < NSTAGE - 1) && newest >= kbeg + t * DEC_TILE && newest < min(kend, kbeg + (t + 1) * DEC_TILE)) {
            // The newest row.  Without rotation here: the tile was copied before the wait and the row may be stale, so it
            // is fetched again (L2, not L1).  With rotation here: the cache does not hold it yet -- this block makes it
            // from the row's q|k|v activation, uses it and writes it into the cache.
            if (threadIdx.x < 2 * CHUNKS_PER_ROW) {
                const int which = threadIdx.x / CHUNKS_PER_ROW, c = (threadIdx.x - which * CHUNKS_PER_ROW) * 8;
                const int r = newest - (kbeg + t * DEC_TILE);
                const int pi = (newest >> p.page_shift) - first_page;
                const int page = pi < DEC_PAGE_SLOTS ? s_pages[pi] : checked_page(table[first_page + pi], page_limit, p.report, MIE_K_ATTENTION_DECODE, first_page + pi);
                const int64_t src = (((int64_t)page * p.num_kv_heads + kvh) * p.page_size + (newest & (p.page_size - 1))) * D + c;
                uint4 v;
                if (rotate) {
                    const bf16* act = p.q + (int64_t)token * p.q_stride + (int64_t)(p.num_heads + (which ? p.num_kv_heads : 0) + kvh) * D;
                    if (which) {
                        v = *reinterpret_cast<const uint4*>(act + c);
                    } else {
                        const int j = c < D / 2 ? c : c - D / 2;           // the pair's index: both halves of it are needed
                        uint4 lo = *reinterpret_cast<const uint4*>(act + j), hi = *reinterpret_cast<const uint4*>(act + j + D / 2), olo, ohi;
                        rotate8(lo, hi, p.cos_t + (int64_t)newest * (D / 2) + j, p.sin_t + (int64_t)newest * (D / 2) + j, olo, ohi);
                        v = c < D / 2 ? olo : ohi;
                    }
                    if (chunk == 0) *reinterpret_cast<uint4*>(const_cast<bf16*>(which ? p.v_cache : p.k_cache) + src) = v;
                } else {
                    v = __ldcg(reinterpret_cast<const uint4*>((which ? p.v_cache : p.k_cache) + src));
                }
                if (TMA) *reinterpret_cast<uint4*>(tma_tiles + (size_t)stage * 2 * KV_TILE_BYTES + which * KV_TILE_BYTES + swz_tile_off(r, c / 8)) = v;
                else *reinterpret_cast<uint4*>((which ? v_s : k_s) + stage * DEC_TILE * DP + r * DP + c) = v;
            }
            __syncthreads();
        }
        const bf16* kt = k_s + stage * DEC_TILE * DP + warp * 16 * DP;
        const bf16* vt = v_s + stage * DEC_TILE * DP + warp * 16 * DP;
        const unsigned char* kt_tma = tma_tiles + (size_t)stage * 2 * KV_TILE_BYTES;   // keys of the stage; values KV_TILE_BYTES behind
        const int key0 = kbeg + t * DEC_TILE + warp * 16;
        if (key0 < kend) {                                          // warp-uniform
            float s[2][4];
#pragma unroll
            for (int n = 0; n < 2; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                unsigned b0, b1, b2, b3;
                if (TMA) ldmatrix_x4(b0, b1, b2, b3, reinterpret_cast<const bf16*>(
                             kt_tma + swz_tile_off(warp * 16 + (lane & 7) + (lane >> 4) * 8, ks * 2 + ((lane >> 3) & 1))));
                else ldmatrix_x4(b0, b1, b2, b3, kt + ((lane & 7) + (lane >> 4) * 8) * DP + ks * 16 + ((lane >> 3) & 1) * 8);
                mma_bf16(s[0], qf[ks], b0, b1);
                mma_bf16(s[1], qf[ks], b2, b3);
            }
            // mask, scale to base 2, running max
            float mx[2] = {-INFINITY, -INFINITY};
            const bool whole = key0 + 16 <= kend && key0 >= first_key;   // no key of the warp's 16 needs a mask (warp-uniform)
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float v = s[n][i] * p.scale_log2e;
                    if (!whole) {
                        const int key = key0 + n * 8 + tq * 2 + (i & 1);
                        if (!(key < kend && key >= first_key)) v = -INFINITY;
                    }
                    s[n][i] = v;
                    mx[i >> 1] = fmaxf(mx[i >> 1], v);
                }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            }
            float alpha[2], sum[2] = {0.f, 0.f};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float mn = fmaxf(m[h], mx[h]);
                alpha[h] = mn == -INFINITY ? 1.f : fast_exp2(m[h] - mn);
                m[h] = mn;
            }
            unsigned pf[4];
            {
                float pv[2][4];
#pragma unroll
                for (int n = 0; n < 2; ++n)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float mm = m[i >> 1];
                        pv[n][i] = mm == -INFINITY ? 0.f : fast_exp2(s[n][i] - mm);
                        sum[i >> 1] += pv[n][i];
                    }
                pf[0] = pack_bf16(pv[0][0], pv[0][1]);
                pf[1] = pack_bf16(pv[0][2], pv[0][3]);
                pf[2] = pack_bf16(pv[1][0], pv[1][1]);
                pf[3] = pack_bf16(pv[1][2], pv[1][3]);
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
            for (int n2 = 0; n2 < NBLK / 2; ++n2) {
                unsigned b0, b1, b2, b3;
                if (TMA) ldmatrix_x4_trans(b0, b1, b2, b3, reinterpret_cast<const bf16*>(
                             kt_tma + KV_TILE_BYTES + swz_tile_off(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, n2 * 2 + (lane >> 4))));
                else ldmatrix_x4_trans(b0, b1, b2, b3, vt + ((lane & 7) + ((lane >> 3) & 1) * 8) * DP + n2 * 16 + (lane >> 4) * 8);
                mma_bf16(o[2 * n2], pf, b0, b1);
                mma_bf16(o[2 * n2 + 1], pf, b2, b3);
            }
        }
        __syncthreads();                                           // the stage may be overwritten next round
    }
    cp_async_wait<0>();
    __syncthreads();
    if (TMA && abort_flag) {                                       // a wait ran out: say so, let copies in flight land
        if (threadIdx.x == 0) atomicExch(p.error, 1);
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
        __syncthreads();
    }

    // merge the four warps: each leaves (m, l, O) in shared memory (the tile buffers are free now)
    float* o_s = reinterpret_cast<float*>(smem_raw);               // [DEC_WARPS][16][D]
    if (tq == 0) { m_s[warp][quad] = m[0]; m_s[warp][quad + 8] = m[1]; l_s[warp][quad] = l[0]; l_s[warp][quad + 8] = l[1]; }
#pragma unroll
    for (int n = 0; n < NBLK; ++n) {
        const int c = n * 8 + tq * 2;
        *reinterpret_cast<float2*>(o_s + (warp * 16 + quad) * D + c) = make_float2(o[n][0], o[n][1]);
        *reinterpret_cast<float2*>(o_s + (warp * 16 + quad + 8) * D + c) = make_float2(o[n][2], o[n][3]);
    }
    __syncthreads();
    const int unit = (row * p.num_kv_heads + kvh) * p.chunks + chunk;
    // The weight of warp w's partial output for head g, 2^(m_w - max) / sum, is the same for all D
    // dimensions: 16 x DEC_WARPS threads work it out once, the element loop below is four multiply-adds.
    __shared__ float f_s[DEC_WARPS][16];
    if (threadIdx.x < 16) {
        const int g = threadIdx.x;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, m_s[w][g]);
        float f[DEC_WARPS], ll = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            f[w] = (mm == -INFINITY || m_s[w][g] == -INFINITY) ? 0.f : fast_exp2(m_s[w][g] - mm);
            ll += f[w] * l_s[w][g];
        }
        const float inv = ll > 0.f ? __frcp_rn(ll) : 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) f_s[w][g] = f[w] * inv;
        c_lse[g] = ll > 0.f ? mm + __log2f(ll) : -INFINITY;           // base-2 log-sum-exp of this block's part
    }
    // Merging the splits inside a cluster: (head, four dimensions) items go round the blocks, item i to
    // block i % S.  Every block sends its normalised partial of an item straight to the item's owner
    // (st.shared::cluster, a slot per sender) and its log-sum-exps to everybody; one cluster barrier; the
    // owner weighs the S partials by 2^(lse_s - max) out of its own shared memory and writes the result.
    const int S = p.splits, items_per_owner = (16 * (D / 4) + S - 1) / S;
    const uint32_t recv_o_addr = (uint32_t)__cvta_generic_to_shared(recv_o);
    if (p.cluster) {
        cluster_wait();                                            // every block of the cluster runs
        if (threadIdx.x < 16) {
            const float v = c_lse[threadIdx.x];
            const uint32_t at = (uint32_t)__cvta_generic_to_shared(&recv_lse[split][threadIdx.x]);
#pragma unroll
            for (int s2 = 0; s2 < 8; ++s2) if (s2 < S) st_cluster_f32(cluster_addr(at, s2), v);
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < gn * (D / 4); idx += DEC_WARPS * 32) {      // one thread: one head, four dimensions
        const int g = idx / (D / 4), d = (idx - g * (D / 4)) * 4;
        float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float f = f_s[w][g];
            const float4 v = *reinterpret_cast<const float4*>(o_s + (w * 16 + g) * D + d);
            val.x += f * v.x; val.y += f * v.y; val.z += f * v.z; val.w += f * v.w;
        }
        const int head = kvh * G + g0 + g;
        if (eff == 1) {
            uint2 packed;
            packed.x = pack_bf16(val.x, val.y);
            packed.y = pack_bf16(val.z, val.w);
            *reinterpret_cast<uint2*>(p.out + ((int64_t)token * p.num_heads + head) * D + d) = packed;
        } else if (p.cluster) {
            const int owner = idx & (S - 1), li = idx >> (31 - __clz(S));            // S is 2, 4 or 8
            st_cluster_f32x4(cluster_addr(recv_o_addr, owner) + (uint32_t)(split * items_per_owner + li) * 16u, val.x, val.y, val.z, val.w);
        } else {
            const int64_t slot = ((int64_t)row * p.num_heads + head) * p.splits + split;
            *reinterpret_cast<float4*>(p.part_o + slot * D + d) = val;
            if (d == 0) p.part_lse[slot] = c_lse[g];
        }
    }
    if (eff == 1) return;

    if (p.cluster) {
        cluster_sync_all();                                        // every partial and log-sum-exp has arrived
        // one thread: one head, four consecutive dimensions, the S partials in rank order
        for (int li = threadIdx.x; li * S + split < gn * (D / 4); li += DEC_WARPS * 32) {
            const int item = li * S + split;
            const int g = item / (D / 4), d4 = (item - g * (D / 4)) * 4;
            float mm = -INFINITY;
#pragma unroll
            for (int s2 = 0; s2 < 8; ++s2) if (s2 < S) mm = fmaxf(mm, recv_lse[s2][g]);
            float acc[4] = {0.f, 0.f, 0.f, 0.f}, wsum = 0.f;
#pragma unroll
            for (int s2 = 0; s2 < 8; ++s2) {
                if (s2 < S) {
                    const float lse = recv_lse[s2][g];
                    const float w = lse == -INFINITY ? 0.f : fast_exp2(lse - mm);
                    const float4 part = recv_o[s2 * items_per_owner + li];
                    acc[0] += w * part.x; acc[1] += w * part.y; acc[2] += w * part.z; acc[3] += w * part.w;
                    wsum += w;
                }
            }
            const float inv = wsum > 0.f ? __frcp_rn(wsum) : 0.f;
            const int head = kvh * G + g0 + g;
            uint2 packed;
            packed.x = pack_bf16(acc[0] * inv, acc[1] * inv);
            packed.y = pack_bf16(acc[2] * inv, acc[3] * inv);
            *reinterpret_cast<uint2*>(p.out + ((int64_t)token * p.num_heads + head) * D + d4) = packed;
        }
        return;                                                    // nobody reads this block's memory any more
    }

    // the last block of this (row, kv head, chunk) merges the splits
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int done = atomicAdd(p.counters + unit, 1);
        s_last = done == eff - 1;
        if (s_last) p.counters[unit] = 0;                          // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int idx = threadIdx.x; idx < gn * D; idx += DEC_WARPS * 32) {
        const int g = idx / D, d = idx - g * D;
        const int head = kvh * G + g0 + g;
        const int64_t base = ((int64_t)row * p.num_heads + head) * p.splits;
        float mm = -INFINITY;
        for (int s2 = 0; s2 < eff; ++s2) mm = fmaxf(mm, __ldcg(p.part_lse + base + s2));
        float acc = 0.f, wsum = 0.f;
        for (int s2 = 0; s2 < eff; ++s2) {
            const float lse = __ldcg(p.part_lse + base + s2);
            if (lse == -INFINITY) continue;
            const float w = fast_exp2(lse - mm);
            acc += w * __ldcg(p.part_o + (base + s2) * D + d);
            wsum += w;
        }
        p.out[((int64_t)token * p.num_heads + head) * D + d] = __float2bfloat16_rn(wsum > 0.f ? acc / wsum : 0.f);
    }
}

// The caches as a 2-D tensor map for the TMA path: rows = (page, kv head, slot), columns = head_dim,
// boxes of {64 columns, box_rows} with the 128-byte swizzle.
struct DecodeMaps { CUtensorMap k, v; bool use; };

static int make_decode_map(CUtensorMap* map, const void* ptr, uint64_t rows, int head_dim, int box_rows) {
    cuuint64_t gdim[2] = {(cuuint64_t)head_dim, rows};
    cuuint64_t gstride[1] = {(cuuint64_t)head_dim * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

template <int D, int NSTAGE, bool TMA>
static int launch_decode_stages(const DecodeParams& p, const DecodeMaps& maps, int num_rows, cudaStream_t stream) {
    // at least the four-warp merge buffer (4 x 16 x D float32) must fit
    size_t smem = TMA ? (size_t)NSTAGE * 2 * ((D + 63) / 64) * 8192 + 1024 : (size_t)NSTAGE * 2 * DEC_TILE * (D + 8) * sizeof(bf16);
    const size_t merge = (size_t)DEC_WARPS * 16 * D * sizeof(float);
    if (smem < merge) smem = merge;
    DecodeParams pp = p;
    pp.recv_offset = (uint32_t)((smem + 15) & ~size_t(15));
    if (p.cluster) smem = pp.recv_offset + (16 * (D / 4) + 8) * sizeof(float4) + 8 * 16 * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel<D, NSTAGE, TMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const dim3 grid(p.splits, p.num_kv_heads * p.chunks, num_rows);
    const dim3 cluster(p.cluster ? p.splits : 1, 1, 1);
    return launch_kernel_cluster(decode_attention_kernel<D, NSTAGE, TMA>, grid, dim3(DEC_WARPS * 32), smem, stream, cluster,
                                 maps.k, maps.v, pp);
}

// Tiles in flight per block.  Few tiles per block (short contexts, many splits): two stages, so that
// more blocks share an SM and hide one another's latencies.  Many tiles per block: a deeper ring.
template <int D, bool TMA>
static int launch_decode_tma(const DecodeParams& p, const DecodeMaps& maps, int num_rows, cudaStream_t stream) {
    if (p.stages <= 2) return launch_decode_stages<D, 2, TMA>(p, maps, num_rows, stream);
    if (p.stages == 3 || D > 64) return launch_decode_stages<D, 3, TMA>(p, maps, num_rows, stream);
    return launch_decode_stages<D, 4, TMA>(p, maps, num_rows, stream);
}

template <int D>
static int launch_decode(const DecodeParams& p, const DecodeMaps& maps, int num_rows, cudaStream_t stream) {
    if constexpr (D == 64 || D == 128) {
        if (maps.use) return launch_decode_tma<D, true>(p, maps, num_rows, stream);
    }
    return launch_decode_tma<D, false>(p, maps, num_rows, stream);
}


// Checks the sizes, fills the parameter block and launches.  With splits > 1 and all three scratch
// pointers null, the splits (2, 4 or 8) form a thread-block cluster and merge through distributed
// shared memory; with scratch given, any number of splits merges through it.
static int decode_attention_launch(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                                   const int* block_tables, int table_stride, const int* row_q_start,
                                   const int* row_q_len, const int* row_ctx_len, int num_rows, void* out,
                                   int num_heads, int num_kv_heads, int head_dim, int page_size, float scale,
                                   int window, int splits, float* part_o, float* part_lse, int* counters,
                                   cudaStream_t stream, int stages = 0, int64_t num_pages = 0,
                                   int64_t check_pages = 0, int* report = nullptr, int min_part_tiles = 0,
                                   const float* cos_t = nullptr, const float* sin_t = nullptr, int max_pos = 0) {
    if (num_rows <= 0) return 0;
    if (head_dim < 16 || head_dim > DEC_MAX_D || head_dim % 16) return MIE_ERR_BAD_ARG;
    if (num_kv_heads <= 0 || num_heads % num_kv_heads) return MIE_ERR_BAD_ARG;
    if (page_size < 1 || (page_size & (page_size - 1))) return MIE_ERR_BAD_ARG;
    const bool cluster = splits > 1 && !part_o && !part_lse && !counters;     // no scratch given: merge inside a cluster
    if (splits < 1 || (splits > 1 && !cluster && (!part_o || !part_lse || !counters))) return MIE_ERR_BAD_ARG;
    if (cluster && splits != 2 && splits != 4 && splits != 8) return MIE_ERR_BAD_ARG;
    if (num_rows > 65535) return MIE_ERR_TOO_LARGE;
    DecodeParams p;
    p.q = (const bf16*)q; p.q_stride = q_stride;
    p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
    p.block_tables = block_tables; p.table_stride = table_stride;
    p.row_q_start = row_q_start; p.row_q_len = row_q_len; p.row_ctx_len = row_ctx_len;
    p.out = (bf16*)out; p.part_o = part_o; p.part_lse = part_lse; p.counters = counters;
    p.num_heads = num_heads; p.num_kv_heads = num_kv_heads; p.page_size = page_size;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.window = window; p.splits = splits; p.cluster = cluster ? 1 : 0;
    p.stages = stages > 0 ? stages : 4;
    p.min_part_tiles = min_part_tiles > 0 ? min_part_tiles : 0;
    const int G = num_heads / num_kv_heads;
    p.chunks = (G + 15) / 16;
    p.scale_log2e = scale * 1.4426950408889634f;
    p.check_pages = check_pages; p.report = report;
    if ((cos_t != nullptr) != (sin_t != nullptr) || (cos_t && (head_dim % 32 || max_pos <= 0))) return MIE_ERR_BAD_ARG;
    p.cos_t = cos_t; p.sin_t = sin_t; p.max_pos = max_pos;
    // TMA copies (see the kernel): head sizes 64 and 128, pages of 8 positions or more, a caller that says
    // how many pages the caches hold (num_pages; the entry point that must not allocate passes 0)
    DecodeMaps maps;
    maps.use = num_pages > 0 && (head_dim == 64 || head_dim == 128) && page_size >= 8 &&
               !((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15);
    p.error = nullptr;
    if (maps.use) {
        int rc = tc_setup();
        if (rc) return rc;
        const int box_rows = page_size < DEC_TILE ? page_size : DEC_TILE;
        const uint64_t rows = (uint64_t)num_pages * num_kv_heads * page_size;
        if ((rc = make_decode_map(&maps.k, k_cache, rows, head_dim, box_rows))) return rc;
        if ((rc = make_decode_map(&maps.v, v_cache, rows, head_dim, box_rows))) return rc;
        p.error = g_error_dev;
    }
    switch (head_dim) {
        case 16: return launch_decode<16>(p, maps, num_rows, stream);
        case 32: return launch_decode<32>(p, maps, num_rows, stream);
        case 48: return launch_decode<48>(p, maps, num_rows, stream);
        case 64: return launch_decode<64>(p, maps, num_rows, stream);
        case 80: return launch_decode<80>(p, maps, num_rows, stream);
        case 96: return launch_decode<96>(p, maps, num_rows, stream);
        case 112: return launch_decode<112>(p, maps, num_rows, stream);
        case 128: return launch_decode<128>(p, maps, num_rows, stream);
    }
    return MIE_ERR_BAD_ARG;
}

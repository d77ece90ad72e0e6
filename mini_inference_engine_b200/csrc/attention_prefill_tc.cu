// Paged causal prefill attention on the 5th-generation tensor cores (head_dim 64 or 128, bfloat16).
//
// One block = 128 consecutive queries of one request and one query head.  Both products of
// attention run as tcgen05.mma with accumulators in tensor memory:
//
//   S = Q K^T   Q [128 x D] and the key tile [128 keys x D] are K-major tiles in shared memory, brought
//               by TMA with the 128-byte swizzle -- Q out of the fused qkv activation, keys out of the
//               cache one page per copy through the request's block table.  S is 128 x 128 float32 in
//               TMEM: one query row per TMEM lane.
//   softmax     four warps, one thread per query row: the thread reads its row of S out of TMEM
//               (tcgen05.ld), masks by position (key <= query, key > query - window), keeps a running
//               max and sum in base 2, and writes P, rounded to bfloat16, back into TMEM (tcgen05.st).
//               No shuffles: a row never leaves its thread.
//   O += P V    P is the A operand straight out of TMEM; V [128 keys x D] sits in shared memory as TMA
//               wrote it, which for this product is an MN-major B operand.  O is 128 x D float32 in
//               TMEM; when the running max of a row moves, its thread rescales its row of O in place.
//
// The reference does this with a library attention call per prompt portion
// (inference_engine/model.py:146-158).  A block works through its key tiles one after the other
// (S, softmax, PV); two blocks share an SM at head_dim 64 (256 TMEM columns and 97 KB of shared
// memory each), so one block's softmax runs under the other's products.  When a launch has more
// query tiles than the GPU runs at a time, a block takes two tiles of a row one after the other,
// the j-th from the end and the j-th from the start: under the causal mask every such pair has the
// same number of key tiles, so the blocks end together instead of leaving a tail of long ones.
//
// Roles: warp 0 = TMA producer (one lane), warp 1 = TMEM owner + MMA issuer (one lane), warps 2..5 =
// softmax and epilogue.  Barriers: q_full, kv_full[2] / kv_empty[2] (two key/value stages; kv_empty
// is the commit behind a PV product, so it also says that P may be overwritten and O rescaled), s_full
// (S is complete), p_full (one arrival per softmax warp: S has been taken, P is written and O
// rescaled), o_full.  The MMA thread issues S of the next tile ahead of PV of this one: issuing costs
// about 50 cycles per MMA and 90 per commit (measured), and the softmax warps wait for the next S only.
// Every wait is bounded (see tcgen05_common.cuh).
#include <type_traits>

#include "tcgen05_common.cuh"
#include "range_check.cuh"

#define FA_BM 128
#define FA_BN 128
#define FA_THREADS 192

struct FaParams {
    const int* block_tables; int table_stride;
    const int* row_q_start; const int* row_q_len; const int* row_ctx_len; int num_rows;
    bf16* out;
    int* error;
    int num_heads, num_kv_heads, page_size, page_shift, window, min_q_len;
    int pair;                // 1: a block takes two query tiles of a row (see the kernel), 0: one
    float scale_log2e;
    int64_t check_pages;     // pages in each cache, for the range check of block-table entries
    int* report;             // range report (range_check.cuh)
};

// MN-major B operand tile with the 128-byte swizzle: 64 elements of N contiguous in a 128-byte row,
// one row per k, 8 rows = one 1024-byte swizzle atom.  Stride between atoms along K (stride byte
// offset) 1024; between 64-element groups along N (leading byte offset) `n_group_bytes`.
__device__ __forceinline__ uint64_t umma_desc_sw128_mn(uint32_t smem_addr, uint32_t n_group_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((n_group_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}


// A quarter of one thread's row of S: 32 float32 columns, asynchronous.  The registers may be read
// only after tmem_ld_wait(r); passing them through the wait keeps the compiler from using them early.
__device__ __forceinline__ void tmem_ld32_async(uint32_t addr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait(uint32_t* r) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31]) :: "memory");
}
// 16 columns (32 entries of P as bfloat16 pairs); completion is awaited by tmem_st_wait().
__device__ __forceinline__ void tmem_st16(uint32_t addr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" :: "r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag));
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int D>
__global__ void __launch_bounds__(FA_THREADS, 2)       // two blocks per SM: at most 168 registers
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q,   // qkv activation [tokens, q_stride], box {64, 128}
                            const __grid_constant__ CUtensorMap map_k,   // key pages as rows [pages * kv_heads * page_size, D], box {64, page rows}
                            const __grid_constant__ CUtensorMap map_v,
                            const FaParams p) {
    constexpr int PARTS = D / 64;                               // 64-column sub-tiles (128 bytes = one swizzle row)
    constexpr uint32_t SUB_BYTES = 128 * 64 * 2;                // one [128 rows x 64] sub-tile
    constexpr uint32_t Q_BYTES = PARTS * SUB_BYTES, KV_BYTES = PARTS * SUB_BYTES;
    constexpr uint32_t TMEM_S = 0, TMEM_P = 128, TMEM_O = 192;  // column offsets: S 128 cols, P 64 cols (bf16 pairs), O D cols
    constexpr uint32_t TMEM_COLS = D == 64 ? 256 : 512;
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t q_full[2], kv_full[2], kv_empty[2], s_full, p_full, o_full;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag, s_row, s_q0[2], s_nsub;

    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char* tiles = smem_dyn + (base - smem_u32(smem_dyn));
    // layout: Q of the first query tile | Q of the second | K stage 0 | V stage 0 | K stage 1 | V stage 1
    auto q_addr = [&](int u) { return base + (uint32_t)u * Q_BYTES; };
    auto k_addr = [&](int s) { return base + 2 * Q_BYTES + (uint32_t)s * 2 * KV_BYTES; };
    auto v_addr = [&](int s) { return base + 2 * Q_BYTES + (uint32_t)s * 2 * KV_BYTES + KV_BYTES; };

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // Which row and which query tiles are this block's?  Asked first, and by a whole warp (warp_find_row): the grid is
    // laid out for the most tiles the step's rows could have, and a block without work leaves before it has set
    // anything up.
    // A block takes two query tiles of a row, one after the other: the j-th from the end and the j-th
    // from the start.  Under the causal mask their key ranges add up to the same length for every j,
    // so all blocks of a row run equally long (the middle tile of an odd count stands alone).
    // Pairing pays once there are more tiles than the GPU runs at a time (p.pair, the host's call):
    // below that every tile has a block of its own and the longest one is the critical path.
    if (warp == 0) {
        int pair, tiles_r;
        const int r = warp_find_row(p.row_q_len, p.num_rows, (int)blockIdx.x, [&](int ql) {
            const int t = ql >= p.min_q_len ? (ql + FA_BM - 1) / FA_BM : 0;
            return p.pair ? (t + 1) / 2 : t;
        }, pair, tiles_r);
        if (lane == 0) {
            s_row = r;
            if (r >= 0) {
                const int ql = p.row_q_len[r];
                tiles_r = (ql + FA_BM - 1) / FA_BM;             // (the count above was of blocks)
                s_q0[0] = (tiles_r - 1 - pair) * FA_BM;         // the longest key ranges start first
                s_q0[1] = pair * FA_BM;
                s_nsub = (p.pair && tiles_r - 1 - pair != pair) ? 2 : 1;
            }
        }
    }
    __syncthreads();
    if (s_row < 0) return;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&q_full[0], 1); mbar_init(&q_full[1], 1);
        mbar_init(&kv_full[0], 1); mbar_init(&kv_full[1], 1);
        mbar_init(&kv_empty[0], 1); mbar_init(&kv_empty[1], 1);
        mbar_init(&s_full, 1); mbar_init(&p_full, 4); mbar_init(&o_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // key/value rows that no copy fills (beyond the context) must hold finite values: 0 * NaN is NaN
    for (uint32_t i = threadIdx.x * 16; i < 4 * KV_BYTES; i += FA_THREADS * 16)
        *reinterpret_cast<uint4*>(tiles + 2 * Q_BYTES + i) = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the TMA unit must see the zeros before it overwrites them
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pdl_wait();                                                  // everything below reads what earlier kernels wrote
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* abort_p = &abort_flag;
    const int row = s_row;

    if (row >= 0) {
        const int q_len = p.row_q_len[row], ctx = p.row_ctx_len[row], q_start = p.row_q_start[row];
        const int head = blockIdx.y;
        const int kvh = head / (p.num_heads / p.num_kv_heads);
        const int nsub = s_nsub;
        // the geometry of query tile u: first query's position, rows, key range in tiles of FA_BN keys
        struct Sub { int q0, pos0, nq, k_hi, k_lo, kbeg, ntiles; };
        Sub sb[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            Sub& g = sb[u];
            g.q0 = s_q0[u < nsub ? u : 0];
            g.pos0 = ctx - q_len + g.q0;                         // position of the tile's first query
            g.nq = min(FA_BM, q_len - g.q0);
            g.k_hi = g.pos0 + g.nq;                              // one past the last key any query here reads
            g.k_lo = p.window > 0 ? max(0, g.pos0 - p.window + 1) : 0;
            g.kbeg = g.k_lo & ~(FA_BN - 1);
            g.ntiles = u < nsub ? (g.k_hi - g.kbeg + FA_BN - 1) / FA_BN : 0;
        }
        const int nA = sb[0].ntiles, G = nA + sb[1].ntiles;      // key tiles of the first query tile, and of both
        // Key tiles are counted through both query tiles (g = 0 .. G-1): stages and barrier phases go on
        // from the first query tile to the second without a break.
        const int rows_per_copy = min(p.page_size, FA_BN);       // one TMA copy = one page (or a 128-row piece of it)

        if (warp == 0) {
            // The producer warp: lane c issues the copies of page c of a tile, and fetches the page id
            // of the NEXT tile one tile ahead, so that no look-up in global memory sits between a
            // freed stage and its refill.
            const int* table = p.block_tables + (int64_t)row * p.table_stride;
            if (lane == 0) {
                for (int u = 0; u < nsub; ++u) {
                    mbar_expect_tx(&q_full[u], Q_BYTES);
#pragma unroll
                    for (int part = 0; part < PARTS; ++part)
                        tma_load_2d(tiles + u * Q_BYTES + part * SUB_BYTES, &map_q, &q_full[u], head * D + part * 64, q_start + sb[u].q0);
                }
            }
            auto key0_of = [&](int g) { return g < nA ? sb[0].kbeg + g * FA_BN : sb[1].kbeg + (g - nA) * FA_BN; };
            auto copies_of = [&](int g) {
                const int key0 = key0_of(g), hi = g < nA ? sb[0].k_hi : sb[1].k_hi;
                return (min(key0 + FA_BN, hi) - key0 + rows_per_copy - 1) / rows_per_copy;
            };
            auto page_of = [&](int g) {                           // lane's page id in key tile g (0 if it has no copy there)
                if (g >= G || lane >= copies_of(g)) return 0;
                const int entry = (key0_of(g) + lane * rows_per_copy) >> p.page_shift;
                return checked_page(table[entry], p.check_pages, p.report, MIE_K_ATTENTION_PREFILL_TC, entry);
            };
            int page_next = page_of(0);
            for (int g = 0; g < G; ++g) {
                const int s = g & 1, round = g >> 1;
                const int page = page_next;
                page_next = page_of(g + 1);
                int ok = 1;
                if (lane == 0) ok = mbar_wait(&kv_empty[s], (round & 1) ^ 1, abort_p) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                const int copies = copies_of(g);
                if (lane == 0) mbar_expect_tx(&kv_full[s], (uint32_t)copies * rows_per_copy * 128u * PARTS * 2u);
                __syncwarp();
                if (lane < copies) {
                    const int key = key0_of(g) + lane * rows_per_copy;
                    const int src_row = (page * p.num_kv_heads + kvh) * p.page_size + (key & (p.page_size - 1));
#pragma unroll
                    for (int part = 0; part < PARTS; ++part) {
                        const uint32_t off = part * SUB_BYTES + (uint32_t)lane * rows_per_copy * 128u;
                        tma_load_2d(tiles + (k_addr(s) - base) + off, &map_k, &kv_full[s], part * 64, src_row);
                        tma_load_2d(tiles + (v_addr(s) - base) + off, &map_v, &kv_full[s], part * 64, src_row);
                    }
                }
            }
        } else if (warp == 1) {
            // Head size 64: the whole warp walks this loop and an elected lane issues, so that what feeds the
            // tensor-core instructions stays uniform across the warp (issued from a loop that one lane ran alone, an
            // MMA cost that lane 90 - 150 cycles): 49.8 -> 45.1 us at 2,048 tokens, 531 -> 496 us at 8,192.  Head size
            // 128 (one block on an SM, twice the exponent-free work per score): one lane alone, the 32 polling lanes
            // cost the softmax warps more than the issue gains (964 -> 1,027 us at 8,192 tokens with the whole warp).
            constexpr bool WARP_ISSUE = D == 64;
            if (WARP_ISSUE || lane == 0) {
                const bool issuer = WARP_ISSUE ? elect_one() : true;
                auto wait_for = [&](uint64_t* bar, uint32_t parity) {
                    return WARP_ISSUE ? mbar_wait_warp(bar, parity, abort_p) : mbar_wait(bar, parity, abort_p);
                };
                auto converge = [&]() { if (WARP_ISSUE) __syncwarp(); };
                // S: M 128, N 128, both operands K-major.  PV: M 128, N D, B (values) MN-major.
                const uint32_t idesc_s = umma_idesc_bf16(FA_BM, FA_BN);
                const uint32_t idesc_o = umma_idesc_bf16(FA_BM, D) | (1u << 16);
                // One thread issues every MMA, and between two of them it can do little: the descriptors
                // of all operand slices are formed once, here, so that an MMA costs its own instruction.
                constexpr int KS = D / 16, KV = FA_BN / 16;
                uint64_t dq[2][KS], dk[2][KS], dv[2][KV];
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    const uint32_t off = (ks / 4) * SUB_BYTES + (ks % 4) * 32;
                    dq[0][ks] = umma_desc_sw128(q_addr(0) + off);
                    dq[1][ks] = umma_desc_sw128(q_addr(1) + off);
                    dk[0][ks] = umma_desc_sw128(k_addr(0) + off);
                    dk[1][ks] = umma_desc_sw128(k_addr(1) + off);
                }
#pragma unroll
                for (int kk = 0; kk < KV; ++kk) {                  // 16 keys per MMA: 8 TMEM columns of P, 2 atoms of V
                    dv[0][kk] = umma_desc_sw128_mn(v_addr(0) + kk * 2048, SUB_BYTES);
                    dv[1][kk] = umma_desc_sw128_mn(v_addr(1) + kk * 2048, SUB_BYTES);
                }
                auto issue_s = [&](int g) {                        // scores of key tile g against its query tile
                    const bool second = g >= nA, st = g & 1;
                    if (issuer) {
#pragma unroll
                        for (int ks = 0; ks < KS; ++ks)
                            umma_bf16(tmem_base + TMEM_S, second ? dq[1][ks] : dq[0][ks], st ? dk[1][ks] : dk[0][ks], idesc_s, ks > 0 ? 1u : 0u);
                        umma_commit(&s_full);
                    }
                    converge();
                };
                // Order per key tile: as soon as the softmax warps have taken S(g) (p_full), S(g+1) is issued
                // ahead of P(g) V(g), so that the next scores are ready while the tensor pipe still works on
                // this tile's values -- the softmax warps never wait for a product that they do not need yet.
                // kv_empty (the commit behind P V) also tells them when P may be overwritten and O rescaled:
                // a commit costs the issuing thread as much as two MMAs, so one serves both.
                bool ok = wait_for(&q_full[0], 0);
                if (ok && nsub > 1) ok = wait_for(&q_full[1], 0);
                if (ok) ok = wait_for(&kv_full[0], 0);
                if (ok) { tc_fence_after(); issue_s(0); }
                for (int g = 0; g < G && ok; ++g) {
                    const int s = g & 1;
                    const int t = g < nA ? g : g - nA;             // key tile within its query tile
                    const bool last_of_tile = g == nA - 1 || g == G - 1;
                    ok = wait_for(&p_full, g & 1);       // P written, O rescaled, S free
                    if (!ok) break;
                    tc_fence_after();
                    bool next_issued = g + 1 >= G;
                    if (!next_issued && (WARP_ISSUE ? __all_sync(0xffffffffu, mbar_try_wait(&kv_full[s ^ 1], ((g + 1) >> 1) & 1)) != 0 : mbar_try_wait(&kv_full[s ^ 1], ((g + 1) >> 1) & 1))) {   // keys of the next tile are here
                        tc_fence_after();
                        issue_s(g + 1);
                        next_issued = true;
                    }
                    if (issuer) {
#pragma unroll
                        for (int kk = 0; kk < KV; ++kk)
                            umma_bf16_ts(tmem_base + TMEM_O, tmem_base + TMEM_P + kk * 8, s ? dv[1][kk] : dv[0][kk], idesc_o,
                                         (t > 0 || kk > 0) ? 1u : 0u);
                        umma_commit(&kv_empty[s]);                 // the stage may be refilled, P overwritten and O rescaled
                        if (last_of_tile) umma_commit(&o_full);    // this query tile's output is complete
                    }
                    converge();
                    if (!next_issued) {                            // the keys were late: wait for them now
                        ok = wait_for(&kv_full[s ^ 1], ((g + 1) >> 1) & 1);
                        if (!ok) break;
                        tc_fence_after();
                        issue_s(g + 1);
                    }
                }
            }
        } else {
            const int q = warp & 3;
            const int r = q * 32 + lane;                           // this thread's query row within the tile
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
            bool ok = true;
            for (int u = 0; u < nsub && ok; ++u) {                 // one query tile after the other
                const int q0 = sb[u].q0, pos0 = sb[u].pos0, nq = sb[u].nq, k_lo = sb[u].k_lo, kbeg = sb[u].kbeg, ntiles = sb[u].ntiles;
                const int g0 = u ? nA : 0;                             // key tiles counted through both query tiles
                const int qpos = pos0 + r;
                float m_run = -INFINITY, l_run = 0.f;
                for (int t = 0; t < ntiles && ok; ++t) {
                    const int g = g0 + t;
                    ok = __all_sync(0xffffffffu, mbar_wait(&s_full, g & 1, abort_p));     // the warp goes on or gives up as one
                    if (!ok) break;
                    tc_fence_after();
                    const int key0 = kbeg + t * FA_BN;
                    // masks are needed only where the tile touches the diagonal, the window's edge or the range's start
                    const bool need_mask = key0 + FA_BN - 1 > pos0 || key0 < k_lo || (p.window > 0 && key0 <= pos0 + FA_BM - 1 - p.window);
                    // The row of S comes out of TMEM in four chunks of 32 columns; the load of the next chunk is
                    // in flight while the current one is worked on.
                    auto for_each_chunk = [&](auto&& body) {
                        uint32_t ca[32], cb[32];
                        tmem_ld32_async(lane_addr + TMEM_S, ca);
                        tmem_ld_wait(ca);
                        tmem_ld32_async(lane_addr + TMEM_S + 32, cb);
                        body(0, ca);
                        tmem_ld_wait(cb);
                        tmem_ld32_async(lane_addr + TMEM_S + 64, ca);
                        body(1, cb);
                        tmem_ld_wait(ca);
                        tmem_ld32_async(lane_addr + TMEM_S + 96, cb);
                        body(2, ca);
                        tmem_ld_wait(cb);
                        body(3, cb);
                    };
                    auto masked = [&](int key) { return !(key <= qpos && (p.window <= 0 || key > qpos - p.window)); };
                    // Reference point of the exponent.  Reading S once per tile is what matters here (TMEM
                    // loads are the slowest part of the step), so the running max is not recomputed up front:
                    // P is formed against the running max as it stands, the row's true max is found on the
                    // way, and only if some entry would exceed 2^8 is the tile redone against the new max
                    // (then O and l are rescaled).  The first tile has no running max and takes a max pass.
                    // The two loops below exist in a masked and an unmasked version, chosen once per tile: a
                    // test per element would double the instructions of the common, unmasked tiles.
                    auto row_max = [&](auto mask_tag) {
                        constexpr bool MASK = decltype(mask_tag)::value;
                        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                        for_each_chunk([&](int ch, const uint32_t* c) {
    #pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                float x = __uint_as_float(c[i]);
                                if (MASK && masked(key0 + ch * 32 + i)) x = -INFINITY;
                                mx4[i & 3] = fmaxf(mx4[i & 3], x);
                            }
                        });
                        return fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                    };
                    if (t == 0) {
                        const float mx = need_mask ? row_max(std::true_type{}) : row_max(std::false_type{});
                        m_run = mx * p.scale_log2e;                    // the scale is positive: max and scaling commute
                    }
                    float alpha = 1.f, sum = 0.f;
                    auto p_pass = [&](auto mask_tag, float neg_m, float& xmax_out) {
                        constexpr bool MASK = decltype(mask_tag)::value;
                        // four independent sums and maxima: one warp per scheduler has nothing else to hide
                        // the latency of a dependent chain behind
                        float xm[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY}, sm[4] = {0.f, 0.f, 0.f, 0.f};
                        for_each_chunk([&](int ch, const uint32_t* c) {
                            uint32_t packed[16];
                            // P(t-1) must have been read by its product before it is overwritten (normally long done)
                            if (ch == 0 && g > 0 && !__all_sync(0xffffffffu, mbar_wait(&kv_empty[(g - 1) & 1], ((g - 1) >> 1) & 1, abort_p))) ok = false;
    #pragma unroll
                            for (int i = 0; i < 32; i += 2) {
                                float x0 = fmaf(__uint_as_float(c[i]), p.scale_log2e, neg_m);
                                float x1 = fmaf(__uint_as_float(c[i + 1]), p.scale_log2e, neg_m);
                                if (MASK) {
                                    if (masked(key0 + ch * 32 + i)) x0 = -INFINITY;
                                    if (masked(key0 + ch * 32 + i + 1)) x1 = -INFINITY;
                                }
                                xm[(i >> 1) & 3] = fmaxf(xm[(i >> 1) & 3], fmaxf(x0, x1));
                                const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
                                sm[(i >> 1) & 3] += p0 + p1;
                                packed[i >> 1] = pack2_bf16(p0, p1);
                            }
                            tmem_st16(lane_addr + TMEM_P + ch * 16, packed);
                        });
                        xmax_out = fmaxf(fmaxf(xm[0], xm[1]), fmaxf(xm[2], xm[3]));
                        return (sm[0] + sm[1]) + (sm[2] + sm[3]);
                    };
                    for (int attempt = 0; attempt < 2; ++attempt) {
                        const float neg_m = m_run == -INFINITY ? 0.f : -m_run;
                        float xmax;
                        sum = need_mask ? p_pass(std::true_type{}, neg_m, xmax) : p_pass(std::false_type{}, neg_m, xmax);
                        // the running max moves only when it has to (warp-wide decision: the loads are warp-wide)
                        const bool moved = xmax > 8.0f || (m_run == -INFINITY && xmax > -INFINITY);
                        if (attempt == 1 || !__any_sync(0xffffffffu, moved)) break;
                        if (moved) {
                            const float m_new = (m_run == -INFINITY ? 0.f : m_run) + xmax;
                            alpha = m_run == -INFINITY ? 1.f : ex2_approx(m_run - m_new);
                            m_run = m_new;
                        }
                    }
                    l_run = l_run * alpha + sum;
                    // rescale this row of O (the PV product of the tile before has finished: s_full came after it)
                    // (tcgen05.ld / st are warp-wide instructions: the whole warp rescales if any of its rows moved)
                    if (t > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
    #pragma unroll 1
                        for (int c = 0; c < D; c += 16) {
                            float v[16];
                            tmem_ld16(lane_addr + TMEM_O + c, v);
                            uint32_t w[16];
    #pragma unroll
                            for (int i = 0; i < 16; ++i) w[i] = __float_as_uint(v[i] * alpha);
                            tmem_st8(lane_addr + TMEM_O + c, w);
                            tmem_st8(lane_addr + TMEM_O + c + 8, w + 8);
                        }
                    }
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&p_full);              // one arrival per warp
                }
                // epilogue: O / l -> bfloat16 -> out[token, head, :]
                if (ok) ok = mbar_wait(&o_full, u & 1, abort_p);
                tc_fence_after();
                __syncwarp();
                if (__all_sync(0xffffffffu, ok)) {                      // warp-wide loads: every lane reads, rows inside the tile store
                    const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
                    bf16* op = p.out + ((int64_t)(q_start + q0 + r) * p.num_heads + head) * D;
    #pragma unroll 1
                    for (int c = 0; c < D; c += 16) {
                        float v[16];
                        tmem_ld16(lane_addr + TMEM_O + c, v);
                        if (r >= nq) continue;
                        uint4 w0, w1;
                        w0.x = pack2_bf16(v[0] * inv, v[1] * inv); w0.y = pack2_bf16(v[2] * inv, v[3] * inv);
                        w0.z = pack2_bf16(v[4] * inv, v[5] * inv); w0.w = pack2_bf16(v[6] * inv, v[7] * inv);
                        w1.x = pack2_bf16(v[8] * inv, v[9] * inv); w1.y = pack2_bf16(v[10] * inv, v[11] * inv);
                        w1.z = pack2_bf16(v[12] * inv, v[13] * inv); w1.w = pack2_bf16(v[14] * inv, v[15] * inv);
                        *reinterpret_cast<uint4*>(op + c) = w0;
                        *reinterpret_cast<uint4*>(op + c + 8) = w1;
                    }
                    // the next query tile's first PV product overwrites O: it follows p_full, which this warp
                    // gives only after these loads
                    tc_fence_before();
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        if (threadIdx.x == 0) atomicExch(p.error, 1);
        for (int i = 0; i < 64; ++i) __nanosleep(2000);           // let copies that are still in flight land
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// --------------------------------------------------------------------------- two query tiles side by side
//
// The kernel above leaves the tensor pipe idle while a block's four softmax warps work and the exponent
// unit idle while its MMA thread issues; two blocks on an SM interleave only by chance.  This one
// makes the interleaving a schedule (head_dim 64): a block holds TWO consecutive query tiles of a row
// (256 queries of one head) and two groups of four softmax warps, one per tile.  They share the key
// and value tiles (loaded once for both) and the MMA thread, which alternates: while group 0 takes its
// scores of key tile j through the softmax, the tensor pipe works on S1(j) and on P1 V of the tile
// before, and the other way round.  TMEM holds S0, S1 (2 x 128 columns), P0, P1 (2 x 64) and O0, O1
// (2 x 64): all 512.  A softmax thread moves its whole row of S into registers at once and gives S back
// (s_free), so that the group's scores of the next key tile are computed while its exponentials run.
// Each group has an MMA-issuing thread of its own (warps 1 and 10): issuing costs a thread 90 - 150
// cycles per tcgen05.mma here (measured with cycle stamps: one thread serving both groups needed 3,400
// cycles a key tile, more than both softmaxes), and twelve MMAs go into every (query tile, key tile).
// Per key tile j the thread of group u issues S_u(j + 1) as soon as s_free says so, then P_u V(j) when
// the group delivers P (p_full).  Blocks are numbered longest first (the last pair of a row has the
// most keys), so that short ones fill the tail.
#define PP_THREADS 352
#define PP_STAGES 3

// Diagnostic build (-DPP_TRACE): cycle stamps of the first block's roles per key tile; not compiled otherwise.
#ifdef PP_TRACE
__device__ long long g_pp_trace[64 * 16];
#define PP_STAMP(who, j, slot) if (blockIdx.x == 0 && blockIdx.y == 0 && (j) < 16) g_pp_trace[((who) * 16 + (j)) * 16 / 4 + (slot)] = clock64()
extern "C" int mie_pp_trace(long long* out, int count) { return (int)cudaMemcpyFromSymbol(out, g_pp_trace, sizeof(long long) * count); }
#else
#define PP_STAMP(who, j, slot)
#endif

__global__ void __launch_bounds__(PP_THREADS, 1)
prefill_attention_pp_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const FaParams p) {
    constexpr int D = 64;
    constexpr uint32_t SUB_BYTES = 128 * 64 * 2;                // one [128 rows x 64] tile
    constexpr uint32_t Q_BYTES = SUB_BYTES, KV_BYTES = SUB_BYTES;
    constexpr uint32_t TMEM_S = 0, TMEM_P = 256, TMEM_O = 384;  // per group u: S + 128 u, P + 64 u, O + 64 u
    constexpr uint32_t TMEM_COLS = 512;
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t q_full[2], kv_full[PP_STAGES], kv_empty[PP_STAGES], s_full[2], s_free[2], p_full[2], pv_done[2], o_full[2];
    __shared__ __align__(8) uint64_t exp_done[2];             // a group has run the exponentials of one more key tile
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag, s_row, s_q0, s_nsub;

    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char* tiles = smem_dyn + (base - smem_u32(smem_dyn));
    // layout: Q0 | Q1 | (K, V) x PP_STAGES
    auto q_addr = [&](int u) { return base + (uint32_t)u * Q_BYTES; };
    auto k_addr = [&](int s) { return base + 2 * Q_BYTES + (uint32_t)s * 2 * KV_BYTES; };
    auto v_addr = [&](int s) { return base + 2 * Q_BYTES + (uint32_t)s * 2 * KV_BYTES + KV_BYTES; };

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // which row and which pair of query tiles (pairs are numbered from the row's end): asked first, by a whole warp;
    // a block without work leaves before it has set anything up
    if (warp == 0) {
        int pair, pairs_r;
        const int r = warp_find_row(p.row_q_len, p.num_rows, (int)blockIdx.y, [&](int ql) {
            return ql >= p.min_q_len ? ((ql + FA_BM - 1) / FA_BM + 1) / 2 : 0;
        }, pair, pairs_r);
        if (lane == 0) {
            s_row = r;
            if (r >= 0) {
                const int tiles_r = (p.row_q_len[r] + FA_BM - 1) / FA_BM;
                const int first = (pairs_r - 1 - pair) * 2;              // the pair's first tile
                s_q0 = first * FA_BM;
                s_nsub = first + 1 < tiles_r ? 2 : 1;
            }
        }
    }
    __syncthreads();
    if (s_row < 0) return;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int u = 0; u < 2; ++u) {
            mbar_init(&q_full[u], 1); mbar_init(&s_full[u], 1); mbar_init(&s_free[u], 4); mbar_init(&p_full[u], 4);
            mbar_init(&pv_done[u], 1); mbar_init(&o_full[u], 1); mbar_init(&exp_done[u], 4);
        }
        for (int s = 0; s < PP_STAGES; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 2); }     // both MMA threads release a stage
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // key/value rows that no copy fills (beyond the context) must hold finite values: 0 * NaN is NaN
    for (uint32_t i = threadIdx.x * 16; i < PP_STAGES * 2 * KV_BYTES; i += PP_THREADS * 16)
        *reinterpret_cast<uint4*>(tiles + 2 * Q_BYTES + i) = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pdl_wait();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* abort_p = &abort_flag;
    const int row = s_row;

    if (row >= 0) {
        const int q_len = p.row_q_len[row], ctx = p.row_ctx_len[row], q_start = p.row_q_start[row];
        const int head = blockIdx.x;                            // heads vary fastest: the longest pairs of ALL heads start first
        const int kvh = head / (p.num_heads / p.num_kv_heads);
        const int nsub = s_nsub;
        struct Sub { int q0, pos0, nq, k_hi, k_lo; };
        Sub sb[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            Sub& g = sb[u];
            g.q0 = s_q0 + (u < nsub ? u : 0) * FA_BM;
            g.pos0 = ctx - q_len + g.q0;
            g.nq = min(FA_BM, q_len - g.q0);
            g.k_hi = g.pos0 + g.nq;
            g.k_lo = p.window > 0 ? max(0, g.pos0 - p.window + 1) : 0;
        }
        // one grid of key tiles for both query tiles, from the first key the first tile reads
        const int kbeg = sb[0].k_lo & ~(FA_BN - 1);
        const int k_hi0 = sb[0].k_hi, k_lo0 = sb[0].k_lo, k_hi1 = nsub > 1 ? sb[1].k_hi : 0, k_lo1 = sb[1].k_lo;
        const int k_end = nsub > 1 ? k_hi1 : k_hi0;
        const int J = (k_end - kbeg + FA_BN - 1) / FA_BN;
        // is key tile j read by query tile u?  (the same answer in every role; the second tile of a lone one reads nothing)
        auto active = [&](int u, int j) {
            const int key0 = kbeg + j * FA_BN;
            return u == 0 ? (key0 < k_hi0 && key0 + FA_BN > k_lo0) : (key0 < k_hi1 && key0 + FA_BN > k_lo1);
        };
        const int rows_per_copy = min(p.page_size, FA_BN);

        if (warp == 0) {
            // ---- producer (as in the kernel above): lane c copies page c of a key tile
            const int* table = p.block_tables + (int64_t)row * p.table_stride;
            if (lane == 0) {
                for (int u = 0; u < nsub; ++u) {
                    mbar_expect_tx(&q_full[u], Q_BYTES);
                    tma_load_2d(tiles + u * Q_BYTES, &map_q, &q_full[u], head * D, q_start + sb[u].q0);
                }
            }
            auto copies_of = [&](int j) {
                const int key0 = kbeg + j * FA_BN;
                return (min(key0 + FA_BN, k_end) - key0 + rows_per_copy - 1) / rows_per_copy;
            };
            auto page_of = [&](int j) {
                if (j >= J || lane >= copies_of(j)) return 0;
                const int entry = (kbeg + j * FA_BN + lane * rows_per_copy) >> p.page_shift;
                return checked_page(table[entry], p.check_pages, p.report, MIE_K_ATTENTION_PREFILL_TC, entry);
            };
            int page_next = page_of(0);
            int s = 0, round = 0;
            for (int j = 0; j < J; ++j) {
                const int page = page_next;
                page_next = page_of(j + 1);
                int ok = 1;
                if (lane == 0 && round > 0) ok = mbar_wait(&kv_empty[s], (round & 1) ^ 1, abort_p) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                const int copies = copies_of(j);
                if (lane == 0) mbar_expect_tx(&kv_full[s], (uint32_t)copies * rows_per_copy * 128u * 2u);
                __syncwarp();
                if (lane < copies) {
                    const int key = kbeg + j * FA_BN + lane * rows_per_copy;
                    const int src_row = (page * p.num_kv_heads + kvh) * p.page_size + (key & (p.page_size - 1));
                    const uint32_t off = (uint32_t)lane * rows_per_copy * 128u;
                    tma_load_2d(tiles + (k_addr(s) - base) + off, &map_k, &kv_full[s], 0, src_row);
                    tma_load_2d(tiles + (v_addr(s) - base) + off, &map_v, &kv_full[s], 0, src_row);
                }
                if (++s == PP_STAGES) { s = 0; ++round; }
            }
        } else if (warp == 1 || warp == 10) {
            if (lane == 0) {
                // ---- the MMA thread of group mu
                const int mu = warp == 1 ? 0 : 1;
                const uint32_t idesc_s = umma_idesc_bf16(FA_BM, FA_BN);
                const uint32_t idesc_o = umma_idesc_bf16(FA_BM, D) | (1u << 16);
                constexpr int KS = D / 16, KV = FA_BN / 16;
                uint64_t dq[KS];
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) dq[ks] = umma_desc_sw128(q_addr(mu) + ks * 32);
                const uint64_t dk0 = umma_desc_sw128(k_addr(0)), dv0 = umma_desc_sw128_mn(v_addr(0), SUB_BYTES);
                constexpr uint64_t STAGE_STEP = (2 * KV_BYTES) >> 4;       // descriptors of another stage differ in the address field only
                const uint32_t s_at = tmem_base + TMEM_S + 128u * mu, p_at = tmem_base + TMEM_P + 64u * mu, o_at = tmem_base + TMEM_O + 64u * mu;
                auto issue_s = [&](int st) {
#pragma unroll
                    for (int ks = 0; ks < KS; ++ks)
                        umma_bf16(s_at, dq[ks], dk0 + STAGE_STEP * st + (uint64_t)(ks * 2), idesc_s, ks > 0 ? 1u : 0u);
                    umma_commit(&s_full[mu]);
                };
                bool ok = mu < nsub ? mbar_wait(&q_full[mu], 0, abort_p) : true;
                int st = 0, round = 0, taken = 0, uses = 0;
                if (ok && active(mu, 0)) {
                    ok = mbar_wait(&kv_full[0], 0, abort_p);
                    if (ok) { tc_fence_after(); issue_s(0); }
                }
                for (int j = 0; j < J && ok; ++j) {
                    const int st_next = st + 1 == PP_STAGES ? 0 : st + 1, round_next = st + 1 == PP_STAGES ? round + 1 : round;
                    const bool now = active(mu, j), next = j + 1 < J && active(mu, j + 1);
                    PP_STAMP(2 + mu, j, 0);
                    if (next) {
                        // the group's next scores: as soon as it has moved its scores of tile j into registers (s_free),
                        // or at once when tile j + 1 is its first
                        if (now) { ok = mbar_wait(&s_free[mu], taken & 1, abort_p); ++taken; }
                        if (ok) ok = mbar_wait(&kv_full[st_next], round_next & 1, abort_p);
                        if (!ok) break;
                        tc_fence_after();
                        issue_s(st_next);
                    }
                    PP_STAMP(2 + mu, j, 1);
                    if (now) {
                        ok = mbar_wait(&p_full[mu], uses & 1, abort_p);    // P(j) is written, O rescaled
                        if (!ok) break;
                        tc_fence_after();
                        PP_STAMP(2 + mu, j, 2);
#pragma unroll
                        for (int kk = 0; kk < KV; ++kk)
                            umma_bf16_ts(o_at, p_at + kk * 8, dv0 + STAGE_STEP * st + (uint64_t)((kk * 2048) >> 4), idesc_o,
                                         (uses > 0 || kk > 0) ? 1u : 0u);
                        umma_commit(&pv_done[mu]);                         // P may be overwritten, O rescaled
                        ++uses;
                        if (!next) {
                            umma_commit(&o_full[mu]);                      // this tile's output is complete
                            ++taken;                                       // (its last s_free is never awaited)
                        }
                    }
                    // A thread whose group does not read this key tile still gives the stage back, but only once the
                    // stage has been filled: running ahead, its arrivals would count for rounds that are not its own.
                    if (!now) { ok = mbar_wait(&kv_full[st], round & 1, abort_p); if (!ok) break; }
                    umma_commit(&kv_empty[st]);                            // what this thread issued on the stage is accounted for
                    PP_STAMP(2 + mu, j, 3);
                    st = st_next; round = round_next;
                }
            }
        } else {
            // ---- softmax group u = 0 (warps 2..5) or 1 (warps 6..9): the row code of the kernel above
            const int u = warp >= 6 ? 1 : 0;
            const int q = warp & 3;                                // TMEM lane quarter = warp id % 4
            const int r = q * 32 + lane;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
            const uint32_t S_AT = lane_addr + TMEM_S + 128u * u, P_AT = lane_addr + TMEM_P + 64u * u, O_AT = lane_addr + TMEM_O + 64u * u;
            bool ok = true;
            if (u < nsub) {
                const int q0 = u ? sb[1].q0 : sb[0].q0, pos0 = u ? sb[1].pos0 : sb[0].pos0, nq = u ? sb[1].nq : sb[0].nq;
                const int k_lo = u ? k_lo1 : k_lo0;
                const int qpos = pos0 + r;
                float m_run = -INFINITY, l_run = 0.f;
                int used = 0;                                      // key tiles this group has taken
                // The two groups take turns at the exponent unit: with both in it at once each takes twice as long
                // and both then wait for their scores at the same time.  Group 0 goes first; the k-th turn of group 1
                // follows the k-th of group 0, the (k+1)-th of group 0 the k-th of group 1, as far as the other has turns.
                int turns_other = 0;
                for (int j = 0; j < J; ++j) turns_other += active(u ^ 1, j) ? 1 : 0;
                for (int j = 0; j < J && ok; ++j) {
                    if (!active(u, j)) continue;
                    ok = __all_sync(0xffffffffu, mbar_wait(&s_full[u], used & 1, abort_p));
                    if (!ok) break;
                    tc_fence_after();
                    if (q == 2 && lane == 0) { PP_STAMP(u, j, 0); }
                    const int key0 = kbeg + j * FA_BN;
                    const bool need_mask = key0 + FA_BN - 1 > pos0 || key0 < k_lo || (p.window > 0 && key0 <= pos0 + FA_BM - 1 - p.window);
                    // The whole row of S moves into registers at once and S is given back (s_free): the MMA thread
                    // issues this group's scores of the next key tile while the exponentials below run out of
                    // registers.  A row that has to be redone against a new maximum is redone from registers too.
                    uint32_t sv[128];
                    tmem_ld32_async(S_AT, sv);
                    tmem_ld32_async(S_AT + 32, sv + 32);
                    tmem_ld32_async(S_AT + 64, sv + 64);
                    tmem_ld32_async(S_AT + 96, sv + 96);
                    tmem_ld_wait(sv); tmem_ld_wait(sv + 32); tmem_ld_wait(sv + 64); tmem_ld_wait(sv + 96);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&s_free[u]);
                    if (q == 2 && lane == 0) { PP_STAMP(u, j, 1); }
                    auto masked = [&](int key) { return !(key <= qpos && (p.window <= 0 || key > qpos - p.window)); };
                    if (need_mask) {                               // masked entries become -inf once, here
#pragma unroll
                        for (int i = 0; i < 128; ++i) if (masked(key0 + i)) sv[i] = __float_as_uint(-INFINITY);
                    }
                    // The row's maximum comes out of the registers first (no second pass over TMEM as in the kernel
                    // above); the reference point of the exponent moves only when an entry would exceed 2^8 against the
                    // one in use, so that O is rescaled in the first tiles of a row and hardly ever after.
                    float alpha = 1.f, sum;
                    {
                        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                        for (int i = 0; i < 128; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[i]));
                        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2e;
                        if (mx > -INFINITY && (m_run == -INFINITY || mx - m_run > 8.0f)) {
                            alpha = m_run == -INFINITY ? 1.f : ex2_approx(m_run - mx);
                            m_run = mx;
                        }
                    }
                    // P of the tile before must have been read by its product before it is overwritten, and O is
                    // rescaled only once that product is complete
                    if (used > 0 && !__all_sync(0xffffffffu, mbar_wait(&pv_done[u], (used - 1) & 1, abort_p))) { ok = false; break; }
                    if (q == 2 && lane == 0) { PP_STAMP(u, j, 2); }
                    {
                        const int wait_for = u == 0 ? used - 1 : used;       // the other group's turn that comes before this one
                        if (wait_for >= 0 && wait_for < turns_other &&
                            !__all_sync(0xffffffffu, mbar_wait(&exp_done[u ^ 1], wait_for & 1, abort_p))) { ok = false; break; }
                    }
                    {
                        const float neg_m = m_run == -INFINITY ? 0.f : -m_run;
                        float sm[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int ch = 0; ch < 4; ++ch) {
                            uint32_t packed[16];
#pragma unroll
                            for (int i = 0; i < 32; i += 2) {
                                const float p0 = ex2_approx(fmaf(__uint_as_float(sv[ch * 32 + i]), p.scale_log2e, neg_m));
                                const float p1 = ex2_approx(fmaf(__uint_as_float(sv[ch * 32 + i + 1]), p.scale_log2e, neg_m));
                                sm[(i >> 1) & 3] += p0 + p1;
                                packed[i >> 1] = pack2_bf16(p0, p1);
                            }
                            tmem_st16(P_AT + ch * 16, packed);
                        }
                        sum = (sm[0] + sm[1]) + (sm[2] + sm[3]);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&exp_done[u]);      // the other group's turn
                    l_run = l_run * alpha + sum;
                    if (used > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
                        for (int c = 0; c < D; c += 16) {
                            float v[16];
                            tmem_ld16(O_AT + c, v);
                            uint32_t w[16];
#pragma unroll
                            for (int i = 0; i < 16; ++i) w[i] = __float_as_uint(v[i] * alpha);
                            tmem_st8(O_AT + c, w);
                            tmem_st8(O_AT + c + 8, w + 8);
                        }
                    }
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&p_full[u]);
                    if (q == 2 && lane == 0) { PP_STAMP(u, j, 3); }
                    ++used;
                }
                if (ok) ok = mbar_wait(&o_full[u], 0, abort_p);
                tc_fence_after();
                __syncwarp();
                if (__all_sync(0xffffffffu, ok)) {
                    const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
                    bf16* op = p.out + ((int64_t)(q_start + q0 + r) * p.num_heads + head) * D;
#pragma unroll 1
                    for (int c = 0; c < D; c += 16) {
                        float v[16];
                        tmem_ld16(O_AT + c, v);
                        if (r >= nq) continue;
                        uint4 w0, w1;
                        w0.x = pack2_bf16(v[0] * inv, v[1] * inv); w0.y = pack2_bf16(v[2] * inv, v[3] * inv);
                        w0.z = pack2_bf16(v[4] * inv, v[5] * inv); w0.w = pack2_bf16(v[6] * inv, v[7] * inv);
                        w1.x = pack2_bf16(v[8] * inv, v[9] * inv); w1.y = pack2_bf16(v[10] * inv, v[11] * inv);
                        w1.z = pack2_bf16(v[12] * inv, v[13] * inv); w1.w = pack2_bf16(v[14] * inv, v[15] * inv);
                        *reinterpret_cast<uint4*>(op + c) = w0;
                        *reinterpret_cast<uint4*>(op + c + 8) = w1;
                    }
                    tc_fence_before();
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        if (threadIdx.x == 0) atomicExch(p.error, 1);
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

static int launch_fa_pp(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const FaParams& p, int work_tokens,
                        int work_rows, cudaStream_t stream) {
    const size_t smem = (size_t)128 * 64 * 2 * (2 + 2 * PP_STAGES) + 1024;
    cudaError_t e = cudaFuncSetAttribute(prefill_attention_pp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const int tiles = (work_tokens + FA_BM - 1) / FA_BM + work_rows;
    const dim3 grid(p.num_heads, (tiles + work_rows + 1) / 2);
    return launch_kernel(prefill_attention_pp_kernel, grid, dim3(PP_THREADS), smem, stream, mq, mk, mv, p);
}

// --------------------------------------------------------------------------- host side

static int make_map_2d(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint64_t row_stride_elems, int box_rows) {
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstride[1] = {row_stride_elems * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

static int g_fa_pp_mode = -1;

template <int D>
static int launch_fa(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const FaParams& p, int work_tokens,
                     int work_rows, cudaStream_t stream) {
    const size_t smem = (size_t)(D / 64) * 128 * 64 * 2 * 6 + 1024;     // 2 x Q + 2 x (K + V)
    cudaError_t e = cudaFuncSetAttribute(prefill_attention_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    // tiles <= tokens / 128 + rows (of the rows that this kernel serves, where the caller knows them); a block takes
    // one tile, or a pair of them (at most (tiles + rows) / 2 pairs) once the tiles of all heads are more than the
    // GPU runs at a time
    const int tiles = (work_tokens + FA_BM - 1) / FA_BM + work_rows;
    FaParams pp = p;
    pp.pair = (int64_t)tiles * p.num_heads > (int64_t)device_sm_count() * (D == 64 ? 2 : 1);
    const dim3 grid(pp.pair ? (tiles + work_rows + 1) / 2 : tiles, p.num_heads);
    return launch_kernel(prefill_attention_tc_kernel<D>, grid, dim3(FA_THREADS), smem, stream, mq, mk, mv, pp);
}

// q: the fused qkv activation [num_tokens, q_stride] bfloat16 (query head h at columns h*D ..), caches
// [num_pages, kv_heads, page_size, D] bfloat16, out [num_tokens, heads, D] bfloat16.  head_dim 64 or
// 128, page_size a power of two >= 8, q_stride % 8 == 0.  Rows with fewer than min_q_len new tokens
// are skipped.  work_rows / work_tokens: how many rows have min_q_len tokens or more, and their tokens in sum, where the
// caller knows (the grid is laid out for the tiles they can have); 0: every row may, num_rows / num_tokens.
extern "C" int mie_prefill_attention_tc(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                                        int64_t num_pages, const int* block_tables, int table_stride, const int* row_q_start,
                                        const int* row_q_len, const int* row_ctx_len, int num_rows, int num_tokens, void* out,
                                        int num_heads, int num_kv_heads, int head_dim, int page_size, float scale, int window,
                                        int min_q_len, int work_rows, int work_tokens, cudaStream_t stream) {
    if (num_rows <= 0 || num_tokens <= 0) return 0;
    if (work_rows <= 0 || work_tokens <= 0 || work_rows > num_rows || work_tokens > num_tokens) { work_rows = num_rows; work_tokens = num_tokens; }
    if (head_dim != 64 && head_dim != 128) return MIE_ERR_BAD_ARG;
    if (num_kv_heads <= 0 || num_heads % num_kv_heads || num_heads > 65535) return MIE_ERR_BAD_ARG;
    if (page_size < 8 || (page_size & (page_size - 1)) || q_stride % 8) return MIE_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
         reinterpret_cast<uintptr_t>(out)) & 15) return MIE_ERR_BAD_ARG;
    int rc = tc_setup();
    if (rc) return rc;
    FaParams p;
    p.block_tables = block_tables; p.table_stride = table_stride;
    p.row_q_start = row_q_start; p.row_q_len = row_q_len; p.row_ctx_len = row_ctx_len; p.num_rows = num_rows;
    p.out = (bf16*)out; p.error = g_error_dev;
    p.num_heads = num_heads; p.num_kv_heads = num_kv_heads; p.page_size = page_size;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.window = window; p.min_q_len = min_q_len; p.pair = 0;
    p.scale_log2e = scale * 1.4426950408889634f;
    p.check_pages = num_pages; p.report = g_range_report;
    CUtensorMap mq, mk, mv;
    const int box_rows = page_size < FA_BN ? page_size : FA_BN;
    const uint64_t cache_rows = (uint64_t)num_pages * num_kv_heads * page_size;
    if ((rc = make_map_2d(&mq, q, (uint64_t)num_tokens, (uint64_t)q_stride, (uint64_t)q_stride, FA_BM))) return rc;
    if ((rc = make_map_2d(&mk, k_cache, cache_rows, (uint64_t)head_dim, (uint64_t)head_dim, box_rows))) return rc;
    if ((rc = make_map_2d(&mv, v_cache, cache_rows, (uint64_t)head_dim, (uint64_t)head_dim, box_rows))) return rc;
    if (head_dim == 64) {
        // two query tiles side by side once there are three pairs for every SM (measured, 32 heads, one tile a block
        // against two side by side: 2,048 tokens 45.1 against 48.5 us, 4,096 tokens 143.7 against 142.4 us, 8,192 tokens
        // 496 against 462 us); below that the one-tile blocks, two on an SM, spread a launch over more SMs
        const int64_t tiles = (work_tokens + FA_BM - 1) / FA_BM;
        if ((tiles + 2 * work_rows) / 2 < 65535 &&
            (g_fa_pp_mode == 1 || (g_fa_pp_mode < 0 && tiles * num_heads >= 6 * (int64_t)device_sm_count())))
            return launch_fa_pp(mq, mk, mv, p, work_tokens, work_rows, stream);
        return launch_fa<64>(mq, mk, mv, p, work_tokens, work_rows, stream);
    }
    return launch_fa<128>(mq, mk, mv, p, work_tokens, work_rows, stream);
}

// Which kernel serves head_dim 64: -1 chooses by the size of the launch (the default), 0 always one query tile a block,
// 1 always two side by side.
extern "C" void mie_prefill_attention_tc_pairs(int mode) { g_fa_pp_mode = mode; }

extern "C" int mie_prefill_attention_tc_error(void) { return g_error_host ? *g_error_host : 0; }
extern "C" void mie_prefill_attention_tc_clear_error(void) { if (g_error_host) *g_error_host = 0; }

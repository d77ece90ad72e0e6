// A chain of few-token products in ONE launch: y_i = x_i W_i^T for up to four products that follow
// one another in a decoder layer (output projection -> gate/up -> down -> the next layer's q|k|v), each
// with the epilogues of gemm_tcgen05.cu (deferred norm factor, SwiGLU, residual sum + next norm's
// input, rotation + cache write).  The reference launches a library product and several elementwise
// kernels for each of them (inference_engine/model.py:169-184).
//
// Why one launch.  At a few tokens a product is pure weight streaming, and a decode step is a chain
// of them: each needs the one before it complete, and between two launches the memory system idles
// while the tail of one kernel (partial sums to their owners, epilogue, exit) and the head of the
// next (dependency, activations) run their latencies.  Here a block never leaves the SM: its
// producer thread streams weight tiles into a deep shared-memory ring and runs AHEAD through the
// products of the chain -- it depends on nothing but free ring slots -- so the weights of product
// i+1 arrive while product i's sums are still on their way; every SM streams all the time, and no
// block enters late.
//
// Work split.  The grid is C clusters of 8 blocks, one block per SM (C = what the device can hold at
// once, 18 on a B200).  Cluster c takes the 128-row tiles c, c + C, ... of every product; the 8
// blocks of a cluster split K eight ways (tcgen05.mma, weights as the 128-row operand, the tokens
// padded to BN = 16 or 32 as the other), send their float32 partial rows to the row's owner block
// (st.async into its shared memory, counted on its mbarrier) and each block adds up and finishes the
// 16 rows it owns.  Two accumulators in tensor memory and two sets of receive slots let the sums and
// the epilogue of one tile run under the products of the next.
//
// Between products every block waits until all blocks have stored their results of the product
// before (a counter in global memory, bounded spin), then fetches its activations by TMA.  The
// counters are touched only after the launch's dependency wait (so launches of this kernel never
// overlap on them) and the last block to leave sets them back to zero.
//
// Every wait is bounded in time; a block that gives up raises the error word, skips what is left,
// still signals what others wait for where it can, frees its tensor memory and returns.
#include "tcgen05_common.cuh"
#include "range_check.cuh"

#define CH_BM 128
#define CH_BK 64
#define CH_S 8                 // blocks of a cluster = splits of K
#define CH_ROWS 16             // rows of a tile that a block owns (CH_BM / CH_S)
#define CH_THREADS 192
#define CH_MAX_OPS 4
#define CH_MAX_STAGES 12
#define CH_COUNTERS 8          // CH_MAX_OPS barriers and the exit counter, padded

struct ChainOp {
    int N, K, k_tiles, tiles_per_split, n_tiles;
    void* out;                 // [M, N] bfloat16 (or [M, N/2] with swiglu); unused with res
    const void* bias; int bias_tag;
    int swiglu;
    int rope;
    const int* positions; const int* slots; const float* cos_t; const float* sin_t; bf16* k_cache; bf16* v_cache;
    int num_heads, num_kv_heads, head_dim, rotary_dim, page_size, page_shift, max_pos, write_cache;
    long long num_pages;
    float* res; const void* norm_w; int norm_w_tag; bf16* xw_out; float* sq_out; int sq_stride;
    const float* sq_in; int sq_slots, sq_in_stride; float sq_width, sq_eps;
};

struct ChainParams {
    int num_ops, M, stages, x_tiles;       // x_tiles: k-tiles of activations the x buffer holds (the longest slice)
    int clusters;                          // C
    unsigned int* counters;                // [CH_COUNTERS], zero between launches
    int* error;                            // host-visible error word
    int* report;                           // range report
    uint32_t x_off, recv_off, table_off, rstd_off;   // byte offsets inside dynamic shared memory (after the ring)
    ChainOp ops[CH_MAX_OPS];
};

struct alignas(64) ChainMaps { CUtensorMap w[CH_MAX_OPS]; CUtensorMap x[CH_MAX_OPS]; };

// Diagnostic build (-DCH_TRACE): the epilogue's first thread of every block stamps the global timer at the
// stations of every product; mie_gemm_chain_trace copies the stamps out.  Not compiled otherwise.
#ifdef CH_TRACE
#define CH_TRACE_SLOTS 8
__device__ unsigned long long g_ch_trace[256 * CH_MAX_OPS * CH_TRACE_SLOTS + 256 * 2];
__device__ __forceinline__ unsigned long long ch_now() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#define CH_STAMP(op, slot) g_ch_trace[((blockIdx.y * CH_S + blockIdx.x) * CH_MAX_OPS + (op)) * CH_TRACE_SLOTS + (slot)] = ch_now()
#define CH_STAMP_BLOCK(which) g_ch_trace[256 * CH_MAX_OPS * CH_TRACE_SLOTS + (blockIdx.y * CH_S + blockIdx.x) * 2 + (which)] = ch_now()
extern "C" int mie_gemm_chain_trace(unsigned long long* out, int count) {
    return (int)cudaMemcpyFromSymbol(out, g_ch_trace, sizeof(unsigned long long) * count);
}
#else
#define CH_STAMP(op, slot)
#define CH_STAMP_BLOCK(which)
#endif

__device__ __forceinline__ float ch_silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

__device__ __forceinline__ void mbar_arrive_remote(uint32_t remote_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// mbarrier wait with acquire at cluster scope: what peers stored before their remote arrive is visible after it
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t i = 1;; ++i) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((i & 63u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > WAIT_LIMIT_CYCLES) break;
        }
    }
    *abort_flag = 1;
    return false;
}

template <int BN>
__global__ void __launch_bounds__(CH_THREADS, 1)
gemm_chain_kernel(const __grid_constant__ ChainMaps maps, const __grid_constant__ ChainParams p) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t full_bar[CH_MAX_STAGES];
    __shared__ __align__(8) uint64_t empty_bar[CH_MAX_STAGES];
    __shared__ __align__(8) uint64_t x_full;                 // the activations of the current product have landed
    __shared__ __align__(8) uint64_t acc_full[2];            // an accumulator is complete (tcgen05.commit)
    __shared__ __align__(8) uint64_t acc_empty[2];           // the epilogue has read it out (128 arrivals)
    __shared__ __align__(8) uint64_t recv_full[2];           // the peers' partial rows of a tile have landed (bytes)
    __shared__ __align__(8) uint64_t send_ok[2];             // all 8 owners are done with a set of receive slots
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    constexpr uint32_t A_BYTES = CH_BM * CH_BK * 2, B_BYTES = BN * CH_BK * 2;
    constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
    constexpr int RED_LD = BN + 4;
    constexpr uint32_t RECV_BYTES = CH_BM * RED_LD * 4;      // one set of receive slots: 8 senders x 16 padded rows
    constexpr uint32_t RECV_TX = CH_BM * BN * 4;             // the bytes that land in it per tile
    const uint32_t tiles_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char* tiles = smem_dyn + (tiles_base - smem_u32(smem_dyn));
    unsigned char* xbuf = tiles + p.x_off;
    float* recv = reinterpret_cast<float*>(tiles + p.recv_off);
    int* rope_pos = reinterpret_cast<int*>(tiles + p.table_off);
    int* rope_slot = rope_pos + BN;
    float* rope_cs = reinterpret_cast<float*>(rope_slot + BN);
    float* rstd_s = reinterpret_cast<float*>(tiles + p.rstd_off);

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 64) { CH_STAMP_BLOCK(0); }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = (int)cluster_rank();                    // = blockIdx.x: the K slice and the owned rows
    const int cl = blockIdx.y;                               // the cluster: tiles cl, cl + C, ...
    const int nblocks = p.clusters * CH_S;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < p.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&x_full, 1);
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 128);
            mbar_init(&recv_full[a], 1);
            mbar_init(&send_ok[a], CH_S);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        for (int a = 0; a < 2; ++a) mbar_expect_tx(&recv_full[a], RECV_TX);     // what this block is owed per tile
    }
    cluster_arrive_release();                                // peers write here and count on these barriers: they must exist
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* abort_p = &abort_flag;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer: weight tiles, through every product
        {                                                   // the whole warp walks the loop, an elected lane issues
            const bool issuer = elect_one();
            int s = 0, round = 0;
            bool ok = true;
            for (int o = 0; o < p.num_ops && ok; ++o) {
                const ChainOp& op = p.ops[o];
                const int kt0 = rank * op.tiles_per_split, kt1 = min(op.k_tiles, kt0 + op.tiles_per_split);
                for (int t = cl; t < op.n_tiles && ok; t += p.clusters) {
                    for (int kt = kt0; kt < kt1; ++kt) {
                        if (round > 0 && !__all_sync(0xffffffffu, mbar_wait(&empty_bar[s], (round & 1) ^ 1, abort_p))) { ok = false; break; }
                        if (issuer) {
                            mbar_expect_tx(&full_bar[s], A_BYTES);
                            tma_load_2d(tiles + (size_t)s * A_BYTES, &maps.w[o], &full_bar[s], kt * CH_BK, t * CH_BM);
                        }
                        __syncwarp();
                        if (++s == p.stages) { s = 0; ++round; }
                    }
                }
            }
        }
        __syncwarp();
        cluster_wait_acquire();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        {                                                   // the whole warp walks the loop, an elected lane issues
            const bool issuer = elect_one();
            const uint32_t idesc = umma_idesc_bf16(CH_BM, BN);
            const uint64_t desc_a0 = umma_desc_sw128(tiles_base), desc_b0 = umma_desc_sw128(tiles_base + p.x_off);
            int s = 0, round = 0, item = 0;
            bool ok = true;
            for (int o = 0; o < p.num_ops && ok; ++o) {
                const ChainOp& op = p.ops[o];
                const int kt0 = rank * op.tiles_per_split, kt1 = min(op.k_tiles, kt0 + op.tiles_per_split);
                const int n_kt = max(0, kt1 - kt0);
                ok = __all_sync(0xffffffffu, mbar_wait(&x_full, o & 1, abort_p));
                for (int t = cl; t < op.n_tiles && ok; t += p.clusters, ++item) {
                    const int a = item & 1;
                    if (item >= 2) ok = __all_sync(0xffffffffu, mbar_wait(&acc_empty[a], ((item >> 1) - 1) & 1, abort_p));
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t tmem_d = tmem_base + (uint32_t)(a * BN);
                    for (int kt = 0; kt < n_kt; ++kt) {
                        ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[s], round & 1, abort_p));
                        if (!ok) break;
                        tc_fence_after();
                        const uint64_t da = desc_a0 + (uint64_t)((uint32_t)s * A_BYTES >> 4);
                        const uint64_t db = desc_b0 + (uint64_t)((uint32_t)kt * B_BYTES >> 4);
                        if (issuer) {
#pragma unroll
                            for (int j = 0; j < CH_BK / 16; ++j)
                                umma_bf16(tmem_d, da + (uint64_t)(j * 2), db + (uint64_t)(j * 2), idesc, (kt > 0 || j > 0) ? 1u : 0u);
                            umma_commit(&empty_bar[s]);
                        }
                        __syncwarp();
                        if (++s == p.stages) { s = 0; ++round; }
                    }
                    if (!ok) break;
                    if (issuer) {
                        if (n_kt > 0) umma_commit(&acc_full[a]);
                        else mbar_arrive(&acc_full[a]);       // an empty slice of K adds a zero tile
                    }
                    __syncwarp();
                }
            }
        }
        __syncwarp();
        cluster_wait_acquire();
    } else {
        // ------------------------------------------------------------------ epilogue warps: dependencies, sends, owners' sums
        cluster_wait_acquire();                              // every block of the cluster runs: its memory and barriers may be written
        const int q = warp & 3, tid = threadIdx.x - 64;
        const int r = q * 32 + lane;                         // this thread's row of the tile (its TMEM lane)
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
        int item = 0;
        bool ok = true;
        for (int o = 0; o < p.num_ops && ok; ++o) {
            const ChainOp& op = p.ops[o];
            const int kt0 = rank * op.tiles_per_split, kt1 = min(op.k_tiles, kt0 + op.tiles_per_split);
            const int n_kt = max(0, kt1 - kt0);
            // ---- the dependency: the launch's own for the first product, all blocks' stores of the product before otherwise
            if (tid == 0) { CH_STAMP(o, 0); }                 // arrives at the product's dependency
            if (o == 0) {
                asm volatile("griddepcontrol.wait;" ::: "memory");
            } else {
                asm volatile("bar.sync 1, 128;" ::: "memory");  // every thread's stores of product o - 1 come before the fence below
                if (tid == 0) {
                    __threadfence();                          // cumulative over the barrier: what all 128 threads stored, device-wide
                    asm volatile("fence.proxy.async;" ::: "memory");
                    atomicAdd(p.counters + (o - 1), 1u);
                    if (ld_acquire_gpu(p.counters + (o - 1)) < (unsigned)nblocks) {
                        const long long t0 = clock64();
                        for (uint32_t i = 1; ld_acquire_gpu(p.counters + (o - 1)) < (unsigned)nblocks; ++i) {
                            if ((i & 15u) == 0u && (*abort_p || clock64() - t0 > WAIT_LIMIT_CYCLES)) { *abort_p = 1; break; }
                        }
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
            if (*abort_p) { ok = false; break; }
            if (tid == 0) { CH_STAMP(o, 1); }                 // dependency resolved
            if (tid == 0) {                                   // this block's slice of the activations, once per product
                asm volatile("fence.proxy.async;" ::: "memory");     // what other SMs stored is read by the TMA unit
                mbar_expect_tx(&x_full, (uint32_t)n_kt * B_BYTES);
                for (int kt = 0; kt < n_kt; ++kt)
                    tma_load_2d(xbuf + (size_t)kt * B_BYTES, &maps.x[o], &x_full, (kt0 + kt) * CH_BK, 0);
            }
            // ---- per-product tables: rotation inputs, the norm factor
            if (op.rope) {
                const int half = op.rotary_dim >> 1;
                for (int i = tid; i < BN; i += 128) {
                    int pos = i < p.M ? op.positions[i] : 0, slot = i < p.M ? op.slots[i] : 0;
                    if (range_position(pos, op.max_pos) != MIE_RANGE_OK) {
                        range_report(p.report, MIE_RANGE_POSITION, MIE_K_GEMM_QKV_ROPE, i, pos);
                        pos = 0; slot = -1;
                    } else if (op.write_cache && range_slot(slot, op.num_pages, op.page_size) != MIE_RANGE_OK) {
                        range_report(p.report, MIE_RANGE_SLOT, MIE_K_GEMM_QKV_ROPE, i, slot);
                        slot = -1;
                    }
                    rope_pos[i] = pos;
                    rope_slot[i] = slot;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                constexpr int TOK_THREADS = 128 / BN;
                for (int tt = tid / TOK_THREADS; tt < BN; tt += 128 / TOK_THREADS) {
                    const int64_t row = (int64_t)rope_pos[tt] * half;
                    for (int jj = tid % TOK_THREADS; jj < half; jj += TOK_THREADS) {
                        rope_cs[tt * half + jj] = op.cos_t[row + jj];
                        rope_cs[BN * half + tt * half + jj] = op.sin_t[row + jj];
                    }
                }
            }
            if (op.sq_in) {
                constexpr int TPT = 128 / BN;
                const int i = tid / TPT, sub = tid % TPT;
                const bool live = i < p.M;
                float v[16];
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    const int sl = sub + k * TPT;
                    v[k] = (live && sl < op.sq_slots) ? __ldcg(op.sq_in + (int64_t)sl * op.sq_in_stride + i) : 0.f;
                }
                float sum = 0.f;
#pragma unroll
                for (int k = 0; k < 16; ++k) sum += v[k];
                if (live)
                    for (int sl = sub + 16 * TPT; sl < op.sq_slots; sl += TPT) sum += __ldcg(op.sq_in + (int64_t)sl * op.sq_in_stride + i);
#pragma unroll
                for (int off = TPT >> 1; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
                if (sub == 0) rstd_s[i] = live ? rsqrtf(sum / op.sq_width + op.sq_eps) : 1.f;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");     // the tables are complete before any owner's sum reads them

            // ---- the tiles of this product, two steps a tile, one tile apart: the partial rows of tile j go out
            // to their owners, then the rows that arrived for tile j - 1 are added up and finished -- their way
            // through the cluster had a whole step to complete, and the products of tile j + 1 run meanwhile
            const bool cyclic = op.rope != 0;                 // with the rotation a block owns every 8th row: a row and its partner share an owner
            const int n_items = op.n_tiles > cl ? (op.n_tiles - cl + p.clusters - 1) / p.clusters : 0;
            constexpr int TK = BN / 8;                        // tokens per thread in the owners' sum: 16 rows x BN / TK = 128 threads
            for (int it = 0; it <= n_items && ok; ++it) {
                if (it < n_items) {                           // ---- send tile `it`
                    const int a = item & 1;
                    const uint32_t ph = (uint32_t)(item >> 1) & 1u;
                    ok = mbar_wait(&acc_full[a], ph, abort_p);
                    if (tid == 0 && it == 0) { CH_STAMP(o, 2); }  // first accumulator of the product complete
                    if (ok && item >= 2) ok = mbar_wait_cluster(&send_ok[a], ph ^ 1u, abort_p);
                    if (!ok) break;
                    if (tid == 0) { CH_STAMP(o, 3); }         // last accumulator complete (overwritten per tile)
                    tc_fence_after();
                    const int owner = cyclic ? (r & (CH_S - 1)) : (r >> 4), sli = cyclic ? (r >> 3) : (r & (CH_ROWS - 1));
                    const uint32_t send_to = cluster_addr(tiles_base + p.recv_off + (uint32_t)a * RECV_BYTES, owner) +
                                             (uint32_t)((rank * CH_ROWS + sli) * RED_LD) * 4u;
                    const uint32_t send_bar = cluster_addr(smem_u32(&recv_full[a]), owner);
#pragma unroll
                    for (int c = 0; c < BN; c += 16) {
                        float v[16];
                        if (n_kt > 0) tmem_ld16(taddr + (uint32_t)(a * BN + c), v);
                        else {
#pragma unroll
                            for (int i = 0; i < 16; ++i) v[i] = 0.f;
                        }
#pragma unroll
                        for (int i = 0; i < 16; i += 4)
                            st_async_cluster_f32x4(send_to + (uint32_t)(c + i) * 4u, send_bar, v[i], v[i + 1], v[i + 2], v[i + 3]);
                    }
                    tc_fence_before();
                    mbar_arrive(&acc_empty[a]);               // the accumulator may be overwritten
                    if (tid == 0) { CH_STAMP(o, 4); }         // rows sent
                    ++item;
                }
                if (it == 0) continue;
                // ---- finish tile `it - 1`: it was item `item - 2` if a tile was sent above, else `item - 1`
                const int fitem = it < n_items ? item - 2 : item - 1;
                const int a = fitem & 1;
                const uint32_t ph = (uint32_t)(fitem >> 1) & 1u;
                const int t = cl + (it - 1) * p.clusters;
                const float* recv_a = recv + (size_t)a * (RECV_BYTES / 4);
                ok = mbar_wait(&recv_full[a], ph, abort_p);
                if (!ok) break;
                if (tid == 0) { CH_STAMP(o, 5); }             // peers' rows have landed

                // one thread: one owned row of the tile, TK consecutive tokens, summed over the senders in rank order
                {
                    const int li = tid & (CH_ROWS - 1), c = (tid >> 4) * TK;
                    const int rr = cyclic ? li * CH_S + rank : rank * CH_ROWS + li;
                    float acc[TK];
#pragma unroll
                    for (int j = 0; j < TK; ++j) acc[j] = 0.f;
                    {
                        float part[CH_S][TK];
#pragma unroll
                        for (int s = 0; s < CH_S; ++s) {
                            const float* src = recv_a + (s * CH_ROWS + li) * RED_LD + c;
                            if (TK == 4) { const float4 f = *reinterpret_cast<const float4*>(src); part[s][0] = f.x; part[s][1] = f.y; part[s][TK - 2] = f.z; part[s][TK - 1] = f.w; }
                            else { const float2 f = *reinterpret_cast<const float2*>(src); part[s][0] = f.x; part[s][1] = f.y; }
                        }
#pragma unroll
                        for (int s = 0; s < CH_S; ++s) {
#pragma unroll
                            for (int j = 0; j < TK; ++j) acc[j] += part[s][j];
                        }
                    }
                    if (op.sq_in) {
#pragma unroll
                        for (int j = 0; j < TK; ++j) acc[j] *= rstd_s[c + j];
                    }
                    const int n = t * CH_BM + rr;
                    if (op.rope) {
                        if (n < op.N) {
                            const int D = op.head_dim, half = op.rotary_dim >> 1;
                            const int hd = n >> (31 - __clz(D)), d = n & (D - 1);
                            const bool rotated = hd < op.num_heads + op.num_kv_heads && d < op.rotary_dim;
                            float pacc[TK];
#pragma unroll
                            for (int j = 0; j < TK; ++j) pacc[j] = 0.f;
                            int np = n;
                            if (rotated) {
                                np = d < half ? n + half : n - half;
                                const int pli = li + ((np - n) >> 3);         // the partner's place in this block's slots
#pragma unroll
                                for (int s2 = 0; s2 < CH_S; ++s2) {
                                    const float* src = recv_a + (s2 * CH_ROWS + pli) * RED_LD + c;
#pragma unroll
                                    for (int j = 0; j < TK; ++j) pacc[j] += src[j];
                                }
                                if (op.sq_in) {
#pragma unroll
                                    for (int j = 0; j < TK; ++j) pacc[j] *= rstd_s[c + j];
                                }
                            }
                            const float b = op.bias ? load_tagged(op.bias, n, op.bias_tag) : 0.f;
                            const float bp = (op.bias && rotated) ? load_tagged(op.bias, np, op.bias_tag) : 0.f;
#pragma unroll
                            for (int j = 0; j < TK; ++j) {
                                const int tk = c + j;
                                if (tk >= p.M) continue;
                                float val = acc[j] + b;
                                if (rotated) {
                                    const int jj = d < half ? d : d - half;
                                    const float cs = rope_cs[tk * half + jj], sn = rope_cs[BN * half + tk * half + jj];
                                    const float other = pacc[j] + bp;
                                    val = d < half ? val * cs - other * sn : val * cs + other * sn;
                                }
                                if (hd < op.num_heads) {
                                    reinterpret_cast<bf16*>(op.out)[(int64_t)tk * op.N + n] = __float2bfloat16_rn(val);
                                } else if (op.write_cache) {
                                    const int slot = rope_slot[tk];
                                    if (slot < 0) continue;
                                    const int page = slot >> op.page_shift, off = slot & (op.page_size - 1);
                                    const bool is_k = hd < op.num_heads + op.num_kv_heads;
                                    const int kvh = hd - op.num_heads - (is_k ? 0 : op.num_kv_heads);
                                    const int64_t dst = (((int64_t)page * op.num_kv_heads + kvh) * op.page_size + off) * D + d;
                                    (is_k ? op.k_cache : op.v_cache)[dst] = __float2bfloat16_rn(val);
                                }
                            }
                        }
                    } else if (op.res) {
                        const bool live = n < op.N;
                        const float b = (op.bias && live) ? load_tagged(op.bias, n, op.bias_tag) : 0.f;
                        const float wn = (op.norm_w && live) ? load_tagged(op.norm_w, n, op.norm_w_tag) : 0.f;
                        float old[TK], sq[TK];
#pragma unroll
                        for (int j = 0; j < TK; ++j) old[j] = (live && c + j < p.M) ? __ldcg(op.res + (int64_t)(c + j) * op.N + n) : 0.f;
#pragma unroll
                        for (int j = 0; j < TK; ++j) {
                            sq[j] = 0.f;
                            if (live && c + j < p.M) {
                                const int64_t at = (int64_t)(c + j) * op.N + n;
                                const float rv = old[j] + acc[j] + b;
                                op.res[at] = rv;
                                if (op.xw_out) op.xw_out[at] = __float2bfloat16_rn(rv * wn);
                                sq[j] = rv * rv;
                            }
                        }
                        if (op.sq_out) {                      // 16 neighbouring lanes hold the same tokens and consecutive features
#pragma unroll
                            for (int off = 1; off <= 8; off <<= 1) {
#pragma unroll
                                for (int j = 0; j < TK; ++j) sq[j] += __shfl_xor_sync(0xffffffffu, sq[j], off);
                            }
                            if (li == 0) {
                                const int slot = t * CH_S + rank;
#pragma unroll
                                for (int j = 0; j < TK; ++j)
                                    if (c + j < op.sq_stride) op.sq_out[(int64_t)slot * op.sq_stride + c + j] = sq[j];
                            }
                        }
                    } else {
                        const float b = (op.bias && n < op.N) ? load_tagged(op.bias, n, op.bias_tag) : 0.f;
#pragma unroll
                        for (int j = 0; j < TK; ++j) {
                            const int tk = c + j;
                            const float val = acc[j] + b;
                            if (op.swiglu) {                  // gate on the even feature, up on the odd one: neighbouring lanes
                                const float other = __shfl_xor_sync(0xffffffffu, val, 1);
                                if (!(rr & 1) && tk < p.M && n < op.N)
                                    reinterpret_cast<bf16*>(op.out)[(int64_t)tk * (op.N / 2) + n / 2] = __float2bfloat16_rn(ch_silu_mul(val, other));
                            } else if (tk < p.M && n < op.N) {
                                reinterpret_cast<bf16*>(op.out)[(int64_t)tk * op.N + n] = __float2bfloat16_rn(val);
                            }
                        }
                    }
                }
                // these receive slots are read out: arm their barrier for their next tile and tell all eight senders
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (tid == 0) { CH_STAMP(o, 6); }             // owners' sum and epilogue of the last tile stored
                if (tid == 0) mbar_expect_tx(&recv_full[a], RECV_TX);
                if (tid < CH_S) mbar_arrive_remote(cluster_addr(smem_u32(&send_ok[a]), tid));
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 64) { CH_STAMP_BLOCK(1); }
    // Nobody may leave while a peer can still write into its shared memory or arrive on its barriers:
    // the whole cluster meets once more.  (A block that gave up still comes here.)
    cluster_sync_all();
    if (threadIdx.x == 0) {
        if (abort_flag) atomicExch(p.error, 1);
        __threadfence();
        const unsigned int left = atomicAdd(p.counters + CH_MAX_OPS, 1u);
        if (left == (unsigned)nblocks - 1u) {                 // the last block out: the counters go back to zero for the next launch
            for (int i = 0; i <= CH_MAX_OPS; ++i) p.counters[i] = 0u;
            __threadfence();
        }
    }
    if (abort_flag) for (int i = 0; i < 64; ++i) __nanosleep(2000);     // let copies that are still in flight land
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// --------------------------------------------------------------------------- host side

static int chain_make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
    cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t gstride[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {CH_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

// One product of a chain as the caller describes it (mirrored field by field by the Python wrapper).
struct ChainOpHost {
    const void* x; const void* w; const void* bias; int bias_tag; void* out; int N, K, swiglu;
    // rotation + cache write (positions non-null)
    const int* positions; const int* slots; const float* cos_t; const float* sin_t; void* k_cache; void* v_cache;
    int num_heads, num_kv_heads, head_dim, rotary_dim, page_size, max_pos, write_cache; long long num_pages;
    // residual epilogue (res non-null) and the norm that goes with it
    void* res; const void* norm_w; int norm_w_tag; void* xw_out; void* sq_out; int sq_stride;
    // deferred norm factor on the input
    const void* sq_in; int sq_slots, sq_in_stride; float sq_width, sq_eps;
};

static unsigned int* g_chain_counters[64] = {nullptr};
static int g_chain_clusters[64][2] = {{0}};      // per device and BN: clusters that fit at once (0 = not asked yet)

template <int BN>
static int chain_smem_plan(ChainParams& p, int x_tiles, bool any_rope, int max_rotary, size_t* smem_out) {
    const size_t A_BYTES = CH_BM * CH_BK * 2, B_BYTES = (size_t)BN * CH_BK * 2;
    const size_t recv = 2 * (size_t)CH_BM * (BN + 4) * 4;
    const size_t xb = ((size_t)x_tiles * B_BYTES + 1023) & ~(size_t)1023;
    const size_t tables = any_rope ? (size_t)BN * 2 * sizeof(int) + (size_t)BN * max_rotary * sizeof(float) : 0;
    const size_t rstd = (size_t)BN * sizeof(float);
    const size_t limit = 227 * 1024 - 1024 - 1024;             // less the alignment slack and the static barriers
    const size_t fixed = xb + recv + tables + rstd;
    if (fixed + 2 * A_BYTES > limit) return MIE_ERR_TOO_LARGE;
    int stages = (int)((limit - fixed) / A_BYTES);
    if (stages > CH_MAX_STAGES) stages = CH_MAX_STAGES;
    if (p.stages > 0 && p.stages < stages) stages = p.stages < 2 ? 2 : p.stages;
    p.stages = stages;
    p.x_tiles = x_tiles;
    p.x_off = (uint32_t)((size_t)stages * A_BYTES);
    p.recv_off = (uint32_t)(p.x_off + xb);
    p.table_off = (uint32_t)(p.recv_off + recv);
    p.rstd_off = (uint32_t)(p.table_off + tables);
    *smem_out = (size_t)p.rstd_off + rstd + 1024;
    return 0;
}

template <int BN>
static int chain_launch(const ChainMaps& maps, ChainParams& p, int x_tiles, bool any_rope, int max_rotary, int pdl, cudaStream_t stream) {
    size_t smem = 0;
    int rc = chain_smem_plan<BN>(p, x_tiles, any_rope, max_rotary, &smem);
    if (rc) return rc;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MIE_ERR_BAD_ARG;
    cudaError_t e = cudaFuncSetAttribute(gemm_chain_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(CH_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = CH_S; attrs[0].val.clusterDim.y = 1; attrs[0].val.clusterDim.z = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 1;
    int& fit = g_chain_clusters[dev][BN == 16 ? 0 : 1];
    if (fit == 0) {
        // every block spins on the others between products, so all of them must run at once: ask how many
        // clusters of 8 the device holds with this much shared memory (the largest the kernel may take)
        cudaFuncSetAttribute(gemm_chain_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024);
        cudaLaunchConfig_t probe = cfg;
        probe.gridDim = dim3(CH_S, device_sm_count() / CH_S);
        probe.dynamicSmemBytes = 227 * 1024 - 1024;
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, gemm_chain_kernel<BN>, &probe);
        if (e != cudaSuccess) return (int)e;
        fit = n < 1 ? -1 : (n > device_sm_count() / CH_S ? device_sm_count() / CH_S : n);
        e = cudaFuncSetAttribute(gemm_chain_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    if (fit < 1) return MIE_ERR_BAD_ARG;
    p.clusters = fit;
    cfg.gridDim = dim3(CH_S, fit);
    if (pdl) {
        attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 2;
    }
    e = cudaLaunchKernelEx(&cfg, gemm_chain_kernel<BN>, maps, p);
    return e != cudaSuccess ? (int)e : launch_status();
}

// Allocates what the chain kernel keeps between launches (its counters, once per device) and looks up
// the tensor-map encoder.  Call it once outside any stream capture; mie_gemm_chain calls it too.
extern "C" int mie_gemm_chain_setup(void) {
    int rc = tc_setup();
    if (rc) return rc;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MIE_ERR_BAD_ARG;
    if (!g_chain_counters[dev]) {
        unsigned int* c = nullptr;
        cudaError_t e = cudaMalloc((void**)&c, CH_COUNTERS * sizeof(unsigned int));
        if (e != cudaSuccess) return (int)e;
        e = cudaMemset(c, 0, CH_COUNTERS * sizeof(unsigned int));
        if (e != cudaSuccess) return (int)e;
        g_chain_counters[dev] = c;
    }
    return 0;
}

// How many clusters of 8 blocks the chain kernel runs as on the current device (after a first launch).
extern "C" int mie_gemm_chain_clusters(int bn) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    return g_chain_clusters[dev][bn == 16 ? 0 : 1];
}

// Runs `num_ops` (1..4) products one after the other in one launch; product i + 1 may read what
// product i wrote.  M tokens (1..32), every x [M, K_i] and w [N_i, K_i] bfloat16, contiguous, 16-byte
// aligned, K_i % 8 == 0, N_i % 8 == 0 (N_i % 16 == 0 with swiglu).  `stages` > 0 caps the ring's depth.
extern "C" int mie_gemm_chain(const ChainOpHost* ops, int num_ops, int M, int stages, int pdl, cudaStream_t stream) {
    if (num_ops < 1 || num_ops > CH_MAX_OPS || M < 1 || M > 32) return MIE_ERR_BAD_ARG;
    int rc = mie_gemm_chain_setup();
    if (rc) return rc;
    int dev = 0;
    cudaGetDevice(&dev);
    const int bn = M <= 16 ? 16 : 32;
    ChainMaps maps;
    ChainParams p;
    p.num_ops = num_ops; p.M = M; p.stages = stages; p.counters = g_chain_counters[dev]; p.error = g_error_dev;
    p.report = g_range_report;
    int x_tiles = 1, max_rotary = 0;
    bool any_rope = false;
    for (int i = 0; i < num_ops; ++i) {
        const ChainOpHost& h = ops[i];
        ChainOp& o = p.ops[i];
        if (h.N <= 0 || h.K <= 0 || h.K % 8 || h.N % 8 || (h.swiglu && h.N % 16)) return MIE_ERR_BAD_ARG;
        if ((reinterpret_cast<uintptr_t>(h.x) | reinterpret_cast<uintptr_t>(h.w)) & 15) return MIE_ERR_BAD_ARG;
        if (!h.res && (!h.out || (reinterpret_cast<uintptr_t>(h.out) & 15))) return MIE_ERR_BAD_ARG;
        o.N = h.N; o.K = h.K;
        o.k_tiles = (h.K + CH_BK - 1) / CH_BK;
        o.tiles_per_split = (o.k_tiles + CH_S - 1) / CH_S;
        o.n_tiles = (h.N + CH_BM - 1) / CH_BM;
        if (o.tiles_per_split > x_tiles) x_tiles = o.tiles_per_split;
        o.out = h.out; o.bias = h.bias; o.bias_tag = h.bias_tag; o.swiglu = h.swiglu;
        o.rope = h.positions != nullptr;
        o.positions = h.positions; o.slots = h.slots; o.cos_t = h.cos_t; o.sin_t = h.sin_t;
        o.k_cache = (bf16*)h.k_cache; o.v_cache = (bf16*)h.v_cache;
        o.num_heads = h.num_heads; o.num_kv_heads = h.num_kv_heads; o.head_dim = h.head_dim; o.rotary_dim = h.rotary_dim;
        o.page_size = h.page_size; o.max_pos = h.max_pos; o.write_cache = h.write_cache;
        o.num_pages = h.num_pages > 0 ? h.num_pages : (1ll << 40);
        o.page_shift = 0;
        if (o.rope) {
            // heads must not straddle tiles, and a row and its rotation partner must share an owner (every 8th row)
            if (h.swiglu || h.res || h.head_dim <= 0 || CH_BM % h.head_dim || (h.rotary_dim & 1) || h.rotary_dim > h.head_dim ||
                (h.rotary_dim / 2) % CH_S || (h.num_heads + 2 * h.num_kv_heads) * h.head_dim != h.N)
                return MIE_ERR_BAD_ARG;
            if (h.page_size < 1 || (h.page_size & (h.page_size - 1))) return MIE_ERR_BAD_ARG;
            while ((1 << o.page_shift) < h.page_size) ++o.page_shift;
            any_rope = true;
            if (h.rotary_dim > max_rotary) max_rotary = h.rotary_dim;
        }
        o.res = (float*)h.res; o.norm_w = h.norm_w; o.norm_w_tag = h.norm_w_tag; o.xw_out = (bf16*)h.xw_out;
        o.sq_out = (float*)h.sq_out; o.sq_stride = h.sq_stride;
        if (h.res) {
            if (h.swiglu || (reinterpret_cast<uintptr_t>(h.res) & 15)) return MIE_ERR_BAD_ARG;
            if ((h.xw_out != nullptr) != (h.norm_w != nullptr) || (h.sq_out && !h.xw_out)) return MIE_ERR_BAD_ARG;
            if (h.sq_out && h.sq_stride < M) return MIE_ERR_BAD_ARG;
        }
        o.sq_in = (const float*)h.sq_in; o.sq_slots = h.sq_slots; o.sq_in_stride = h.sq_in_stride;
        o.sq_width = h.sq_width; o.sq_eps = h.sq_eps;
        if (h.sq_in && (h.sq_slots < 1 || h.sq_in_stride < M || !(h.sq_width > 0.f))) return MIE_ERR_BAD_ARG;
        if ((rc = chain_make_map(&maps.w[i], h.w, h.N, h.K, CH_BM))) return rc;
        if ((rc = chain_make_map(&maps.x[i], h.x, M, h.K, bn))) return rc;
    }
    for (int i = num_ops; i < CH_MAX_OPS; ++i) { maps.w[i] = maps.w[0]; maps.x[i] = maps.x[0]; p.ops[i] = p.ops[0]; }
    if ((size_t)bn * max_rotary * sizeof(float) > 16 * 1024) return MIE_ERR_BAD_ARG;
    if (bn == 16) return chain_launch<16>(maps, p, x_tiles, any_rope, max_rotary, pdl, stream);
    return chain_launch<32>(maps, p, x_tiles, any_rope, max_rotary, pdl, stream);
}

extern "C" int mie_gemm_chain_error(void) { return g_error_host ? *g_error_host : 0; }
extern "C" void mie_gemm_chain_clear_error(void) { if (g_error_host) *g_error_host = 0; }

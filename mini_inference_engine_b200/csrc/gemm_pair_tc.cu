// The matrix product for many tokens, y[M, N] = x[M, K] w[N, K]^T, on pairs of SMs (bfloat16 operands, float32
// accumulation, sm_100a).  The reference calls the vendor library for every product (F.linear,
// inference_engine/model.py:172,178,180,181,185); this is the package's own kernel for prompt-sized M.
//
// Two blocks form a cluster and work on one 256 x 256 tile of y with cta_group::2 instructions: block r of
// the pair holds 128 rows of x (tokens) and 128 rows of w (half of the tile's 256 output features) per
// 64-wide k-tile, 32 KB a stage instead of the 48 KB a lone block needs for 128 x 256, and the pair's MMA
// (M = 256, N = 256, K = 16) reads both halves of w from the two shared memories.  Each block's tensor
// memory holds its 128 rows x 256 columns of the tile, twice: the pair runs persistently over tiles
// pair, pair + pairs, ... (tokens fastest, so that the pairs of a wave share a panel of w), and while the
// four epilogue warps of both blocks take accumulator b out of tensor memory the MMAs of the next tile
// fill accumulator b ^ 1 and the copies run further ahead still.
//
// Roles per block (192 threads): warp 0 lane 0 issues this block's TMA copies (their bytes are counted on
// the `full` barrier of the leader, block 0 of the pair, whose copy instruction names it: that is what
// `.cta_group::2` on a copy allows); warp 1 lane 0 of the LEADER issues the MMAs and commits them to the
// `empty` and `acc_full` barriers of both blocks (one commit each, the peer's by its cluster address);
// warps 2 - 5 are the epilogue (a thread a row) and give the accumulator back on the leader's `acc_empty`.
// Every wait is bounded; a block that gives up raises the error word and leaves.
//
// Epilogues: bias; SwiGLU on interleaved rows of w (row 2i the gate, 2i + 1 the value: y has N / 2
// columns); float32 or bfloat16 output; the two halves of an RMSNorm without a kernel of its own, as in the
// few-token product (csrc/gemm_tcgen05.cu): with `res` the product is added to the float32 residual stream in
// place and, for the norm that reads the stream next, xw = bfloat16(res * norm_weight) and the row's share of
// sum(res^2) over this tile's columns go out (one slot per 256-column tile: sq_out[tile_n][row]); with `sq_in`
// the float32 sums are scaled by rsqrt(sum over slots / width + eps) before anything else, which is that norm
// applied to the operand x = xw of a producer (a row factor commutes with the product).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tcgen05_common.cuh"

typedef __nv_bfloat16 bf16;

#define GP_THREADS 192
#define GP_BM 128                 // rows of x per block; the pair's tile is 256 rows
#define GP_BNH 128                // rows of w per block; the pair's tile is 256 columns
#define GP_BK 64
#define GP_MAX_STAGES 6
#define GP_STAGE_BYTES 32768u     // 16 KB of x and 16 KB of w per block and k-tile

struct GpParams {
    void* out;               // [M, N] (or [M, N / 2] with SwiGLU), bfloat16 or float32
    const void* bias;        // [N] or null
    int bias_tag, out_f32, swiglu;
    int M, N, K;
    int tiles_m, num_tiles, k_tiles, stages;
    int* error;
    float* res; const void* norm_w; int norm_w_tag; bf16* xw_out; float* sq_out; int sq_stride;
    const float* sq_in; int sq_slots, sq_in_stride; float sq_width, sq_eps;
};

__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t leader_bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(leader_bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// All MMAs this thread has issued so far arrive, when they are complete, on the barrier at this offset in BOTH
// blocks of the pair (an arrival sent to several blocks of the cluster; no data moves).
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void tmem_ld32(uint32_t addr, float* v) {
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
                   "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
                   "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(addr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__global__ void __launch_bounds__(GP_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const GpParams p) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t full[GP_MAX_STAGES], empty[GP_MAX_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;       // tiles on 1024-byte lines (128-byte swizzle)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();                                // 0: the leader of the pair
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int S = p.stages;
    volatile int* abort_p = &abort_flag;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < GP_MAX_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }   // 4 epilogue warps of 2 blocks
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();                  // both blocks' barriers exist before a copy or a commit of the peer names them
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    pdl_wait();

    if (warp == 0) {
        // ---- producer: this block's half of every k-tile, counted on the leader's barrier (the warp as a whole
        // walks the loop, an elected lane issues)
        int s = 0;
        uint32_t round = 0;
        const uint32_t bar0 = cluster_addr(smem_u32(&full[0]), 0);
        bool ok = true;
        for (int tile = pair; tile < p.num_tiles && ok; tile += pairs) {
            const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
            const int row_x = tm * 2 * GP_BM + (int)rank * GP_BM, row_w = tn * 2 * GP_BNH + (int)rank * GP_BNH;
            for (int kt = 0; kt < p.k_tiles; ++kt) {
                if (round > 0 && !__all_sync(0xffffffffu, mbar_wait(&empty[s], (round - 1) & 1, abort_p))) { ok = false; break; }
                if (elect_one()) {
                    if (rank == 0) mbar_expect_tx(&full[s], 2 * GP_STAGE_BYTES);
                    const uint32_t bar = bar0 + (uint32_t)s * 8u;
                    const uint32_t dst = base + (uint32_t)s * GP_STAGE_BYTES;
                    tma_load_2d_pair(dst, &map_x, bar, kt * GP_BK, row_x);
                    tma_load_2d_pair(dst + GP_STAGE_BYTES / 2, &map_w, bar, kt * GP_BK, row_w);
                }
                __syncwarp();
                if (++s == S) { s = 0; ++round; }
            }
        }
    } else if (warp == 1) {
        if (rank == 0) {
            // ---- the pair's MMAs: 256 x 256 x 16, four per k-tile; the whole warp walks the loop, one lane issues
            const uint32_t idesc = umma_idesc_bf16(2 * GP_BM, 2 * GP_BNH);
            const uint64_t da0 = umma_desc_sw128(base), db0 = umma_desc_sw128(base + GP_STAGE_BYTES / 2);
            constexpr uint64_t STAGE_STEP = GP_STAGE_BYTES >> 4;       // descriptors of another stage differ in the address field
            int s = 0, t_local = 0;
            uint32_t round = 0;
            uint64_t da = da0, db = db0;
            bool ok = true;
            for (int tile = pair; tile < p.num_tiles && ok; tile += pairs, ++t_local) {
                const int buf = t_local & 1, use = t_local >> 1;
                if (use > 0 && !__all_sync(0xffffffffu, mbar_wait(&acc_empty[buf], (use - 1) & 1, abort_p))) break;   // both epilogues have read it
                tc_fence_after();
                const uint32_t d_at = tmem_base + (uint32_t)buf * 256u;
                for (int kt = 0; kt < p.k_tiles; ++kt) {
                    if (!__all_sync(0xffffffffu, mbar_wait(&full[s], round & 1, abort_p))) { ok = false; break; }
                    if (elect_one()) {
#pragma unroll
                        for (int ks = 0; ks < GP_BK / 16; ++ks)
                            umma_bf16_pair(d_at, da + (uint64_t)(ks * 2), db + (uint64_t)(ks * 2), idesc, (kt > 0 || ks > 0) ? 1u : 0u);
                        umma_commit_pair(&empty[s]);                   // the stage is free in both blocks once these are done
                    }
                    __syncwarp();
                    if (++s == S) { s = 0; ++round; da = da0; db = db0; }
                    else { da += STAGE_STEP; db += STAGE_STEP; }
                }
                if (ok && elect_one()) umma_commit_pair(&acc_full[buf]);
                __syncwarp();
            }
        }
    } else {
        // ---- epilogue: a thread a row of this block's 128; 256 columns in eight loads of 32
        const int q = warp & 3;                                          // the quarter of tensor memory this warp may read
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        const uint32_t acc_empty_leader[2] = {cluster_addr(smem_u32(&acc_empty[0]), 0), cluster_addr(smem_u32(&acc_empty[1]), 0)};
        int t_local = 0;
        for (int tile = pair; tile < p.num_tiles; tile += pairs, ++t_local) {
            const int buf = t_local & 1, use = t_local >> 1;
            const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
            if (!__all_sync(0xffffffffu, mbar_wait(&acc_full[buf], use & 1, abort_p))) break;
            tc_fence_after();
            const int row = tm * 2 * GP_BM + (int)rank * GP_BM + q * 32 + lane;
            const int col0 = tn * 2 * GP_BNH;
            float rstd = 1.f, ssq = 0.f;
            if (p.sq_in && row < p.M) {                                  // the norm in front of this product, as a row factor
                float sum = 0.f;
                for (int sl = 0; sl < p.sq_slots; ++sl) sum += __ldcg(p.sq_in + (int64_t)sl * p.sq_in_stride + row);
                rstd = rsqrtf(sum / p.sq_width + p.sq_eps);
            }
#pragma unroll 1
            for (int c = 0; c < 2 * GP_BNH; c += 32) {
                float v[32];
                tmem_ld32(lane_addr + (uint32_t)buf * 256u + (uint32_t)c, v);
                const int col = col0 + c;
                if (row >= p.M || col >= p.N) continue;
                if (p.sq_in) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] *= rstd;
                }
                if (p.bias) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) if (col + i < p.N) v[i] += load_tagged(p.bias, col + i, p.bias_tag);
                }
                if (p.res) {
                    // the stream takes the sum; the next norm's operand and its sum of squares ride along
                    float* rp = p.res + (int64_t)row * p.N + col;
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        if (col + i >= p.N) break;
                        float4 r = *reinterpret_cast<const float4*>(rp + i);
                        r.x += v[i]; r.y += v[i + 1]; r.z += v[i + 2]; r.w += v[i + 3];
                        *reinterpret_cast<float4*>(rp + i) = r;
                        v[i] = r.x; v[i + 1] = r.y; v[i + 2] = r.z; v[i + 3] = r.w;
                        ssq += r.x * r.x + r.y * r.y + r.z * r.z + r.w * r.w;
                    }
                    if (p.xw_out) {
                        bf16* op = p.xw_out + (int64_t)row * p.N + col;
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            if (col + i >= p.N) break;
                            float wn[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) wn[j] = load_tagged(p.norm_w, col + i + j, p.norm_w_tag);
                            uint4 w;
                            w.x = pack_bf16x2(v[i] * wn[0], v[i + 1] * wn[1]); w.y = pack_bf16x2(v[i + 2] * wn[2], v[i + 3] * wn[3]);
                            w.z = pack_bf16x2(v[i + 4] * wn[4], v[i + 5] * wn[5]); w.w = pack_bf16x2(v[i + 6] * wn[6], v[i + 7] * wn[7]);
                            *reinterpret_cast<uint4*>(op + i) = w;
                        }
                    }
                    continue;
                }
                if (p.swiglu) {
                    // interleaved rows of w: column 2i the gate, 2i + 1 the value
                    float o[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float g = v[2 * i], u = v[2 * i + 1];
                        o[i] = __fdividef(g, 1.f + __expf(-g)) * u;
                    }
                    const int64_t at = (int64_t)row * (p.N / 2) + col / 2;
                    if (p.out_f32) {
                        float* op = reinterpret_cast<float*>(p.out) + at;
#pragma unroll
                        for (int i = 0; i < 16; i += 4)
                            if (col + 2 * i < p.N) *reinterpret_cast<float4*>(op + i) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
                    } else {
                        bf16* op = reinterpret_cast<bf16*>(p.out) + at;
#pragma unroll
                        for (int i = 0; i < 16; i += 8) {
                            if (col + 2 * i >= p.N) break;
                            uint4 w;
                            w.x = pack_bf16x2(o[i], o[i + 1]); w.y = pack_bf16x2(o[i + 2], o[i + 3]);
                            w.z = pack_bf16x2(o[i + 4], o[i + 5]); w.w = pack_bf16x2(o[i + 6], o[i + 7]);
                            *reinterpret_cast<uint4*>(op + i) = w;
                        }
                    }
                } else if (p.out_f32) {
                    float* op = reinterpret_cast<float*>(p.out) + (int64_t)row * p.N + col;
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        if (col + i < p.N) *reinterpret_cast<float4*>(op + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                } else {
                    bf16* op = reinterpret_cast<bf16*>(p.out) + (int64_t)row * p.N + col;
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        if (col + i >= p.N) break;
                        uint4 w;
                        w.x = pack_bf16x2(v[i], v[i + 1]); w.y = pack_bf16x2(v[i + 2], v[i + 3]);
                        w.z = pack_bf16x2(v[i + 4], v[i + 5]); w.w = pack_bf16x2(v[i + 6], v[i + 7]);
                        *reinterpret_cast<uint4*>(op + i) = w;
                    }
                }
            }
            if (p.sq_out && row < p.M) p.sq_out[(int64_t)tn * p.sq_stride + row] = ssq;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_leader[buf]);
        }
    }

    // Nobody leaves while the peer may still read this block's shared memory (the leader's MMAs read both) or
    // signal its barriers; a block that gave up says so and lets copies in flight land first.
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        if (threadIdx.x == 0) atomicExch(p.error, 1);
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    cluster_sync_all();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

// --------------------------------------------------------------------------- host side

static int make_map_rows(CUtensorMap* map, const void* ptr, int rows, int K) {
    cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t gstride[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {GP_BK, 128};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

// The fused epilogues (see the header): the layout the few-token product's entry point takes.
struct GpFuse {
    void* res; const void* norm_w; int norm_w_tag; void* xw_out; void* sq_out; int sq_stride;
    const void* sq_in; int sq_slots; int sq_in_stride; float sq_width; float sq_eps;
};

// How many slots of sum(res^2) a product with N columns leaves per row (one per 256-column tile).
extern "C" int mie_gemm_pair_slots(int N) { return (N + 2 * GP_BNH - 1) / (2 * GP_BNH); }

// y = x w^T (+ bias) (then SwiGLU over interleaved columns).  x [M, K], w [N, K] bfloat16 row-major, K % 8 == 0,
// N % 8 == 0 (N % 16 == 0 with SwiGLU), all pointers 16-byte aligned.  y_tag: MIE_BF16 or MIE_F32.  With
// fuse->res, y is not written (may be null): res [M, N] float32 += the product; with fuse->norm_w also
// xw_out [M, N] bfloat16 and sq_out [mie_gemm_pair_slots(N)][sq_stride >= M] float32.  With fuse->sq_in
// [sq_slots][sq_in_stride >= M] the sums are scaled by rsqrt(sum over slots / sq_width + sq_eps) first.
extern "C" int mie_gemm_pair(const void* x, const void* w, const void* bias, int bias_tag, void* y, int y_tag, int M, int N,
                             int K, int swiglu, const GpFuse* fuse, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (K % 8 || N % 8 || (swiglu && N % 16)) return MIE_ERR_BAD_ARG;
    const bool into_stream = fuse && fuse->res;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | (into_stream ? 0 : reinterpret_cast<uintptr_t>(y))) & 15) return MIE_ERR_BAD_ARG;
    if (!into_stream && (!y || (y_tag != MIE_BF16 && y_tag != MIE_F32))) return MIE_ERR_BAD_ARG;
    if (into_stream) {
        if (swiglu || (reinterpret_cast<uintptr_t>(fuse->res) & 15)) return MIE_ERR_BAD_ARG;
        if ((fuse->xw_out != nullptr) != (fuse->norm_w != nullptr) || (fuse->sq_out != nullptr) != (fuse->norm_w != nullptr)) return MIE_ERR_BAD_ARG;
        if (fuse->norm_w && (fuse->sq_stride < M || (reinterpret_cast<uintptr_t>(fuse->xw_out) & 15))) return MIE_ERR_BAD_ARG;
    }
    if (fuse && fuse->sq_in && (fuse->sq_slots < 1 || fuse->sq_in_stride < M || !(fuse->sq_width > 0.f))) return MIE_ERR_BAD_ARG;
    int rc = tc_setup();
    if (rc) return rc;
    CUtensorMap mx, mw;
    if ((rc = make_map_rows(&mx, x, M, K))) return rc;
    if ((rc = make_map_rows(&mw, w, N, K))) return rc;
    GpParams p;
    p.out = y; p.bias = bias; p.bias_tag = bias_tag; p.out_f32 = y_tag == MIE_F32; p.swiglu = swiglu ? 1 : 0;
    p.M = M; p.N = N; p.K = K;
    p.tiles_m = (M + 2 * GP_BM - 1) / (2 * GP_BM);
    p.num_tiles = p.tiles_m * ((N + 2 * GP_BNH - 1) / (2 * GP_BNH));
    p.k_tiles = (K + GP_BK - 1) / GP_BK;
    p.stages = GP_MAX_STAGES;
    p.error = g_error_dev;
    p.res = nullptr; p.norm_w = nullptr; p.norm_w_tag = 0; p.xw_out = nullptr; p.sq_out = nullptr; p.sq_stride = 0;
    p.sq_in = nullptr; p.sq_slots = 0; p.sq_in_stride = 0; p.sq_width = 1.f; p.sq_eps = 0.f;
    if (fuse) {
        p.res = (float*)fuse->res; p.norm_w = fuse->norm_w; p.norm_w_tag = fuse->norm_w_tag;
        p.xw_out = (bf16*)fuse->xw_out; p.sq_out = (float*)fuse->sq_out; p.sq_stride = fuse->sq_stride;
        p.sq_in = (const float*)fuse->sq_in; p.sq_slots = fuse->sq_slots; p.sq_in_stride = fuse->sq_in_stride;
        p.sq_width = fuse->sq_width; p.sq_eps = fuse->sq_eps;
    }
    const size_t smem = (size_t)p.stages * GP_STAGE_BYTES + 1024;
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    int pairs = device_sm_count() / 2;
    if (pairs > p.num_tiles) pairs = p.num_tiles;
    return launch_kernel_cluster(gemm_pair_kernel, dim3(2 * pairs), dim3(GP_THREADS), smem, stream, dim3(2, 1, 1), mx, mw, p);
}

extern "C" int mie_gemm_pair_error(void) { return g_error_host ? *g_error_host : 0; }
extern "C" void mie_gemm_pair_clear_error(void) { if (g_error_host) *g_error_host = 0; }

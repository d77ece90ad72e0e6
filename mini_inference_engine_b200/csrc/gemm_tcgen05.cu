// y[M, N] = x[M, K] * W[N, K]^T (+ bias) in bfloat16 on the 5th-generation tensor cores:
// tcgen05.mma issued by one thread, operands staged in shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle), the float32 accumulator in tensor memory (TMEM), read
// back with tcgen05.ld for the epilogue.  The reference calls the vendor library for these products
// (F.linear, inference_engine/model.py:172,178,180,181,185).
//
// Both operands are K-major (x rows and W rows are contiguous in K), so one kernel serves both
// orientations of the 128-row MMA:
//   NORMAL  (many tokens):  MMA rows = 128 tokens, MMA columns = BN output features.
//   SWAPPED (few tokens, decode): MMA rows = 128 output features (the weight streams through the
//           128-row operand at full tile height), MMA columns = the tokens padded to BN in
//           {16, 32, 64, 128, 256}.  The step is then pure weight streaming.
//
// Split-K without scratch memory: the blocks that share an output tile form a thread-block cluster
// along grid.z (2, 4 or 8 blocks), and every block owns a share of the tile's rows.  SWAPPED (the
// decode path, where the tail of the kernel is most of its time): each block sends its float32
// partial rows straight from TMEM into the owner's shared memory (st.async to shared::cluster, one
// slot per sender, every store counted on the owner's own mbarrier), and the owner adds up its slots
// locally as soon as its 128 x BN sums have landed: no barrier across the cluster.  NORMAL: each
// block leaves its partial tile in its own shared memory and, after a barrier, reads its share out
// of the others' (ld.shared::cluster); a second barrier keeps everyone's memory alive meanwhile.
// Either way the sum runs in rank order -- the same order every time -- with no global partial
// sums, no atomics and no second kernel.  SWAPPED with 64 tokens or more (BN >= 64): a block owns
// TOKENS, not rows -- BN / splits tokens of every row of the tile.  Its peers stage their partial
// tile in their own shared memory, laid out by owner, and send each owner its 4 KB with ONE bulk copy
// (cp.async.bulk shared::cta -> shared::cluster, counted on the owner's mbarrier) instead of two
// thousand 16-byte remote stores; the owner's thread r adds up row r for its tokens, and what it then
// writes -- a token's features, side by side across the warp -- is contiguous in memory.
//
// Programmatic dependent launch: the kernel lets its successor start at once
// (griddepcontrol.launch_dependents) and itself may start while its predecessor still runs.  Weights
// do not depend on the predecessor, so the producer fills the whole shared-memory ring with weight
// tiles first and only then waits for the predecessor (griddepcontrol.wait) to fetch the activations:
// the weight stream of one product overlaps the tail of the kernel before it.
//
// Optional rotation epilogue for the fused q|k|v projection (few tokens, split-K): the block that adds
// up a row of the tile also adds up the row's rotation partner (rotate-half pairs are half a head
// apart, inside the same 128-row tile when the head size divides 128), rotates by the token's
// position, and writes q to the activation and k, v straight into their cache pages -- the work of the
// separate rotation kernel (inference_engine/model.py:174-176,130-134), on float32 sums.
//
// Optional residual epilogue, and the norm that goes with it (few tokens, split-K): the owner of a
// row adds its sum to the float32 residual stream, res += y, in place.  For the RMSNorm that reads
// the stream next it also writes xw = bf16(res * norm_weight) and its share of sum(res^2) per token
// into a slot of its own (sq_out[slot][token]; slots = 128-row tiles x max(splits, 4)).  The product
// that consumes xw then owes the factor rsqrt(mean(res^2) + eps), which is a scalar per token and so
// commutes with the product: it adds up the slots (in slot order) while its weights stream and scales
// its float32 sums by it before bias, rotation or SwiGLU.  Two kernels fewer per layer than norm
// kernels between the products (inference_engine/model.py:169-184 launches a fused add+norm there).
//
// Optional SwiGLU epilogue: with gate and up rows interleaved in W (row 2i = gate_i, row 2i+1 = up_i)
// the epilogue writes silu(gate) * up, N/2 wide, from the float32 accumulators
// (inference_engine/model.py:180-181 does this with two more kernels on rounded values).
//
// Roles in a block of 6 warps: warp 0 = TMA producer (one lane), warp 1 = TMEM owner and MMA issuer
// (one lane), warps 2..5 = epilogue (each reads the TMEM lane quarter warp_id % 4).  A ring of
// `stages` shared-memory slots is handed back and forth through mbarriers: full[s] (TMA bytes have
// landed) and empty[s] (tcgen05.commit: the MMAs that read the slot are done).
//
// Every wait on an mbarrier is bounded: after WAIT_LIMIT_CYCLES the block raises an error word in
// host-visible memory, stops issuing work, lets copies in flight land, still takes part in the
// cluster's barriers, frees its TMEM and returns.
#include "tcgen05_common.cuh"
#include "range_check.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_MAX_STAGES 8
#define TC_THREADS 192


struct TcParams {
    void* out;               // [M, N] (or [M, N/2] with the SwiGLU epilogue) bfloat16 or float32
    const void* bias;        // [N] or null
    int bias_tag;
    int* error;              // host-visible error word
    int M, N, K;             // tokens, output features (rows of W), inner size
    int k_tiles, tiles_per_split, splits, stages;
    int l2_ahead;            // weight k-tiles beyond the ring that the copy warp asks into L2 before the dependency wait
    int swiglu;              // 1: rows 2i / 2i+1 of W are gate_i / up_i; the output is silu(gate) * up, N/2 wide
    // Optional fused rotation + cache write for a q|k|v projection (see the header comment): rows of W
    // are [heads*D of q | kv_heads*D of k | kv_heads*D of v]; q is rotated and written to `out`, k is
    // rotated and v copied into their cache pages at slots[token]; the k and v columns of `out` are not
    // written.
    int rope;
    const int* positions; const int* slots;
    const float* cos_t; const float* sin_t;          // [max_pos, rotary_dim / 2]
    bf16* k_cache; bf16* v_cache;                    // [pages, kv_heads, page_size, head_dim]
    int num_heads, num_kv_heads, head_dim, rotary_dim, page_size, page_shift, max_pos, write_cache;
    int64_t num_pages;                               // pages in each cache, for the range check of the slots
    int* report;                                     // range report (range_check.cuh)
    uint32_t rope_smem_offset;                       // where the rotation's tables start inside dynamic shared memory
    uint32_t recv_smem_offset;                       // with `push`: where the slots for the peers' partial rows start
    int push;                                        // split-K by sending partial rows to their owners (SWAPPED, when the slots fit)
    // Optional residual epilogue (see the header comment): res [M, N] float32 in place; with norm_w also
    // xw_out [M, N] bfloat16 and sq_out [tiles * max(splits, 4)][sq_stride] float32.  `out` is not written.
    float* res; const void* norm_w; int norm_w_tag; bf16* xw_out; float* sq_out; int sq_stride;
    // Optional: the input x is xw of an earlier residual epilogue; scale the sums of token t by
    // rsqrt(sum over slots of sq_in[slot][t] / sq_width + sq_eps).
    const float* sq_in; int sq_slots, sq_in_stride; float sq_width, sq_eps;
    uint32_t rstd_smem_offset;
};

template <bool OUT_F32>
__device__ __forceinline__ void store_out(void* out, int64_t idx, float v) {
    if (OUT_F32) reinterpret_cast<float*>(out)[idx] = v;
    else reinterpret_cast<bf16*>(out)[idx] = __float2bfloat16_rn(v);
}

// 16 consecutive output columns of one row, starting at a multiple of 8 (N % 8 == 0, so groups of 8
// are wholly inside or outside the row).
template <bool OUT_F32>
__device__ __forceinline__ void store_row16(void* out, int64_t row_off, int n, int N, const float* v) {
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        if (n + g * 8 >= N) return;
        if (OUT_F32) {
            float4* p = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + row_off + n + g * 8);
            p[0] = make_float4(v[g * 8], v[g * 8 + 1], v[g * 8 + 2], v[g * 8 + 3]);
            p[1] = make_float4(v[g * 8 + 4], v[g * 8 + 5], v[g * 8 + 6], v[g * 8 + 7]);
        } else {
            uint4 w;
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
            for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[g * 8 + 2 * i], v[g * 8 + 2 * i + 1]);
            *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(out) + row_off + n + g * 8) = w;
        }
    }
}


__device__ __forceinline__ void grid_dep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// silu(g) * u with the fast exponential and division (a few ulp; the result is rounded to bfloat16 or
// added to float32 sums of bfloat16 products)
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

template <int BN, bool SWAPPED, bool OUT_F32>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a,     // the 128-row operand: x (NORMAL) or W (SWAPPED)
               const __grid_constant__ CUtensorMap map_b,     // the BN-row operand:  W (NORMAL) or x (SWAPPED)
               const TcParams p) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t full_bar[TC_MAX_STAGES];
    __shared__ __align__(8) uint64_t empty_bar[TC_MAX_STAGES];
    __shared__ __align__(8) uint64_t tmem_full_bar;
    __shared__ __align__(8) uint64_t recv_bar;               // push: counts the bytes of the peers' partial rows as they land
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    constexpr int RED_LD = BN + 4;                            // padded row of the float32 partial tile, 16-byte aligned
    const uint32_t tiles_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;        // swizzled tiles sit on 1024-byte lines
    unsigned char* tiles = smem_dyn + (tiles_base - smem_u32(smem_dyn));
    // behind the ring (only with the rotation epilogue): positions, slots, cos | sin rows of the tile's tokens
    int* rope_pos = reinterpret_cast<int*>(tiles + p.rope_smem_offset);
    int* rope_slot = rope_pos + BN;
    float* rope_cs = reinterpret_cast<float*>(rope_slot + BN);
    float* rstd_s = reinterpret_cast<float*>(tiles + p.rstd_smem_offset);      // [BN], only with sq_in

    grid_dep_launch_dependents();                             // the next kernel may start its own prologue now
    // SWAPPED split-K sends partial rows into the peers' shared memory.  A block may be written to only
    // once it runs: everybody arrives here, and waits (long since satisfied) before its first send.
    const bool push = SWAPPED && p.push;
    // tokens, not rows, are owned (see the header comment): 4 to 16 tokens per owner
    const int tpo = BN / (p.splits > 0 ? p.splits : 1);
    const bool tok = push && BN >= 64 && tpo >= 4 && tpo <= 16;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a0 = blockIdx.x * TC_BM;          // first row of the 128-row operand
    const int b0 = blockIdx.y * BN;             // first row of the BN-row operand
    const int split = blockIdx.z;               // = rank in the cluster
    const int kt0 = split * p.tiles_per_split;
    const int kt1 = min(p.k_tiles, kt0 + p.tiles_per_split);
    const int n_kt = kt1 - kt0;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < p.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&tmem_full_bar, 1);
        mbar_init(&recv_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the barriers are used by the TMA unit
        // what this block is owed: every block of the cluster sends it rows_per rows of BN sums
        if (push) mbar_expect_tx(&recv_bar, (uint32_t)(TC_BM * BN * sizeof(float)));
    }
    // Peers write into this block's memory and count on its barrier: both must exist first.  Everybody
    // arrives here (thread 0 after it has set the barriers up) and waits, long since satisfied, before
    // its first send.
    if (push) cluster_arrive_release();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* abort_p = &abort_flag;
    float pre_res[4] = {0.f, 0.f, 0.f, 0.f}, pre_wn = 0.f, pre_b = 0.f;     // residual epilogue: fetched ahead by the epilogue warps

    // The copy warp and the MMA warp walk their loops as whole warps and an elected lane issues: what feeds the
    // TMA and tensor-core instructions (descriptors, coordinates, barrier addresses, counters) then stays uniform
    // across the warp.  Issued from a loop that one lane ran alone, each tcgen05.mma cost that lane 90 - 150 cycles,
    // which the last k-tiles of a product pay in full (nothing else is left to hide them).
    if (warp == 0) {
        {
            // weights first: they do not depend on the kernel before this one
            const bool issuer = elect_one();
            const CUtensorMap* map_w = SWAPPED ? &map_a : &map_b;
            const CUtensorMap* map_x = SWAPPED ? &map_b : &map_a;
            const uint32_t w_off = SWAPPED ? 0 : A_BYTES, x_off = SWAPPED ? A_BYTES : 0;
            const int w0 = SWAPPED ? a0 : b0, x0 = SWAPPED ? b0 : a0;
            const int ahead = min(n_kt, p.stages);
            if (issuer) {
                for (int it = 0; it < ahead; ++it) {
                    mbar_expect_tx(&full_bar[it], STAGE_BYTES);
                    tma_load_2d(tiles + (size_t)it * STAGE_BYTES + w_off, map_w, &full_bar[it], (kt0 + it) * TC_BK, w0);
                }
            }
            // the block's weight tiles beyond the ring: asked into L2 while the kernel before this one finishes
            if (issuer) {
                for (int it = ahead; it < min(n_kt, ahead + p.l2_ahead); ++it) tma_prefetch_l2_2d(map_w, (kt0 + it) * TC_BK, w0);
            }
            __syncwarp();
            grid_dep_wait();                                  // the activations are the previous kernel's output
            if (issuer) {
                for (int it = 0; it < ahead; ++it)
                    tma_load_2d(tiles + (size_t)it * STAGE_BYTES + x_off, map_x, &full_bar[it], (kt0 + it) * TC_BK, x0);
            }
            __syncwarp();
            // slot and round by counting: a division by the (run-time) ring depth costs more than the MMAs of a
            // k-tile cost to issue
            int s = ahead == p.stages ? 0 : ahead, round = ahead == p.stages ? 1 : 0;
            for (int it = ahead; it < n_kt; ++it) {
                if (!__all_sync(0xffffffffu, mbar_wait(&empty_bar[s], (round & 1) ^ 1, abort_p))) break;
                if (issuer) {
                    mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                    unsigned char* slot = tiles + (size_t)s * STAGE_BYTES;
                    const int k = (kt0 + it) * TC_BK;
                    tma_load_2d(slot + w_off, map_w, &full_bar[s], k, w0);
                    tma_load_2d(slot + x_off, map_x, &full_bar[s], k, x0);
                }
                __syncwarp();
                if (++s == p.stages) { s = 0; ++round; }
            }
        }
        __syncwarp();
        if (push) cluster_wait_acquire();
    } else if (warp == 1) {
        {
            const bool issuer = elect_one();
            const uint32_t idesc = umma_idesc_bf16(TC_BM, BN);
            bool ok = true;
            int s = 0, round = 0;
            const uint64_t desc_a0 = umma_desc_sw128(tiles_base), desc_b0 = umma_desc_sw128(tiles_base + A_BYTES);
            for (int it = 0; it < n_kt && ok; ++it) {
                ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[s], round & 1, abort_p));
                if (!ok) break;
                tc_fence_after();
                // the descriptors of a slot's slices differ from the first slot's only in the address field
                // (units of 16 bytes, 14 bits: shared memory ends below 2^18 bytes, so the sum cannot carry)
                const uint64_t step = (uint64_t)((uint32_t)s * STAGE_BYTES >> 4);
                if (issuer) {
#pragma unroll
                    for (int j = 0; j < TC_BK / 16; ++j) {   // 16 elements = 32 bytes of K per MMA, inside the swizzle row
                        umma_bf16(tmem_base, desc_a0 + step + (uint64_t)(j * 2), desc_b0 + step + (uint64_t)(j * 2), idesc,
                                  (it > 0 || j > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty_bar[s]);              // frees the slot once these MMAs have read it
                }
                __syncwarp();
                if (++s == p.stages) { s = 0; ++round; }
            }
            if (ok && issuer) umma_commit(&tmem_full_bar);   // the accumulator is complete
        }
        __syncwarp();
        if (push) cluster_wait_acquire();
    } else {
        if (push) cluster_wait_acquire();                    // every block of the cluster runs: its memory and barrier may be written
        // epilogue: warp q reads TMEM lanes 32q .. 32q+31; thread r owns row r of the MMA tile
        const int q = warp & 3;
        const int r = q * 32 + lane;
        if (p.rope) {
            // what the rotation needs of this step -- positions, cache slots and the cos/sin rows of the
            // tile's tokens -- goes to shared memory now, while the weights stream, so that no look-up in
            // global memory is left for the end of the kernel.  Positions and slots are inputs of the step
            // and the tables are constants: none of them is the previous kernel's output, so this does
            // not wait for it.
            const int half = p.rotary_dim >> 1, et = threadIdx.x - 64;
            for (int i = et; i < BN; i += 128) {
                const int t = b0 + i;
                // a position or slot out of range is reported; its token is rotated by row 0 and not stored
                int pos = t < p.M ? p.positions[t] : 0, slot = t < p.M ? p.slots[t] : 0;
                if (range_position(pos, p.max_pos) != MIE_RANGE_OK) {
                    range_report(p.report, MIE_RANGE_POSITION, MIE_K_GEMM_QKV_ROPE, t, pos);
                    pos = 0; slot = -1;
                } else if (p.write_cache && range_slot(slot, p.num_pages, p.page_size) != MIE_RANGE_OK) {
                    range_report(p.report, MIE_RANGE_SLOT, MIE_K_GEMM_QKV_ROPE, t, slot);
                    slot = -1;
                }
                rope_pos[i] = pos;
                rope_slot[i] = slot;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");       // the four epilogue warps only
            // 128 / BN threads share a token's row of angles (no division by the run-time half in the loop)
            constexpr int TOK_THREADS = BN >= 128 ? 1 : 128 / BN;     // threads that share a token's row of angles
            for (int tt = et / TOK_THREADS; tt < BN; tt += 128 / TOK_THREADS) {
                const int64_t row = (int64_t)rope_pos[tt] * half;
                for (int jj = et % TOK_THREADS; jj < half; jj += TOK_THREADS) {
                    rope_cs[tt * half + jj] = p.cos_t[row + jj];
                    rope_cs[BN * half + tt * half + jj] = p.sin_t[row + jj];
                }
            }
        }
        if (p.sq_in) {
            // the factor the norm before this product left for it: 128 / BN threads add up a token's slots,
            // each its share in slot order, then the shares in lane order -- the same order every time
            grid_dep_wait();
            constexpr int TPT = BN >= 128 ? 1 : 128 / BN;    // threads per token
            const int et = threadIdx.x - 64;
            for (int i0 = 0; i0 < BN; i0 += 128 / TPT) {
                const int i = i0 + et / TPT, sub = et % TPT, t = b0 + i;
                // the first sixteen shares per thread are fetched together (one round trip, not sixteen), then
                // added in slot order; more than that (hundreds of slots) go one by one
                const bool live = i < BN && t < p.M;
                float v[16];
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    const int sl = sub + k * TPT;
                    v[k] = (live && sl < p.sq_slots) ? __ldcg(p.sq_in + (int64_t)sl * p.sq_in_stride + t) : 0.f;
                }
                float sum = 0.f;
#pragma unroll
                for (int k = 0; k < 16; ++k) sum += v[k];
                if (live)
                    for (int sl = sub + 16 * TPT; sl < p.sq_slots; sl += TPT) sum += __ldcg(p.sq_in + (int64_t)sl * p.sq_in_stride + t);
#pragma unroll
                for (int o = TPT >> 1; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                if (sub == 0 && i < BN) rstd_s[i] = t < p.M ? rsqrtf(sum / p.sq_width + p.sq_eps) : 1.f;
            }                                                // read after the block-wide barrier below
        }
        if (p.res && !tok) {
            // the stream values that this thread will add to (its first item of the owners' sum below) and
            // the norm weight of its feature are fetched now, not at the end of the kernel
            grid_dep_wait();
            const int rows_per = TC_BM / p.splits, idx = threadIdx.x - 64;
            if (idx < rows_per * (BN / 4)) {
                const int n = a0 + split * rows_per + (idx & (rows_per - 1)), c = (idx >> (31 - __clz(rows_per))) * 4;
                if (n < p.N) {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (b0 + c + j < p.M) pre_res[j] = __ldcg(p.res + (int64_t)(b0 + c + j) * p.N + n);
                    if (p.norm_w) pre_wn = load_tagged(p.norm_w, n, p.norm_w_tag);
                    if (p.bias) pre_b = load_tagged(p.bias, n, p.bias_tag);
                }
            }
        }
        const bool have_work = n_kt > 0;                     // a split beyond the last k-tile adds a zero tile
        const bool ready = have_work ? mbar_wait(&tmem_full_bar, 0, abort_p) : true;
        tc_fence_after();
        if (ready) {
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
            float* red = reinterpret_cast<float*>(tiles);     // the ring is free: every MMA has read its slot
            // where row r of the partial tile goes: the owner's slot for this sender (see the sum below)
            uint32_t send_to = 0, send_bar = 0;
            if (tok) {
                // the partial tile goes to this block's own shared memory first, laid out [owner][row][tpo tokens];
                // then one bulk copy per owner
                const int t_shift = 31 - __clz(tpo);
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    float v[16];
                    if (have_work) tmem_ld16(taddr + c, v);
                    else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = 0.f;
                    }
#pragma unroll
                    for (int i = 0; i < 16; i += 4) {
                        const int tk = c + i, o = tk >> t_shift, j = tk & (tpo - 1);
                        *reinterpret_cast<float4*>(red + ((o * TC_BM + r) << t_shift) + j) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the copy engine reads what these threads wrote
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const int et = threadIdx.x - 64;
                if (et < p.splits) {
                    const uint32_t bytes = (uint32_t)(TC_BM * tpo) * 4u;
                    const uint32_t dst = cluster_addr(tiles_base + p.recv_smem_offset, et) + (uint32_t)split * bytes;
                    const uint32_t bar = cluster_addr(smem_u32(&recv_bar), et);
                    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(dst), "r"(tiles_base + (uint32_t)et * bytes), "r"(bytes), "r"(bar) : "memory");
                }
            } else {
            if (push) {
                const int S = p.splits, rows_per = TC_BM / S;              // powers of two: masks and shifts
                const int s_shift = 31 - __clz(S), rows_shift = 31 - __clz(rows_per);
                const int owner = p.rope ? r & (S - 1) : r >> rows_shift, li = p.rope ? r >> s_shift : r & (rows_per - 1);
                send_to = cluster_addr(tiles_base + p.recv_smem_offset, owner) + (uint32_t)((split * rows_per + li) * RED_LD) * 4u;
                send_bar = cluster_addr(smem_u32(&recv_bar), owner);
            }
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                float v[16];
                if (have_work) tmem_ld16(taddr + c, v);
                else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = 0.f;
                }
                if (push) {
#pragma unroll
                    for (int i = 0; i < 16; i += 4)
                        st_async_cluster_f32x4(send_to + (uint32_t)(c + i) * 4u, send_bar, v[i], v[i + 1], v[i + 2], v[i + 3]);
                } else if (p.splits > 1) {                     // leave the partial tile for the cluster
#pragma unroll
                    for (int i = 0; i < 16; ++i) red[r * RED_LD + c + i] = v[i];
                } else if (!SWAPPED) {
                    const int m = a0 + r, n = b0 + c;
                    if (m < p.M && n < p.N) {
                        if (p.bias) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) if (n + i < p.N) v[i] += load_tagged(p.bias, n + i, p.bias_tag);
                        }
                        if (p.swiglu) {
                            float h[16];
#pragma unroll
                            for (int i = 0; i < 8; ++i) h[i] = silu_mul(v[2 * i], v[2 * i + 1]);
#pragma unroll
                            for (int i = 8; i < 16; ++i) h[i] = 0.f;
                            // 8 outputs starting at column n / 2 of a row N / 2 wide
                            if (OUT_F32) {
                                float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + (int64_t)m * (p.N / 2) + n / 2);
                                o[0] = make_float4(h[0], h[1], h[2], h[3]);
                                o[1] = make_float4(h[4], h[5], h[6], h[7]);
                            } else {
                                uint4 w;
                                __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
                                for (int i = 0; i < 4; ++i) hp[i] = __floats2bfloat162_rn(h[2 * i], h[2 * i + 1]);
                                *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.out) + (int64_t)m * (p.N / 2) + n / 2) = w;
                            }
                        } else {
                            store_row16<OUT_F32>(p.out, (int64_t)m * p.N, n, p.N, v);
                        }
                    }
                } else {
                    const int n = a0 + r;
                    const float b = (p.bias && n < p.N) ? load_tagged(p.bias, n, p.bias_tag) : 0.f;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int t = b0 + c + i;
                        float val = v[i] + b;
                        if (p.swiglu) {                        // gate on the even lane, up on the odd one
                            const float other = __shfl_xor_sync(0xffffffffu, val, 1);
                            if (!(lane & 1) && t < p.M && n < p.N)
                                store_out<OUT_F32>(p.out, (int64_t)t * (p.N / 2) + n / 2, silu_mul(val, other));
                        } else if (t < p.M && n < p.N) {
                            store_out<OUT_F32>(p.out, (int64_t)t * p.N + n, val);
                        }
                    }
                }
            }
            }
        }
    }

    tc_fence_before();
    __syncthreads();                                         // every role is done; nothing waits on an mbarrier any more
    const bool aborted = abort_flag != 0;

    if (p.splits > 1) {
        // split-K: add the partial tiles of the cluster's blocks, each block its share of the rows.
        // With `push` the partial rows arrive in this block's slots (slot s = what rank s sent) and are
        // counted on its own barrier: it waits for its 128 x BN sums and nobody else's, no barrier across
        // the cluster; with the rotation a block owns every S-th row, which keeps a row and its partner
        // (half a rotation apart, a multiple of S) with the same owner.
        bool have_all = true;
        if (push) { if (warp >= 2) have_all = mbar_wait(&recv_bar, 0, abort_p); }
        else cluster_sync_all();
        // bulk copies read the SENDER's shared memory: nobody leaves before every owner has what it is owed
        if (tok) cluster_arrive_release();
        const int S = p.splits;
        const int rows_per = TC_BM / S;                      // S is 2, 4 or 8
        const int rows_shift = 31 - __clz(rows_per);         // rows_per is a power of two: shifts, no divisions, on this last stretch
        const int r_lo = split * rows_per;
        if (tok && warp >= 2 && !aborted && have_all) {
            // ---- tokens are owned: thread r adds up row r of the tile for this block's tpo tokens
            const int r = threadIdx.x - 64, t_shift = 31 - __clz(tpo);
            float* recv = reinterpret_cast<float*>(tiles + p.recv_smem_offset);        // [sender][row][tpo]
            float acc[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] = 0.f;
#pragma unroll
            for (int s2 = 0; s2 < 8; ++s2) {
                if (s2 < S) {
                    const float4* src = reinterpret_cast<const float4*>(recv + ((s2 * TC_BM + r) << t_shift));
#pragma unroll
                    for (int j4 = 0; j4 < 4; ++j4) {
                        if (j4 * 4 < tpo) {
                            const float4 f = src[j4];
                            acc[j4 * 4] += f.x; acc[j4 * 4 + 1] += f.y; acc[j4 * 4 + 2] += f.z; acc[j4 * 4 + 3] += f.w;
                        }
                    }
                }
            }
            const int tk0 = split * tpo;                     // this block's first token within the tile
            if (p.sq_in) {
#pragma unroll
                for (int j = 0; j < 16; ++j) if (j < tpo) acc[j] *= rstd_s[tk0 + j];
            }
            const int n = a0 + r;
            const bool live = n < p.N;
            const float b = (p.bias && live) ? load_tagged(p.bias, n, p.bias_tag) : 0.f;
            if (p.rope) {
                // the rotation partner's sums come through shared memory: every row of the tile is here
                const int D = p.head_dim, half = p.rotary_dim >> 1;
                const int hd = n >> (31 - __clz(D)), d = n & (D - 1);
                const bool rotated = live && hd < p.num_heads + p.num_kv_heads && d < p.rotary_dim;
#pragma unroll
                for (int j = 0; j < 16; ++j) if (j < tpo) recv[(r << t_shift) + j] = acc[j] + b;      // slot 0 of this row: read by this thread only, above
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const int rp = rotated ? (d < half ? r + half : r - half) : r;
                if (live) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int tk = tk0 + j, t = b0 + tk;
                        if (j >= tpo || t >= p.M) continue;
                        float val = acc[j] + b;
                        if (rotated) {
                            const int jj = d < half ? d : d - half;
                            const float cs = rope_cs[tk * half + jj], sn = rope_cs[BN * half + tk * half + jj];
                            const float other = recv[(rp << t_shift) + j];
                            val = d < half ? val * cs - other * sn : val * cs + other * sn;
                        }
                        if (hd < p.num_heads) {
                            store_out<OUT_F32>(p.out, (int64_t)t * p.N + n, val);
                        } else if (p.write_cache) {
                            const int slot = rope_slot[tk];
                            if (slot < 0) continue;
                            const int page = slot >> p.page_shift, off = slot & (p.page_size - 1);
                            const bool is_k = hd < p.num_heads + p.num_kv_heads;
                            const int kvh = hd - p.num_heads - (is_k ? 0 : p.num_kv_heads);
                            const int64_t dst = (((int64_t)page * p.num_kv_heads + kvh) * p.page_size + off) * D + d;
                            (is_k ? p.k_cache : p.v_cache)[dst] = __float2bfloat16_rn(val);
                        }
                    }
                }
            } else if (p.res) {
                const float wn = (p.norm_w && live) ? load_tagged(p.norm_w, n, p.norm_w_tag) : 0.f;
                float old[16];
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    old[j] = (j < tpo && live && b0 + tk0 + j < p.M) ? __ldcg(p.res + (int64_t)(b0 + tk0 + j) * p.N + n) : 0.f;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (j >= tpo) continue;
                    const int t = b0 + tk0 + j;
                    float sq = 0.f;
                    if (live && t < p.M) {
                        const int64_t at = (int64_t)t * p.N + n;
                        const float rv = old[j] + acc[j] + b;
                        p.res[at] = rv;
                        if (p.xw_out) p.xw_out[at] = __float2bfloat16_rn(rv * wn);
                        sq = rv * rv;
                    }
                    if (p.sq_out) {                            // a warp holds 32 rows of the tile: one slot per warp and tile
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                        if (lane == 0 && t < p.sq_stride) p.sq_out[(int64_t)(blockIdx.x * 4 + (warp - 2)) * p.sq_stride + t] = sq;
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (j >= tpo) continue;
                    const int t = b0 + tk0 + j;
                    const float val = acc[j] + b;
                    if (p.swiglu) {                            // gate on the even row, up on the odd one: neighbouring lanes
                        const float other = __shfl_xor_sync(0xffffffffu, val, 1);
                        if (!(r & 1) && t < p.M && live) store_out<OUT_F32>(p.out, (int64_t)t * (p.N / 2) + n / 2, silu_mul(val, other));
                    } else if (t < p.M && live) {
                        store_out<OUT_F32>(p.out, (int64_t)t * p.N + n, val);
                    }
                }
            }
        } else if (warp >= 2 && !aborted && have_all) {
            const int tid = threadIdx.x - 64;                // 0..127
            uint32_t peer[8];
#pragma unroll
            for (int s = 0; s < 8; ++s) peer[s] = push ? 0u : cluster_addr(tiles_base, s < S ? s : 0);
            const float* recv = reinterpret_cast<const float*>(tiles + p.recv_smem_offset);
            const bool cyclic = push && p.rope;
            // one thread: one row of the tile, four consecutive columns, summed over the blocks in rank order
            for (int idx = tid; idx < rows_per * (BN / 4); idx += 128) {
                int rr, c, li = 0;
                if (SWAPPED) { li = idx & (rows_per - 1); c = (idx >> rows_shift) * 4; rr = cyclic ? li * S + split : r_lo + li; }   // neighbours: consecutive features
                else { rr = r_lo + idx / (BN / 4); c = (idx % (BN / 4)) * 4; }             // neighbours: consecutive columns
                const uint32_t off = (uint32_t)(rr * RED_LD + c) * 4u;
                float4 part[8];
#pragma unroll
                for (int s = 0; s < 8; ++s)
                    if (s < S) part[s] = push ? *reinterpret_cast<const float4*>(recv + (s * rows_per + li) * RED_LD + c)
                                              : ld_cluster_f32x4(peer[s] + off);
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int s = 0; s < 8; ++s)
                    if (s < S) { acc[0] += part[s].x; acc[1] += part[s].y; acc[2] += part[s].z; acc[3] += part[s].w; }
                if (SWAPPED && p.sq_in) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[j] *= rstd_s[c + j];
                }
                if (!SWAPPED) {
                    const int m = a0 + rr, n = b0 + c;
                    if (m >= p.M || n >= p.N) continue;
                    if (p.bias) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) acc[j] += load_tagged(p.bias, n + j, p.bias_tag);
                    }
                    if (p.swiglu) {
                        store_out<OUT_F32>(p.out, (int64_t)m * (p.N / 2) + n / 2, silu_mul(acc[0], acc[1]));
                        store_out<OUT_F32>(p.out, (int64_t)m * (p.N / 2) + n / 2 + 1, silu_mul(acc[2], acc[3]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) store_out<OUT_F32>(p.out, (int64_t)m * p.N + n + j, acc[j]);
                    }
                } else if (p.rope) {
                    const int n = a0 + rr;
                    if (n < p.N) {
                        const int D = p.head_dim, half = p.rotary_dim >> 1;
                        const int hd = n >> (31 - __clz(D)), d = n & (D - 1); // head (over q, k, v together) and place in it; D divides 128
                        const bool rotated = hd < p.num_heads + p.num_kv_heads && d < p.rotary_dim;
                        float pacc[4] = {0.f, 0.f, 0.f, 0.f};
                        int np = n;
                        if (rotated) {                                       // the partner row: half a rotation apart, same tile
                            np = d < half ? n + half : n - half;
                            const int pli = li + ((np - n) >> (31 - __clz(S)));   // the partner's place in this block's slots (half is a multiple of S)
                            float4 pp[8];
#pragma unroll
                            for (int s2 = 0; s2 < 8; ++s2)
                                if (s2 < S) pp[s2] = *reinterpret_cast<const float4*>(recv + (s2 * rows_per + pli) * RED_LD + c);
#pragma unroll
                            for (int s2 = 0; s2 < 8; ++s2)
                                if (s2 < S) { pacc[0] += pp[s2].x; pacc[1] += pp[s2].y; pacc[2] += pp[s2].z; pacc[3] += pp[s2].w; }
                            if (p.sq_in) {
#pragma unroll
                                for (int j = 0; j < 4; ++j) pacc[j] *= rstd_s[c + j];
                            }
                        }
                        const float b = p.bias ? load_tagged(p.bias, n, p.bias_tag) : 0.f;
                        const float bp = (p.bias && rotated) ? load_tagged(p.bias, np, p.bias_tag) : 0.f;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int t = b0 + c + j;
                            if (t >= p.M) continue;
                            float val = acc[j] + b;
                            if (rotated) {
                                const int jj = d < half ? d : d - half;
                                const float cs = rope_cs[(c + j) * half + jj], sn = rope_cs[BN * half + (c + j) * half + jj];
                                const float other = pacc[j] + bp;
                                val = d < half ? val * cs - other * sn : val * cs + other * sn;
                            }
                            if (hd < p.num_heads) {
                                store_out<OUT_F32>(p.out, (int64_t)t * p.N + n, val);
                            } else if (p.write_cache) {
                                const int slot = rope_slot[c + j];
                                if (slot < 0) continue;                 // out of range: reported when it was fetched
                                const int page = slot >> p.page_shift, off = slot & (p.page_size - 1);
                                const bool is_k = hd < p.num_heads + p.num_kv_heads;
                                const int kvh = hd - p.num_heads - (is_k ? 0 : p.num_kv_heads);
                                const int64_t dst = (((int64_t)page * p.num_kv_heads + kvh) * p.page_size + off) * D + d;
                                (is_k ? p.k_cache : p.v_cache)[dst] = __float2bfloat16_rn(val);
                            }
                        }
                    }
                } else if (p.res) {
                    // res += y in place; for the norm that reads the stream next, xw = bf16(res * w) and this
                    // group of lanes' share of sum(res^2): min(rows_per, 32) neighbouring lanes hold the same four
                    // tokens and consecutive features, so a shuffle tree over them adds up the features
                    const int n = a0 + rr;
                    const bool live = n < p.N, ahead = idx == tid;           // the first item's values are here already
                    float b = pre_b, wn = pre_wn, old[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) old[j] = pre_res[j];
                    if (!ahead) {
                        b = (p.bias && live) ? load_tagged(p.bias, n, p.bias_tag) : 0.f;
                        wn = (p.norm_w && live) ? load_tagged(p.norm_w, n, p.norm_w_tag) : 0.f;
#pragma unroll
                        for (int j = 0; j < 4; ++j)                        // all four loads before the first store
                            old[j] = (live && b0 + c + j < p.M) ? __ldcg(p.res + (int64_t)(b0 + c + j) * p.N + n) : 0.f;
                    }
                    float sq[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int t = b0 + c + j;
                        sq[j] = 0.f;
                        if (live && t < p.M) {
                            const int64_t at = (int64_t)t * p.N + n;
                            const float rv = old[j] + acc[j] + b;
                            p.res[at] = rv;
                            if (p.xw_out) p.xw_out[at] = __float2bfloat16_rn(rv * wn);
                            sq[j] = rv * rv;
                        }
                    }
                    if (p.sq_out) {
                        const int width = rows_per < 32 ? rows_per : 32;         // 16 or 32
#pragma unroll
                        for (int o = 1; o <= 8; o <<= 1) {                       // four independent trees, step by step
#pragma unroll
                            for (int j = 0; j < 4; ++j) sq[j] += __shfl_xor_sync(0xffffffffu, sq[j], o);
                        }
                        if (width == 32) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) sq[j] += __shfl_xor_sync(0xffffffffu, sq[j], 16);
                        }
                        if ((li & (width - 1)) == 0) {
                            const int groups = TC_BM / width;                     // slots per 128-row tile = max(S, 4)
                            const int slot = blockIdx.x * groups + ((split * rows_per + li) >> (width == 32 ? 5 : 4));
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                if (b0 + c + j < p.sq_stride) p.sq_out[(int64_t)slot * p.sq_stride + b0 + c + j] = sq[j];
                        }
                    }
                } else {
                    const int n = a0 + rr;
                    const float b = (p.bias && n < p.N) ? load_tagged(p.bias, n, p.bias_tag) : 0.f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int t = b0 + c + j;
                        const float val = acc[j] + b;
                        if (p.swiglu) {                        // gate on the even feature, up on the odd one: neighbouring threads
                            const float other = __shfl_xor_sync(0xffffffffu, val, 1);
                            if (!(rr & 1) && t < p.M && n < p.N)
                                store_out<OUT_F32>(p.out, (int64_t)t * (p.N / 2) + n / 2, silu_mul(val, other));
                        } else if (t < p.M && n < p.N) {
                            store_out<OUT_F32>(p.out, (int64_t)t * p.N + n, val);
                        }
                    }
                }
            }
        }
        if (!push) cluster_sync_all();                       // nobody leaves while its shared memory is being read
        if (tok) cluster_wait_acquire();                     // every owner has received: the staged tile may go
    }

    __syncthreads();
    if (abort_flag) {
        if (threadIdx.x == 0) atomicExch(p.error, 1);
        for (int i = 0; i < 64; ++i) __nanosleep(2000);       // let copies that are still in flight land
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// --------------------------------------------------------------------------- host side

// A [rows, K] bfloat16 row-major matrix as a 2-D tensor map with boxes of {64, box_rows} elements
// and the 128-byte swizzle; rows and columns outside the matrix read as zero.
static int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
    cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t gstride[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

template <int BN, bool SWAPPED, bool OUT_F32>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, dim3 grid, int pdl, cudaStream_t stream) {
    const size_t red = (size_t)TC_BM * (BN + 4) * sizeof(float);           // the partial tile: S slots of 128 / S rows
    const size_t stage = TC_BM * TC_BK * 2 + BN * TC_BK * 2;
    const size_t tables = (p.rope ? (size_t)BN * 2 * sizeof(int) + (size_t)BN * p.rotary_dim * sizeof(float) : 0) +
                          (p.sq_in ? (size_t)BN * sizeof(float) : 0);
    const size_t limit = 227 * 1024 - 1024 - 512;                           // less the alignment slack and the static barriers
    TcParams pp = p;
    // Peers write their partial rows while this block's ring is still live, so the slots lie beside the
    // ring: where even a ring of two stages leaves no room for them, the partial tile stays at home
    // (in the ring, once it is done) and the owners fetch it.  A ring that would not fit is made
    // shorter, never refused.
    pp.push = SWAPPED && p.splits > 1 && 2 * stage + red + tables <= limit;
    if ((p.rope || p.res || p.sq_in) && !pp.push) return MIE_ERR_BAD_ARG;   // these live in the owners' sum
    const size_t beside = (pp.push ? red : 0) + tables;
    while (pp.stages > 2 && pp.stages * stage + beside > limit) --pp.stages;
    size_t smem = (size_t)pp.stages * stage;
    pp.recv_smem_offset = 0;
    if (pp.push) { pp.recv_smem_offset = (uint32_t)smem; smem += red; }
    else if (p.splits > 1 && red > smem) smem = red;
    pp.rope_smem_offset = (uint32_t)smem;
    if (p.rope) smem += (size_t)BN * 2 * sizeof(int) + (size_t)BN * p.rotary_dim * sizeof(float);
    pp.rstd_smem_offset = (uint32_t)smem;
    if (p.sq_in) smem += (size_t)BN * sizeof(float);
    smem += 1024;
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, SWAPPED, OUT_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    int na = 0;
    if (p.splits > 1) {
        attrs[na].id = cudaLaunchAttributeClusterDimension;
        attrs[na].val.clusterDim.x = 1; attrs[na].val.clusterDim.y = 1; attrs[na].val.clusterDim.z = p.splits;
        ++na;
    }
    if (pdl) {
        attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = na;
    e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, SWAPPED, OUT_F32>, ma, mb, pp);
    return e != cudaSuccess ? (int)e : launch_status();
}

template <bool SWAPPED, bool OUT_F32>
static int dispatch_bn(int bn, const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, dim3 grid, int pdl, cudaStream_t stream) {
    switch (bn) {
        case 16: return launch_tc<16, SWAPPED, OUT_F32>(ma, mb, p, grid, pdl, stream);
        case 32: return launch_tc<32, SWAPPED, OUT_F32>(ma, mb, p, grid, pdl, stream);
        case 64: return launch_tc<64, SWAPPED, OUT_F32>(ma, mb, p, grid, pdl, stream);
        case 128: return launch_tc<128, SWAPPED, OUT_F32>(ma, mb, p, grid, pdl, stream);
        case 256: return launch_tc<256, SWAPPED, OUT_F32>(ma, mb, p, grid, pdl, stream);
    }
    return MIE_ERR_BAD_ARG;
}

// x [M, K] and w [N, K] bfloat16, y [M, N] (with `swiglu`: [M, N/2]) bfloat16 (y_tag MIE_BF16) or
// float32.  `swapped` puts the weight on the 128-row side (few tokens), `bn` is the other side's
// tile (16..256), `splits` in {1, 2, 4, 8} cuts K across a cluster, `pdl` launches with programmatic
// stream serialization.  Needs K % 8 == 0, N % 8 == 0 (N % 16 == 0 with swiglu) and 16-byte aligned
// pointers; refuses anything else.
struct RopeFuseArgs {
    const int* positions; const int* slots; const float* cos_t; const float* sin_t; void* k_cache; void* v_cache;
    int num_heads, num_kv_heads, head_dim, rotary_dim, page_size, max_pos, write_cache;
    long long num_pages;
};

// The residual epilogue and the deferred norm factor (see the header comment); null pointers switch a
// half off.  Mirrored field by field by the Python wrapper.
struct TcFuse {
    void* res; const void* norm_w; int norm_w_tag; void* xw_out; void* sq_out; int sq_stride;
    const void* sq_in; int sq_slots; int sq_in_stride; float sq_width; float sq_eps;
};

static int gemm_tc_launch(const void* x, const void* w, const void* bias, int bias_tag, void* y, int y_tag, int M, int N,
                          int K, int swapped, int bn, int splits, int stages, int swiglu, int pdl, const RopeFuseArgs* rope,
                          cudaStream_t stream, const TcFuse* fuse = nullptr) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || N % 8 || (swiglu && N % 16)) return MIE_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(y)) & 15) return MIE_ERR_BAD_ARG;
    const bool to_res = fuse && fuse->res;
    if (stages < 2 || stages > TC_MAX_STAGES) return MIE_ERR_BAD_ARG;
    if (splits != 1 && splits != 2 && splits != 4 && splits != 8) return MIE_ERR_BAD_ARG;
    int rc = tc_setup();
    if (rc) return rc;
    TcParams p;
    p.out = y; p.bias = bias; p.bias_tag = bias_tag; p.error = g_error_dev;
    p.M = M; p.N = N; p.K = K; p.swiglu = swiglu;
    p.res = nullptr; p.norm_w = nullptr; p.norm_w_tag = 0; p.xw_out = nullptr; p.sq_out = nullptr; p.sq_stride = 0;
    p.sq_in = nullptr; p.sq_slots = 0; p.sq_in_stride = 0; p.sq_width = 1.f; p.sq_eps = 0.f;
    if (fuse) {
        if (to_res) {
            // the owners' sum adds to the stream: needs the weight on the 128-row side and a split K
            if (!swapped || splits < 2 || swiglu || rope || (reinterpret_cast<uintptr_t>(fuse->res) & 15)) return MIE_ERR_BAD_ARG;
            if ((fuse->xw_out != nullptr) != (fuse->norm_w != nullptr) || (fuse->sq_out && !fuse->xw_out)) return MIE_ERR_BAD_ARG;
            if (fuse->sq_out && fuse->sq_stride < M) return MIE_ERR_BAD_ARG;
            p.res = (float*)fuse->res; p.norm_w = fuse->norm_w; p.norm_w_tag = fuse->norm_w_tag;
            p.xw_out = (bf16*)fuse->xw_out; p.sq_out = (float*)fuse->sq_out; p.sq_stride = fuse->sq_stride;
        }
        if (fuse->sq_in) {
            if (!swapped || splits < 2 || fuse->sq_slots < 1 || fuse->sq_in_stride < M || !(fuse->sq_width > 0.f)) return MIE_ERR_BAD_ARG;
            p.sq_in = (const float*)fuse->sq_in; p.sq_slots = fuse->sq_slots; p.sq_in_stride = fuse->sq_in_stride;
            p.sq_width = fuse->sq_width; p.sq_eps = fuse->sq_eps;
        }
    }
    p.rope = 0;
    if (rope) {
        // needs the cluster reduction with the weight on the 128-row side, heads that do not straddle tiles
        if (!swapped || splits < 2 || swiglu || y_tag != MIE_BF16 || rope->head_dim <= 0 || TC_BM % rope->head_dim ||
            (rope->rotary_dim & 1) || rope->rotary_dim > rope->head_dim ||
            (rope->num_heads + 2 * rope->num_kv_heads) * rope->head_dim != N)
            return MIE_ERR_BAD_ARG;
        if ((size_t)bn * rope->rotary_dim * sizeof(float) > 16 * 1024) return MIE_ERR_BAD_ARG;   // the tables must stay small
        p.rope = 1;
        p.positions = rope->positions; p.slots = rope->slots; p.cos_t = rope->cos_t; p.sin_t = rope->sin_t;
        p.k_cache = (bf16*)rope->k_cache; p.v_cache = (bf16*)rope->v_cache;
        p.num_heads = rope->num_heads; p.num_kv_heads = rope->num_kv_heads; p.head_dim = rope->head_dim;
        p.rotary_dim = rope->rotary_dim; p.page_size = rope->page_size; p.max_pos = rope->max_pos;
        if (rope->page_size < 1 || (rope->page_size & (rope->page_size - 1))) return MIE_ERR_BAD_ARG;
        p.page_shift = 0;
        while ((1 << p.page_shift) < rope->page_size) ++p.page_shift;
        p.write_cache = rope->write_cache;
        p.num_pages = rope->num_pages > 0 ? (int64_t)rope->num_pages : ((int64_t)1 << 40);
        p.report = g_range_report;
    }
    p.k_tiles = (K + TC_BK - 1) / TC_BK;
    while (splits > 1 && splits > p.k_tiles) splits >>= 1;
    p.tiles_per_split = (p.k_tiles + splits - 1) / splits;
    p.splits = splits;             // a block whose range is empty still joins the cluster with a zero tile
    if ((p.rope || p.res || p.sq_in) && p.splits < 2) return MIE_ERR_BAD_ARG;   // these live in the cluster reduction
    if (p.rope && (p.rotary_dim / 2) % p.splits) return MIE_ERR_BAD_ARG;   // a row and its partner must have one owner
    p.stages = stages;
    {
        // Eight tiles of the block's weights beyond the ring go into L2 before the dependency wait -- for a matrix that
        // L2 holds beside everything else (up to 64 MB: every product of a 1B model, q|k|v and the output projection
        // of an 8B one).  Measured on the whole decode step: 0.817 -> 0.778 ms at TinyLlama-1.1B's sizes with 8 or 16
        // tiles; at Llama-3-8B's, with every product asking, 8 tiles cost 0.5 % and 64 tiles 17 %.
        static int l2_ahead = -1, l2_ahead_mb = 64;
        if (l2_ahead < 0) {
            const char* e = getenv("MIE_B200_L2_AHEAD");
            l2_ahead = e ? atoi(e) : 8;
            const char* m = getenv("MIE_B200_L2_AHEAD_MB");
            if (m) l2_ahead_mb = atoi(m);
        }
        p.l2_ahead = (int64_t)N * K * 2 <= (int64_t)l2_ahead_mb << 20 ? l2_ahead : 0;
    }
    CUtensorMap ma, mb;
    dim3 grid;
    if (swapped) {
        if ((rc = make_map(&ma, w, N, K, TC_BM))) return rc;
        if ((rc = make_map(&mb, x, M, K, bn))) return rc;
        grid = dim3((N + TC_BM - 1) / TC_BM, (M + bn - 1) / bn, p.splits);
    } else {
        if ((rc = make_map(&ma, x, M, K, TC_BM))) return rc;
        if ((rc = make_map(&mb, w, N, K, bn))) return rc;
        grid = dim3((M + TC_BM - 1) / TC_BM, (N + bn - 1) / bn, p.splits);
    }
    if (grid.y > 65535) return MIE_ERR_TOO_LARGE;
    const bool f32 = y_tag == MIE_F32;
    if (swapped) return f32 ? dispatch_bn<true, true>(bn, ma, mb, p, grid, pdl, stream) : dispatch_bn<true, false>(bn, ma, mb, p, grid, pdl, stream);
    return f32 ? dispatch_bn<false, true>(bn, ma, mb, p, grid, pdl, stream) : dispatch_bn<false, false>(bn, ma, mb, p, grid, pdl, stream);
}

extern "C" int mie_gemm_tc(const void* x, const void* w, const void* bias, int bias_tag, void* y, int y_tag, int M, int N,
                           int K, int swapped, int bn, int splits, int stages, int swiglu, int pdl, cudaStream_t stream) {
    return gemm_tc_launch(x, w, bias, bias_tag, y, y_tag, M, N, K, swapped, bn, splits, stages, swiglu, pdl, nullptr, stream);
}

// The q|k|v projection with the rotation and the cache write in its epilogue: y [M, N] bfloat16
// receives the rotated q columns only; rotated k and plain v go to slots[token] of the caches.
// Needs swapped = 1, splits in {2, 4, 8}, head_dim dividing 128.
extern "C" int mie_gemm_tc_qkv_rope(const void* x, const void* w, const void* bias, int bias_tag, void* y, int M, int N, int K,
                                    int bn, int splits, int stages, int pdl, const int* positions, const int* slots,
                                    const float* cos_t, const float* sin_t, void* k_cache, void* v_cache, int num_heads,
                                    int num_kv_heads, int head_dim, int rotary_dim, int page_size, int max_pos,
                                    int write_cache, long long num_pages, cudaStream_t stream) {
    RopeFuseArgs r = {positions, slots, cos_t, sin_t, k_cache, v_cache, num_heads, num_kv_heads, head_dim, rotary_dim,
                      page_size, max_pos, write_cache, num_pages};
    return gemm_tc_launch(x, w, bias, bias_tag, y, MIE_BF16, M, N, K, 1, bn, splits, stages, 0, pdl, &r, stream);
}

// The product with the residual epilogue and / or the deferred norm factor (`fuse`), optionally with
// the rotation epilogue too (`positions` non-null; then as mie_gemm_tc_qkv_rope).  With fuse->res set
// `y` is not written and may be null.
extern "C" int mie_gemm_tc_fused(const void* x, const void* w, const void* bias, int bias_tag, void* y, int y_tag, int M, int N,
                                 int K, int bn, int splits, int stages, int swiglu, int pdl, const TcFuse* fuse,
                                 const int* positions, const int* slots, const float* cos_t, const float* sin_t,
                                 void* k_cache, void* v_cache, int num_heads, int num_kv_heads, int head_dim, int rotary_dim,
                                 int page_size, int max_pos, int write_cache, long long num_pages, cudaStream_t stream) {
    RopeFuseArgs r = {positions, slots, cos_t, sin_t, k_cache, v_cache, num_heads, num_kv_heads, head_dim, rotary_dim,
                      page_size, max_pos, write_cache, num_pages};
    return gemm_tc_launch(x, w, bias, bias_tag, y, y_tag, M, N, K, 1, bn, splits, stages, swiglu, pdl, positions ? &r : nullptr,
                          stream, fuse);
}

// Non-zero when a block of any launch so far gave up a bounded wait.  Reads host memory that the
// kernel writes directly; meaningful after the launches have completed (a stream synchronise).
extern "C" int mie_gemm_tc_error(void) { return g_error_host ? *g_error_host : 0; }
extern "C" void mie_gemm_tc_clear_error(void) { if (g_error_host) *g_error_host = 0; }

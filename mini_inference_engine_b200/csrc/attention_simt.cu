// Paged, causal, variable-length attention on CUDA cores: the one kernel that serves prompt
// portions and single decoded tokens alike, in float32 (the true 32-bit path) and in bfloat16
// (the reference path that the tensor-core kernels are checked against).
//
// A batch row is a request: q_len new tokens whose keys and values were already written to the
// cache, ctx_len = tokens in the cache including them.  Query i of the row sits at position
// p = ctx_len - q_len + i and reads keys j <= p (and j > p - window when window > 0) through the
// row's block table.  Query head h reads kv head h / (H / H_kv).  Scores, softmax and the
// accumulator are float32; online softmax over tiles of 32 keys.
//
// This replaces the reference's three code paths (Triton decode kernel for single tokens,
// SDPA on local k/v for a fresh prompt, SDPA on gathered k/v + mask for a continued one,
// inference_engine/model.py:128-159, inference_engine/kernels/decode_attention.py:20-82).
//
// Work split: one block = one row, one tile of QT consecutive queries, one kv head and up to
// HG <= 8 query heads of its group; each of the 8 warps owns one (query, head) pair, so a key
// tile staged in shared memory is used by up to 8 pairs.  Within a warp, lane j scores key j of
// the tile, then each lane owns output dimensions lane, lane+32, ...
#include "common.cuh"
#include "range_check.cuh"

#define ATT_WARPS 8
#define ATT_KEYS 32
#define ATT_MAX_D 256

template <typename T> struct Vec;
template <> struct Vec<float> {
    static constexpr int N = 4;
    __device__ static void load(const float* p, float* dst) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
    }
};
template <> struct Vec<bf16> {
    static constexpr int N = 8;
    __device__ static void load(const bf16* p, float* dst) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            dst[2 * i] = f.x; dst[2 * i + 1] = f.y;
        }
    }
};

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
paged_attention_kernel(const T* __restrict__ q, int64_t q_stride, const T* __restrict__ k_cache,
                       const T* __restrict__ v_cache, const int* __restrict__ block_tables,
                       int table_stride, const int* __restrict__ row_q_start,
                       const int* __restrict__ row_q_len, const int* __restrict__ row_ctx_len,
                       int num_rows, T* __restrict__ out, int num_heads, int num_kv_heads,
                       int head_dim, int page_size, int page_shift, float scale, int window,
                       int QT, int HG, int min_q_len, int64_t num_pages, int* report) {
    extern __shared__ __align__(16) float smem[];
    __shared__ int s_row, s_q0;
    const int D = head_dim, DP = head_dim + 4;
    float* q_s = smem;                          // [ATT_WARPS][D]
    float* k_s = q_s + ATT_WARPS * D;           // [ATT_KEYS][DP]
    float* v_s = k_s + ATT_KEYS * DP;           // [ATT_KEYS][DP]

    pdl_launch_dependents();
    // which row and query tile is this block's?  (a whole warp asks: warp_find_row)
    if (threadIdx.x < 32) {
        int tile, tiles;
        const int found = warp_find_row(row_q_len, num_rows, (int)blockIdx.x,
                                        [&](int ql) { return ql >= min_q_len ? (ql + QT - 1) / QT : 0; },   // shorter rows belong to another kernel
                                        tile, tiles);
        if (threadIdx.x == 0) { s_row = found; s_q0 = tile * QT; }
    }
    __syncthreads();
    const int r = s_row;
    if (r < 0) return;
    pdl_wait();
    const int q0 = s_q0;
    const int q_len = row_q_len[r], ctx_len = row_ctx_len[r], q_start = row_q_start[r];
    if (ctx_len > table_stride * page_size) {      // more positions than the row's block table covers: reported, row left alone
        if (threadIdx.x == 0) range_report(report, MIE_RANGE_POSITION, MIE_K_ATTENTION_SIMT, r, ctx_len);
        return;
    }
    const int G = num_heads / num_kv_heads;
    const int chunks = (G + HG - 1) / HG;
    const int kvh = blockIdx.y / chunks, chunk = blockIdx.y - kvh * chunks;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qi = warp / HG, g = chunk * HG + (warp - qi * HG);
    const bool active = warp < QT * HG && (q0 + qi) < q_len && g < G;
    const int head = kvh * G + g;
    const int pos_q = ctx_len - q_len + q0 + qi;
    const int token = q_start + q0 + qi;

    if (active) {
        const T* qp = q + (int64_t)token * q_stride + (int64_t)head * D;
        for (int d = lane; d < D; d += 32) q_s[warp * D + d] = to_f32<T>(qp[d]) * scale;
    }

    const int q_last = min(q0 + QT, q_len) - 1;
    const int k_hi = ctx_len - q_len + q_last + 1;                       // one past the last key any query here reads
    const int k_lo = window > 0 ? max(0, ctx_len - q_len + q0 - window + 1) : 0;

    float m = -INFINITY, l = 0.f;
    float acc[ATT_MAX_D / 32];
#pragma unroll
    for (int i = 0; i < ATT_MAX_D / 32; ++i) acc[i] = 0.f;

    const int vecs_per_row = D / Vec<T>::N;
    const int* table = block_tables + (int64_t)r * table_stride;

    for (int k0 = k_lo & ~(ATT_KEYS - 1); k0 < k_hi; k0 += ATT_KEYS) {
        __syncthreads();                     // the previous tile (and q_s on the first pass) is done with
        for (int idx = threadIdx.x; idx < ATT_KEYS * vecs_per_row; idx += blockDim.x) {
            const int jj = idx / vecs_per_row, c = (idx - jj * vecs_per_row) * Vec<T>::N;
            const int key = k0 + jj;
            float kf[Vec<T>::N], vf[Vec<T>::N];
            if (key >= k_lo && key < k_hi) {
                const int page = checked_page(table[key >> page_shift], num_pages, report, MIE_K_ATTENTION_SIMT, key >> page_shift);
                const int off = key & (page_size - 1);
                const int64_t src = (((int64_t)page * num_kv_heads + kvh) * page_size + off) * D + c;
                Vec<T>::load(k_cache + src, kf);
                Vec<T>::load(v_cache + src, vf);
            } else {
#pragma unroll
                for (int i = 0; i < Vec<T>::N; ++i) { kf[i] = 0.f; vf[i] = 0.f; }
            }
#pragma unroll
            for (int i = 0; i < Vec<T>::N; ++i) { k_s[jj * DP + c + i] = kf[i]; v_s[jj * DP + c + i] = vf[i]; }
        }
        __syncthreads();
        if (active) {
            const int key = k0 + lane;
            const bool valid = key <= pos_q && (window <= 0 || key > pos_q - window);
            float s = 0.f;
            const float4* kr = reinterpret_cast<const float4*>(k_s + lane * DP);
            const float4* qr = reinterpret_cast<const float4*>(q_s + warp * D);
            for (int d4 = 0; d4 < D / 4; ++d4) {
                const float4 a = qr[d4], b = kr[d4];
                s = fmaf(a.x, b.x, s); s = fmaf(a.y, b.y, s); s = fmaf(a.z, b.z, s); s = fmaf(a.w, b.w, s);
            }
            s = valid ? s : -INFINITY;
            const float m_new = fmaxf(m, warp_max(s));
            if (m_new > -INFINITY) {           // else every key of this tile is masked for this query
                const float alpha = expf(m - m_new);          // m = -inf gives 0
                const float p = valid ? expf(s - m_new) : 0.f;
                l = l * alpha + warp_sum(p);
                m = m_new;
#pragma unroll
                for (int i = 0; i < ATT_MAX_D / 32; ++i) acc[i] *= alpha;
                for (int j = 0; j < ATT_KEYS; ++j) {
                    const float pj = __shfl_sync(0xffffffffu, p, j);
                    const float* vr = v_s + j * DP;
#pragma unroll
                    for (int i = 0; i < ATT_MAX_D / 32; ++i) {
                        const int d = lane + 32 * i;
                        if (d < D) acc[i] = fmaf(pj, vr[d], acc[i]);
                    }
                }
            }
        }
    }
    if (active) {
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        T* op = out + ((int64_t)token * num_heads + head) * D;
#pragma unroll
        for (int i = 0; i < ATT_MAX_D / 32; ++i) {
            const int d = lane + 32 * i;
            if (d < D) op[d] = from_f32<T>(acc[i] * inv);
        }
    }
}

static size_t att_smem_bytes(int head_dim) {
    return sizeof(float) * ((size_t)ATT_WARPS * head_dim + 2 * (size_t)ATT_KEYS * (head_dim + 4));
}

// Rows with fewer than `min_q_len` new tokens are skipped (another kernel serves them).
// q: [num_tokens, ...] with `q_stride` elements between tokens and heads packed [H, D] at the row
// start; out: [num_tokens, H, D] contiguous; caches: [pages, H_kv, page_size, D].
extern "C" int mie_paged_attention(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                                   const int* block_tables, int table_stride, const int* row_q_start,
                                   const int* row_q_len, const int* row_ctx_len, int num_rows,
                                   int num_tokens, void* out, int act_tag, int num_heads, int num_kv_heads,
                                   int head_dim, int page_size, float scale, int window, int min_q_len,
                                   long long num_pages, cudaStream_t stream) {
    if (num_rows <= 0 || num_tokens <= 0) return 0;
    if (head_dim < 16 || head_dim > ATT_MAX_D || head_dim % 16) return MIE_ERR_BAD_ARG;
    if (num_kv_heads <= 0 || num_heads % num_kv_heads) return MIE_ERR_BAD_ARG;
    if (page_size < 1 || (page_size & (page_size - 1))) return MIE_ERR_BAD_ARG;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    const int G = num_heads / num_kv_heads;
    const int HG = G < ATT_WARPS ? G : ATT_WARPS;
    const int QT = ATT_WARPS / HG;
    const int chunks = (G + HG - 1) / HG;
    const dim3 grid((num_tokens + QT - 1) / QT + num_rows, num_kv_heads * chunks);
    const size_t smem = att_smem_bytes(head_dim);
    cudaError_t e;
    if (act_tag == MIE_F32) {
        e = cudaFuncSetAttribute(paged_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        return launch_kernel(paged_attention_kernel<float>, grid, dim3(ATT_WARPS * 32), smem, stream,
            (const float*)q, q_stride, (const float*)k_cache, (const float*)v_cache, block_tables, table_stride,
            row_q_start, row_q_len, row_ctx_len, num_rows, (float*)out, num_heads, num_kv_heads, head_dim,
            page_size, page_shift, scale, window, QT, HG, min_q_len, (int64_t)num_pages, g_range_report);
    } else if (act_tag == MIE_BF16) {
        e = cudaFuncSetAttribute(paged_attention_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        return launch_kernel(paged_attention_kernel<bf16>, grid, dim3(ATT_WARPS * 32), smem, stream,
            (const bf16*)q, q_stride, (const bf16*)k_cache, (const bf16*)v_cache, block_tables, table_stride,
            row_q_start, row_q_len, row_ctx_len, num_rows, (bf16*)out, num_heads, num_kv_heads, head_dim,
            page_size, page_shift, scale, window, QT, HG, min_q_len, (int64_t)num_pages, g_range_report);
    }
    return MIE_ERR_BAD_ARG;
}

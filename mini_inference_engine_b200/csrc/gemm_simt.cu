// y[M, N] = x[M, K] * W[N, K]^T (+ bias[N]) on CUDA cores with float32 FMA.
//
// This is the matrix product of the true 32-bit path (no tensor-core mode of reduced precision:
// tcgen05 has no float32 x float32 product) and the product used when a bfloat16 model holds a
// matrix in 32 bits.  Operands may be float32 or bfloat16 (widened on load, exact); the
// accumulator is float32; the result is rounded once on store.  Any M, N, K: edges are guarded,
// and rows that are not 16-byte aligned fall back to scalar loads.
// (The reference calls F.linear / cuBLAS here: inference_engine/model.py:172,178,180,181,185.)
//
// Two kernels: a tiled one (BM x BN block tile, BK = 16, TM x TN per thread) for many rows and a
// row-streaming one for a handful of rows (decode), where each warp owns output columns and reads
// its weight rows exactly once.
#include "common.cuh"

template <typename T> __device__ __forceinline__ void load4(const T* p, float* dst);
template <> __device__ __forceinline__ void load4<float>(const float* p, float* dst) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
}
template <> __device__ __forceinline__ void load4<bf16>(const bf16* p, float* dst) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    dst[0] = a.x; dst[1] = a.y; dst[2] = b.x; dst[3] = b.y;
}

constexpr int BK = 16;

// Stage a [ROWS x BK] tile of a K-major matrix into shared memory transposed: dst[k][row].
template <typename T, int ROWS, int THREADS>
__device__ __forceinline__ void stage_tile(const T* __restrict__ src, int rows_total, int K, int row0,
                                           int k0, float (*dst)[ROWS + 4], bool vec_ok) {
    for (int idx = threadIdx.x; idx < ROWS * (BK / 4); idx += THREADS) {
        const int r = idx / (BK / 4), c = (idx - r * (BK / 4)) * 4;
        const int row = row0 + r, k = k0 + c;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (row < rows_total) {
            const T* p = src + (int64_t)row * K + k;
            if (vec_ok && k + 3 < K) load4<T>(p, v);
            else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (k + i < K) v[i] = to_f32<T>(p[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[c + i][r] = v[i];
    }
}

template <typename TA, typename TW, typename TC, int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_tiled_kernel(const TA* __restrict__ A, const TW* __restrict__ W, const void* __restrict__ bias,
                  int bias_tag, TC* __restrict__ C, int M, int N, int K, bool vec_a, bool vec_w) {
    constexpr int THREADS = (BM / TM) * (BN / TN);
    pdl_enter();
    __shared__ __align__(16) float As[BK][BM + 4];
    __shared__ __align__(16) float Ws[BK][BN + 4];
    const int tx = threadIdx.x % (BN / TN), ty = threadIdx.x / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        stage_tile<TA, BM, THREADS>(A, M, K, m0, k0, As, vec_a);
        stage_tile<TW, BN, THREADS>(W, N, K, n0, k0, Ws, vec_w);
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; i += 4) {
                const float4 v = *reinterpret_cast<const float4*>(&As[k][ty * TM + i]);
                a[i] = v.x; a[i + 1] = v.y; a[i + 2] = v.z; a[i + 3] = v.w;
            }
#pragma unroll
            for (int j = 0; j < TN; j += 4) {
                const float4 v = *reinterpret_cast<const float4*>(&Ws[k][tx * TN + j]);
                b[j] = v.x; b[j + 1] = v.y; b[j + 2] = v.z; b[j + 3] = v.w;
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += load_tagged(bias, n, bias_tag);
            C[(int64_t)m * N + n] = from_f32<TC>(v);
        }
    }
}

// Few rows: block = 8 warps, each warp computes ROWS x 1 outputs per column it owns; x rows are
// read through L1/L2 (they are small), each weight row is read once per group of ROWS rows.
template <typename TA, typename TW, typename TC, int ROWS>
__global__ void __launch_bounds__(256)
gemm_rows_kernel(const TA* __restrict__ A, const TW* __restrict__ W, const void* __restrict__ bias,
                 int bias_tag, TC* __restrict__ C, int M, int N, int K, bool vec_ok) {
    pdl_enter();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    const int m0 = blockIdx.y * ROWS;
    if (n >= N) return;
    float acc[ROWS];
#pragma unroll
    for (int i = 0; i < ROWS; ++i) acc[i] = 0.f;
    const TW* w = W + (int64_t)n * K;
    if (vec_ok) {
        for (int k = lane * 4; k < K; k += 128) {
            float wv[4];
            load4<TW>(w + k, wv);
#pragma unroll
            for (int i = 0; i < ROWS; ++i) {
                if (m0 + i < M) {
                    float av[4];
                    load4<TA>(A + (int64_t)(m0 + i) * K + k, av);
                    acc[i] = fmaf(av[0], wv[0], acc[i]); acc[i] = fmaf(av[1], wv[1], acc[i]);
                    acc[i] = fmaf(av[2], wv[2], acc[i]); acc[i] = fmaf(av[3], wv[3], acc[i]);
                }
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) {
            const float wv = to_f32<TW>(w[k]);
#pragma unroll
            for (int i = 0; i < ROWS; ++i)
                if (m0 + i < M) acc[i] = fmaf(to_f32<TA>(A[(int64_t)(m0 + i) * K + k]), wv, acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
        const float v = warp_sum(acc[i]);
        if (lane == 0 && m0 + i < M) {
            const float b = bias ? load_tagged(bias, n, bias_tag) : 0.f;
            C[(int64_t)(m0 + i) * N + n] = from_f32<TC>(v + b);
        }
    }
}

template <typename TA, typename TW, typename TC>
static int launch_gemm(const void* A, const void* W, const void* bias, int bias_tag, void* C, int M,
                       int N, int K, cudaStream_t stream) {
    const bool al_a = (reinterpret_cast<uintptr_t>(A) % 16 == 0) && ((int64_t)K * sizeof(TA)) % 16 == 0;
    const bool al_w = (reinterpret_cast<uintptr_t>(W) % 16 == 0) && ((int64_t)K * sizeof(TW)) % 16 == 0;
    // vector loads of 4 elements need K % 4 == 0 as well, which the byte test implies for both types
    if (M <= 16) {
        constexpr int ROWS = 8;
        const dim3 grid((N + 7) / 8, (M + ROWS - 1) / ROWS);
        return launch_kernel(gemm_rows_kernel<TA, TW, TC, ROWS>, grid, dim3(256), 0, stream,
                             (const TA*)A, (const TW*)W, bias, bias_tag, (TC*)C, M, N, K, al_a && al_w);
    } else if (M <= 192 || N < 128) {
        const dim3 grid((N + 63) / 64, (M + 63) / 64);
        return launch_kernel(gemm_tiled_kernel<TA, TW, TC, 64, 64, 4, 4>, grid, dim3(256), 0, stream,
                             (const TA*)A, (const TW*)W, bias, bias_tag, (TC*)C, M, N, K, al_a, al_w);
    } else {
        const dim3 grid((N + 127) / 128, (M + 127) / 128);
        return launch_kernel(gemm_tiled_kernel<TA, TW, TC, 128, 128, 8, 8>, grid, dim3(256), 0, stream,
                             (const TA*)A, (const TW*)W, bias, bias_tag, (TC*)C, M, N, K, al_a, al_w);
    }
}

// Tags: MIE_F32 / MIE_BF16 for x, W and y.  bias may be null.
extern "C" int mie_gemm_simt(const void* x, int x_tag, const void* w, int w_tag, const void* bias,
                             int bias_tag, void* y, int y_tag, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return MIE_ERR_BAD_ARG;
    if (x_tag == MIE_F32 && w_tag == MIE_F32 && y_tag == MIE_F32)
        return launch_gemm<float, float, float>(x, w, bias, bias_tag, y, M, N, K, stream);
    if (x_tag == MIE_BF16 && w_tag == MIE_BF16 && y_tag == MIE_BF16)
        return launch_gemm<bf16, bf16, bf16>(x, w, bias, bias_tag, y, M, N, K, stream);
    if (x_tag == MIE_BF16 && w_tag == MIE_BF16 && y_tag == MIE_F32)
        return launch_gemm<bf16, bf16, float>(x, w, bias, bias_tag, y, M, N, K, stream);
    if (x_tag == MIE_BF16 && w_tag == MIE_F32 && y_tag == MIE_BF16)
        return launch_gemm<bf16, float, bf16>(x, w, bias, bias_tag, y, M, N, K, stream);
    if (x_tag == MIE_BF16 && w_tag == MIE_F32 && y_tag == MIE_F32)
        return launch_gemm<bf16, float, float>(x, w, bias, bias_tag, y, M, N, K, stream);
    return MIE_ERR_BAD_ARG;
}

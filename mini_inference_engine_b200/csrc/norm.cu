// Fused residual-add + RMSNorm.
//   res[r, :] += delta[r, :]            (float32 residual stream, updated in place)
//   out[r, :]  = res[r, :] * rsqrt(mean(res[r, :]^2) + eps) * w[:]
// One block per row; the summed row stays in shared memory between the two passes, so each
// input is read once.  Statistics, the sum and the scaling are float32; only `out` is rounded
// to the activation type.  The reference's Triton kernel does the same in one program per row
// but keeps the residual in the model dtype (inference_engine/kernels/rmsnorm.py:13-32).
//
// `rows` (optional) gathers: output row b is computed from input row rows[b] and the residual
// is left untouched -- the row selection before the final norm (inference_engine/model.py:182-184).
#include "common.cuh"
#include "range_check.cuh"

template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(const TD* __restrict__ delta, float* __restrict__ res,
                                   const void* __restrict__ w, int w_tag, TO* __restrict__ out,
                                   const int* __restrict__ rows, int n, float eps, int use_smem,
                                   int num_in_rows, int* report) {
    extern __shared__ float row_cache[];
    __shared__ float red[33];
    pdl_enter();
    const int b = blockIdx.x;
    const int64_t r = rows ? rows[b] : b;
    if (rows && range_row(r, num_in_rows) != MIE_RANGE_OK) {      // a gathered row that does not exist: reported, not read
        if (threadIdx.x == 0) range_report(report, MIE_RANGE_ROW, MIE_K_NORM, b, (int)r);
        return;
    }
    float* res_row = res + r * n;
    const TD* d_row = delta ? delta + r * n : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = res_row[i];
        if (d_row) v += to_f32<TD>(d_row[i]);
        if (use_smem) row_cache[i] = v;
        if (!rows && d_row) res_row[i] = v;
        ss += v * v;
    }
    const float total = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(total / (float)n + eps);
    TO* o_row = out + (int64_t)b * n;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v;
        if (use_smem) v = row_cache[i];
        else { v = res_row[i]; if (rows && d_row) v += to_f32<TD>(d_row[i]); }
        o_row[i] = from_f32<TO>(v * rstd * load_tagged(w, i, w_tag));
    }
}

// The same with 16-byte accesses: bfloat16 delta/out, n % 8 == 0, the row kept in registers (up to
// 8 x 1024 x 8 elements), float32 residual read and written as float4 pairs.
template <int PER_THREAD>
__global__ void add_rmsnorm_bf16x8_kernel(const bf16* __restrict__ delta, float* __restrict__ res, const void* __restrict__ w,
                                          int w_tag, bf16* __restrict__ out, const int* __restrict__ rows, int n, float eps,
                                          int num_in_rows, int* report) {
    __shared__ float red[33];
    pdl_enter();
    const int b = blockIdx.x;
    const int64_t r = rows ? rows[b] : b;
    if (rows && range_row(r, num_in_rows) != MIE_RANGE_OK) {
        if (threadIdx.x == 0) range_report(report, MIE_RANGE_ROW, MIE_K_NORM, b, (int)r);
        return;
    }
    float* res_row = res + r * n;
    const bf16* d_row = delta ? delta + r * n : nullptr;
    float v[PER_THREAD][8];
    float ss = 0.f;
    const int n8 = n >> 3;
#pragma unroll
    for (int it = 0; it < PER_THREAD; ++it) {
        const int i8 = threadIdx.x + it * blockDim.x;
        if (i8 < n8) {
            const float4 a = *reinterpret_cast<const float4*>(res_row + 8 * i8), c = *reinterpret_cast<const float4*>(res_row + 8 * i8 + 4);
            v[it][0] = a.x; v[it][1] = a.y; v[it][2] = a.z; v[it][3] = a.w; v[it][4] = c.x; v[it][5] = c.y; v[it][6] = c.z; v[it][7] = c.w;
            if (d_row) {
                const uint4 d = *reinterpret_cast<const uint4*>(d_row + 8 * i8);
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
                for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); v[it][2 * j] += f.x; v[it][2 * j + 1] += f.y; }
                if (!rows) {
                    *reinterpret_cast<float4*>(res_row + 8 * i8) = make_float4(v[it][0], v[it][1], v[it][2], v[it][3]);
                    *reinterpret_cast<float4*>(res_row + 8 * i8 + 4) = make_float4(v[it][4], v[it][5], v[it][6], v[it][7]);
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += v[it][j] * v[it][j];
        }
    }
    const float total = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(total / (float)n + eps);
    bf16* o_row = out + (int64_t)b * n;
#pragma unroll
    for (int it = 0; it < PER_THREAD; ++it) {
        const int i8 = threadIdx.x + it * blockDim.x;
        if (i8 < n8) {
            uint4 o;
            __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                ho[j] = __floats2bfloat162_rn(v[it][2 * j] * rstd * load_tagged(w, 8 * i8 + 2 * j, w_tag),
                                              v[it][2 * j + 1] * rstd * load_tagged(w, 8 * i8 + 2 * j + 1, w_tag));
            *reinterpret_cast<uint4*>(o_row + 8 * i8) = o;
        }
    }
}

// act_tag: type of delta and out (MIE_F32 or MIE_BF16).  delta may be null (first layer: the
// residual already holds the embedding).
extern "C" int mie_add_rmsnorm(const void* delta, float* res, const void* w, int w_tag, void* out,
                               int act_tag, const int* rows, int num_rows, int n, float eps,
                               int num_in_rows, cudaStream_t stream) {
    if (num_rows <= 0) return 0;
    if (n <= 0) return MIE_ERR_BAD_ARG;
    const bool aligned = ((reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(res) | reinterpret_cast<uintptr_t>(out)) % 16) == 0;
    if (act_tag == MIE_BF16 && n % 8 == 0 && n <= 8 * 1024 * 4 && aligned) {
        const int n8 = n / 8;
        int threads = 32;
        while (threads < 256 && threads < n8) threads <<= 1;       // 2048-wide rows: 256 threads, one 16-byte piece each
        const int per = (n8 + threads - 1) / threads;
        if (per <= 1)
            return launch_kernel(add_rmsnorm_bf16x8_kernel<1>, dim3(num_rows), dim3(threads), 0, stream, (const bf16*)delta, res, w,
                                 w_tag, (bf16*)out, rows, n, eps, num_in_rows, g_range_report);
        if (per <= 2)
            return launch_kernel(add_rmsnorm_bf16x8_kernel<2>, dim3(num_rows), dim3(threads), 0, stream, (const bf16*)delta, res, w,
                                 w_tag, (bf16*)out, rows, n, eps, num_in_rows, g_range_report);
        if (per <= 4)
            return launch_kernel(add_rmsnorm_bf16x8_kernel<4>, dim3(num_rows), dim3(threads), 0, stream, (const bf16*)delta, res, w,
                                 w_tag, (bf16*)out, rows, n, eps, num_in_rows, g_range_report);
        if (per <= 16)
            return launch_kernel(add_rmsnorm_bf16x8_kernel<16>, dim3(num_rows), dim3(threads), 0, stream, (const bf16*)delta, res, w,
                                 w_tag, (bf16*)out, rows, n, eps, num_in_rows, g_range_report);
    }
    int threads = 32;
    while (threads < 1024 && threads * 4 < n) threads <<= 1;
    const size_t smem_bytes = (size_t)n * sizeof(float);
    const int use_smem = smem_bytes <= 40 * 1024;
    const size_t smem = use_smem ? smem_bytes : 0;
    if (act_tag == MIE_F32)
        return launch_kernel(add_rmsnorm_kernel<float, float>, dim3(num_rows), dim3(threads), smem, stream,
                             (const float*)delta, res, w, w_tag, (float*)out, rows, n, eps, use_smem, num_in_rows, g_range_report);
    else if (act_tag == MIE_BF16)
        return launch_kernel(add_rmsnorm_kernel<bf16, bf16>, dim3(num_rows), dim3(threads), smem, stream,
                             (const bf16*)delta, res, w, w_tag, (bf16*)out, rows, n, eps, use_smem, num_in_rows, g_range_report);
    return MIE_ERR_BAD_ARG;
}

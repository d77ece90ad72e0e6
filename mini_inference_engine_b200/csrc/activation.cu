// SwiGLU on a fused gate/up projection: out[t, i] = silu(gu[t, i]) * gu[t, I + i],
// silu(z) = z / (1 + exp(-z)), computed in float32 (inference_engine/model.py:180-181, where the
// two halves come from `.chunk(2)` of the fused projection).  With `interleaved` the projection's
// columns alternate gate_i, up_i (the layout the tensor-core product's fused epilogue wants of the
// weight): out[t, i] = silu(gu[t, 2i]) * gu[t, 2i + 1].
#include "common.cuh"

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t total, int inter, int interleaved) {
    pdl_enter();
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / inter;
        const int i = (int)(idx - t * inter);
        const float g = to_f32<T>(gu[t * 2 * inter + (interleaved ? 2 * i : i)]);
        const float u = to_f32<T>(gu[t * 2 * inter + (interleaved ? 2 * i + 1 : inter + i)]);
        out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
    }
}

// Eight outputs per thread with 16-byte loads and stores (bfloat16, inter % 8 == 0).  The result is
// rounded to bfloat16, so the exponential and the division are the hardware approximations (two ulp
// each in float32): with the library's the kernel issued instructions all the time and reached 0.6 of
// the memory bandwidth on 2,048 tokens.  Token and place within it are counted along the grid-stride
// loop instead of divided out of a 64-bit index every time.
__global__ void swiglu_bf16x8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int64_t total8, int inter8,
                                     int interleaved) {
    pdl_enter();
    const unsigned stride = gridDim.x * blockDim.x, first = blockIdx.x * blockDim.x + threadIdx.x;   // the grid is capped: both fit
    const unsigned stride_t = stride / (unsigned)inter8, stride_i = stride - stride_t * (unsigned)inter8;
    int64_t t = first / (unsigned)inter8;
    int i8 = (int)(first - (unsigned)t * (unsigned)inter8);
    for (int64_t idx = first; idx < total8; idx += stride, t += stride_t, i8 += (int)stride_i) {
        if (i8 >= inter8) { i8 -= inter8; ++t; }
        const bf16* row = gu + t * 16 * inter8;
        float g[8], u[8];
        if (interleaved) {
            const uint4 a = *reinterpret_cast<const uint4*>(row + 16 * i8), b = *reinterpret_cast<const uint4*>(row + 16 * i8 + 8);
            const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
            const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 x = __bfloat1622float2(ha[j]), y = __bfloat1622float2(hb[j]);
                g[j] = x.x; u[j] = x.y; g[4 + j] = y.x; u[4 + j] = y.y;
            }
        } else {
            const uint4 a = *reinterpret_cast<const uint4*>(row + 8 * i8), b = *reinterpret_cast<const uint4*>(row + 8 * inter8 + 8 * i8);
            const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
            const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 x = __bfloat1622float2(ha[j]), y = __bfloat1622float2(hb[j]);
                g[2 * j] = x.x; g[2 * j + 1] = x.y; u[2 * j] = y.x; u[2 * j + 1] = y.y;
            }
        }
        uint4 o;
        __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            ho[j] = __floats2bfloat162_rn(__fdividef(g[2 * j], 1.0f + __expf(-g[2 * j])) * u[2 * j],
                                          __fdividef(g[2 * j + 1], 1.0f + __expf(-g[2 * j + 1])) * u[2 * j + 1]);
        *reinterpret_cast<uint4*>(out + idx * 8) = o;
    }
}

extern "C" int mie_swiglu(const void* gu, void* out, int act_tag, int num_tokens, int inter, int interleaved,
                          cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (inter <= 0) return MIE_ERR_BAD_ARG;
    const int64_t total = (int64_t)num_tokens * inter;
    const int threads = 256;
    if (act_tag == MIE_BF16 && inter % 8 == 0 && (reinterpret_cast<uintptr_t>(gu) | reinterpret_cast<uintptr_t>(out)) % 16 == 0) {
        int64_t blocks8 = (total / 8 + threads - 1) / threads;
        if (blocks8 > device_sm_count() * 16) blocks8 = device_sm_count() * 16;
        return launch_kernel(swiglu_bf16x8_kernel, dim3((int)blocks8), dim3(threads), 0, stream, (const bf16*)gu, (bf16*)out,
                             total / 8, inter / 8, interleaved);
    }
    int64_t blocks = (total + threads - 1) / threads;
    if (blocks > device_sm_count() * 16) blocks = device_sm_count() * 16;
    if (act_tag == MIE_F32)
        return launch_kernel(swiglu_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (const float*)gu, (float*)out, total, inter, interleaved);
    else if (act_tag == MIE_BF16)
        return launch_kernel(swiglu_kernel<bf16>, dim3((int)blocks), dim3(threads), 0, stream, (const bf16*)gu, (bf16*)out, total, inter, interleaved);
    return MIE_ERR_BAD_ARG;
}

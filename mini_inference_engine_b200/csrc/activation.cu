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

extern "C" int mie_swiglu(const void* gu, void* out, int act_tag, int num_tokens, int inter, int interleaved,
                          cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (inter <= 0) return MIE_ERR_BAD_ARG;
    const int64_t total = (int64_t)num_tokens * inter;
    const int threads = 256;
    int64_t blocks = (total + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (act_tag == MIE_F32)
        return launch_kernel(swiglu_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (const float*)gu, (float*)out, total, inter, interleaved);
    else if (act_tag == MIE_BF16)
        return launch_kernel(swiglu_kernel<bf16>, dim3((int)blocks), dim3(threads), 0, stream, (const bf16*)gu, (bf16*)out, total, inter, interleaved);
    return MIE_ERR_BAD_ARG;
}

// Sampling over float32 logits [rows, vocab]: one block per row, no host synchronisation.
//   temperature == 0: argmax (the lowest index wins a tie), inference_engine/sampling.py:15
//   temperature  > 0: argmax(logit / t + g), g = -log(-log(u)) Gumbel noise.  This draws from
//     softmax(logit / t) like the reference's exponential race argmax(p / E)
//     (inference_engine/sampling.py:18-22), because log(p / E) = logit/t - const - log E and
//     -log E is Gumbel-distributed for E = -log u.
// The noise is a counter-based hash of (seed, request id, output position, vocabulary entry), so
// a request's tokens do not depend on what else is in the batch or on how steps were cut.
#include "common.cuh"

__device__ __forceinline__ uint64_t mix64(uint64_t x) {
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__global__ void sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                              const int64_t* __restrict__ request, const int* __restrict__ position,
                              uint64_t seed, int* __restrict__ out, int vocab) {
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    pdl_enter();
    const int row = blockIdx.x;
    const float* lg = logits + (int64_t)row * vocab;
    const float t = temperature[row];
    uint64_t key = 0;
    if (t > 0.f) {
        key = mix64(seed * 0x9E3779B97F4A7C15ull + (uint64_t)request[row]);
        key = mix64(key ^ ((uint64_t)position[row] * 0xD1B54A32D192ED03ull));
    }
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        float v = lg[i];
        if (t > 0.f) {
            const uint64_t h = mix64(key + (uint64_t)i);
            const float u = ((float)(h >> 41) + 0.5f) * (1.0f / 8388608.0f);   // 23 bits + 0.5: never 0 or 1
            v = v / t - logf(-logf(u));
        }
        if (v > bv || (v == bv && i < bi) || bi == 0x7fffffff) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        bv = lane < nw ? best_v[lane] : -INFINITY;
        bi = lane < nw ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) out[row] = bi < vocab ? bi : 0;
    }
}

extern "C" int mie_sample(const float* logits, const float* temperature, const int64_t* request,
                          const int* position, uint64_t seed, int* out, int rows, int vocab,
                          cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return MIE_ERR_BAD_ARG;
    const int threads = vocab >= 8192 ? 1024 : (vocab >= 1024 ? 256 : 64);
    return launch_kernel(sample_kernel, dim3(rows), dim3(threads), 0, stream, logits, temperature, request, position, seed, out, vocab);
}

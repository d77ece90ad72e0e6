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

// A row is cut into SAMPLE_PARTS slices, one block each; the blocks of a row form a thread-block cluster
// and the first of them picks the winner out of the others' shared memory.  One block per row left the
// GPU idle at decode batch sizes (8 rows: 8 of 148 SMs, 9 us for 128 KB a row) and made the noise of a
// sampled row -- a hash and two logarithms per vocabulary entry -- one SM's work.
#define SAMPLE_PARTS 8
#define SAMPLE_THREADS 256

__device__ __forceinline__ void take(float& bv, int& bi, float v, int i) {
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
}

template <bool CLUSTER>
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const int64_t* __restrict__ request, const int* __restrict__ position,
              uint64_t seed, int* __restrict__ out, int vocab,
              int* __restrict__ host_out, const int* __restrict__ host_turn, int host_stride) {
    __shared__ float best_v[SAMPLE_THREADS / 32];
    __shared__ int best_i[SAMPLE_THREADS / 32];
    __shared__ float part_v;
    __shared__ int part_i;
    pdl_enter();
    const int row = blockIdx.y, part = blockIdx.x, parts = gridDim.x;
    const float* lg = logits + (int64_t)row * vocab;
    const float t = temperature[row];
    uint64_t key = 0;
    if (t > 0.f) {
        key = mix64(seed * 0x9E3779B97F4A7C15ull + (uint64_t)request[row]);
        key = mix64(key ^ ((uint64_t)position[row] * 0xD1B54A32D192ED03ull));
    }
    auto score = [&](float v, int i) {
        if (t > 0.f) {
            const uint64_t h = mix64(key + (uint64_t)i);
            const float u = ((float)(h >> 41) + 0.5f) * (1.0f / 8388608.0f);   // 23 bits + 0.5: never 0 or 1
            v = v / t - logf(-logf(u));
        }
        return v;
    };
    // this block's slice: whole groups of four entries, so that aligned rows can be read 16 bytes at a time
    const int per = ((vocab + parts - 1) / parts + 3) & ~3;
    const int lo = min(vocab, part * per), hi = min(vocab, lo + per);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    if ((reinterpret_cast<uintptr_t>(lg) & 15) == 0) {
        const int hi4 = lo + ((hi - lo) & ~3);
        for (int i = lo + threadIdx.x * 4; i < hi4; i += SAMPLE_THREADS * 4) {
            const float4 v = *reinterpret_cast<const float4*>(lg + i);
            take(bv, bi, score(v.x, i), i);
            take(bv, bi, score(v.y, i + 1), i + 1);
            take(bv, bi, score(v.z, i + 2), i + 2);
            take(bv, bi, score(v.w, i + 3), i + 3);
        }
        for (int i = hi4 + threadIdx.x; i < hi; i += SAMPLE_THREADS) take(bv, bi, score(lg[i], i), i);
    } else {
        for (int i = lo + threadIdx.x; i < hi; i += SAMPLE_THREADS) take(bv, bi, score(lg[i], i), i);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        take(bv, bi, ov, oi);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = lane < SAMPLE_THREADS / 32 ? best_v[lane] : -INFINITY;
        bi = lane < SAMPLE_THREADS / 32 ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            take(bv, bi, ov, oi);
        }
        if (lane == 0) { part_v = bv; part_i = bi; }
    }
    if (!CLUSTER) {
        if (threadIdx.x == 0) {
            const int tok = bi < vocab ? bi : 0;
            out[row] = tok;
            if (host_out) host_out[(host_turn ? *host_turn : 0) * host_stride + row] = tok;
        }
        return;
    }
    cluster_sync_all();                                          // every slice's winner is in its block's shared memory
    if (part == 0 && warp == 0) {
        bv = -INFINITY;
        bi = 0x7fffffff;
        if (lane < parts) {
            bv = ld_cluster_f32(cluster_addr((uint32_t)__cvta_generic_to_shared(&part_v), lane));
            bi = __float_as_int(ld_cluster_f32(cluster_addr((uint32_t)__cvta_generic_to_shared(&part_i), lane)));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            take(bv, bi, ov, oi);
        }
        if (lane == 0) {
            const int tok = bi < vocab ? bi : 0;
            out[row] = tok;
            // the host's copy, written straight into its (pinned, device-visible) memory: a copy engine
            // would take longer to start than this step's 32 bytes take to cross
            if (host_out) host_out[(host_turn ? *host_turn : 0) * host_stride + row] = tok;
        }
    }
    cluster_sync_all();                                          // nobody leaves while its shared memory is being read
}

// `host_out` (optional): pinned host memory [turns][host_stride] that the device can address; row r's
// token also goes to host_out[*host_turn][r] (host_turn: a device pointer to the turn, or null for 0).
extern "C" int mie_sample(const float* logits, const float* temperature, const int64_t* request,
                          const int* position, uint64_t seed, int* out, int rows, int vocab,
                          int* host_out, const int* host_turn, int host_stride, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return MIE_ERR_BAD_ARG;
    if (rows > 65535) return MIE_ERR_TOO_LARGE;
    if (vocab < 4096)                                            // a small vocabulary: one block a row
        return launch_kernel(sample_kernel<false>, dim3(1, rows), dim3(SAMPLE_THREADS), 0, stream, logits, temperature,
                             request, position, seed, out, vocab, host_out, host_turn, host_stride);
    return launch_kernel_cluster(sample_kernel<true>, dim3(SAMPLE_PARTS, rows), dim3(SAMPLE_THREADS), 0, stream,
                                 dim3(SAMPLE_PARTS, 1, 1), logits, temperature, request, position, seed, out, vocab,
                                 host_out, host_turn, host_stride);
}

// Rotary position encoding and the write of new keys and values into cache pages.
//
// Tables: cos/sin[p, j] of ang = p * inv_freq[j] in float32, j < rotary_dim/2
// (inference_engine/model.py:56-61, which rounds its tables to the model dtype; these stay 32-bit).
//
// Rotation (rotate-half pairing, inference_engine/model.py:64-69), for j < rotary_dim/2:
//   x'[j]        = x[j] * cos - x[j + half] * sin
//   x'[j + half] = x[j + half] * cos + x[j] * sin
// and dimensions >= rotary_dim pass through.  q is rotated in place inside the fused qkv rows;
// rotated k and plain v go to slot `slots[t]` of the layer's pages
// (inference_engine/model.py:130-134), page layout [page, kv_head, slot_in_page, head_dim].
#include "common.cuh"
#include "rope_math.cuh"
#include "range_check.cuh"

__global__ void rope_table_kernel(const float* __restrict__ inv_freq, float* __restrict__ cos_t,
                                  float* __restrict__ sin_t, int max_pos, int half) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)max_pos * half) return;
    const int p = (int)(idx / half), j = (int)(idx % half);
    const float ang = (float)p * inv_freq[j];
    float s, c;
    sincosf(ang, &s, &c);
    cos_t[idx] = c;
    sin_t[idx] = s;
}

extern "C" int mie_rope_table(const float* inv_freq, float* cos_t, float* sin_t, int max_pos,
                              int half, cudaStream_t stream) {
    if (max_pos <= 0 || half <= 0) return MIE_ERR_BAD_ARG;
    const int64_t total = (int64_t)max_pos * half;
    rope_table_kernel<<<(int)((total + 255) / 256), 256, 0, stream>>>(inv_freq, cos_t, sin_t, max_pos, half);
    return launch_status();
}

template <typename T>
__global__ void rope_cache_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                  const int* __restrict__ slots, const float* __restrict__ cos_t,
                                  const float* __restrict__ sin_t, T* __restrict__ k_cache,
                                  T* __restrict__ v_cache, int num_heads, int num_kv_heads,
                                  int head_dim, int rotary_dim, int page_size, int max_pos,
                                  int write_cache, int64_t num_pages, int* report) {
    pdl_enter();
    const int t = blockIdx.x;
    const int half = rotary_dim >> 1;
    const int pos = positions[t];
    // positions and slots are made on the host; one out of range is reported and its token left alone
    if (half > 0 && range_position(pos, max_pos) != MIE_RANGE_OK) {
        if (threadIdx.x == 0) range_report(report, MIE_RANGE_POSITION, MIE_K_ROPE_CACHE, t, pos);
        return;
    }
    if (write_cache && range_slot(slots[t], num_pages, page_size) != MIE_RANGE_OK) {
        if (threadIdx.x == 0) range_report(report, MIE_RANGE_SLOT, MIE_K_ROPE_CACHE, t, slots[t]);
        return;
    }
    const float* cs = cos_t + (int64_t)pos * half;
    const float* sn = sin_t + (int64_t)pos * half;
    T* row = qkv + (int64_t)t * (num_heads + 2 * num_kv_heads) * head_dim;

    // q heads: rotate in place
    for (int idx = threadIdx.x; idx < num_heads * half; idx += blockDim.x) {
        const int h = idx / half, j = idx - h * half;
        T* x = row + h * head_dim;
        const float a = to_f32<T>(x[j]), b = to_f32<T>(x[j + half]);
        const float c = cs[j], s = sn[j];
        x[j] = from_f32<T>(a * c - b * s);
        x[j + half] = from_f32<T>(b * c + a * s);
    }
    if (!write_cache) return;
    const int slot = slots[t];
    const int page = slot / page_size, off = slot - page * page_size;
    const T* k_row = row + num_heads * head_dim;
    const T* v_row = k_row + num_kv_heads * head_dim;
    // k heads: rotate into the cache; the pass-through tail and v are copied
    for (int idx = threadIdx.x; idx < num_kv_heads * head_dim; idx += blockDim.x) {
        const int h = idx / head_dim, d = idx - h * head_dim;
        const int64_t dst = (((int64_t)page * num_kv_heads + h) * page_size + off) * head_dim + d;
        const T* x = k_row + h * head_dim;
        float kv;
        if (d < half) kv = to_f32<T>(x[d]) * cs[d] - to_f32<T>(x[d + half]) * sn[d];
        else if (d < rotary_dim) kv = to_f32<T>(x[d]) * cs[d - half] + to_f32<T>(x[d - half]) * sn[d - half];
        else kv = to_f32<T>(x[d]);
        k_cache[dst] = from_f32<T>(kv);
        v_cache[dst] = v_row[idx];
    }
}

// bfloat16 with 16-byte accesses: eight rotation pairs per thread (rotary_dim % 16 == 0, head_dim % 8 == 0): rotate8 of rope_math.cuh.
__global__ void rope_cache_bf16x8_kernel(bf16* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ slots,
                                         const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                         bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, int num_heads, int num_kv_heads,
                                         int head_dim, int rotary_dim, int page_size, int max_pos, int write_cache,
                                         int64_t num_pages, int* report) {
    pdl_enter();
    const int t = blockIdx.x;
    const int half = rotary_dim >> 1, h8 = half >> 3, d8 = head_dim >> 3, tail8 = (head_dim - rotary_dim) >> 3;
    const int pos = positions[t];
    if (range_position(pos, max_pos) != MIE_RANGE_OK) {
        if (threadIdx.x == 0) range_report(report, MIE_RANGE_POSITION, MIE_K_ROPE_CACHE, t, pos);
        return;
    }
    if (write_cache && range_slot(slots[t], num_pages, page_size) != MIE_RANGE_OK) {
        if (threadIdx.x == 0) range_report(report, MIE_RANGE_SLOT, MIE_K_ROPE_CACHE, t, slots[t]);
        return;
    }
    const float* cs = cos_t + (int64_t)pos * half;
    const float* sn = sin_t + (int64_t)pos * half;
    bf16* row = qkv + (int64_t)t * (num_heads + 2 * num_kv_heads) * head_dim;
    for (int idx = threadIdx.x; idx < num_heads * h8; idx += blockDim.x) {
        const int h = idx / h8, j = (idx - h * h8) * 8;
        bf16* x = row + h * head_dim;
        uint4 lo = *reinterpret_cast<const uint4*>(x + j), hi = *reinterpret_cast<const uint4*>(x + j + half), olo, ohi;
        rotate8(lo, hi, cs + j, sn + j, olo, ohi);
        *reinterpret_cast<uint4*>(x + j) = olo;
        *reinterpret_cast<uint4*>(x + j + half) = ohi;
    }
    if (!write_cache) return;
    const int slot = slots[t];
    const int page = slot / page_size, off = slot - page * page_size;
    const bf16* k_row = row + num_heads * head_dim;
    const bf16* v_row = k_row + num_kv_heads * head_dim;
    for (int idx = threadIdx.x; idx < num_kv_heads * h8; idx += blockDim.x) {
        const int h = idx / h8, j = (idx - h * h8) * 8;
        const bf16* x = k_row + h * head_dim;
        const int64_t dst = (((int64_t)page * num_kv_heads + h) * page_size + off) * head_dim;
        uint4 lo = *reinterpret_cast<const uint4*>(x + j), hi = *reinterpret_cast<const uint4*>(x + j + half), olo, ohi;
        rotate8(lo, hi, cs + j, sn + j, olo, ohi);
        *reinterpret_cast<uint4*>(k_cache + dst + j) = olo;
        *reinterpret_cast<uint4*>(k_cache + dst + j + half) = ohi;
    }
    for (int idx = threadIdx.x; idx < num_kv_heads * (tail8 + d8); idx += blockDim.x) {
        const int h = idx / (tail8 + d8), c = idx - h * (tail8 + d8);
        const int64_t dst = (((int64_t)page * num_kv_heads + h) * page_size + off) * head_dim;
        if (c < tail8) {       // dimensions of k beyond the rotated ones pass through
            const int d = rotary_dim + c * 8;
            *reinterpret_cast<uint4*>(k_cache + dst + d) = *reinterpret_cast<const uint4*>(k_row + h * head_dim + d);
        } else {
            const int d = (c - tail8) * 8;
            *reinterpret_cast<uint4*>(v_cache + dst + d) = *reinterpret_cast<const uint4*>(v_row + h * head_dim + d);
        }
    }
}

extern "C" int mie_rope_cache_write(void* qkv, int act_tag, const int* positions, const int* slots,
                                    const float* cos_t, const float* sin_t, void* k_cache, void* v_cache,
                                    int num_tokens, int num_heads, int num_kv_heads, int head_dim,
                                    int rotary_dim, int page_size, int max_pos, int write_cache,
                                    long long num_pages, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (head_dim <= 0 || rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1) || page_size <= 0)
        return MIE_ERR_BAD_ARG;
    const int work = num_heads * (rotary_dim / 2) > num_kv_heads * head_dim ? num_heads * (rotary_dim / 2)
                                                                             : num_kv_heads * head_dim;
    int threads = 64;
    while (threads < 512 && threads < work) threads <<= 1;
    const bool aligned = ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) % 16) == 0;
    if (act_tag == MIE_BF16 && rotary_dim > 0 && rotary_dim % 16 == 0 && head_dim % 8 == 0 && aligned) {
        int t8 = 32;
        while (t8 < 256 && t8 * 8 < work) t8 <<= 1;
        return launch_kernel(rope_cache_bf16x8_kernel, dim3(num_tokens), dim3(t8), 0, stream, (bf16*)qkv, positions, slots, cos_t,
                             sin_t, (bf16*)k_cache, (bf16*)v_cache, num_heads, num_kv_heads, head_dim, rotary_dim, page_size,
                             max_pos, write_cache, (int64_t)num_pages, g_range_report);
    }
    if (act_tag == MIE_F32)
        return launch_kernel(rope_cache_kernel<float>, dim3(num_tokens), dim3(threads), 0, stream,
            (float*)qkv, positions, slots, cos_t, sin_t, (float*)k_cache, (float*)v_cache, num_heads,
            num_kv_heads, head_dim, rotary_dim, page_size, max_pos, write_cache, (int64_t)num_pages, g_range_report);
    else if (act_tag == MIE_BF16)
        return launch_kernel(rope_cache_kernel<bf16>, dim3(num_tokens), dim3(threads), 0, stream,
            (bf16*)qkv, positions, slots, cos_t, sin_t, (bf16*)k_cache, (bf16*)v_cache, num_heads,
            num_kv_heads, head_dim, rotary_dim, page_size, max_pos, write_cache, (int64_t)num_pages, g_range_report);
    return MIE_ERR_BAD_ARG;
}

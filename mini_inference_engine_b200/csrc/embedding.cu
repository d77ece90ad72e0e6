// Embedding gather: res[t, :] = table[ids[t], :], written as float32 because the gathered row
// opens the residual stream, which this engine keeps in 32-bit
// (what F.embedding does at inference_engine/model.py:168).
// A negative id -(k+1) stands for "the k-th token the previous step sampled": it is read from the
// `feedback` buffer on the device, so a step can be launched before the host has seen that token.
#include "common.cuh"
#include "range_check.cuh"

template <typename TT>
__global__ void embedding_kernel(const TT* __restrict__ table, const int* __restrict__ ids,
                                 const int* __restrict__ feedback, float* __restrict__ out, int hidden, int vocab,
                                 int feedback_len, int* report) {
    pdl_enter();
    const int t = blockIdx.x;
    int id = ids[t];
    // ids are checked on the host when a request is added; one out of range here is reported and its
    // row left as it is (both the id in the batch and the token it may stand for are checked)
    bool ok = range_token(id, vocab, feedback ? feedback_len : 0) == MIE_RANGE_OK;
    if (ok && id < 0) { id = feedback[-id - 1]; ok = id >= 0 && id < vocab; }
    if (!ok) {
        if (threadIdx.x == 0) range_report(report, MIE_RANGE_TOKEN, MIE_K_EMBEDDING, t, id);
        return;
    }
    const TT* src = table + (int64_t)id * hidden;
    float* dst = out + (int64_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32<TT>(src[i]);
}

extern "C" int mie_embedding(const void* table, int table_tag, const int* ids, const int* feedback, float* out,
                             int num_tokens, int hidden, int vocab, int feedback_len, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (hidden <= 0 || vocab <= 0) return MIE_ERR_BAD_ARG;
    const int threads = hidden >= 1024 ? 256 : (hidden >= 256 ? 128 : 64);
    if (table_tag == MIE_F32)
        return launch_kernel(embedding_kernel<float>, dim3(num_tokens), dim3(threads), 0, stream, (const float*)table, ids, feedback, out, hidden, vocab, feedback_len, g_range_report);
    else if (table_tag == MIE_BF16)
        return launch_kernel(embedding_kernel<bf16>, dim3(num_tokens), dim3(threads), 0, stream, (const bf16*)table, ids, feedback, out, hidden, vocab, feedback_len, g_range_report);
    return MIE_ERR_BAD_ARG;
}

// Decode attention with its scratch memory inside the library: see attention_decode_static.h for
// who needs this and the rules of use.  The kernel is the one of attention_decode.cu.
#include "attention_decode.cuh"
#include "attention_decode_static.h"

#include <stdio.h>

// partial outputs | partial log-sum-exps | split counters
static __device__ __align__(256) unsigned char g_static_scratch[MIE_STATIC_SCRATCH_BYTES];

#define MIE_STATIC_MAX_DEVICES 64
static unsigned char* g_scratch_address[MIE_STATIC_MAX_DEVICES];   // device address per device, 0 = not looked up yet
static thread_local char g_error[256];

extern "C" const char* mie_decode_attention_static_error(void) { return g_error; }

// In host code `g_static_scratch` is only a handle for the runtime, not a device address; the
// address a kernel can use comes from cudaGetSymbolAddress, once per device with that device current.
static int scratch_for_current_device(unsigned char** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { snprintf(g_error, sizeof g_error, "cudaGetDevice failed: %s", cudaGetErrorString(e)); return (int)e; }
    if (dev < 0 || dev >= MIE_STATIC_MAX_DEVICES) {
        snprintf(g_error, sizeof g_error, "device %d is beyond the %d devices this entry point keeps addresses for", dev,
                 MIE_STATIC_MAX_DEVICES);
        return MIE_ERR_TOO_LARGE;
    }
    if (!g_scratch_address[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) {
            snprintf(g_error, sizeof g_error, "cudaGetSymbolAddress of the static scratch failed on device %d: %s", dev,
                     cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : MIE_ERR_BAD_ARG;
        }
        g_scratch_address[dev] = (unsigned char*)p;
    }
    *out = g_scratch_address[dev];
    return 0;
}

extern "C" int mie_decode_attention_static(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                                           const int* block_tables, int table_stride, const int* row_q_start,
                                           const int* row_q_len, const int* row_ctx_len, int num_rows, void* out,
                                           int num_heads, int num_kv_heads, int head_dim, int page_size, float scale,
                                           int window, int splits, cudaStream_t stream) {
    g_error[0] = 0;
    if (num_rows <= 0) return 0;
    float* part_o = nullptr;
    float* part_lse = nullptr;
    int* counters = nullptr;
    if (splits > 1) {
        if (num_kv_heads <= 0 || num_heads <= 0 || num_heads % num_kv_heads || head_dim <= 0) {
            snprintf(g_error, sizeof g_error, "bad head counts or head size (%d heads, %d kv heads, head_dim %d)", num_heads,
                     num_kv_heads, head_dim);
            return MIE_ERR_BAD_ARG;
        }
        const long long lse = (long long)num_rows * num_heads * splits;
        const long long po = lse * head_dim;
        const long long units = (long long)num_rows * num_kv_heads * ((num_heads / num_kv_heads + 15) / 16);
        if (po > MIE_STATIC_MAX_PART_O || lse > MIE_STATIC_MAX_PART_LSE || units > MIE_STATIC_MAX_UNITS) {
            snprintf(g_error, sizeof g_error,
                     "too large for the static scratch: rows*heads*splits*head_dim = %lld (max %d), rows*heads*splits = %lld "
                     "(max %d), rows*kv_heads*chunks = %lld (max %d); use fewer splits or mie_decode_attention with your own scratch",
                     po, MIE_STATIC_MAX_PART_O, lse, MIE_STATIC_MAX_PART_LSE, units, MIE_STATIC_MAX_UNITS);
            return MIE_ERR_TOO_LARGE;
        }
        unsigned char* base = nullptr;
        const int rc = scratch_for_current_device(&base);
        if (rc) return rc;
        part_o = reinterpret_cast<float*>(base);
        part_lse = part_o + MIE_STATIC_MAX_PART_O;
        counters = reinterpret_cast<int*>(part_lse + MIE_STATIC_MAX_PART_LSE);
        // the counters must start at zero whatever the last call (or an aborted one) left
        const cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)units * sizeof(int), stream);
        if (e != cudaSuccess) { snprintf(g_error, sizeof g_error, "cudaMemsetAsync failed: %s", cudaGetErrorString(e)); return (int)e; }
    }
    const int rc = decode_attention_launch(q, q_stride, k_cache, v_cache, block_tables, table_stride, row_q_start,
                                           row_q_len, row_ctx_len, num_rows, out, num_heads, num_kv_heads, head_dim,
                                           page_size, scale, window, splits, part_o, part_lse, counters, stream);
    if (rc < 0) snprintf(g_error, sizeof g_error, "the decode kernel refused the sizes (code %d): head_dim a multiple of 16 up to %d, "
                         "page_size a power of two, heads a multiple of kv heads", rc, DEC_MAX_D);
    else if (rc > 0) snprintf(g_error, sizeof g_error, "launch failed: %s", cudaGetErrorString((cudaError_t)rc));
    return rc;
}

// Range checks on the integers a step hands the kernels: token ids, positions, cache slots, page
// ids and row indices.  The host builds them and is trusted, but a fault there would read or write
// outside an allocation, and nothing else on the device would notice.  A kernel that meets a value
// out of range records it in a four-word report (first one wins), skips the access -- or, for a page
// id inside an attention loop, reads the scratch page 0 instead -- and goes on; the engine reads the
// report after the step's synchronisation and raises.  The report lives in host-mapped memory; a
// null pointer means "check and skip, report nowhere".
//
// The predicates are __host__ __device__ so that their arithmetic is tested on the host.
#pragma once
#include <stdint.h>

#define MIE_RANGE_OK 0
#define MIE_RANGE_TOKEN 1       // token id outside [-feedback_len, vocab)
#define MIE_RANGE_POSITION 2    // position outside [0, table length)
#define MIE_RANGE_SLOT 3        // cache slot outside [0, pages * page_size)
#define MIE_RANGE_PAGE 4        // block-table entry outside [0, pages)
#define MIE_RANGE_ROW 5         // row index outside [0, rows)

#ifdef __CUDACC__
#define MIE_HD __host__ __device__ __forceinline__
#else
#define MIE_HD inline
#endif

// A token id is a vocabulary entry, or -(k+1) for entry k of the previous step's sampled tokens.
MIE_HD int range_token(int id, int vocab, int feedback_len) {
    return (id >= 0 ? id < vocab : -(int64_t)id - 1 < (int64_t)feedback_len) ? MIE_RANGE_OK : MIE_RANGE_TOKEN;
}
MIE_HD int range_position(int pos, int table_len) {
    return (pos >= 0 && pos < table_len) ? MIE_RANGE_OK : MIE_RANGE_POSITION;
}
MIE_HD int range_slot(int slot, int64_t num_pages, int page_size) {
    return (slot >= 0 && (int64_t)slot < num_pages * (int64_t)page_size) ? MIE_RANGE_OK : MIE_RANGE_SLOT;
}
MIE_HD int range_page(int page, int64_t num_pages) {
    return (page >= 0 && (int64_t)page < num_pages) ? MIE_RANGE_OK : MIE_RANGE_PAGE;
}
MIE_HD int range_row(int64_t row, int64_t num_rows) {
    return (row >= 0 && row < num_rows) ? MIE_RANGE_OK : MIE_RANGE_ROW;
}

#ifdef __CUDACC__
// report = {code, kernel id, index (which token / row / table entry), value}
#define MIE_K_EMBEDDING 1
#define MIE_K_ROPE_CACHE 2
#define MIE_K_NORM 3
#define MIE_K_ATTENTION_SIMT 4
#define MIE_K_ATTENTION_DECODE 5
#define MIE_K_ATTENTION_PREFILL 6
#define MIE_K_ATTENTION_PREFILL_TC 7
#define MIE_K_GEMM_QKV_ROPE 8

__device__ __forceinline__ void range_report(int* report, int code, int kernel, int index, int value) {
    if (report == nullptr) return;
    if (atomicCAS_system(report, 0, code) == 0) {
        report[1] = kernel;
        report[2] = index;
        report[3] = value;
        __threadfence_system();
    }
}
// Every library that checks ranges holds the report's device address, set once after loading.
static int* g_range_report = nullptr;
extern "C" void mie_set_range_report(int* report) { g_range_report = report; }
// The predicates as the host compiles them (for tests of their arithmetic): kind = MIE_RANGE_*.
extern "C" int mie_range_predicate(int kind, long long value, long long limit, long long limit2) {
    switch (kind) {
        case MIE_RANGE_TOKEN: return range_token((int)value, (int)limit, (int)limit2);
        case MIE_RANGE_POSITION: return range_position((int)value, (int)limit);
        case MIE_RANGE_SLOT: return range_slot((int)value, limit, (int)limit2);
        case MIE_RANGE_PAGE: return range_page((int)value, limit);
        case MIE_RANGE_ROW: return range_row(value, limit);
    }
    return -1;
}

// The page id to read: itself when in range, else the scratch page, with a report.
__device__ __forceinline__ int checked_page(int page, int64_t num_pages, int* report, int kernel, int index) {
    if (range_page(page, num_pages) == MIE_RANGE_OK) return page;
    range_report(report, MIE_RANGE_PAGE, kernel, index, page);
    return 0;
}
#endif

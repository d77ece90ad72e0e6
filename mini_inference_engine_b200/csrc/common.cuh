// Shared device helpers for the kernels of this package (sm_100a only).
// Every launcher is an extern "C" function that takes raw device pointers, sizes and a
// stream, launches on that stream and returns the cudaError_t of the launch (0 = ok), or a
// negative code of its own for arguments it refuses.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MIE_ERR_BAD_ARG (-1)      // a size or option this kernel does not take
#define MIE_ERR_TOO_LARGE (-2)    // beyond a stated maximum

// element type tags shared with the Python side
#define MIE_F32 0
#define MIE_BF16 1

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// load by runtime tag (norm weights and tables may be stored in either type)
__device__ __forceinline__ float load_tagged(const void* p, int64_t i, int tag) {
    return tag == MIE_F32 ? reinterpret_cast<const float*>(p)[i]
                          : __bfloat162float(reinterpret_cast<const bf16*>(p)[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `red` is 33 floats of
// shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();                       // protect `red` against a previous use
    if (lane == 0) red[warp] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    if (warp == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// The row that work item `index` belongs to when row r has items_of(row_q_len[r]) items (0 for a row that another
// kernel serves), found by the 32 lanes of a warp together -- 32 rows a round, a prefix sum by shuffles -- instead of
// one thread walking the rows: a step may hold hundreds of one-token rows in front of the row a block is looking
// for.  Returns the row (-1: there is no such item), the item's number within the row and the row's item count;
// every lane gets the same answer.  Row lengths belong to the step's inputs, copied to the device before its first
// kernel: they may be read before the dependency wait.
template <typename F>
__device__ __forceinline__ int warp_find_row(const int* __restrict__ row_q_len, int num_rows, int index, F items_of,
                                             int& within, int& items_r) {
    const int lane = threadIdx.x & 31;
    for (int base = 0; base < num_rows; base += 32) {
        const int r = base + lane;
        const int n = r < num_rows ? items_of(row_q_len[r]) : 0;
        int incl = n;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        const int total = __shfl_sync(0xffffffffu, incl, 31);
        if (index < total) {
            const int l = __ffs(__ballot_sync(0xffffffffu, incl > index)) - 1;
            items_r = __shfl_sync(0xffffffffu, n, l);
            within = index - (__shfl_sync(0xffffffffu, incl, l) - items_r);
            return base + l;
        }
        index -= total;
    }
    within = 0;
    items_r = 0;
    return -1;
}

static inline int launch_status() { return (int)cudaGetLastError(); }

// Streaming multiprocessors of the current device, asked once per device.
static inline int device_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
        cached[dev] = n;
    }
    return cached[dev];
}

// Programmatic dependent launch.  Every kernel of this package starts with pdl_enter(): it lets the
// next kernel in the stream be scheduled at once (its blocks become resident and run their own
// prologue) and then waits until the kernels before it have completed and their writes are visible.
// What is gained is the launch gap between dependent kernels; what keeps it correct is that no
// kernel writes global memory, or reads anything that a kernel of the same step writes, before its
// wait, and that every block of every kernel waits, so "the kernel before me is complete" carries
// over the whole chain.  Three kernels do read before their wait, and only what is older than the
// step: the tcgen05 product its weights (and, with the rotation epilogue, positions, slots and the
// cos/sin rows), decode attention the lengths, block tables and every cached row but the newest.  Launched without the
// attribute (MIE_B200_PDL=0), both instructions do nothing.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_enter() { pdl_launch_dependents(); pdl_wait(); }

#include <stdlib.h>
static inline bool pdl_enabled() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("MIE_B200_PDL"); v = (e && e[0] == '0') ? 0 : 1; }
    return v == 1;
}

// kernel<<<grid, block, smem, stream>>>(args...) with the programmatic-serialization attribute and,
// when `cluster` has more than one block, as thread-block clusters of that shape.
template <typename... KArgs, typename... Args>
static inline int launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                        cudaStream_t stream, dim3 cluster, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (cluster.x * cluster.y * cluster.z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster.x; attr[n].val.clusterDim.y = cluster.y; attr[n].val.clusterDim.z = cluster.z;
        ++n;
    }
    if (pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    return e != cudaSuccess ? (int)e : launch_status();
}
template <typename... KArgs, typename... Args>
static inline int launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                Args... args) {
    return launch_kernel_cluster(kernel, grid, block, smem, stream, dim3(1, 1, 1), args...);
}

// Thread-block clusters: a barrier over all threads of all blocks of the cluster, and loads from
// another block's shared memory (distributed shared memory).
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The two halves of the cluster barrier, for a barrier whose arrival and wait lie apart.
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The address of `local_addr` (a shared::cta address of this block) in block `rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_addr(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    return remote;
}
// Plain (not volatile) so that the loads of all ranks are in flight together; ordering against the
// peers' writes comes from the cluster barrier before the first load.
__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t addr) {
    float4 v;
    asm("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
// A store into another block's shared memory; the cluster barrier after it (release / acquire)
// makes it visible there.
__device__ __forceinline__ void st_cluster_f32x4(uint32_t addr, float a, float b, float c, float d) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
// The same store, asynchronous: it also counts its 16 bytes on an mbarrier of the block it writes to
// (`bar`, an address in that block's shared memory), so the receiver can wait for exactly what it is
// owed instead of the whole cluster meeting at a barrier.
__device__ __forceinline__ void st_async_cluster_f32x4(uint32_t addr, uint32_t bar, float a, float b, float c, float d) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];"
                 ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d), "r"(bar) : "memory");
}
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float a) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(a) : "memory");
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
    float v;
    asm("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}

// Shared by every kernel file: element types, small reductions, error reporting.
//
// Launchers are plain C functions taking raw device pointers and a stream, so a
// library builds in seconds with nvcc alone and loads through ctypes. A launcher
// returns 0, a CUDA error code (> 0) or ABK_REFUSED (< 0: the sizes are not ones
// this kernel takes; abk_last_error() says why).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define ABK_REFUSED (-1)
enum { ABK_F32 = 0, ABK_BF16 = 1 };

#ifdef ABK_DEFINE_ERROR
static thread_local char abk_error_text[512];
extern "C" const char *abk_last_error() { return abk_error_text; }
#define ABK_REFUSE(...)                                                  \
    do {                                                                 \
        snprintf(abk_error_text, sizeof abk_error_text, __VA_ARGS__);    \
        return ABK_REFUSED;                                              \
    } while (0)
#endif

#define ABK_LAUNCH_RESULT() ((int)cudaGetLastError())

// Programmatic dependent launch. A kernel that starts with pdl_wait() may be launched with
// abk_launch(): its CTAs are then scheduled, and run whatever stands before pdl_wait(), while the
// kernel before it in the stream is still finishing, and pdl_wait() returns once that kernel has
// completed and its writes are visible. Nothing before pdl_wait() may read what the kernel just before
// writes (what kernels further back wrote is complete by then), nor write global memory. In a step of a few hundred small kernels this hides most of the
// launch latency of each. Kernels launched the ordinary way are unaffected by pdl_wait().
//
// Built with -DABK_TRACE=<number of the source file> (see kernels/trace.py), thread 0 of the first CTA
// of every launch also records when it reached pdl_wait() and when it was let go, on the device-wide
// nanosecond timer: the second time of a launch is the moment the launch before it had finished, so a
// step's records give its timeline without a profiler serialising it.
#ifdef ABK_TRACE
#define ABK_TRACE_MAX 16384
struct AbkTraceRecord {
    unsigned long long reached, released;
    int file, grid, block, pad;
};
__device__ AbkTraceRecord abk_trace_records[ABK_TRACE_MAX];
__device__ unsigned int abk_trace_count;
__device__ __forceinline__ unsigned long long abk_trace_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#ifdef ABK_DEFINE_ERROR
// Copies the records made so far to `out` (room for `max`) and starts over; returns how many there were.
extern "C" int abk_trace_read(void *out, int max) {
    unsigned int n = 0, zero = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&n, abk_trace_count, sizeof n) != cudaSuccess) return -1;
    if (n > ABK_TRACE_MAX) n = ABK_TRACE_MAX;
    if ((int)n > max) n = max;
    if (n && cudaMemcpyFromSymbol(out, abk_trace_records, n * sizeof(AbkTraceRecord)) != cudaSuccess) return -1;
    if (cudaMemcpyToSymbol(abk_trace_count, &zero, sizeof zero) != cudaSuccess) return -1;
    return (int)n;
}
#endif
#endif
__device__ __forceinline__ void pdl_wait() {
#ifdef ABK_TRACE
    const unsigned long long reached = abk_trace_ns();
#endif
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#ifdef ABK_TRACE
    if (threadIdx.x == 0 && threadIdx.y == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
        unsigned int i = atomicAdd(&abk_trace_count, 1u);
        if (i < ABK_TRACE_MAX)
            abk_trace_records[i] = {reached, abk_trace_ns(), ABK_TRACE, (int)(gridDim.x * gridDim.y * gridDim.z),
                                    (int)(blockDim.x * blockDim.y), 0};
    }
#endif
}

#ifdef __CUDACC__
#include <cstdlib>
#include <mutex>
#include <map>
#include <utility>
// Lets `kernel` use `bytes` of dynamic shared memory (more than the 48 KB a kernel gets unasked). The setting is per
// device and per kernel: it is made when a pair first asks, and again when it asks for more than it has; other
// calls cost a lookup under a lock.
static inline cudaError_t abk_allow_shared_memory(const void *kernel, int bytes) {
    static std::mutex lock;
    static std::map<std::pair<int, const void *>, int> allowed;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> guard(lock);
    auto it = allowed.find({device, kernel});
    if (it != allowed.end() && it->second >= bytes) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) allowed[{device, kernel}] = bytes;
    return e;
}
// SMs of the current device (148 on a B200), asked once per device.
static inline int abk_sm_count() {
    static std::mutex lock;
    static int of_device[64];
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
    std::lock_guard<std::mutex> guard(lock);
    if (!of_device[device]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
        of_device[device] = n;
    }
    return of_device[device];
}
static inline bool abk_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char *e = getenv("ABACUS_PDL");
        on = !(e && e[0] == '0');
    }
    return on != 0;
}
// The grid's CTAs come as clusters of `cluster` CTAs (each grid dimension must be a multiple of the cluster's).
template <typename... KArgs, typename... Args>
static inline void abk_launch_clusters(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                       dim3 cluster, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (cluster.x * cluster.y * cluster.z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster.x, attr[n].val.clusterDim.y = cluster.y, attr[n].val.clusterDim.z = cluster.z;
        n++;
    }
    if (abk_pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    cfg.attrs = attr, cfg.numAttrs = n;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);  // the error, if any, is read by ABK_LAUNCH_RESULT
}
template <typename... KArgs, typename... Args>
static inline void abk_launch_clusters(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                       int cluster_x, Args &&...args) {
    abk_launch_clusters(kernel, grid, block, smem, stream, dim3(cluster_x, 1, 1), std::forward<Args>(args)...);
}
template <typename... KArgs, typename... Args>
static inline void abk_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args &&...args) {
    abk_launch_clusters(kernel, grid, block, smem, stream, dim3(1, 1, 1), std::forward<Args>(args)...);
}
#endif

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// silu(gate) * up for the bfloat16 path (src/model.c:274-282): the exponential and the reciprocal by the
// special-function unit (a few units in the last place of float32, far below the bfloat16 the result is
// stored in). Every bfloat16 kernel uses this one, so a token's activation is the same on every way.
__device__ __forceinline__ float silu_mul_fast(float gate, float up) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(gate * -1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return gate * r * up;
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

// Sum over a block of up to 1024 threads; every thread gets the result. `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float *scratch) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < n_warps ? scratch[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float *scratch) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < n_warps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Where a position of a sequence lies in a paged cache.
//   tokens_per_page keys per page; a sequence's pages are listed in its row of the page table.
//   ring_pages > 0: the sequence keeps only that many pages and position p lives in
//   logical page (p / tokens_per_page) % ring_pages (a window of the most recent keys).
struct PagedCache {
    const int *page_table;  // [slots, table_width]
    int table_width;
    int ring_pages;         // 0: all pages are kept
    int tokens_per_page;
};
__device__ __forceinline__ int cache_page(const PagedCache &c, int slot, int pos) {
    int logical = pos / c.tokens_per_page;
    if (c.ring_pages > 0) logical %= c.ring_pages;
    return c.page_table[(long long)slot * c.table_width + logical];
}
// Element offset of (page, kv head, position, 0) in a pool laid out [pages, kv heads, tokens_per_page, head_dim].
__device__ __forceinline__ long long cache_offset(const PagedCache &c, int page, int kv_head, int n_kv_heads, int pos,
                                                  int head_dim) {
    return (((long long)page * n_kv_heads + kv_head) * c.tokens_per_page + pos % c.tokens_per_page) * head_dim;
}

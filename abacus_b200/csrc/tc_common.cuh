// Blackwell (sm_100a) building blocks in inline PTX: mbarriers with bounded waits, TMA tile
// loads, tensor memory (TMEM) allocation, tcgen05.mma issue and commit, tcgen05.ld.
//
// Every wait gives up after a limit and reports it; no loop here can spin for ever.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tc {

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
// Waits for the phase with the given parity; false if it did not come within the library's limit of wall time. The
// limit starts at a quarter of a second: thousands of times longer than any wait of a working kernel, and short
// enough that a kernel whose barriers are wrong ends at once instead of spinning for minutes. It is a variable of
// the library on the device, so a caller (a test that lets a wait run out on purpose) can set it at run time.
#define TC_WAIT_NS 250000000ull
__device__ unsigned long long abk_wait_limit_ns = TC_WAIT_NS;
#ifdef ABK_DEFINE_ERROR
// Sets the limit of every bounded wait of this library's kernels on the current device, in nanoseconds.
extern "C" int abk_set_wait_limit_ns(unsigned long long ns) {
    return (int)cudaMemcpyToSymbol(abk_wait_limit_ns, &ns, sizeof ns);
}
#endif
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t start = global_ns(), limit = abk_wait_limit_ns;
    for (;;) {
        for (int i = 0; i < 64; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_ns() - start > limit) return false;
    }
}

// ------------------------------------------------------------------ thread-block clusters
// Rank of this CTA in its cluster and the cluster's size (0 and 1 for a launch without clusters).
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
    uint32_t n;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(n));
    return n;
}
// Barrier over all threads of all CTAs of the cluster; every thread must reach it, converged. What
// was written to shared memory before it is visible to the other CTAs after it.
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address, in the cluster's window, of CTA `rank`'s copy of this CTA's shared address `addr`.
__device__ __forceinline__ uint32_t peer_smem(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float2 ld_cluster_f2(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}

// ------------------------------------------------------------------ TMA
// Loads the box of `map` whose first element is (x, y) (x: innermost, in elements) into shared
// memory and signals `bar` with the bytes written. x * element size must be a multiple of 16.
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_addr(dst)), "l"((uint64_t)map), "r"(smem_addr(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)map) : "memory");
}

// ------------------------------------------------------------------ tensor memory
// One whole warp allocates `columns` (a power of two >= 32) and writes the address to *holder.
__device__ __forceinline__ void tmem_alloc(uint32_t *holder, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(holder)),
                 "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t addr, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(columns) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ------------------------------------------------------------------ tcgen05.mma
// Shared-memory operand descriptor for a K-major tile stored as rows of 128 bytes with the
// 128-byte swizzle (what a TMA load with CU_TENSOR_MAP_SWIZZLE_128B writes): groups of 8 rows
// are 1024 bytes apart. `addr` is the shared address of the tile's first row (+ 32 bytes per
// step of 16 bfloat16 along K inside the 128-byte row).
__device__ __forceinline__ uint64_t smem_desc_k_sw128(uint32_t addr) {
    uint64_t d = (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;          // leading byte offset (unused with swizzled K-major tiles)
    d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset: 8 rows of 128 bytes
    d |= (uint64_t)1 << 46;          // descriptor version of sm_100
    d |= (uint64_t)2 << 61;          // 128-byte swizzle
    return d;
}
// Instruction descriptor: bfloat16 A and B (both K-major), float32 accumulator, tile M x N.
__host__ __device__ constexpr uint32_t idesc_bf16_f32(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// D[tmem] (+)= A[smem] . B[smem]^T, issued by one thread.
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                       bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// The barrier gets one arrival when all tcgen05.mma issued so far by this thread are done.
__device__ __forceinline__ void mma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar))
                 : "memory");
}

// ------------------------------------------------------------------ pairs of CTAs on one tile (cta_group::2)
// Two CTAs of a cluster (ranks 2i and 2i + 1, on the two SMs of a pair) share one product: each holds half of A's
// rows and half of B's rows in its own shared memory, at the same offsets, and gets its half of the accumulator's rows
// in its own tensor memory; the even CTA (the leader) issues the instruction for both. Every load is a CTA's own,
// plain copy into its own shared memory (no multicast); only its completion is reported to the leader's barrier.
//
// Both CTAs allocate together: one warp of each, the same warp in both, the same `holder` offset.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *holder, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(holder)),
                 "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free_pair(uint32_t addr, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(columns) : "memory");
}
// A CTA's own box into its own shared memory; the bytes are reported to the barrier at `bar_in_cluster`, an address
// in the cluster's window (peer_smem of the leader's barrier).
__device__ __forceinline__ void tma_load_2d_pair(void *dst, const CUtensorMap *map, int x, int y, uint32_t bar_in_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_addr(dst)), "l"((uint64_t)map), "r"(bar_in_cluster), "r"(x), "r"(y)
        : "memory");
}
// D[tensor memory of both CTAs] (+)= A . B^T over the pair: M = 256 (128 rows from each CTA), N columns (N / 2 rows of B
// from each CTA). Issued by one thread of the leader.
__device__ __forceinline__ void mma_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// The barrier at this offset in both CTAs of the pair gets one arrival when all tcgen05.mma issued so far are done.
__device__ __forceinline__ void mma_commit_pair(uint64_t *bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_addr(bar)),
        "h"((uint16_t)3)
        : "memory");
}
// One arrival on a barrier of another CTA of the cluster.
__device__ __forceinline__ void mbar_arrive_in_cluster(uint32_t bar_in_cluster) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_in_cluster) : "memory");
}

// ------------------------------------------------------------------ tcgen05.ld
// 32 lanes x 16 columns of 32 bits: thread t of the warp gets lane (base lane + t), v[j] = column j.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t *v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace tc

// Warp-level tensor-core tiles for the attention kernels: ldmatrix from TMA-swizzled boxes, mma.sync
// m16n8k16 in bfloat16 with float32 accumulation, and the two products of attention on them.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

#define PAGE 64
#define BOX_BYTES 8192  // 64 rows of 128 bytes

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
// c (16 x 8, float32) += a (16 x 16, bfloat16, row-major) . b (16 x 8, bfloat16, column-major)
__device__ __forceinline__ void mma_bf16(float *c, const uint32_t *a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Address of the 16-byte chunk `chunk` (0..7) of row `row` in a box written by TMA with the 128-byte swizzle.
__device__ __forceinline__ uint32_t sw128(uint32_t base, int row, int chunk) {
    return base + row * 128 + ((chunk ^ (row & 7)) << 4);
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *(uint32_t *)&t;
}
__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// S (16 rows x 8 * NT keys) = Q . K^T for one warp: q fragments in registers, keys `key0 ..` of the
// page at `k_base` (boxes of 64 columns, BOX_BYTES apart).
template <int HD, int NT>
__device__ __forceinline__ void scores(float (*s)[4], const uint32_t (*qf)[4], uint32_t k_base, int key0, int lane) {
#pragma unroll
    for (int nt = 0; nt < NT; nt++) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
    const int j = lane >> 3, r8 = lane & 7;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ks++) {
        const uint32_t box = k_base + (ks / 4) * BOX_BYTES;
        const int c0 = (ks % 4) * 2;
#pragma unroll
        for (int ntp = 0; ntp < NT / 2; ntp++) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4(sw128(box, key0 + 8 * (2 * ntp + (j >> 1)) + r8, c0 + (j & 1)), b0, b1, b2, b3);
            mma_bf16(s[2 * ntp], qf[ks], b0, b1);
            mma_bf16(s[2 * ntp + 1], qf[ks], b2, b3);
        }
    }
}

// O (16 rows x HD) += P (16 x 16 * KS keys, as A fragments) . V, values of keys `key0 ..` of the page at v_base.
template <int HD, int KS>
__device__ __forceinline__ void weighted_values(float (*o)[4], const uint32_t (*pf)[4], uint32_t v_base, int key0, int lane) {
    const int j = lane >> 3, r8 = lane & 7;
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
#pragma unroll
        for (int ntp = 0; ntp < HD / 16; ntp++) {
            const int nt = 2 * ntp;
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t(sw128(v_base + (nt / 8) * BOX_BYTES, key0 + 16 * ks + 8 * (j & 1) + r8, (nt % 8) + (j >> 1)), b0, b1, b2, b3);
            mma_bf16(o[nt], pf[ks], b0, b1);
            mma_bf16(o[nt + 1], pf[ks], b2, b3);
        }
    }
}

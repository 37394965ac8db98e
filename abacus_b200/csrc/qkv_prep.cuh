// What is done to one head of one token between the q/k/v product and attention (src/model.c:247-259), for the
// kernels that hold a bfloat16 head as 8 consecutive elements a lane: RMSNorm over the head with a weight shared by
// all heads (q and k, not v), then the rotary encoding over the whole head in halves (element i pairs with
// i + HD / 2). The q/k/v preparation kernels and the decode attention that prepares its own heads both use it, so a
// head comes out the same whichever prepares it.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

// The arithmetic, every rounding written out, so that the two ways of holding a head below give the same bits.
template <int HD> __device__ __forceinline__ float prep_scale(float ss, float eps) { return 1.0f / sqrtf(__fadd_rn(ss / (float)HD, eps)); }
__device__ __forceinline__ float prep_normed(float w, float v, float scale) { return __fmul_rn(w, __fmul_rn(v, scale)); }
// element i of the lower half with its partner i + HD / 2, angle i: (lo cos - hi sin, hi cos + lo sin)
__device__ __forceinline__ float prep_rotated_lower(float lo, float hi, float c, float s) { return __fmaf_rn(lo, c, -__fmul_rn(hi, s)); }
__device__ __forceinline__ float prep_rotated_upper(float hi, float lo, float c, float s) { return __fmaf_rn(hi, c, __fmul_rn(lo, s)); }

// raw: this lane's 8 elements (16 bytes) of the head; l: which 8 of the head (lane within the head's HD / 8 lanes, which
// are consecutive lanes of the warp); upper: l >= HD / 16. prepared: a q or k head (a v head comes back as it is).
// w: the norm's weights, or null; eps. rotate: with the lane's angles cs / sn (8 each: of elements 8 l .. of the
// lower half, or of their partners' for an upper lane). Whole warps call it (it shuffles).
template <int HD>
__device__ __forceinline__ uint4 prep_head_values(uint4 raw, bool prepared, const float *w, float eps, bool rotate, int l,
                                                  bool upper, const float *cs, const float *sn) {
    constexpr int LPH = HD / 8;
    const uint32_t in[4] = {raw.x, raw.y, raw.z, raw.w};
    float v[8];
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const float2 f = __bfloat1622float2(*(const __nv_bfloat162 *)&in[e]);
        v[2 * e] = f.x, v[2 * e + 1] = f.y;
    }
    float ss = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; e++) ss = __fmaf_rn(v[e], v[e], ss);
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));  // over the head's lanes
    if (prepared && w) {
        const float scale = prep_scale<HD>(ss, eps);
        const float4 w0 = __ldg((const float4 *)(w + l * 8)), w1 = __ldg((const float4 *)(w + l * 8 + 4));
        const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int e = 0; e < 8; e++) v[e] = prep_normed(wv[e], v[e], scale);
    }
    // the element HD / 2 above or below each of this lane's, from the lane that holds it
    float other[8];
#pragma unroll
    for (int e = 0; e < 8; e++) other[e] = __shfl_xor_sync(0xffffffffu, v[e], LPH / 2);
    uint32_t outw[4] = {in[0], in[1], in[2], in[3]};
    if (prepared) {
        if (rotate) {
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = upper ? prep_rotated_upper(v[e], other[e], cs[e], sn[e]) : prep_rotated_lower(v[e], other[e], cs[e], sn[e]);
        }
#pragma unroll
        for (int e = 0; e < 4; e++) {
            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
            outw[e] = *(uint32_t *)&h2;
        }
    }
    return make_uint4(outw[0], outw[1], outw[2], outw[3]);
}

// The same for a thread that holds a head, or a part of one, as float32 (the accumulators of a product whose rows are
// tokens: a row of the tile is one thread's) is put together from the pieces above by its kernel (gemm_tc.cu). The values
// pass through bfloat16 first, as they do where the product stores them for the kernel above, and the sums of squares
// are taken eight at a time and folded as the lanes above fold them:
__device__ __forceinline__ float prep_through_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
// the sum of squares of 8 consecutive elements (a lane's share above)
__device__ __forceinline__ float prep_sumsq8(const float *v) {
    float ss = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; e++) ss = __fmaf_rn(v[e], v[e], ss);
    return ss;
}
// the HD / 8 shares folded into the head's sum (lanes l and l ^ o above add the same two numbers: one sum serves both)
template <int HD> __device__ __forceinline__ float prep_fold(float *part) {
#pragma unroll
    for (int o = HD / 16; o > 0; o >>= 1)
#pragma unroll
        for (int l = 0; l < o; l++) part[l] = __fadd_rn(part[l], part[l + o]);
    return part[0];
}

// out[M, N] = x[M, K] . w[N, K]^T for a handful of rows (M <= 16: a decode step of a small batch),
// where the product is nothing but streaming the weights once.
//
// A CTA of eight warps owns 16 output features (rows of w) over the whole of K; warp i takes every
// eighth block of 32 columns. Each lane reads 16 consecutive bytes of a weight row straight from
// global memory into the A fragment of a warp-level tensor-core product (mma.sync m16n8k16, the 8
// columns being 8 tokens); x is read the same way into the B fragment, so both agree on which of
// the 32 columns sit in which slot of the product. No shared-memory staging, no barrier in the
// loop, no scratch memory: the eight partial tiles are added in warp order at the end, so the
// result does not depend on timing. float32 accumulation.
//
// A matrix with few rows and a long K (the projections back to the model's width) gives few CTAs, each
// with several turns of loads one after the other. Its CTAs come as clusters of up to 8 that split K
// between them, one turn each; the first CTA of a cluster adds the others' sums, in their order,
// reading them through distributed shared memory.
// Formula: src/model.c:299, 302, 307, 309.
#define ABK_DEFINE_ERROR
#include "common.cuh"
#include "tc_common.cuh"

#define ROWS_WARPS 8
#define ROWS_THREADS (32 * ROWS_WARPS)

__device__ __forceinline__ void mma_bf16(float *c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// A 16-byte read-only load (zeros if !ok). Written as volatile asm so that the loads of a turn stay
// ahead of its products, in program order: all of them are in flight before the first is needed.
__device__ __forceinline__ uint4 load16(const __nv_bfloat16 *p, bool ok) {
    uint4 v;
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "mov.b32 %0, 0;\n\tmov.b32 %1, 0;\n\tmov.b32 %2, 0;\n\tmov.b32 %3, 0;\n\t"
        "@q ld.global.nc.v4.b32 {%0, %1, %2, %3}, [%4];\n\t}"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
        : "l"(p), "r"((int)ok));
    return v;
}

// NT: tiles of 8 tokens (1, 2, 4 or 8: up to 64 rows; every CTA reads all of x, which stays in the L2).
// TILE: output features a CTA owns, 16 or 8. With 8 the upper half of the 16-row product is zero and
// twice as many CTAs share the matrix: for matrices with too few rows to give every SM a tile of 16.
// GATED: w holds gate and up rows in turns of `block` rows (gate of features [0, block), up of the same, gate of
// the next block, ...; block = N: all gates, then all ups, src/model.c:98); a CTA owns 8 outputs, takes their
// gate rows as the lower and their up rows as the upper half of the product, and stores silu(gate) * up
// (src/model.c:274-282) instead of the two sums: the feed-forward's first product and its activation in one.
__device__ __forceinline__ void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

template <int NT, int TILE, bool GATED, typename TO>
__global__ void __launch_bounds__(ROWS_THREADS) gemm_rows_kernel(const __nv_bfloat16 *__restrict__ x,
                                                                 const __nv_bfloat16 *__restrict__ w, TO *__restrict__ out,
                                                                 int M, int N, int K, long long ldx, long long ldw,
                                                                 long long ldo, int block) {
    __shared__ float part[ROWS_WARPS][16][8 * NT + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, r = lane >> 2, c = lane & 3;
    const int ranks = (int)tc::cluster_size(), rank = (int)tc::cluster_rank();  // the cluster splits K
    const int n0 = (blockIdx.x / ranks) * TILE;
    const bool row_lo = n0 + r < N, row_hi = GATED ? row_lo : TILE == 16 && n0 + r + 8 < N;
    // (a turn of gate rows is a multiple of 8 long, so a CTA's 8 outputs lie in one turn)
    const long long w_row = GATED ? (long long)(n0 / block) * 2 * block + n0 % block + r : n0 + r;
    const __nv_bfloat16 *w_lo = w + w_row * ldw + 8 * c, *w_hi = w_lo + (GATED ? (long long)block : 8) * ldw;
    const __nv_bfloat16 *x0 = x + (long long)r * ldx + 8 * c;  // token r of tile t is 8 t rows further
    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; t++) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f;
    const int blocks = (rank + 1) * (K / 32 / ranks), first = rank * (K / 32 / ranks) + warp;  // this CTA's part of K
    // several blocks of 32 columns a turn, so that eight 16-byte loads of weights are in flight per lane
    constexpr int TURN = NT <= 2 ? 4 : 2;
    uint4 a_lo[TURN], a_hi[TURN], b[TURN][NT];
    auto load_weights = [&](int kb) {
#pragma unroll
        for (int u = 0; u < TURN; u++) {
            int k = (kb + u * ROWS_WARPS) * 32;
            bool in = kb + u * ROWS_WARPS < blocks;
            a_lo[u] = load16(w_lo + k, in && row_lo);
            a_hi[u] = TILE == 16 || GATED ? load16(w_hi + k, in && row_hi) : make_uint4(0, 0, 0, 0);
        }
    };
    // The weights are nobody's output: the first turn's are fetched, and the later turns' called into the L2,
    // before pdl_wait(), while the kernel that writes x is still running.
    load_weights(first);
    for (int kb = first + TURN * ROWS_WARPS; kb < blocks; kb += ROWS_WARPS) {
        if (row_lo) prefetch_l2(w_lo + kb * 32);
        if ((TILE == 16 || GATED) && row_hi) prefetch_l2(w_hi + kb * 32);
    }
    pdl_wait();
    for (int kb = first; kb < blocks; kb += TURN * ROWS_WARPS) {
        if (kb != first) load_weights(kb);
#pragma unroll
        for (int u = 0; u < TURN; u++) {
            int k = (kb + u * ROWS_WARPS) * 32;
            bool in = kb + u * ROWS_WARPS < blocks;
#pragma unroll
            for (int t = 0; t < NT; t++) b[u][t] = load16(x0 + (long long)(8 * t) * ldx + k, in && 8 * t + r < M);
        }
#pragma unroll
        for (int u = 0; u < TURN; u++) {
#pragma unroll
            for (int t = 0; t < NT; t++) {
                mma_bf16(acc[t], a_lo[u].x, a_hi[u].x, a_lo[u].y, a_hi[u].y, b[u][t].x, b[u][t].y);
                mma_bf16(acc[t], a_lo[u].z, a_hi[u].z, a_lo[u].w, a_hi[u].w, b[u][t].z, b[u][t].w);
            }
        }
    }
    // accumulator: rows r and r + 8 (features), columns 2c and 2c + 1 (tokens) of each tile
#pragma unroll
    for (int t = 0; t < NT; t++) {
        part[warp][r][8 * t + 2 * c] = acc[t][0], part[warp][r][8 * t + 2 * c + 1] = acc[t][1];
        part[warp][r + 8][8 * t + 2 * c] = acc[t][2], part[warp][r + 8][8 * t + 2 * c + 1] = acc[t][3];
    }
    __syncthreads();
    if (ranks > 1) {
        // the warps' sums become the CTA's (kept in the first warp's tile), the first CTA adds the other CTAs'
        for (int i = threadIdx.x; i < 16 * 8 * NT; i += ROWS_THREADS) {
            int row = i / (8 * NT), token = i % (8 * NT);
            float sum = 0.0f;
#pragma unroll
            for (int wv = 0; wv < ROWS_WARPS; wv++) sum += part[wv][row][token];
            part[0][row][token] = sum;  // each element is read and written by this thread alone
        }
        tc::cluster_sync();
        if (rank == 0) {
            for (int i = threadIdx.x; i < TILE * 8 * NT; i += ROWS_THREADS) {
                int token = i / TILE, row = i % TILE;
                if (token < M && n0 + row < N) {
                    float sum = part[0][row][token];
                    const uint32_t at = (uint32_t)__cvta_generic_to_shared(&part[0][row][token]);
                    // the other CTAs' sums: all loads in flight before the first is added (in the CTAs' order)
                    float v[8];
#pragma unroll
                    for (int c = 1; c < 8; c++) {
                        v[c] = 0.0f;
                        if (c < ranks) asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v[c]) : "r"(tc::peer_smem(at, c)));
                    }
#pragma unroll
                    for (int c = 1; c < 8; c++) sum += v[c];
                    out[(long long)token * ldo + n0 + row] = from_float<TO>(sum);
                }
            }
        }
        tc::cluster_sync();  // nobody leaves while its sums may still be read
        return;
    }
    for (int i = threadIdx.x; i < TILE * 8 * NT; i += ROWS_THREADS) {
        int token = i / TILE, row = i % TILE;  // consecutive threads write consecutive features of a token
        if (token < M && n0 + row < N) {
            float sum = 0.0f, up = 0.0f;
#pragma unroll
            for (int wv = 0; wv < ROWS_WARPS; wv++) sum += part[wv][row][token];
            if (GATED) {
#pragma unroll
                for (int wv = 0; wv < ROWS_WARPS; wv++) up += part[wv][row + 8][token];
                // gate and up pass through bfloat16, as they do where they are stored between the product
                // and the activation (larger steps): a token's result is the same on either way
                sum = __bfloat162float(__float2bfloat16_rn(sum)), up = __bfloat162float(__float2bfloat16_rn(up));
                sum = silu_mul_fast(sum, up);
            }
            out[(long long)token * ldo + n0 + row] = from_float<TO>(sum);
        }
    }
}

// x [M, K], w [N, K] bfloat16 (row pitches ldx, ldw in elements); out [M, N] bfloat16 or float32.
// M <= 16, K a multiple of 32, rows 16-byte aligned.
extern "C" int abk_gemm_rows(const void *x, const void *w, void *out, int out_dtype, int M, int N, int K, long long ldx,
                             long long ldw, long long ldo, void *stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64) ABK_REFUSE("gemm_rows: %d rows are more than 64", M);
    if (K <= 0 || K % 32 || ldx % 8 || ldw % 8) ABK_REFUSE("gemm_rows: K = %d must be a multiple of 32 and the pitches of 8", K);
    if (((uintptr_t)x | (uintptr_t)w) & 15) ABK_REFUSE("gemm_rows: operands must be 16-byte aligned");
    const bool narrow = (N + 15) / 16 < 2 * abk_sm_count();  // too few tiles of 16 for two CTAs on every SM
    const int tiles = narrow ? (N + 7) / 8 : (N + 15) / 16;
    // a long K over few tiles: clusters that split K, one turn of loads to a CTA, while the grid stays small
    const int turn = 32 * ROWS_WARPS * (M <= 16 ? 4 : 2);
    int ranks = narrow ? K / turn : 1;
    if (ranks > 8) ranks = 8;
    while (ranks > 1 && ((K / 32) % ranks || (long long)tiles * ranks > 8 * abk_sm_count())) ranks--;
    if (ranks < 1) ranks = 1;
    dim3 grid(tiles * ranks);
    cudaStream_t s = (cudaStream_t)stream;
    const __nv_bfloat16 *xb = (const __nv_bfloat16 *)x, *wb = (const __nv_bfloat16 *)w;
#define ROWS_LAUNCH(NT, TILE, TO)                                                                                     \
    abk_launch_clusters(gemm_rows_kernel<NT, TILE, false, TO>, grid, dim3(ROWS_THREADS), 0, s, ranks, xb, wb, (TO *)out, M, \
                        N, K, ldx, ldw, ldo, 0)
#define ROWS_BY_M(TO)                                                                     \
    if (M <= 8) { if (narrow) ROWS_LAUNCH(1, 8, TO); else ROWS_LAUNCH(1, 16, TO); }       \
    else if (M <= 16) { if (narrow) ROWS_LAUNCH(2, 8, TO); else ROWS_LAUNCH(2, 16, TO); } \
    else if (M <= 32) { if (narrow) ROWS_LAUNCH(4, 8, TO); else ROWS_LAUNCH(4, 16, TO); } \
    else { if (narrow) ROWS_LAUNCH(8, 8, TO); else ROWS_LAUNCH(8, 16, TO); }
    if (out_dtype == ABK_BF16) { ROWS_BY_M(__nv_bfloat16) } else { ROWS_BY_M(float) }
#undef ROWS_BY_M
#undef ROWS_LAUNCH
    return ABK_LAUNCH_RESULT();
}

// act[M, N] = silu(x . w_gate^T) * (x . w_up^T) where w [2 N, K] holds gate and up rows in turns of `block`
// rows (a multiple of 8 that divides N; N itself: all gates, then all ups).
// x, w bfloat16; act bfloat16. M <= 64, K a multiple of 32.
extern "C" int abk_gemm_rows_swiglu(const void *x, const void *w, void *act, int M, int N, int K, long long ldx,
                                    long long ldw, long long ldo, int block, void *stream) {
    if (M <= 0 || N <= 0) return 0;
    if (block <= 0 || N % block || (block % 8 && block != N)) ABK_REFUSE("gemm_rows_swiglu: turns of %d rows do not fit %d features", block, N);
    if (M > 64) ABK_REFUSE("gemm_rows_swiglu: %d rows are more than 64", M);
    if (K <= 0 || K % 32 || ldx % 8 || ldw % 8) ABK_REFUSE("gemm_rows_swiglu: K = %d must be a multiple of 32 and the pitches of 8", K);
    if (((uintptr_t)x | (uintptr_t)w) & 15) ABK_REFUSE("gemm_rows_swiglu: operands must be 16-byte aligned");
    dim3 grid((N + 7) / 8);
    cudaStream_t s = (cudaStream_t)stream;
    const __nv_bfloat16 *xb = (const __nv_bfloat16 *)x, *wb = (const __nv_bfloat16 *)w;
#define GATED_LAUNCH(NT) \
    abk_launch(gemm_rows_kernel<NT, 8, true, __nv_bfloat16>, grid, dim3(ROWS_THREADS), 0, s, xb, wb, (__nv_bfloat16 *)act, M, N, K, ldx, ldw, ldo, block)
    if (M <= 8) GATED_LAUNCH(1);
    else if (M <= 16) GATED_LAUNCH(2);
    else if (M <= 32) GATED_LAUNCH(4);
    else GATED_LAUNCH(8);
#undef GATED_LAUNCH
    return ABK_LAUNCH_RESULT();
}

// Attention over the paged bfloat16 cache on the warp-level tensor-core path (mma.sync m16n8k16),
// for head sizes 64 and 128: a prefill kernel (many tokens of a sequence at once, causal) and a
// decode kernel (one token per sequence, split along the keys). Pages of the cache ([64 keys,
// head_dim], contiguous) and query tiles come in by TMA as boxes of [64 rows, 64 columns] with
// the 128-byte swizzle, so that ldmatrix reads them without bank conflicts.
//
// Scores, softmax and the running maximum/sum are float32; probabilities are rounded to
// bfloat16 for the second product, as the tensor cores need. Formula: src/model.c:197-211.
//
// What these kernels do not take (windows, the float32 cache, other head sizes, groups of more
// than 16 query heads) goes to the general kernel.
#define ABK_DEFINE_ERROR
#include "common.cuh"
#include "tc_common.cuh"
#include "tensor_map.cuh"

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

// ------------------------------------------------------------------ prefill
struct AttnPrefill {
    __nv_bfloat16 *out;  // [tokens, n_heads * head_dim]
    int n_heads, n_kv_heads;
    float scale_log2;  // score scale times log2(e)
    const int *tiles;  // [n_tiles][2]: sequence of the step, first of its 64 rows among the sequence's new tokens
    const int *seq_start, *seq_pos0, *seq_len_after, *seq_slot;
    PagedCache cache;
    int *status;
};

#define PRE_STAGES 3
#define PRE_THREADS 160  // four warps of 16 query rows each, and one that issues the copies

template <int HD>
__global__ void __launch_bounds__(PRE_THREADS) attn_prefill_kernel(const __grid_constant__ CUtensorMap q_map,
                                                                   const __grid_constant__ CUtensorMap k_map,
                                                                   const __grid_constant__ CUtensorMap v_map,
                                                                   AttnPrefill p) {
    constexpr int TILE_BYTES = PAGE * HD * 2;  // a page of keys, or of values, or the query tile
    extern __shared__ uint8_t pre_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)pre_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *q_s = smem, *k_s = q_s + TILE_BYTES, *v_s = k_s + PRE_STAGES * TILE_BYTES;
    uint64_t *full = (uint64_t *)(v_s + PRE_STAGES * TILE_BYTES), *empty = full + PRE_STAGES, *q_full = empty + PRE_STAGES;
    __shared__ int failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = p.tiles[2 * blockIdx.x], row0 = p.tiles[2 * blockIdx.x + 1], h = blockIdx.y;
    const int kvh = h / (p.n_heads / p.n_kv_heads);
    const int start = p.seq_start[seq], pos0 = p.seq_pos0[seq], n_new = p.seq_len_after[seq] - pos0;
    const int last_row = min(row0 + PAGE - 1, n_new - 1);
    const int n_tiles = (pos0 + last_row) / PAGE + 1;  // pages of keys the tile's last row sees

    if (threadIdx.x == 0) {
        failed = 0;
        for (int s = 0; s < PRE_STAGES; s++) tc::mbar_init(&full[s], 1), tc::mbar_init(&empty[s], 4);
        tc::mbar_init(q_full, 1);
        tc::mbar_init_fence();
    }
    __syncthreads();

    if (warp == 4) {
        if (lane == 0) {
            tc::mbar_expect_tx(q_full, TILE_BYTES);
#pragma unroll
            for (int half = 0; half < HD / 64; half++)
                tc::tma_load_2d(q_s + half * BOX_BYTES, &q_map, h * HD + half * 64, start + row0, q_full);
            const int slot = p.seq_slot[seq];
            int issued = 0;
            for (int jt = 0; jt < n_tiles; jt++, issued++) {
                int s = jt % PRE_STAGES;
                if (!tc::mbar_wait(&empty[s], ((jt / PRE_STAGES) & 1) ^ 1)) {
                    failed = 1;
                    break;
                }
                int y = (cache_page(p.cache, slot, jt * PAGE) * p.n_kv_heads + kvh) * PAGE;
                tc::mbar_expect_tx(&full[s], 2 * TILE_BYTES);
#pragma unroll
                for (int half = 0; half < HD / 64; half++) {
                    tc::tma_load_2d(k_s + s * TILE_BYTES + half * BOX_BYTES, &k_map, half * 64, y, &full[s]);
                    tc::tma_load_2d(v_s + s * TILE_BYTES + half * BOX_BYTES, &v_map, half * 64, y, &full[s]);
                }
            }
            if (failed)  // let the copies in flight land before the CTA's memory goes away
                for (int i = max(0, issued - PRE_STAGES); i < issued; i++) tc::mbar_wait(&full[i % PRE_STAGES], (i / PRE_STAGES) & 1);
        }
    } else {
        const int r_lo = row0 + 16 * warp + (lane >> 2), r_hi = r_lo + 8;  // this thread's two rows (of the sequence's new tokens)
        const int qpos_lo = pos0 + r_lo, qpos_hi = pos0 + r_hi;
        const int warp_first = pos0 + row0 + 16 * warp, warp_last = warp_first + 15;
        uint32_t qf[HD / 16][4];
        bool ok = tc::mbar_wait(q_full, 0);
        {
            const int j = lane >> 3, r8 = lane & 7;
            const uint32_t qb = tc::smem_addr(q_s);
#pragma unroll
            for (int ks = 0; ks < HD / 16; ks++)
                ldsm_x4(sw128(qb + (ks / 4) * BOX_BYTES, 16 * warp + 8 * (j & 1) + r8, (ks % 4) * 2 + (j >> 1)), qf[ks][0],
                        qf[ks][1], qf[ks][2], qf[ks][3]);
        }
        float o[HD / 8][4];
#pragma unroll
        for (int nt = 0; nt < HD / 8; nt++) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f;
        float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;

        for (int jt = 0; jt < n_tiles && ok; jt++) {
            const int s = jt % PRE_STAGES;
            if (!tc::mbar_wait(&full[s], (jt / PRE_STAGES) & 1)) {
                ok = false;
                break;
            }
            if (jt * PAGE <= warp_last) {  // else every key of this page lies after all of this warp's rows
                float sc[8][4];
                scores<HD, 8>(sc, qf, tc::smem_addr(k_s + s * TILE_BYTES), 0, lane);
                const bool edge = jt * PAGE + PAGE - 1 > warp_first;  // some key may lie after some row
                float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
                for (int nt = 0; nt < 8; nt++) {
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        float v = sc[nt][e] * p.scale_log2;
                        if (edge) {
                            int key = jt * PAGE + 8 * nt + 2 * (lane & 3) + (e & 1);
                            if (key > (e < 2 ? qpos_lo : qpos_hi)) v = -INFINITY;
                        }
                        sc[nt][e] = v;
                    }
                    mx_lo = fmaxf(mx_lo, fmaxf(sc[nt][0], sc[nt][1]));
                    mx_hi = fmaxf(mx_hi, fmaxf(sc[nt][2], sc[nt][3]));
                }
                const float n_lo = fmaxf(m_lo, quad_max(mx_lo)), n_hi = fmaxf(m_hi, quad_max(mx_hi));
                const float ref_lo = n_lo == -INFINITY ? 0.0f : n_lo, ref_hi = n_hi == -INFINITY ? 0.0f : n_hi;
                const float c_lo = exp2f(m_lo - ref_lo), c_hi = exp2f(m_hi - ref_hi);
                m_lo = n_lo, m_hi = n_hi;
                float sum_lo = 0.0f, sum_hi = 0.0f;
                uint32_t pf[4][4];
#pragma unroll
                for (int nt = 0; nt < 8; nt++) {
                    float p0 = exp2f(sc[nt][0] - ref_lo), p1 = exp2f(sc[nt][1] - ref_lo);
                    float p2 = exp2f(sc[nt][2] - ref_hi), p3 = exp2f(sc[nt][3] - ref_hi);
                    sum_lo += p0 + p1, sum_hi += p2 + p3;
                    pf[nt >> 1][(nt & 1) * 2] = pack_bf16(p0, p1);
                    pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
                }
                l_lo = l_lo * c_lo + sum_lo, l_hi = l_hi * c_hi + sum_hi;
#pragma unroll
                for (int nt = 0; nt < HD / 8; nt++) o[nt][0] *= c_lo, o[nt][1] *= c_lo, o[nt][2] *= c_hi, o[nt][3] *= c_hi;
                weighted_values<HD, 4>(o, pf, tc::smem_addr(v_s + s * TILE_BYTES), 0, lane);
            }
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&empty[s]);
        }
        if (!ok) failed = 1;
        l_lo = quad_sum(l_lo), l_hi = quad_sum(l_hi);
        const float i_lo = 1.0f / l_lo, i_hi = 1.0f / l_hi;
        __nv_bfloat16 *dst_lo = p.out + ((long long)(start + r_lo) * p.n_heads + h) * HD + 2 * (lane & 3);
        __nv_bfloat16 *dst_hi = dst_lo + (long long)8 * p.n_heads * HD;
#pragma unroll
        for (int nt = 0; nt < HD / 8; nt++) {
            if (ok && r_lo < n_new) *(uint32_t *)(dst_lo + 8 * nt) = pack_bf16(o[nt][0] * i_lo, o[nt][1] * i_lo);
            if (ok && r_hi < n_new) *(uint32_t *)(dst_hi + 8 * nt) = pack_bf16(o[nt][2] * i_hi, o[nt][3] * i_hi);
        }
    }
    __syncthreads();
    if (failed && threadIdx.x == 0) atomicOr(p.status + 3, 1);
}

// q: the step's qkv rows [n_rows, row_width] (q columns first); out [n_rows, n_heads * head_dim].
// tiles: int32 [n_tiles, 2] on the device. The sequences must have no window. status word 3 is set if a wait ran out.
extern "C" int abk_attention_prefill(const void *qkv, long long row_width, int n_rows, void *out, int n_heads,
                                     int n_kv_heads, int head_dim, float scale, const int *tiles, int n_tiles,
                                     const int *seq_start, const int *seq_pos0, const int *seq_len_after,
                                     const int *seq_slot, const void *k_pool, const void *v_pool, long long pool_rows,
                                     const int *page_table, int table_width, int tokens_per_page, int *status,
                                     void *stream) {
    if (n_tiles <= 0) return 0;
    if (head_dim != 64 && head_dim != 128) ABK_REFUSE("attention_prefill: head_dim %d is not 64 or 128", head_dim);
    if (tokens_per_page != PAGE) ABK_REFUSE("attention_prefill: pages of %d tokens, not %d", tokens_per_page, PAGE);
    if (n_kv_heads < 1 || n_heads % n_kv_heads || n_heads > 65535) ABK_REFUSE("attention_prefill: %d heads, %d kv heads", n_heads, n_kv_heads);
    CUtensorMap qm, km, vm;
    int rc = tmap::bf16_rows_of_128_bytes(qkv, n_rows, row_width, row_width, PAGE, &qm);
    if (!rc) rc = tmap::bf16_rows_of_128_bytes(k_pool, pool_rows, head_dim, head_dim, PAGE, &km);
    if (!rc) rc = tmap::bf16_rows_of_128_bytes(v_pool, pool_rows, head_dim, head_dim, PAGE, &vm);
    if (rc) return rc;
    AttnPrefill p;
    p.out = (__nv_bfloat16 *)out, p.n_heads = n_heads, p.n_kv_heads = n_kv_heads;
    p.scale_log2 = scale * 1.4426950408889634f, p.tiles = tiles, p.seq_start = seq_start, p.seq_pos0 = seq_pos0;
    p.seq_len_after = seq_len_after, p.seq_slot = seq_slot, p.status = status;
    p.cache.page_table = page_table, p.cache.table_width = table_width, p.cache.ring_pages = 0;
    p.cache.tokens_per_page = tokens_per_page;
    const int smem = (1 + 2 * PRE_STAGES) * PAGE * head_dim * 2 + 1024 + 128;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 120 * 1024);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 120 * 1024);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(n_tiles, n_heads);
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim == 64) attn_prefill_kernel<64><<<grid, PRE_THREADS, smem, s>>>(qm, km, vm, p);
    else attn_prefill_kernel<128><<<grid, PRE_THREADS, smem, s>>>(qm, km, vm, p);
    return ABK_LAUNCH_RESULT();
}

// ------------------------------------------------------------------ decode
// One new token per row. A CTA takes one (row, kv head, chunk of 128 keys = two pages); the query
// heads of the group are the rows of the products (up to 16, the rest of the 16-row tile is zero).
// Each of the four warps takes 32 keys; the CTA leaves (max, sum, weighted values) per query head
// in scratch memory and takes a ticket; the last CTA of a (row, kv head) folds the chunks in chunk
// order. Chunks are aligned to absolute positions, so a row's result does not depend on its batch.
#define DEC_CHUNK 128
#define DEC_THREADS 128

struct AttnDecodeMma {
    const __nv_bfloat16 *q;  // row r, head h at q + r * q_row + h * head_dim
    long long q_row;
    __nv_bfloat16 *out;  // [rows, n_heads * head_dim]
    int n_heads, n_kv_heads;
    float scale_log2;
    int window;
    const int *token_seq, *token_pos, *seq_slot;
    PagedCache cache;
    float *part_o;   // [rows, n_heads, max_chunks, head_dim]
    float *part_ml;  // [rows, n_heads, max_chunks, 2]: maximum (in units of log2) and sum
    int *tickets;    // [rows, n_kv_heads], zero before and after
    int max_chunks;
    int *status;
};

template <int HD>
__global__ void __launch_bounds__(DEC_THREADS) attn_decode_mma_kernel(const __grid_constant__ CUtensorMap k_map,
                                                                      const __grid_constant__ CUtensorMap v_map,
                                                                      AttnDecodeMma p) {
    constexpr int TILE_BYTES = PAGE * HD * 2;
    extern __shared__ uint8_t dec_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)dec_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *k_s = smem, *v_s = k_s + 2 * TILE_BYTES;
    const int group = p.n_heads / p.n_kv_heads;
    float *warp_o = (float *)(v_s + 2 * TILE_BYTES);   // [4 warps][group][HD]
    float *warp_ml = warp_o + 4 * group * HD;          // [4 warps][group][2]
    uint64_t *bars = (uint64_t *)(warp_ml + 4 * group * 2);
    __shared__ int failed, ticket;

    const int chunk = blockIdx.x, kvh = blockIdx.y, r = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = p.token_seq[r];
    if (seq < 0) {  // padding: zeros, written by the CTAs of chunk 0
        if (chunk == 0)
            for (int i = threadIdx.x; i < group * HD; i += DEC_THREADS)
                p.out[((long long)r * p.n_heads + kvh * group) * HD + i] = __float2bfloat16_rn(0.0f);
        return;
    }
    const int pos = p.token_pos[r];
    const int lo = p.window > 0 && pos - p.window + 1 > 0 ? pos - p.window + 1 : 0;
    const int first = chunk * DEC_CHUNK;
    if (first > pos || first + DEC_CHUNK <= lo) return;  // none of this chunk's keys is visible

    if (threadIdx.x == 0) {
        failed = 0;
        tc::mbar_init(&bars[0], 1), tc::mbar_init(&bars[1], 1);
        tc::mbar_init_fence();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const int slot = p.seq_slot[seq];
        for (int pg = 0; pg < 2; pg++) {
            int p_first = first + pg * PAGE;
            if (p_first > pos || p_first + PAGE <= lo) continue;
            int y = (cache_page(p.cache, slot, p_first) * p.n_kv_heads + kvh) * PAGE;
            tc::mbar_expect_tx(&bars[pg], 2 * TILE_BYTES);
#pragma unroll
            for (int half = 0; half < HD / 64; half++) {
                tc::tma_load_2d(k_s + pg * TILE_BYTES + half * BOX_BYTES, &k_map, half * 64, y, &bars[pg]);
                tc::tma_load_2d(v_s + pg * TILE_BYTES + half * BOX_BYTES, &v_map, half * 64, y, &bars[pg]);
            }
        }
    }
    // warp w takes keys first + 32 w .. + 31: rows 32 (w & 1) .. of page w / 2
    const int j0 = first + warp * 32, pg = warp >> 1, key0 = (warp & 1) * 32;
    const bool any = j0 <= pos && j0 + 32 > lo;
    const int g_lo = lane >> 2, g_hi = g_lo + 8;  // this thread's two rows: query heads of the group
    uint32_t qf[HD / 16][4];
    {
        const __nv_bfloat16 *q_lo = p.q + (long long)r * p.q_row + (long long)(kvh * group + g_lo) * HD + 2 * (lane & 3);
        const __nv_bfloat16 *q_hi = q_lo + 8 * HD;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++) {
            qf[ks][0] = g_lo < group ? *(const uint32_t *)(q_lo + 16 * ks) : 0u;
            qf[ks][1] = g_hi < group ? *(const uint32_t *)(q_hi + 16 * ks) : 0u;
            qf[ks][2] = g_lo < group ? *(const uint32_t *)(q_lo + 16 * ks + 8) : 0u;
            qf[ks][3] = g_hi < group ? *(const uint32_t *)(q_hi + 16 * ks + 8) : 0u;
        }
    }
    float o[HD / 8][4];
#pragma unroll
    for (int nt = 0; nt < HD / 8; nt++) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;
    if (any) {
        if (!tc::mbar_wait(&bars[pg], 0)) failed = 1;
        float sc[4][4];
        scores<HD, 4>(sc, qf, tc::smem_addr(k_s + pg * TILE_BYTES), key0, lane);
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                int key = j0 + 8 * nt + 2 * (lane & 3) + (e & 1);
                sc[nt][e] = key >= lo && key <= pos ? sc[nt][e] * p.scale_log2 : -INFINITY;
            }
            mx_lo = fmaxf(mx_lo, fmaxf(sc[nt][0], sc[nt][1]));
            mx_hi = fmaxf(mx_hi, fmaxf(sc[nt][2], sc[nt][3]));
        }
        m_lo = quad_max(mx_lo), m_hi = quad_max(mx_hi);  // finite: at least one of the warp's keys is visible
        uint32_t pf[2][4];
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
            float p0 = exp2f(sc[nt][0] - m_lo), p1 = exp2f(sc[nt][1] - m_lo);
            float p2 = exp2f(sc[nt][2] - m_hi), p3 = exp2f(sc[nt][3] - m_hi);
            l_lo += p0 + p1, l_hi += p2 + p3;
            pf[nt >> 1][(nt & 1) * 2] = pack_bf16(p0, p1);
            pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
        l_lo = quad_sum(l_lo), l_hi = quad_sum(l_hi);
        weighted_values<HD, 2>(o, pf, tc::smem_addr(v_s + pg * TILE_BYTES), key0, lane);
    }
#pragma unroll
    for (int nt = 0; nt < HD / 8; nt++) {
        int d = 8 * nt + 2 * (lane & 3);
        if (g_lo < group) *(float2 *)(warp_o + (warp * group + g_lo) * HD + d) = make_float2(o[nt][0], o[nt][1]);
        if (g_hi < group) *(float2 *)(warp_o + (warp * group + g_hi) * HD + d) = make_float2(o[nt][2], o[nt][3]);
    }
    if ((lane & 3) == 0) {
        if (g_lo < group) warp_ml[(warp * group + g_lo) * 2] = m_lo, warp_ml[(warp * group + g_lo) * 2 + 1] = l_lo;
        if (g_hi < group) warp_ml[(warp * group + g_hi) * 2] = m_hi, warp_ml[(warp * group + g_hi) * 2 + 1] = l_hi;
    }
    __syncthreads();
    if (failed && threadIdx.x == 0) atomicOr(p.status + 2, 1);
    // fold the four warps, in warp order, and leave the chunk's partial result
    for (int i = threadIdx.x; i < group * HD; i += DEC_THREADS) {
        int g = i / HD, d = i - g * HD, h = kvh * group + g;
        float m = -INFINITY;
        for (int w = 0; w < 4; w++) m = fmaxf(m, warp_ml[(w * group + g) * 2]);
        float acc = 0.0f, l = 0.0f;
        for (int w = 0; w < 4; w++) {
            float mw = warp_ml[(w * group + g) * 2];
            float f = mw == -INFINITY ? 0.0f : exp2f(mw - m);
            acc = fmaf(f, warp_o[(w * group + g) * HD + d], acc);
            l = fmaf(f, warp_ml[(w * group + g) * 2 + 1], l);
        }
        long long at = ((long long)r * p.n_heads + h) * p.max_chunks + chunk;
        p.part_o[at * HD + d] = acc;
        if (d == 0) p.part_ml[at * 2] = m, p.part_ml[at * 2 + 1] = l;
    }
    // the last CTA of this (row, kv head) folds the chunks, in chunk order
    const int c_lo = lo / DEC_CHUNK, c_hi = pos / DEC_CHUNK;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) ticket = atomicAdd(&p.tickets[r * p.n_kv_heads + kvh], 1);
    __syncthreads();
    if (ticket != c_hi - c_lo) return;
    __threadfence();
    for (int i = threadIdx.x; i < group * HD; i += DEC_THREADS) {
        int g = i / HD, d = i - g * HD, h = kvh * group + g;
        const long long base = ((long long)r * p.n_heads + h) * p.max_chunks;
        float m = -INFINITY;
        for (int c = c_lo; c <= c_hi; c++) m = fmaxf(m, __ldcg(p.part_ml + (base + c) * 2));
        float acc = 0.0f, l = 0.0f;
        for (int c0 = c_lo; c0 <= c_hi; c0 += 4) {
            float mc[4], ov[4], lv[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                bool in = c0 + u <= c_hi;
                mc[u] = in ? __ldcg(p.part_ml + (base + c0 + u) * 2) : -INFINITY;
                lv[u] = in ? __ldcg(p.part_ml + (base + c0 + u) * 2 + 1) : 0.0f;
                ov[u] = in ? __ldcg(p.part_o + (base + c0 + u) * HD + d) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                float w = mc[u] == -INFINITY ? 0.0f : exp2f(mc[u] - m);
                acc = fmaf(w, ov[u], acc), l = fmaf(w, lv[u], l);
            }
        }
        p.out[((long long)r * p.n_heads + h) * HD + d] = __float2bfloat16_rn(acc / l);
    }
    if (threadIdx.x == 0) p.tickets[r * p.n_kv_heads + kvh] = 0;
}

extern "C" long long abk_attention_decode_mma_scratch_floats(int rows, int n_heads, int head_dim, int max_chunks) {
    return (long long)rows * n_heads * max_chunks * (head_dim + 2);
}

// max_positions: no row's position reaches it (it sizes the grid; a captured graph passes its bound).
// scratch: float32 [abk_attention_decode_mma_scratch_floats(...)]; tickets: int32 [n_rows * n_kv_heads], zero
// before and after. status word 2 is set if a wait ran out.
extern "C" int abk_attention_decode_mma(const void *q, long long q_row, void *out, int n_rows, int n_heads,
                                        int n_kv_heads, int head_dim, float scale, int window, const int *token_seq,
                                        const int *token_pos, const int *seq_slot, const void *k_pool,
                                        const void *v_pool, long long pool_rows, const int *page_table, int table_width,
                                        int ring_pages, int tokens_per_page, int max_positions, float *scratch,
                                        int *tickets, int *status, void *stream) {
    if (n_rows <= 0) return 0;
    if (head_dim != 64 && head_dim != 128) ABK_REFUSE("attention_decode_mma: head_dim %d is not 64 or 128", head_dim);
    if (tokens_per_page != PAGE) ABK_REFUSE("attention_decode_mma: pages of %d tokens, not %d", tokens_per_page, PAGE);
    if (n_kv_heads < 1 || n_heads % n_kv_heads || n_heads / n_kv_heads > 16)
        ABK_REFUSE("attention_decode_mma: %d heads in %d groups (at most 16 to a group)", n_heads, n_kv_heads);
    if (n_kv_heads > 65535 || n_rows > 65535) ABK_REFUSE("attention_decode_mma: %d rows or %d kv heads exceed a grid", n_rows, n_kv_heads);
    if (((uintptr_t)q & 3) || (q_row & 1)) ABK_REFUSE("attention_decode_mma: q must be 4-byte aligned");
    CUtensorMap km, vm;
    int rc = tmap::bf16_rows_of_128_bytes(k_pool, pool_rows, head_dim, head_dim, PAGE, &km);
    if (!rc) rc = tmap::bf16_rows_of_128_bytes(v_pool, pool_rows, head_dim, head_dim, PAGE, &vm);
    if (rc) return rc;
    int max_chunks = (max_positions + DEC_CHUNK - 1) / DEC_CHUNK;
    if (max_chunks < 1) max_chunks = 1;
    int group = n_heads / n_kv_heads;
    AttnDecodeMma p;
    p.q = (const __nv_bfloat16 *)q, p.q_row = q_row, p.out = (__nv_bfloat16 *)out, p.n_heads = n_heads;
    p.n_kv_heads = n_kv_heads, p.scale_log2 = scale * 1.4426950408889634f, p.window = window;
    p.token_seq = token_seq, p.token_pos = token_pos, p.seq_slot = seq_slot;
    p.cache.page_table = page_table, p.cache.table_width = table_width, p.cache.ring_pages = ring_pages;
    p.cache.tokens_per_page = tokens_per_page;
    p.part_o = scratch, p.part_ml = scratch + (long long)n_rows * n_heads * max_chunks * head_dim;
    p.tickets = tickets, p.max_chunks = max_chunks, p.status = status;
    const int smem = 4 * PAGE * head_dim * 2 + 4 * group * (head_dim + 2) * 4 + 1024 + 64;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 120 * 1024);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_decode_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 120 * 1024);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(max_chunks, n_kv_heads, n_rows);
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim == 64) attn_decode_mma_kernel<64><<<grid, DEC_THREADS, smem, s>>>(km, vm, p);
    else attn_decode_mma_kernel<128><<<grid, DEC_THREADS, smem, s>>>(km, vm, p);
    return ABK_LAUNCH_RESULT();
}

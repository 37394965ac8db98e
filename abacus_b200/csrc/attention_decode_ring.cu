// Decode attention over the paged bfloat16 cache on the warp-level tensor-core path, head sizes 64
// and 128, groups of up to 16 query heads, with or without a window.
//
// One new token per row. The pages of a (row, kv head) are dealt out to S CTAs, page p to CTA
// p mod S; S is chosen so that the whole grid is about two CTAs per SM, whatever the batch. A CTA
// has one warp that issues TMA loads (a page of keys and a page of values, [64, head_dim] each, as
// swizzled boxes) into a ring of three stages, and four warps that each take 16 keys of every
// page: scores of the group's query heads (the rows of the product; the rest of the 16-row tile is
// zero), running maximum and sum in float32, probabilities times values. Loads therefore run two
// pages ahead of the arithmetic. At the end the four warps are folded in warp order, the CTA
// leaves (max, sum, weighted values) per query head in scratch memory and takes a ticket, and the
// last CTA of the (row, kv head) folds the S partial results in CTA order.
//
// A row's result depends on S, that is on the size of the batch, only in the order of float32
// sums. Formula: src/model.c:197-211.
#define ABK_DEFINE_ERROR
#include "common.cuh"
#include "tc_common.cuh"
#include "tensor_map.cuh"
#include "mma_tiles.cuh"

#define RING_STAGES 3
#define RING_THREADS 160  // four warps of 16 keys each, and one that issues the copies
#define RING_MAX_SPLITS 64

struct AttnDecodeRing {
    const __nv_bfloat16 *q;  // row r, head h at q + r * q_row + h * head_dim
    long long q_row;
    __nv_bfloat16 *out;  // [rows, n_heads * head_dim]
    int n_heads, n_kv_heads;
    float scale_log2;
    int window;
    const int *token_seq, *token_pos, *seq_slot;
    PagedCache cache;
    float *part_o;   // [rows, n_heads, splits, head_dim]
    float *part_ml;  // [rows, n_heads, splits, 2]: maximum (in units of log2) and sum
    int *tickets;    // [rows, n_kv_heads], zero before and after
    int splits;
    int *status;
};

template <int HD>
__global__ void __launch_bounds__(RING_THREADS) attn_decode_ring_kernel(const __grid_constant__ CUtensorMap k_map,
                                                                        const __grid_constant__ CUtensorMap v_map,
                                                                        AttnDecodeRing p) {
    constexpr int TILE_BYTES = PAGE * HD * 2;
    extern __shared__ uint8_t ring_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)ring_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *k_s = smem, *v_s = k_s + RING_STAGES * TILE_BYTES;
    const int group = p.n_heads / p.n_kv_heads;
    float *warp_o = (float *)(v_s + RING_STAGES * TILE_BYTES);  // [4 warps][group][HD]
    float *warp_ml = warp_o + 4 * group * HD;                   // [4 warps][group][2]
    uint64_t *full = (uint64_t *)(warp_ml + 4 * group * 2), *empty = full + RING_STAGES;
    __shared__ int failed, ticket;

    const int split = blockIdx.x, kvh = blockIdx.y, r = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 128) tc::tma_prefetch_map(&k_map), tc::tma_prefetch_map(&v_map);
    pdl_wait();
    const int seq = p.token_seq[r];
    if (seq < 0) {  // padding: zeros, written by the first CTA
        if (split == 0)
            for (int i = threadIdx.x; i < group * HD; i += RING_THREADS)
                p.out[((long long)r * p.n_heads + kvh * group) * HD + i] = __float2bfloat16_rn(0.0f);
        return;
    }
    const int pos = p.token_pos[r];
    const int lo = p.window > 0 && pos - p.window + 1 > 0 ? pos - p.window + 1 : 0;
    const int first_page = lo / PAGE, last_page = pos / PAGE, n_pages = last_page - first_page + 1;
    if (split >= n_pages) return;  // fewer pages than CTAs: the others have nothing to do
    const int active = min(p.splits, n_pages);

    if (threadIdx.x == 0) {
        failed = 0;
        for (int s = 0; s < RING_STAGES; s++) tc::mbar_init(&full[s], 1), tc::mbar_init(&empty[s], 4);
        tc::mbar_init_fence();
    }
    __syncthreads();

    if (warp == 4) {
        if (lane == 0) {
            const int slot = p.seq_slot[seq];
            int issued = 0;
            for (int pg = first_page + split; pg <= last_page; pg += p.splits, issued++) {
                int s = issued % RING_STAGES;
                if (!tc::mbar_wait(&empty[s], ((issued / RING_STAGES) & 1) ^ 1)) {
                    failed = 1;
                    break;
                }
                int y = (cache_page(p.cache, slot, pg * PAGE) * p.n_kv_heads + kvh) * PAGE;
                tc::mbar_expect_tx(&full[s], 2 * TILE_BYTES);
#pragma unroll
                for (int half = 0; half < HD / 64; half++) {
                    tc::tma_load_2d(k_s + s * TILE_BYTES + half * BOX_BYTES, &k_map, half * 64, y, &full[s]);
                    tc::tma_load_2d(v_s + s * TILE_BYTES + half * BOX_BYTES, &v_map, half * 64, y, &full[s]);
                }
            }
            if (failed)  // let the copies in flight land before the CTA's memory goes away
                for (int i = max(0, issued - RING_STAGES); i < issued; i++) tc::mbar_wait(&full[i % RING_STAGES], (i / RING_STAGES) & 1);
        }
    } else {
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
        bool ok = true;
        int done = 0;
        for (int pg = first_page + split; pg <= last_page && ok; pg += p.splits, done++) {
            const int s = done % RING_STAGES;
            if (!tc::mbar_wait(&full[s], (done / RING_STAGES) & 1)) {
                ok = false;
                break;
            }
            const int j0 = pg * PAGE + 16 * warp;  // this warp's 16 keys of the page
            if (j0 <= pos && j0 + 16 > lo) {
                float sc[2][4];
                scores<HD, 2>(sc, qf, tc::smem_addr(k_s + s * TILE_BYTES), 16 * warp, lane);
                float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
                for (int nt = 0; nt < 2; nt++) {
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        int key = j0 + 8 * nt + 2 * (lane & 3) + (e & 1);
                        sc[nt][e] = key >= lo && key <= pos ? sc[nt][e] * p.scale_log2 : -INFINITY;
                    }
                    mx_lo = fmaxf(mx_lo, fmaxf(sc[nt][0], sc[nt][1]));
                    mx_hi = fmaxf(mx_hi, fmaxf(sc[nt][2], sc[nt][3]));
                }
                // at least one of the warp's 16 keys is visible, so the new maxima are finite
                const float n_lo = fmaxf(m_lo, quad_max(mx_lo)), n_hi = fmaxf(m_hi, quad_max(mx_hi));
                const float c_lo = exp2f(m_lo - n_lo), c_hi = exp2f(m_hi - n_hi);
                m_lo = n_lo, m_hi = n_hi;
                uint32_t pf[1][4];
                float sum_lo = 0.0f, sum_hi = 0.0f;
#pragma unroll
                for (int nt = 0; nt < 2; nt++) {
                    float p0 = exp2f(sc[nt][0] - n_lo), p1 = exp2f(sc[nt][1] - n_lo);
                    float p2 = exp2f(sc[nt][2] - n_hi), p3 = exp2f(sc[nt][3] - n_hi);
                    sum_lo += p0 + p1, sum_hi += p2 + p3;
                    pf[0][nt * 2] = pack_bf16(p0, p1);
                    pf[0][nt * 2 + 1] = pack_bf16(p2, p3);
                }
                l_lo = l_lo * c_lo + sum_lo, l_hi = l_hi * c_hi + sum_hi;
#pragma unroll
                for (int nt = 0; nt < HD / 8; nt++) o[nt][0] *= c_lo, o[nt][1] *= c_lo, o[nt][2] *= c_hi, o[nt][3] *= c_hi;
                weighted_values<HD, 1>(o, pf, tc::smem_addr(v_s + s * TILE_BYTES), 16 * warp, lane);
            }
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&empty[s]);
        }
        if (!ok) failed = 1;
        l_lo = quad_sum(l_lo), l_hi = quad_sum(l_hi);
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
    }
    __syncthreads();
    if (failed && threadIdx.x == 0) atomicOr(p.status + 2, 1);
    // fold the four warps, in warp order, and leave this CTA's partial result
    for (int i = threadIdx.x; i < group * HD; i += RING_THREADS) {
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
        long long at = ((long long)r * p.n_heads + h) * p.splits + split;
        p.part_o[at * HD + d] = acc;
        if (d == 0) p.part_ml[at * 2] = m, p.part_ml[at * 2 + 1] = l;
    }
    // the last CTA of this (row, kv head) folds the partial results, in CTA order
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) ticket = atomicAdd(&p.tickets[r * p.n_kv_heads + kvh], 1);
    __syncthreads();
    if (ticket != active - 1) return;
    __threadfence();
    // weights of the partial results: all (max, sum) pairs come in with one round of loads
    float *fold_w = warp_o;                     // [group][active]: e^(m_c - m), reusing the warps' buffer
    float *fold_l = warp_o + group * RING_MAX_SPLITS;  // [group]: the total sum
    for (int i = threadIdx.x; i < group * active; i += RING_THREADS) {
        int g = i / active, c = i - g * active;
        long long at = ((long long)r * p.n_heads + kvh * group + g) * p.splits + c;
        fold_w[g * RING_MAX_SPLITS + c] = __ldcg(p.part_ml + at * 2);
    }
    __syncthreads();
    if (threadIdx.x < group) {
        const int g = threadIdx.x;
        const long long base = ((long long)r * p.n_heads + kvh * group + g) * p.splits;
        float m = -INFINITY, l = 0.0f;
        for (int c = 0; c < active; c++) m = fmaxf(m, fold_w[g * RING_MAX_SPLITS + c]);
        for (int c = 0; c < active; c++) {  // in CTA order
            float mc = fold_w[g * RING_MAX_SPLITS + c];
            float w = mc == -INFINITY ? 0.0f : exp2f(mc - m);
            fold_w[g * RING_MAX_SPLITS + c] = w;
            l = fmaf(w, __ldcg(p.part_ml + (base + c) * 2 + 1), l);
        }
        fold_l[g] = l;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < group * HD; i += RING_THREADS) {
        int g = i / HD, d = i - g * HD, h = kvh * group + g;
        const float *po = p.part_o + ((long long)r * p.n_heads + h) * p.splits * HD + d;
        float acc = 0.0f;
        for (int c0 = 0; c0 < active; c0 += 8) {  // eight loads in flight, added in CTA order
            float ov[8];
#pragma unroll
            for (int u = 0; u < 8; u++) ov[u] = c0 + u < active ? __ldcg(po + (long long)(c0 + u) * HD) : 0.0f;
#pragma unroll
            for (int u = 0; u < 8; u++)
                if (c0 + u < active) acc = fmaf(fold_w[g * RING_MAX_SPLITS + c0 + u], ov[u], acc);
        }
        p.out[((long long)r * p.n_heads + h) * HD + d] = __float2bfloat16_rn(acc / fold_l[g]);
    }
    if (threadIdx.x == 0) p.tickets[r * p.n_kv_heads + kvh] = 0;
}

// CTAs per (row, kv head): about two CTAs per SM over the whole grid, at most one per page.
extern "C" int abk_attention_decode_ring_splits(int rows, int n_kv_heads, int max_positions) {
    long long pairs = (long long)rows * n_kv_heads;
    int pages = (max_positions + PAGE - 1) / PAGE;
    long long s = (2 * 148 + pairs - 1) / pairs;
    if (s > RING_MAX_SPLITS) s = RING_MAX_SPLITS;
    if (s > pages) s = pages;
    return s < 1 ? 1 : (int)s;
}

extern "C" long long abk_attention_decode_ring_scratch_floats(int rows, int n_heads, int n_kv_heads, int head_dim,
                                                              int max_positions) {
    return (long long)rows * n_heads * abk_attention_decode_ring_splits(rows, n_kv_heads, max_positions) * (head_dim + 2);
}

// max_positions: no row's position reaches it (with the number of rows it fixes the grid; a captured graph
// passes its bound). scratch: float32 [abk_attention_decode_ring_scratch_floats(...)]; tickets: int32
// [n_rows * n_kv_heads], zero before and after. status word 2 is set if a wait ran out.
extern "C" int abk_attention_decode_ring(const void *q, long long q_row, void *out, int n_rows, int n_heads,
                                         int n_kv_heads, int head_dim, float scale, int window, const int *token_seq,
                                         const int *token_pos, const int *seq_slot, const void *k_pool,
                                         const void *v_pool, long long pool_rows, const int *page_table, int table_width,
                                         int ring_pages, int tokens_per_page, int max_positions, float *scratch,
                                         int *tickets, int *status, void *stream) {
    if (n_rows <= 0) return 0;
    if (head_dim != 64 && head_dim != 128) ABK_REFUSE("attention_decode_ring: head_dim %d is not 64 or 128", head_dim);
    if (tokens_per_page != PAGE) ABK_REFUSE("attention_decode_ring: pages of %d tokens, not %d", tokens_per_page, PAGE);
    if (n_kv_heads < 1 || n_heads % n_kv_heads || n_heads / n_kv_heads > 16)
        ABK_REFUSE("attention_decode_ring: %d heads in %d groups (at most 16 to a group)", n_heads, n_kv_heads);
    if (n_kv_heads > 65535 || n_rows > 65535) ABK_REFUSE("attention_decode_ring: %d rows or %d kv heads exceed a grid", n_rows, n_kv_heads);
    if (((uintptr_t)q & 3) || (q_row & 1)) ABK_REFUSE("attention_decode_ring: q must be 4-byte aligned");
    CUtensorMap km, vm;
    int rc = tmap::bf16_rows_of_128_bytes(k_pool, pool_rows, head_dim, head_dim, PAGE, &km);
    if (!rc) rc = tmap::bf16_rows_of_128_bytes(v_pool, pool_rows, head_dim, head_dim, PAGE, &vm);
    if (rc) return rc;
    int group = n_heads / n_kv_heads;
    AttnDecodeRing p;
    p.q = (const __nv_bfloat16 *)q, p.q_row = q_row, p.out = (__nv_bfloat16 *)out, p.n_heads = n_heads;
    p.n_kv_heads = n_kv_heads, p.scale_log2 = scale * 1.4426950408889634f, p.window = window;
    p.token_seq = token_seq, p.token_pos = token_pos, p.seq_slot = seq_slot;
    p.cache.page_table = page_table, p.cache.table_width = table_width, p.cache.ring_pages = ring_pages;
    p.cache.tokens_per_page = tokens_per_page;
    p.splits = abk_attention_decode_ring_splits(n_rows, n_kv_heads, max_positions);
    p.part_o = scratch, p.part_ml = scratch + (long long)n_rows * n_heads * p.splits * head_dim;
    p.tickets = tickets, p.status = status;
    const int smem = 2 * RING_STAGES * PAGE * head_dim * 2 + 4 * group * (head_dim + 2) * 4 + 1024 + 64;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_ring_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_decode_ring_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(p.splits, n_kv_heads, n_rows);
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim == 64) abk_launch(attn_decode_ring_kernel<64>, grid, dim3(RING_THREADS), smem, s, km, vm, p);
    else abk_launch(attn_decode_ring_kernel<128>, grid, dim3(RING_THREADS), smem, s, km, vm, p);
    return ABK_LAUNCH_RESULT();
}

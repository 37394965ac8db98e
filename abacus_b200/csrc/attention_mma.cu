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
#include "mma_tiles.cuh"

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

#define PRE_STAGES 2  // 80 KB of shared memory with the query tile: two CTAs to an SM
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
    if (seq < 0) return;  // padding of the work list (a captured step has a fixed number of tiles)
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
                // the reference of a row's exponentials is a whole power of two (the maximum rounded up, in units
                // of log2): whatever tile a key falls into, its probability is the same bits times a power of two,
                // so the bfloat16 it is rounded to does not depend on how the keys were tiled, split or cut
                const float n_lo = fmaxf(m_lo, ceilf(quad_max(mx_lo))), n_hi = fmaxf(m_hi, ceilf(quad_max(mx_hi)));
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
    {   // once per device
        cudaError_t e = abk_allow_shared_memory((const void *)attn_prefill_kernel<64>, 120 * 1024);
        if (e == cudaSuccess) e = abk_allow_shared_memory((const void *)attn_prefill_kernel<128>, 120 * 1024);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid(n_tiles, n_heads);
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim == 64) attn_prefill_kernel<64><<<grid, PRE_THREADS, smem, s>>>(qm, km, vm, p);
    else attn_prefill_kernel<128><<<grid, PRE_THREADS, smem, s>>>(qm, km, vm, p);
    return ABK_LAUNCH_RESULT();
}


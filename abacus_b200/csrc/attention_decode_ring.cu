// Decode attention over the paged bfloat16 cache on the warp-level tensor-core path, head sizes 64
// and 128, groups of up to 16 query heads, with or without a window.
//
// One new token per row. The pages of a (row, kv head) are dealt out to the S CTAs of a thread-block
// cluster, page p to CTA p mod S; S (at most 8) is chosen so that the whole grid is about two CTAs
// per SM, whatever the batch. A CTA has one warp that issues TMA loads (a page of keys and a page of
// values, [64, head_dim] each, as swizzled boxes) into a ring of stages, and four warps that each
// take 16 keys of every page: scores of the group's query heads (the rows of the product; the rest
// of the 16-row tile is zero), running maximum and sum in float32, probabilities times values. The
// loads run ahead of the arithmetic by the depth of the ring, which is twice as deep when the grid
// is so small that an SM holds one CTA. At the end the four warps are folded in warp order into the
// CTA's partial result (max, sum, weighted values per query head) in its own shared memory; after a
// cluster barrier every CTA folds a share of the output columns over all S partial results, in CTA
// order, reading the others' through distributed shared memory. No scratch memory, no atomics.
//
// A row's result depends on S, that is on the size of the batch, only in the order of float32
// sums. Formula: src/model.c:197-211.
//
// The kernel may also take the step between the q/k/v product and attention into itself (src/model.c:247-259: the
// per-head norm of q and k, their rotary encoding, the new token's key and value into the cache): a launch less in
// every layer of a decode step. Every CTA of a cluster then prepares the group's query heads for itself, into shared
// memory; the CTA that holds the new token's page prepares its key and value as well, writes them to the cache, and
// the warp whose 16 keys include the new token puts them into the page's copy in shared memory once that has landed
// (the copy may have read the page before or after the write: either way the row is then the new one). The
// arithmetic is that of the preparation's own kernel (qkv_prep.cuh), so the result is the same to the bit.
#define ABK_DEFINE_ERROR
#include "common.cuh"
#include "tc_common.cuh"
#include "tensor_map.cuh"
#include "mma_tiles.cuh"
#include "qkv_prep.cuh"

#define RING_MAX_STAGES 12
#define RING_STAGE_BYTES (96 * 1024)  // keys and values in flight per CTA when an SM holds two
#define RING_THREADS 160  // four warps of 16 keys each, and one that issues the copies
#define RING_MAX_SPLITS 8  // the portable size of a cluster

struct AttnDecodeRing {
    const __nv_bfloat16 *q;  // row r, head h at q + r * q_row + h * head_dim
    long long q_row;
    __nv_bfloat16 *out;  // [rows, n_heads * head_dim]
    int n_heads, n_kv_heads;
    float scale_log2;
    int window;
    const int *token_seq, *token_pos, *seq_slot;
    PagedCache cache;
    int stages;  // depth of the ring
    int *status;
    // prepare != 0: q, and the new token's k and v beside it in the row (k head h at q + (n_heads + h) * head_dim, v head h
    // n_kv_heads heads further), are as the product left them, and are prepared here
    int prepare;
    const float *q_norm, *k_norm;  // null: no norm
    float eps;
    const float *cos, *sin;  // [positions, head_dim / 2]; null: no rotation
    __nv_bfloat16 *k_pool, *v_pool;  // where the new key and value are kept; null: nowhere (the cache is another layer's)
};

template <int HD>
__global__ void __launch_bounds__(RING_THREADS) attn_decode_ring_kernel(const __grid_constant__ CUtensorMap k_map,
                                                                        const __grid_constant__ CUtensorMap v_map,
                                                                        AttnDecodeRing p) {
    constexpr int TILE_BYTES = PAGE * HD * 2;
    extern __shared__ uint8_t ring_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)ring_raw + 1023) & ~(uintptr_t)1023);
    const int stages = p.stages;
    uint8_t *k_s = smem, *v_s = k_s + stages * TILE_BYTES;
    const int group = p.n_heads / p.n_kv_heads;
    float *cta_o = (float *)(v_s + stages * TILE_BYTES);  // [group][HD]: what the other CTAs read
    float *cta_ml = cta_o + group * HD;                   // [group][2]: maximum (in units of log2) and sum
    float *warp_o = cta_ml + group * 2;                   // [4 warps][group][HD]
    float *warp_ml = warp_o + 4 * group * HD;             // [4 warps][group][2]
    __nv_bfloat16 *q_s = (__nv_bfloat16 *)(((uintptr_t)(warp_ml + 4 * group * 2) + 15) & ~(uintptr_t)15);  // [group][HD]: the prepared query heads
    __shared__ uint64_t full[RING_MAX_STAGES], empty[RING_MAX_STAGES];
    __shared__ int failed;

    const int split = (int)tc::cluster_rank(), splits = (int)tc::cluster_size();
    const int kvh = blockIdx.y, r = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 128) tc::tma_prefetch_map(&k_map), tc::tma_prefetch_map(&v_map);
    // Before pdl_wait() only what kernels further back than the one just before this wrote is read: the
    // step's index arrays and the page table, and (by the copy warp) every page but the one of the new
    // token, which the kernel just before this one may still be writing.
    const int seq = p.token_seq[r];
    if (seq < 0) {  // padding: zeros, written by the first CTA; the whole cluster leaves here
        pdl_wait();
        if (split == 0)
            for (int i = threadIdx.x; i < group * HD; i += RING_THREADS)
                p.out[((long long)r * p.n_heads + kvh * group) * HD + i] = __float2bfloat16_rn(0.0f);
        return;
    }
    const int pos = p.token_pos[r];
    const int lo = p.window > 0 && pos - p.window + 1 > 0 ? pos - p.window + 1 : 0;
    const int first_page = lo / PAGE, last_page = pos / PAGE, n_pages = last_page - first_page + 1;
    const int active = min(splits, n_pages);  // CTAs with fewer pages than ranks have nothing to add
    const int mine = split < n_pages ? (n_pages - 1 - split) / splits + 1 : 0;  // this CTA's pages

    if (threadIdx.x == 0) {
        failed = 0;
        for (int s = 0; s < stages; s++) tc::mbar_init(&full[s], 1), tc::mbar_init(&empty[s], 4);
        tc::mbar_init_fence();
    }
    __syncthreads();
    // the lane's part in preparing heads: 8 elements of one of the 32 * 8 / HD heads a warp holds at a time
    constexpr int LPH = HD / 8, HPW = 32 / LPH;
    const int sub = lane / LPH, l = lane % LPH;
    const bool upper = l >= LPH / 2;
    float cs[8], sn[8];
    if (p.prepare && warp != 4 && mine > 0 && p.cos) {  // the angles of the new token's position: nobody's output
        const int at = (upper ? l - LPH / 2 : l) * 8;
        const float4 *c4 = (const float4 *)(p.cos + (long long)pos * (HD / 2) + at), *s4 = (const float4 *)(p.sin + (long long)pos * (HD / 2) + at);
        const float4 c0 = c4[0], c1 = c4[1], s0 = s4[0], s1 = s4[1];
        cs[0] = c0.x, cs[1] = c0.y, cs[2] = c0.z, cs[3] = c0.w, cs[4] = c1.x, cs[5] = c1.y, cs[6] = c1.z, cs[7] = c1.w;
        sn[0] = s0.x, sn[1] = s0.y, sn[2] = s0.z, sn[3] = s0.w, sn[4] = s1.x, sn[5] = s1.y, sn[6] = s1.z, sn[7] = s1.w;
    }
    if (warp != 4) pdl_wait();

    if (warp == 4) {
        // every lane looks up the pool row of one of the CTA's pages, so that the table's latency is
        // paid once for 32 pages and not before every copy
        const int slot = p.seq_slot[seq];
        int issued = 0;
        bool go = true;
        for (int base = 0; base < mine && go; base += 32) {
            int y_lane = 0;
            if (base + lane < mine) {
                int pg = first_page + split + (base + lane) * splits;
                y_lane = (cache_page(p.cache, slot, pg * PAGE) * p.n_kv_heads + kvh) * PAGE;
            }
            const int n = min(32, mine - base);
            for (int i = 0; i < n && go; i++, issued++) {
                const int y = __shfl_sync(0xffffffffu, y_lane, i);
                int bad = 0;
                // the new token's page: the kernel before this one may still be writing it, unless the new token
                // is written here (then the page holds earlier steps' tokens, and the new row is put in after the copy)
                if (!p.prepare && first_page + split + issued * splits == last_page) pdl_wait();
                if (lane == 0) {
                    const int s = issued % stages;
                    if (!tc::mbar_wait(&empty[s], ((issued / stages) & 1) ^ 1)) {
                        bad = 1;
                    } else {
                        tc::mbar_expect_tx(&full[s], 2 * TILE_BYTES);
#pragma unroll
                        for (int half = 0; half < HD / 64; half++) {
                            tc::tma_load_2d(k_s + s * TILE_BYTES + half * BOX_BYTES, &k_map, half * 64, y, &full[s]);
                            tc::tma_load_2d(v_s + s * TILE_BYTES + half * BOX_BYTES, &v_map, half * 64, y, &full[s]);
                        }
                    }
                }
                if (__shfl_sync(0xffffffffu, bad, 0)) go = false;
            }
        }
        pdl_wait();  // every thread has waited before the result is written (a second wait returns at once)
        if (!go && lane == 0) {  // let the copies in flight land before the CTA's memory goes away
            failed = 1;
            issued--;  // the copy that was not issued
            for (int i = max(0, issued - stages); i < issued; i++) tc::mbar_wait(&full[i % stages], (i / stages) & 1);
        }
    } else if (mine > 0) {
        const int g_lo = lane >> 2, g_hi = g_lo + 8;  // this thread's two rows: query heads of the group
        // the new token's key and value, held by the warp whose 16 keys include it in the CTA that has its page
        const bool has_new = p.prepare && (last_page - first_page) % splits == split && (pos % PAGE) / 16 == warp;
        uint4 new_kv = make_uint4(0, 0, 0, 0);  // lanes of head 0: the key's elements 8 l .., of head 1: the value's
        if (p.prepare) {
            const __nv_bfloat16 *row = p.q + (long long)r * p.q_row + l * 8;
            for (int g0 = warp * HPW; g0 < group; g0 += 4 * HPW) {  // (the same for a whole warp)
                const int g = g0 + sub;
                const uint4 raw = g < group ? *(const uint4 *)(row + (long long)(kvh * group + g) * HD) : make_uint4(0, 0, 0, 0);
                const uint4 done = prep_head_values<HD>(raw, true, p.q_norm, p.eps, p.cos != nullptr, l, upper, cs, sn);
                if (g < group) *(uint4 *)(q_s + g * HD + l * 8) = done;
            }
            if (has_new) {
                const long long head = sub == 0 ? p.n_heads + kvh : p.n_heads + p.n_kv_heads + kvh;
                const uint4 raw = sub < 2 ? *(const uint4 *)(row + head * HD) : make_uint4(0, 0, 0, 0);
                new_kv = prep_head_values<HD>(raw, sub == 0, p.k_norm, p.eps, p.cos != nullptr, l, upper, cs, sn);
                if (sub < 2 && p.k_pool) {
                    const int page = cache_page(p.cache, p.seq_slot[seq], pos);
                    __nv_bfloat16 *pool = sub == 0 ? p.k_pool : p.v_pool;
                    *(uint4 *)(pool + cache_offset(p.cache, page, kvh, p.n_kv_heads, pos, HD) + l * 8) = new_kv;
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");  // the four warps that multiply: all heads are in q_s
        }
        uint32_t qf[HD / 16][4];
        {
            const __nv_bfloat16 *q_lo = p.prepare ? q_s + g_lo * HD + 2 * (lane & 3)
                                                  : p.q + (long long)r * p.q_row + (long long)(kvh * group + g_lo) * HD + 2 * (lane & 3);
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
        int done = 0, s = 0, phase = 0;
        for (int pg = first_page + split; pg <= last_page && ok; pg += splits, done++) {
            if (!tc::mbar_wait(&full[s], phase)) {
                ok = false;
                break;
            }
            const int j0 = pg * PAGE + 16 * warp;  // this warp's 16 keys of the page
            if (has_new && pg == last_page) {  // the new token's row of the page's copy (only this warp reads it)
                if (sub < 2) {
                    uint8_t *tile = (sub == 0 ? k_s : v_s) + s * TILE_BYTES + (l / 8) * BOX_BYTES;
                    *(uint4 *)(tile + sw128(0, pos % PAGE, l % 8)) = new_kv;
                }
                __syncwarp();
            }
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
                // The reference is a whole power of two (the maximum rounded up, in units of log2), so a key's
                // probability rounds to the same bfloat16 whichever CTA, warp or step meets it.
                const float n_lo = fmaxf(m_lo, ceilf(quad_max(mx_lo))), n_hi = fmaxf(m_hi, ceilf(quad_max(mx_hi)));
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
            if (++s == stages) s = 0, phase ^= 1;
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
    // fold the four warps, in warp order, into this CTA's partial result
    if (mine > 0) {
        for (int i = threadIdx.x; i < group * HD; i += RING_THREADS) {
            int g = i / HD, d = i - g * HD;
            float m = -INFINITY;
            for (int w = 0; w < 4; w++) m = fmaxf(m, warp_ml[(w * group + g) * 2]);
            float acc = 0.0f, l = 0.0f;
            for (int w = 0; w < 4; w++) {
                float mw = warp_ml[(w * group + g) * 2];
                float f = mw == -INFINITY ? 0.0f : exp2f(mw - m);
                acc = fmaf(f, warp_o[(w * group + g) * HD + d], acc);
                l = fmaf(f, warp_ml[(w * group + g) * 2 + 1], l);
            }
            cta_o[i] = acc;
            if (d == 0) cta_ml[g * 2] = m, cta_ml[g * 2 + 1] = l;
        }
    }
    tc::cluster_sync();
    // every CTA folds its share of the output (four columns a thread) over the partial results, in CTA order
    const uint32_t o_addr = tc::smem_addr(cta_o), ml_addr = tc::smem_addr(cta_ml);
    for (int i = split + splits * threadIdx.x; i < group * (HD / 4); i += splits * RING_THREADS) {
        const int g = i / (HD / 4), d = 4 * (i - g * (HD / 4));
        float2 ml[RING_MAX_SPLITS];
        float4 ov[RING_MAX_SPLITS];
#pragma unroll
        for (int c = 0; c < RING_MAX_SPLITS; c++) {
            if (c < active) {
                ml[c] = tc::ld_cluster_f2(tc::peer_smem(ml_addr + g * 8, c));
                ov[c] = tc::ld_cluster_f4(tc::peer_smem(o_addr + (g * HD + d) * 4, c));
            }
        }
        float m = -INFINITY;
#pragma unroll
        for (int c = 0; c < RING_MAX_SPLITS; c++)
            if (c < active) m = fmaxf(m, ml[c].x);
        float l = 0.0f, a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll
        for (int c = 0; c < RING_MAX_SPLITS; c++) {
            if (c < active) {
                float w = ml[c].x == -INFINITY ? 0.0f : exp2f(ml[c].x - m);
                l = fmaf(w, ml[c].y, l);
                a0 = fmaf(w, ov[c].x, a0), a1 = fmaf(w, ov[c].y, a1), a2 = fmaf(w, ov[c].z, a2), a3 = fmaf(w, ov[c].w, a3);
            }
        }
        const float inv = 1.0f / l;
        uint2 packed = make_uint2(pack_bf16(a0 * inv, a1 * inv), pack_bf16(a2 * inv, a3 * inv));
        *(uint2 *)(p.out + ((long long)r * p.n_heads + kvh * group + g) * HD + d) = packed;
    }
    tc::cluster_sync();  // nobody leaves while its partial result may still be read
}

// How many clusters of `splits` CTAs with `smem` bytes each the device holds at once (looked up once per shape).
template <int HD>
static int resident_clusters(int splits, int smem) {
    struct Known { int splits, smem, clusters; };
    static Known known[64];
    static int n_known = 0;
    for (int i = 0; i < n_known; i++)
        if (known[i].splits == splits && known[i].smem == smem) return known[i].clusters;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits, 1, 1), cfg.blockDim = dim3(RING_THREADS), cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = splits, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr, cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, attn_decode_ring_kernel<HD>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        clusters = 0;
    }
    if (n_known < 64) known[n_known++] = {splits, smem, clusters};
    return clusters;
}

struct RingPrepare {  // what the kernel needs to prepare q, k and v itself
    const float *q_norm, *k_norm, *cos, *sin;
    float eps;
    int keep;  // the new key and value go to the cache (not where the cache is another layer's)
};
static int ring_launch(const void *q, long long q_row, void *out, int n_rows, int n_heads, int n_kv_heads, int head_dim,
                       float scale, int window, const int *token_seq, const int *token_pos, const int *seq_slot,
                       const void *k_pool, const void *v_pool, long long pool_rows, const int *page_table, int table_width,
                       int ring_pages, int tokens_per_page, int max_positions, int *status, const RingPrepare *prepare,
                       void *stream) {
    if (n_rows <= 0) return 0;
    if (head_dim != 64 && head_dim != 128) ABK_REFUSE("attention_decode_ring: head_dim %d is not 64 or 128", head_dim);
    if (tokens_per_page != PAGE) ABK_REFUSE("attention_decode_ring: pages of %d tokens, not %d", tokens_per_page, PAGE);
    if (n_kv_heads < 1 || n_heads % n_kv_heads || n_heads / n_kv_heads > 16)
        ABK_REFUSE("attention_decode_ring: %d heads in %d groups (at most 16 to a group)", n_heads, n_kv_heads);
    if (n_kv_heads > 65535 || n_rows > 65535) ABK_REFUSE("attention_decode_ring: %d rows or %d kv heads exceed a grid", n_rows, n_kv_heads);
    if (((uintptr_t)q & 3) || (q_row & 1)) ABK_REFUSE("attention_decode_ring: q must be 4-byte aligned");
    if (prepare && ((((uintptr_t)q | (uintptr_t)prepare->q_norm | (uintptr_t)prepare->k_norm | (uintptr_t)prepare->cos |
                      (uintptr_t)prepare->sin | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) || (q_row & 7) || !prepare->cos != !prepare->sin))
        ABK_REFUSE("attention_decode_ring: rows, norms, angles and pools must be 16-byte aligned to be prepared here");
    if ((uintptr_t)out & 7) ABK_REFUSE("attention_decode_ring: out must be 8-byte aligned");
    CUtensorMap km, vm;
    int rc = tmap::bf16_rows_of_128_bytes(k_pool, pool_rows, head_dim, head_dim, PAGE, &km);
    if (!rc) rc = tmap::bf16_rows_of_128_bytes(v_pool, pool_rows, head_dim, head_dim, PAGE, &vm);
    if (rc) return rc;
    const int group = n_heads / n_kv_heads;
    AttnDecodeRing p;
    p.q = (const __nv_bfloat16 *)q, p.q_row = q_row, p.out = (__nv_bfloat16 *)out, p.n_heads = n_heads;
    p.n_kv_heads = n_kv_heads, p.scale_log2 = scale * 1.4426950408889634f, p.window = window;
    p.token_seq = token_seq, p.token_pos = token_pos, p.seq_slot = seq_slot;
    p.cache.page_table = page_table, p.cache.table_width = table_width, p.cache.ring_pages = ring_pages;
    p.cache.tokens_per_page = tokens_per_page;
    p.prepare = prepare != nullptr;
    p.q_norm = prepare ? prepare->q_norm : nullptr, p.k_norm = prepare ? prepare->k_norm : nullptr;
    p.cos = prepare ? prepare->cos : nullptr, p.sin = prepare ? prepare->sin : nullptr, p.eps = prepare ? prepare->eps : 0.0f;
    p.k_pool = prepare && prepare->keep ? (__nv_bfloat16 *)k_pool : nullptr;
    p.v_pool = prepare && prepare->keep ? (__nv_bfloat16 *)v_pool : nullptr;
    {   // once per device
        cudaError_t e = abk_allow_shared_memory((const void *)attn_decode_ring_kernel<64>, 224 * 1024);
        if (e == cudaSuccess) e = abk_allow_shared_memory((const void *)attn_decode_ring_kernel<128>, 224 * 1024);
        if (e != cudaSuccess) return (int)e;
    }
    // CTAs per (row, kv head): as many as a cluster holds (8) and the pages allow, as long as all of the grid's
    // clusters are on the device at once; a grid so small that they still are with a ring twice as deep
    // (one CTA to an SM) gets that, for the same bytes in flight per SM
    const long long pairs = (long long)n_rows * n_kv_heads;
    const int pages = (max_positions + PAGE - 1) / PAGE;
    const int tile_pair = 2 * PAGE * head_dim * 2;
    // partial results, the prepared query heads, and room to align them and the ring
    const int fold_bytes = 5 * group * (head_dim + 2) * 4 + group * head_dim * 2 + 16 + 1024 + 64;
    int stages = RING_STAGE_BYTES / tile_pair;
    if (stages > (224 * 1024 - fold_bytes) / tile_pair) stages = (224 * 1024 - fold_bytes) / tile_pair;
    if (stages < 2) ABK_REFUSE("attention_decode_ring: a group of %d heads of %d leaves no room for a ring", group, head_dim);
    int deep = 2 * stages;
    if (deep > RING_MAX_STAGES) deep = RING_MAX_STAGES;
    if (deep > (224 * 1024 - fold_bytes) / tile_pair) deep = (224 * 1024 - fold_bytes) / tile_pair;
    auto resident = [&](int s, int st) {
        int smem = st * tile_pair + fold_bytes;
        return head_dim == 64 ? resident_clusters<64>(s, smem) : resident_clusters<128>(s, smem);
    };
    int splits = pages < RING_MAX_SPLITS ? pages : RING_MAX_SPLITS;
    while (splits > 1 && resident(splits, stages) < pairs) splits--;
    p.stages = deep > stages && resident(splits, deep) >= pairs ? deep : stages;
    p.status = status;
    const int smem = p.stages * tile_pair + fold_bytes;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits, n_kv_heads, n_rows), cfg.blockDim = dim3(RING_THREADS), cfg.dynamicSmemBytes = smem;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = splits, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = abk_pdl_enabled() ? 2 : 1;
    if (head_dim == 64) cudaLaunchKernelEx(&cfg, attn_decode_ring_kernel<64>, km, vm, p);
    else cudaLaunchKernelEx(&cfg, attn_decode_ring_kernel<128>, km, vm, p);
    return ABK_LAUNCH_RESULT();
}

// max_positions: no row's position reaches it (with the number of rows it fixes the grid; a captured graph
// passes its bound). status word 2 is set if a wait ran out.
extern "C" int abk_attention_decode_ring(const void *q, long long q_row, void *out, int n_rows, int n_heads,
                                         int n_kv_heads, int head_dim, float scale, int window, const int *token_seq,
                                         const int *token_pos, const int *seq_slot, const void *k_pool,
                                         const void *v_pool, long long pool_rows, const int *page_table, int table_width,
                                         int ring_pages, int tokens_per_page, int max_positions, int *status,
                                         void *stream) {
    return ring_launch(q, q_row, out, n_rows, n_heads, n_kv_heads, head_dim, scale, window, token_seq, token_pos, seq_slot, k_pool,
                       v_pool, pool_rows, page_table, table_width, ring_pages, tokens_per_page, max_positions, status, nullptr,
                       stream);
}

// The same with q/k/v preparation taken in (src/model.c:247-259): the rows at q are as the q/k/v product left them
// (q heads, then k heads, then v heads); q and k are normed with q_norm / k_norm [head_dim] (null: not) and eps, rotated
// over the whole head in halves with cos / sin [positions, head_dim / 2] (null: not), and with keep != 0 the new
// token's key and value are written to the pools. Rows, norms, angles and pools 16-byte aligned.
extern "C" int abk_attention_decode_ring_prepare(const void *qkv, long long q_row, void *out, int n_rows, int n_heads,
                                                 int n_kv_heads, int head_dim, float scale, int window,
                                                 const int *token_seq, const int *token_pos, const int *seq_slot,
                                                 void *k_pool, void *v_pool, long long pool_rows, const int *page_table,
                                                 int table_width, int ring_pages, int tokens_per_page, int max_positions,
                                                 const float *q_norm, const float *k_norm, float eps, const float *cos,
                                                 const float *sin, int keep, int *status, void *stream) {
    RingPrepare prepare = {q_norm, k_norm, cos, sin, eps, keep};
    return ring_launch(qkv, q_row, out, n_rows, n_heads, n_kv_heads, head_dim, scale, window, token_seq, token_pos, seq_slot,
                       k_pool, v_pool, pool_rows, page_table, table_width, ring_pages, tokens_per_page, max_positions, status,
                       &prepare, stream);
}

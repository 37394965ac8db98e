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
#define ABK_DEFINE_ERROR
#include "common.cuh"
#include "tc_common.cuh"
#include "tensor_map.cuh"
#include "mma_tiles.cuh"

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
                if (first_page + split + issued * splits == last_page) pdl_wait();  // the new token's page
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
        int done = 0, s = 0, phase = 0;
        for (int pg = first_page + split; pg <= last_page && ok; pg += splits, done++) {
            if (!tc::mbar_wait(&full[s], phase)) {
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

// max_positions: no row's position reaches it (with the number of rows it fixes the grid; a captured graph
// passes its bound). status word 2 is set if a wait ran out.
extern "C" int abk_attention_decode_ring(const void *q, long long q_row, void *out, int n_rows, int n_heads,
                                         int n_kv_heads, int head_dim, float scale, int window, const int *token_seq,
                                         const int *token_pos, const int *seq_slot, const void *k_pool,
                                         const void *v_pool, long long pool_rows, const int *page_table, int table_width,
                                         int ring_pages, int tokens_per_page, int max_positions, int *status,
                                         void *stream) {
    if (n_rows <= 0) return 0;
    if (head_dim != 64 && head_dim != 128) ABK_REFUSE("attention_decode_ring: head_dim %d is not 64 or 128", head_dim);
    if (tokens_per_page != PAGE) ABK_REFUSE("attention_decode_ring: pages of %d tokens, not %d", tokens_per_page, PAGE);
    if (n_kv_heads < 1 || n_heads % n_kv_heads || n_heads / n_kv_heads > 16)
        ABK_REFUSE("attention_decode_ring: %d heads in %d groups (at most 16 to a group)", n_heads, n_kv_heads);
    if (n_kv_heads > 65535 || n_rows > 65535) ABK_REFUSE("attention_decode_ring: %d rows or %d kv heads exceed a grid", n_rows, n_kv_heads);
    if (((uintptr_t)q & 3) || (q_row & 1)) ABK_REFUSE("attention_decode_ring: q must be 4-byte aligned");
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
    const int fold_bytes = 5 * group * (head_dim + 2) * 4 + 1024 + 64;  // partial results, and room to align the ring
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

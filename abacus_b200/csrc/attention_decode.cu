// Decode attention: one new token per sequence against its keys and values in the paged cache.
// bfloat16 cache, head sizes 64, 128 and 256, any number of heads and groups, with or without a
// window. Other sizes and the float32 cache go to the general kernel.
//
// The work is split along the keys so that a single long sequence still fills the GPU: a CTA
// takes one (row, kv head, chunk of 128 keys = two pages). It copies the chunk's two key pages
// and two value pages (each [64, head_dim], contiguous in the cache) into shared memory with
// bulk async copies (cp.async.bulk) signalled on mbarriers, then each of its four warps takes
// 32 keys: scores, their maximum and sum, and the weighted values, for every query head of the
// group in turn. A lane owns head_dim / 32 consecutive elements; the dot products of eight keys
// are reduced across the warp together (9 shuffles for 8 keys) so that the shuffles of one key
// do not wait on each other. The CTA leaves (max, sum, weighted values) per query head in
// scratch memory and takes a ticket; the last CTA of a (row, kv head) folds the chunks together
// in chunk order. Chunks are aligned to absolute positions, so what a row computes does not
// depend on the batch it is in, nor on which CTA came last.
//
// Formula: src/model.c:197-211; softmax and accumulation in float32.
#define ABK_DEFINE_ERROR
#include "common.cuh"
#include "tc_common.cuh"

#define DEC_THREADS 128
#define DEC_CHUNK 128
#define DEC_PAGE 64

struct AttnDecode {
    const __nv_bfloat16 *q;  // row r, head h at q + r * q_row + h * head_dim
    long long q_row;
    __nv_bfloat16 *out;  // [rows, n_heads * head_dim]
    int n_heads, n_kv_heads, head_dim;
    float scale;  // score scale times log2(e): scores and references are in units of log2
    int window;
    const int *token_seq, *token_pos, *seq_slot;
    const __nv_bfloat16 *k_pool, *v_pool;
    PagedCache cache;
    float *part_o;   // [rows, n_heads, max_chunks, head_dim]
    float *part_ml;  // [rows, n_heads, max_chunks, 2]
    int *tickets;    // [rows, n_kv_heads], zero before and after
    int max_chunks;
    int *status;
};

__device__ __forceinline__ void bulk_copy(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     tc::smem_addr(dst)),
                 "l"(src), "r"(bytes), "r"(tc::smem_addr(bar))
                 : "memory");
}

template <int EPL> __device__ __forceinline__ void load_slice(const __nv_bfloat16 *p, float *f);
template <> __device__ __forceinline__ void load_slice<2>(const __nv_bfloat16 *p, float *f) {
    float2 t = __bfloat1622float2(*(const __nv_bfloat162 *)p);
    f[0] = t.x, f[1] = t.y;
}
template <> __device__ __forceinline__ void load_slice<4>(const __nv_bfloat16 *p, float *f) {
    uint2 raw = *(const uint2 *)p;
    float2 a = __bfloat1622float2(*(const __nv_bfloat162 *)&raw.x), b = __bfloat1622float2(*(const __nv_bfloat162 *)&raw.y);
    f[0] = a.x, f[1] = a.y, f[2] = b.x, f[3] = b.y;
}
template <> __device__ __forceinline__ void load_slice<8>(const __nv_bfloat16 *p, float *f) {
    uint4 raw = *(const uint4 *)p;
    const __nv_bfloat162 *h = (const __nv_bfloat162 *)&raw;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float2 t = __bfloat1622float2(h[i]);
        f[2 * i] = t.x, f[2 * i + 1] = t.y;
    }
}

// Sums part[0..7] over the warp, eight values at once: afterwards part[0] of lane L is the total of
// value number 4 * bit4(L) + 2 * bit3(L) + bit2(L). Every step halves what a lane still carries.
__device__ __forceinline__ float reduce8(float *part, int lane) {
    const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float send = b4 ? part[i] : part[i + 4], keep = b4 ? part[i + 4] : part[i];
        part[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        float send = b3 ? part[i] : part[i + 2], keep = b3 ? part[i + 2] : part[i];
        part[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
    float send = b2 ? part[0] : part[1], keep = b2 ? part[1] : part[0];
    float v = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v;
}

// HD = 32 * EPL: every lane owns EPL consecutive elements of a head.
template <int EPL> __global__ void __launch_bounds__(DEC_THREADS) attn_decode_kernel(AttnDecode p) {
    constexpr int HD = 32 * EPL;
    extern __shared__ __align__(128) uint8_t dec_smem[];
    __nv_bfloat16 *k_s = (__nv_bfloat16 *)dec_smem;            // [2 pages][64][HD]
    __nv_bfloat16 *v_s = k_s + 2 * DEC_PAGE * HD;              // [2 pages][64][HD]
    float *warp_o = (float *)(v_s + 2 * DEC_PAGE * HD);        // [4 warps][group][HD]
    const int group = p.n_heads / p.n_kv_heads;
    float *warp_ml = warp_o + 4 * group * HD;                  // [4 warps][group][2]
    uint64_t *bars = (uint64_t *)(warp_ml + 4 * group * 2);    // one per page
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
    if (pos >= p.max_chunks * DEC_CHUNK) {
        // The row lies beyond the bound the grid was sized for: not all of its chunks have a CTA, so nobody would
        // draw the last ticket. Say so in the status word, leave zeros, and touch no ticket.
        if (chunk == 0) {
            if (threadIdx.x == 0) atomicOr(p.status + 2, 2);
            for (int i = threadIdx.x; i < group * HD; i += DEC_THREADS)
                p.out[((long long)r * p.n_heads + kvh * group) * HD + i] = __float2bfloat16_rn(0.0f);
        }
        return;
    }
    const int lo = p.window > 0 && pos - p.window + 1 > 0 ? pos - p.window + 1 : 0;
    const int first = chunk * DEC_CHUNK;
    if (first > pos || first + DEC_CHUNK <= lo) return;  // none of this chunk's keys is visible
    const int slot = p.seq_slot[seq];

    if (threadIdx.x == 0) {
        failed = 0;
        tc::mbar_init(&bars[0], 1), tc::mbar_init(&bars[1], 1);
        tc::mbar_init_fence();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int pg = 0; pg < 2; pg++) {
            int p_first = first + pg * DEC_PAGE;
            if (p_first > pos || p_first + DEC_PAGE <= lo) continue;
            int rows = min(DEC_PAGE, pos - p_first + 1);
            uint32_t bytes = (uint32_t)rows * HD * 2;
            int page = cache_page(p.cache, slot, p_first);
            long long off = cache_offset(p.cache, page, kvh, p.n_kv_heads, p_first, HD);
            tc::mbar_expect_tx(&bars[pg], 2 * bytes);
            bulk_copy(k_s + pg * DEC_PAGE * HD, p.k_pool + off, bytes, &bars[pg]);
            bulk_copy(v_s + pg * DEC_PAGE * HD, p.v_pool + off, bytes, &bars[pg]);
        }
    }
    // warp w takes keys first + 32 w .. + 31, which lie in page w / 2
    const int j0 = first + warp * 32, pg = warp >> 1;
    const bool any = j0 <= pos && j0 + 32 > lo;
    if (any && !tc::mbar_wait(&bars[pg], 0)) failed = 1;
    const __nv_bfloat16 *kw = k_s + (warp * 32) * HD + lane * EPL, *vw = v_s + (warp * 32) * HD + lane * EPL;
    const int n_keys = any ? min(32, pos - j0 + 1) : 0;  // keys j0 .. j0 + n_keys - 1 exist
    const int skip = any && lo > j0 ? lo - j0 : 0;       // and the first `skip` of them are outside the window
    const int my_key = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);  // see reduce8

    for (int g = 0; g < group; g++) {
        const int h = kvh * group + g;
        float q[EPL], o[EPL], sc[4];
        load_slice<EPL>(p.q + (long long)r * p.q_row + (long long)h * HD + lane * EPL, q);
#pragma unroll
        for (int rd = 0; rd < 4; rd++) {
            sc[rd] = -INFINITY;
            if (rd * 8 < n_keys) {  // rows beyond n_keys were not copied; what they hold is never used
                float part[8];
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    float kf[EPL];
                    load_slice<EPL>(kw + (rd * 8 + i) * HD, kf);
                    part[i] = 0.0f;
#pragma unroll
                    for (int e = 0; e < EPL; e++) part[i] = fmaf(q[e], kf[e], part[i]);
                }
                float s = reduce8(part, lane) * p.scale;
                int kk = rd * 8 + my_key;
                if (kk >= skip && kk < n_keys) sc[rd] = s;
            }
        }
        // scores are in units of log2 and the reference is the maximum rounded up to a whole number: a key's
        // probability is then the same bits times a power of two whichever warp or chunk it falls into
        float m = ceilf(warp_max(fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]))));
        float pr[4];
#pragma unroll
        for (int rd = 0; rd < 4; rd++) pr[rd] = sc[rd] == -INFINITY ? 0.0f : exp2f(sc[rd] - m);
        float l = warp_sum((pr[0] + pr[1]) + (pr[2] + pr[3])) * 0.25f;  // four lanes hold each key
        // summed unrounded, multiplied with the values as bfloat16: what the tensor-core kernels do, so that a
        // row's result does not depend on which kernel ran it beyond rounding
#pragma unroll
        for (int rd = 0; rd < 4; rd++) pr[rd] = __bfloat162float(__float2bfloat16_rn(pr[rd]));
#pragma unroll
        for (int e = 0; e < EPL; e++) o[e] = 0.0f;
#pragma unroll
        for (int rd = 0; rd < 4; rd++) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
                int kk = rd * 8 + i;
                if (kk < n_keys) {
                    float vf[EPL];
                    float pk = __shfl_sync(0xffffffffu, pr[rd], ((i >> 2) & 1) * 16 + ((i >> 1) & 1) * 8 + (i & 1) * 4);
                    load_slice<EPL>(vw + kk * HD, vf);
#pragma unroll
                    for (int e = 0; e < EPL; e++) o[e] = fmaf(pk, vf[e], o[e]);
                }
            }
        }
        float *wo = warp_o + (warp * group + g) * HD + lane * EPL;
#pragma unroll
        for (int e = 0; e < EPL; e++) wo[e] = o[e];
        if (lane == 0) warp_ml[(warp * group + g) * 2] = m, warp_ml[(warp * group + g) * 2 + 1] = l;
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
            float f[4], ov[4], lv[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                bool in = c0 + u <= c_hi;
                f[u] = in ? __ldcg(p.part_ml + (base + c0 + u) * 2) : -INFINITY;
                lv[u] = in ? __ldcg(p.part_ml + (base + c0 + u) * 2 + 1) : 0.0f;
                ov[u] = in ? __ldcg(p.part_o + (base + c0 + u) * HD + d) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                float w = f[u] == -INFINITY ? 0.0f : exp2f(f[u] - m);
                acc = fmaf(w, ov[u], acc), l = fmaf(w, lv[u], l);
            }
        }
        p.out[((long long)r * p.n_heads + h) * HD + d] = __float2bfloat16_rn(acc / l);
    }
    if (threadIdx.x == 0) p.tickets[r * p.n_kv_heads + kvh] = 0;
}

// floats of scratch: partial values and (max, sum) pairs; then the tickets, as int32 (zero at first).
extern "C" long long abk_attention_decode_scratch_floats(int rows, int n_heads, int head_dim, int max_chunks) {
    return (long long)rows * n_heads * max_chunks * (head_dim + 2);
}

// max_positions: no row's position reaches it (it sizes the grid; a captured graph passes its bound).
// scratch: float32 [abk_attention_decode_scratch_floats(...)]; tickets: int32 [n_rows * n_kv_heads], zero
// before and after. status word 2 is set if a wait ran out.
extern "C" int abk_attention_decode(const void *q, long long q_row, void *out, int n_rows, int n_heads, int n_kv_heads,
                                    int head_dim, float scale, int window, const int *token_seq, const int *token_pos,
                                    const int *seq_slot, const void *k_pool, const void *v_pool, const int *page_table,
                                    int table_width, int ring_pages, int tokens_per_page, int max_positions,
                                    float *scratch, int *tickets, int *status, void *stream) {
    if (n_rows <= 0) return 0;
    if (head_dim != 64 && head_dim != 128 && head_dim != 256)
        ABK_REFUSE("attention_decode: head_dim %d is not 64, 128 or 256", head_dim);
    if (tokens_per_page != DEC_PAGE) ABK_REFUSE("attention_decode: pages of %d tokens, not %d", tokens_per_page, DEC_PAGE);
    if (n_kv_heads < 1 || n_heads % n_kv_heads) ABK_REFUSE("attention_decode: %d heads, %d kv heads", n_heads, n_kv_heads);
    if (n_kv_heads > 65535 || n_rows > 65535) ABK_REFUSE("attention_decode: %d rows or %d kv heads exceed a grid", n_rows, n_kv_heads);
    if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15 || (q_row * 2) % 16)
        ABK_REFUSE("attention_decode: q and the cache must be 16-byte aligned");
    int max_chunks = (max_positions + DEC_CHUNK - 1) / DEC_CHUNK;
    if (max_chunks < 1) max_chunks = 1;
    int group = n_heads / n_kv_heads;
    AttnDecode p;
    p.q = (const __nv_bfloat16 *)q, p.q_row = q_row, p.out = (__nv_bfloat16 *)out, p.n_heads = n_heads;
    p.n_kv_heads = n_kv_heads, p.head_dim = head_dim, p.scale = scale * 1.4426950408889634f, p.window = window, p.token_seq = token_seq;
    p.token_pos = token_pos, p.seq_slot = seq_slot, p.k_pool = (const __nv_bfloat16 *)k_pool;
    p.v_pool = (const __nv_bfloat16 *)v_pool;
    p.cache.page_table = page_table, p.cache.table_width = table_width, p.cache.ring_pages = ring_pages;
    p.cache.tokens_per_page = tokens_per_page;
    p.part_o = scratch, p.part_ml = scratch + (long long)n_rows * n_heads * max_chunks * head_dim;
    p.tickets = tickets, p.max_chunks = max_chunks, p.status = status;
    size_t smem = (size_t)4 * DEC_PAGE * head_dim * 2 + (size_t)4 * group * (head_dim + 2) * 4 + 64;
    if (smem > 200 * 1024) ABK_REFUSE("attention_decode: a group of %d query heads needs %zu bytes of shared memory", group, smem);
    dim3 grid(max_chunks, n_kv_heads, n_rows);
    cudaStream_t s = (cudaStream_t)stream;
    {   // once per device, and not inside a stream capture
        cudaError_t e = abk_allow_shared_memory((const void *)attn_decode_kernel<2>, 200 * 1024);
        if (e == cudaSuccess) e = abk_allow_shared_memory((const void *)attn_decode_kernel<4>, 200 * 1024);
        if (e == cudaSuccess) e = abk_allow_shared_memory((const void *)attn_decode_kernel<8>, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
    }
    if (head_dim == 64) attn_decode_kernel<2><<<grid, DEC_THREADS, smem, s>>>(p);
    else if (head_dim == 128) attn_decode_kernel<4><<<grid, DEC_THREADS, smem, s>>>(p);
    else attn_decode_kernel<8><<<grid, DEC_THREADS, smem, s>>>(p);
    return ABK_LAUNCH_RESULT();
}

// Row-wise kernels around the matrix products: embedding, residual add + RMSNorm,
// SwiGLU, and the preparation of q/k/v (per-head norm, rotary encoding, cache write).
// All arithmetic is float32; only what is stored may be bfloat16.
#define ABK_DEFINE_ERROR
#include "common.cuh"
#include "qkv_prep.cuh"

// ------------------------------------------------------------------ embedding
// x[t, :] = float(table[tokens[t], :])                      (src/model.c:290-291)
template <typename TW>
__global__ void embed_kernel(const int *__restrict__ tokens, const TW *__restrict__ table, float *__restrict__ x,
                             int d, int vocab, int *status) {
    pdl_wait();
    int t = blockIdx.x;
    int tok = tokens[t];
    bool bad = tok < 0 || tok >= vocab;
    if (bad && threadIdx.x == 0) atomicOr(status, 1);
    const TW *row = table + (long long)(bad ? 0 : tok) * d;
    float *out = x + (long long)t * d;
    for (int j = threadIdx.x; j < d; j += blockDim.x) out[j] = bad ? 0.0f : to_float(row[j]);
}

extern "C" int abk_embed(const int *tokens, const void *table, int table_dtype, float *x, int n_tokens, int d, int vocab,
                         int *status, void *stream) {
    if (n_tokens <= 0) return 0;
    int threads = d >= 1024 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    if (table_dtype == ABK_BF16)
        abk_launch(embed_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, s, tokens, (const __nv_bfloat16 *)table, x, d, vocab, status);
    else
        abk_launch(embed_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, tokens, (const float *)table, x, d, vocab, status);
    return ABK_LAUNCH_RESULT();
}

// ------------------------------------------------------------------ residual add + RMSNorm
// x += y (when y is given); out = w * (x / sqrt(mean(x^2) + eps))      (src/model.c:238-244, 164-169)
// With `rows`, output row r is made from row rows[r] of x (+ y) and x is left as it is: the
// final norm of the rows whose logits are wanted.
__device__ __forceinline__ void store4(float *p, float a, float b, float c, float d) { *(float4 *)p = make_float4(a, b, c, d); }
__device__ __forceinline__ void store4(__nv_bfloat16 *p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *(uint2 *)p = make_uint2(*(uint32_t *)&lo, *(uint32_t *)&hi);
}

template <typename TO>
__global__ void add_rmsnorm_kernel(float *__restrict__ x, const float *__restrict__ y, const float *__restrict__ w,
                                   TO *__restrict__ out, const int *__restrict__ rows, int d, float eps) {
    __shared__ float scratch[33];
    pdl_wait();
    int r = blockIdx.x;
    long long src = rows ? rows[r] : r;
    float *xr = x + src * d;
    const float *yr = y ? y + src * d : nullptr;
    bool update = yr && !rows;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        float v = xr[j];
        if (yr) v += yr[j];
        if (update) xr[j] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    float scale = 1.0f / sqrtf(ss / (float)d + eps);
    TO *o = out + (long long)r * d;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        float v = xr[j];
        if (yr && !update) v += yr[j];
        o[j] = from_float<TO>(w[j] * (v * scale));
    }
}

// The same with a row in registers (d a multiple of 4 up to 1024 * V, V float4 a thread): the weights come
// in before pdl_wait(), x and y are read once, and every access is 16 bytes wide.
template <typename TO, int V>
__global__ void __launch_bounds__(256) add_rmsnorm_row_kernel(float *__restrict__ x, const float *__restrict__ y,
                                                              const float *__restrict__ w, TO *__restrict__ out,
                                                              const int *__restrict__ rows, int d, float eps) {
    __shared__ float scratch[33];
    float4 wv[V], v[V];
#pragma unroll
    for (int i = 0; i < V; i++) {
        int j = 4 * (threadIdx.x + 256 * i);
        wv[i] = j < d ? *(const float4 *)(w + j) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    pdl_wait();
    const int r = blockIdx.x;
    const long long src = rows ? rows[r] : r;
    float *xr = x + src * d;
    const float *yr = y ? y + src * d : nullptr;
    const bool update = yr && !rows;
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < V; i++) {
        int j = 4 * (threadIdx.x + 256 * i);
        v[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (j < d) {
            v[i] = *(const float4 *)(xr + j);
            if (yr) {
                float4 t = *(const float4 *)(yr + j);
                v[i].x += t.x, v[i].y += t.y, v[i].z += t.z, v[i].w += t.w;
            }
            if (update) *(float4 *)(xr + j) = v[i];
        }
        ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    TO *o = out + (long long)r * d;
#pragma unroll
    for (int i = 0; i < V; i++) {
        int j = 4 * (threadIdx.x + 256 * i);
        if (j < d) store4(o + j, wv[i].x * (v[i].x * scale), wv[i].y * (v[i].y * scale), wv[i].z * (v[i].z * scale),
                          wv[i].w * (v[i].w * scale));
    }
}

extern "C" int abk_add_rmsnorm(float *x, const float *y, const float *w, void *out, int out_dtype, const int *rows,
                               int n_rows, int d, float eps, void *stream) {
    if (n_rows <= 0) return 0;
    int threads = d >= 2048 ? 512 : d >= 512 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    const bool aligned = !(((uintptr_t)x | (uintptr_t)y | (uintptr_t)w | (uintptr_t)out) & 15);
    if (d % 4 == 0 && d <= 4096 && aligned) {
#define ROW_LAUNCH(TO, V) \
    abk_launch(add_rmsnorm_row_kernel<TO, V>, dim3(n_rows), dim3(256), 0, s, x, y, w, (TO *)out, rows, d, eps)
#define ROW_BY_D(TO)                       \
    if (d <= 1024) ROW_LAUNCH(TO, 1);      \
    else if (d <= 2048) ROW_LAUNCH(TO, 2); \
    else ROW_LAUNCH(TO, 4);
        if (out_dtype == ABK_BF16) { ROW_BY_D(__nv_bfloat16) } else { ROW_BY_D(float) }
#undef ROW_BY_D
#undef ROW_LAUNCH
        return ABK_LAUNCH_RESULT();
    }
    if (out_dtype == ABK_BF16)
        abk_launch(add_rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, s, x, y, w, (__nv_bfloat16 *)out, rows, d, eps);
    else
        abk_launch(add_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, s, x, y, w, (float *)out, rows, d, eps);
    return ABK_LAUNCH_RESULT();
}

// ------------------------------------------------------------------ SwiGLU
// act[t, j] = silu(gate[t, j]) * up[t, j]                              (src/model.c:274-282)
// A row of gate_up holds gate and up in turns of `block` columns: gate of features [0, block), up of the same,
// gate of [block, 2 block), ... With block = inter that is all gates and then all ups (src/model.c:98).
__device__ __forceinline__ long long gate_column(int j, int block) { return (long long)(j / block) * 2 * block + j % block; }
template <typename T>
__global__ void swiglu_kernel(const T *__restrict__ gate_up, T *__restrict__ act, long long total, int inter, int block) {
    pdl_wait();
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (long long)gridDim.x * blockDim.x) {
        long long t = e / inter;
        int j = (int)(e - t * inter);
        float g = to_float(gate_up[t * 2 * inter + gate_column(j, block)]);
        float u = to_float(gate_up[t * 2 * inter + gate_column(j, block) + block]);
        act[e] = from_float<T>(sizeof(T) == 2 ? silu_mul_fast(g, u) : g / (1.0f + expf(-g)) * u);
    }
}

// bfloat16 with inter and block multiples of 8: eight elements a thread, read and written as 16-byte vectors.
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16 *__restrict__ gate_up, __nv_bfloat16 *__restrict__ act,
                                     long long groups, int inter, int block) {
    pdl_wait();
    const int per_row = inter >> 3;
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += (long long)gridDim.x * blockDim.x) {
        long long t = g / per_row;
        int j = (int)(g - t * per_row) << 3;
        const __nv_bfloat16 *gcol = gate_up + t * 2 * inter + gate_column(j, block);
        uint4 graw = *(const uint4 *)gcol, uraw = *(const uint4 *)(gcol + block);
        const __nv_bfloat162 *gp = (const __nv_bfloat162 *)&graw, *up = (const __nv_bfloat162 *)&uraw;
        uint4 out;
        __nv_bfloat162 *op = (__nv_bfloat162 *)&out;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            float2 gv = __bfloat1622float2(gp[e]), uv = __bfloat1622float2(up[e]);
            op[e] = __floats2bfloat162_rn(silu_mul_fast(gv.x, uv.x), silu_mul_fast(gv.y, uv.y));
        }
        *(uint4 *)(act + t * inter + j) = out;
    }
}

extern "C" int abk_swiglu(const void *gate_up, void *act, int dtype, int n_tokens, int inter, int block, void *stream) {
    long long total = (long long)n_tokens * inter;
    if (total <= 0) return 0;
    if (block <= 0 || inter % block) ABK_REFUSE("swiglu: turns of %d columns do not divide %d", block, inter);
    if (dtype == ABK_BF16 && inter % 8 == 0 && block % 8 == 0 && ((uintptr_t)gate_up | (uintptr_t)act) % 16 == 0) {
        long long groups = total >> 3, want = (groups + 255) / 256;
        int blocks = (int)(want > abk_sm_count() * 16 ? abk_sm_count() * 16 : want);
        abk_launch(swiglu_bf16x8_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16 *)gate_up,
                   (__nv_bfloat16 *)act, groups, inter, block);
        return ABK_LAUNCH_RESULT();
    }
    int threads = 256;
    long long blocks = (total + threads - 1) / threads;
    if (blocks > abk_sm_count() * 32) blocks = abk_sm_count() * 32;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ABK_BF16)
        abk_launch(swiglu_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, s, (const __nv_bfloat16 *)gate_up, (__nv_bfloat16 *)act, total, inter, block);
    else
        abk_launch(swiglu_kernel<float>, dim3((int)blocks), dim3(threads), 0, s, (const float *)gate_up, (float *)act, total, inter, block);
    return ABK_LAUNCH_RESULT();
}

// ------------------------------------------------------------------ q/k/v preparation
// Per token and head (src/model.c:247-259): RMSNorm over the head with a weight shared by all
// heads (q and k, not v), then the rotary encoding of q and k, in place; k and v are also
// written to their place in the paged cache.
//
// One warp per (token, head). Heads are numbered q heads, then k heads, then v heads, as they
// lie in a row of qkv. Tokens whose sequence index is negative are padding and are skipped.
struct QkvPrep {
    void *qkv;
    int n_heads, n_kv_heads, head_dim;
    int q_only;  // only the q heads are prepared (keys and values come from elsewhere)
    const int *token_seq, *token_pos, *seq_slot, *seq_len_after;
    const float *q_norm, *k_norm;
    float eps;
    const float *cos, *sin;  // [positions, rotary_dim / 2]; null: no rotation
    int rotary_dim, interleaved;
    void *k_pool, *v_pool;  // null: nothing is cached (the layer reads another layer's cache)
    PagedCache cache;
};

#define PREP_WARPS 4
#define MAX_HEAD_DIM 256

template <typename T> __global__ void qkv_prep_kernel(QkvPrep p) {
    __shared__ float buf[PREP_WARPS][MAX_HEAD_DIM];
    pdl_wait();
    int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int head = blockIdx.y * PREP_WARPS + warp;
    int total_heads = p.n_heads + 2 * p.n_kv_heads;
    if (head >= (p.q_only ? p.n_heads : total_heads)) return;
    int seq = p.token_seq[t];
    if (seq < 0) return;
    int pos = p.token_pos[t];
    int hd = p.head_dim;
    T *row = (T *)p.qkv + ((long long)t * total_heads + head) * hd;
    bool is_q = head < p.n_heads, is_k = !is_q && head < p.n_heads + p.n_kv_heads;
    int kv_head = is_q ? 0 : is_k ? head - p.n_heads : head - p.n_heads - p.n_kv_heads;
    float *b = buf[warp];

    if (is_q || is_k) {
        float ss = 0.0f;
        for (int j = lane; j < hd; j += 32) {
            float v = to_float(row[j]);
            b[j] = v;
            ss += v * v;
        }
        const float *w = is_q ? p.q_norm : p.k_norm;
        if (w) {
            ss = warp_sum(ss);
            float scale = 1.0f / sqrtf(ss / (float)hd + p.eps);
            for (int j = lane; j < hd; j += 32) b[j] = w[j] * (b[j] * scale);
        }
        __syncwarp();
        if (p.cos) {
            int half = p.rotary_dim / 2;
            const float *c = p.cos + (long long)pos * half, *s = p.sin + (long long)pos * half;
            for (int i = lane; i < half; i += 32) {
                int ia = p.interleaved ? 2 * i : i, ib = p.interleaved ? 2 * i + 1 : i + half;
                float a = b[ia], bb = b[ib];
                b[ia] = a * c[i] - bb * s[i];
                b[ib] = bb * c[i] + a * s[i];
            }
            __syncwarp();
        }
        for (int j = lane; j < hd; j += 32) row[j] = from_float<T>(b[j]);
    }
    if (is_q || !p.k_pool) return;
    // A windowed cache keeps ring_pages pages; of the positions that share a place only the last is written.
    if (p.cache.ring_pages > 0 &&
        pos + p.cache.ring_pages * p.cache.tokens_per_page <= p.seq_len_after[seq] - 1)
        return;
    int page = cache_page(p.cache, p.seq_slot[seq], pos);
    T *dst = (T *)(is_k ? p.k_pool : p.v_pool) + cache_offset(p.cache, page, kv_head, p.n_kv_heads, pos, hd);
    if (is_k)
        for (int j = lane; j < hd; j += 32) dst[j] = from_float<T>(b[j]);
    else
        for (int j = lane; j < hd; j += 32) dst[j] = row[j];
}

// The same for bfloat16 heads of 64 * EPH elements that are rotated whole in half pairing (or not at
// all): each lane owns EPH consecutive elements of the first half and their partners in the second,
// read and written as one vector each, with no shared-memory staging.
#define FAST_WARPS 4
#define FAST_SLOTS 4  // groups of heads a warp has in flight at a time (its share of a prompt token's 32 heads of 128)
// One head of one token in the fast kernels: this lane's 8 elements `raw` of head `head` (q, k or v by its number) are
// normed, rotated with the lane's angles cs/sn, written back to the row, and k and v go to the cache at kept_at (the
// token's place in the pools for kv head 0; negative: not kept). Whole warps call it (shuffles); lanes past the
// end of the heads have live = false.
template <int HD>
__device__ __forceinline__ void prep_head(const QkvPrep &p, uint4 raw_u, int head, bool live, int l, bool upper,
                                          const float *cs, const float *sn, __nv_bfloat16 *row0, long long kept_at) {
    const bool is_q = head < p.n_heads, is_k = !is_q && head < p.n_heads + p.n_kv_heads;
    const int kv_head = is_q ? 0 : is_k ? head - p.n_heads : head - p.n_heads - p.n_kv_heads;
    const uint4 done = prep_head_values<HD>(raw_u, is_q || is_k, is_q ? p.q_norm : p.k_norm, p.eps, p.cos != nullptr, l, upper, cs, sn);
    if (live && (is_q || is_k)) *(uint4 *)(row0 + (long long)head * HD) = done;
    if (live && !is_q && kept_at >= 0) {
        __nv_bfloat16 *dst = (__nv_bfloat16 *)(is_k ? p.k_pool : p.v_pool) + kept_at +
                             (long long)kv_head * p.cache.tokens_per_page * HD + l * 8;
        *(uint4 *)dst = done;
    }
}

// bfloat16, head sizes 64, 128 and 256, rotation over the whole head in halves: a lane holds 8 consecutive
// elements (16 bytes) of a head, so HD / 8 lanes hold a head and a warp 32 * 8 / HD heads at a time. A CTA
// takes `heads_per_cta` heads of one token (q, then k, then v): all of them for a prompt, where the
// token's indices, page, weights and angles are then looked up once for 32 heads; a warp's worth for a
// decode step, so that its few tokens still spread over the SMs. Everything but the rows themselves (the step's index
// arrays, the page table, the norms' weights, the angles) was written by kernels further back than the one
// just before this, and is read before pdl_wait().
template <int HD> __global__ void __launch_bounds__(FAST_WARPS * 32) qkv_prep_fast_kernel(QkvPrep p, int heads_per_cta) {
    constexpr int LPH = HD / 8, HPW = 32 / LPH;  // lanes per head, heads per warp
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / LPH, l = lane % LPH;  // which of the warp's heads, and which 8 elements of it
    const bool upper = l >= LPH / 2;             // the elements that pair with those HD / 2 below them
    const int total_heads = p.n_heads + 2 * p.n_kv_heads;
    const int n_work = p.q_only ? p.n_heads : total_heads;
    const int base = blockIdx.y * heads_per_cta, limit = min(base + heads_per_cta, n_work);
    // A warp issues its instructions in order and stops at the first whose operand is still on its way, so the
    // order of the loads is the depth of the chain: sequence and position together; then, with them, the angles,
    // the slot and the length; then the rows (they need none of these); the page, which needs the slot, last.
    const int seq = p.token_seq[t], pos = p.token_pos[t];
    if (seq < 0) return;
    float cs[8], sn[8];
    const int at = (upper ? l - LPH / 2 : l) * 8;  // of this lane's elements among the HD / 2 angles
    float4 c0, c1, s0, s1;
    if (p.cos) {
        const float4 *c4 = (const float4 *)(p.cos + (long long)pos * (HD / 2) + at), *s4 = (const float4 *)(p.sin + (long long)pos * (HD / 2) + at);
        c0 = c4[0], c1 = c4[1], s0 = s4[0], s1 = s4[1];
    }
    const bool caching = !p.q_only && p.k_pool;
    const int slot = caching ? p.seq_slot[seq] : 0, len_after = caching ? p.seq_len_after[seq] : 0;
    if (p.q_norm) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.q_norm + l * 8));  // read where they are used: few registers,
    if (p.k_norm) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.k_norm + l * 8));  // so that more warps fit an SM
    __nv_bfloat16 *row0 = (__nv_bfloat16 *)p.qkv + (long long)t * total_heads * HD + l * 8;
    pdl_wait();
    long long kept_at = -1;  // where the token's keys and values go in the pools (kv head 0), if they are kept
    bool first_round = true;
    for (int h0 = base + warp * HPW + sub; h0 - sub < limit; h0 += FAST_WARPS * HPW * FAST_SLOTS) {
        uint4 raw[FAST_SLOTS];
#pragma unroll
        for (int u = 0; u < FAST_SLOTS; u++) {
            const int head = h0 + u * FAST_WARPS * HPW;
            raw[u] = head < limit ? *(const uint4 *)(row0 + (long long)head * HD) : make_uint4(0, 0, 0, 0);
        }
        if (first_round) {  // (after the rows are on their way)
            first_round = false;
            if (caching && !(p.cache.ring_pages > 0 && pos + p.cache.ring_pages * p.cache.tokens_per_page <= len_after - 1))
                kept_at = cache_offset(p.cache, cache_page(p.cache, slot, pos), 0, p.n_kv_heads, pos, HD);
            if (p.cos) {
                cs[0] = c0.x, cs[1] = c0.y, cs[2] = c0.z, cs[3] = c0.w, cs[4] = c1.x, cs[5] = c1.y, cs[6] = c1.z, cs[7] = c1.w;
                sn[0] = s0.x, sn[1] = s0.y, sn[2] = s0.z, sn[3] = s0.w, sn[4] = s1.x, sn[5] = s1.y, sn[6] = s1.z, sn[7] = s1.w;
            }
        }
#pragma unroll
        for (int u = 0; u < FAST_SLOTS; u++) {
            const int head = h0 + u * FAST_WARPS * HPW;
            if (head - sub >= limit) break;  // the whole warp is past the end (the shuffles below are for whole warps)
            prep_head<HD>(p, raw[u], head, head < limit, l, upper, cs, sn, row0, kept_at);
        }
    }
}

// The same for the many tokens of a prompt. One token to a CTA gives more CTAs than the GPU holds at a time, and
// every wave of them walks the chain token -> sequence -> slot -> page -> rows anew. Here a CTA takes PROMPT_TOKENS
// tokens in a row: it looks up the indices, pages and angles of all of them at once, before pdl_wait() (they are
// written by kernels further back than the one just before), and then streams the rows, loading the next
// token's while it works on this one's, so that all the CTAs of a prompt of a few thousand tokens are resident
// together and the chain is walked once.
#define PROMPT_TOKENS 4
template <int HD> __global__ void __launch_bounds__(FAST_WARPS * 32) qkv_prep_prompt_kernel(QkvPrep p, int n_tokens) {
    constexpr int LPH = HD / 8, HPW = 32 / LPH, ROUND = FAST_WARPS * HPW * FAST_SLOTS;  // heads of a token a CTA has in flight
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / LPH, l = lane % LPH;
    const bool upper = l >= LPH / 2;
    const int total_heads = p.n_heads + 2 * p.n_kv_heads;
    const int limit = p.q_only ? p.n_heads : total_heads;
    const int rounds = (limit + ROUND - 1) / ROUND;
    const int t0 = blockIdx.x * PROMPT_TOKENS;
    const int at = (upper ? l - LPH / 2 : l) * 8;
    const bool caching = !p.q_only && p.k_pool;
    int seq[PROMPT_TOKENS], pos[PROMPT_TOKENS], slot[PROMPT_TOKENS], len_after[PROMPT_TOKENS];
    long long kept[PROMPT_TOKENS];
#pragma unroll
    for (int i = 0; i < PROMPT_TOKENS; i++) {
        const bool in = t0 + i < n_tokens;
        seq[i] = in ? p.token_seq[t0 + i] : -1, pos[i] = in ? p.token_pos[t0 + i] : 0;
    }
#pragma unroll
    for (int i = 0; i < PROMPT_TOKENS; i++) {
        const bool on = seq[i] >= 0;
        slot[i] = caching && on ? p.seq_slot[seq[i]] : 0, len_after[i] = caching && on ? p.seq_len_after[seq[i]] : 0;
        if (on && p.cos && threadIdx.x < HD / 64) {  // the token's angles, HD / 2 float32 of each kind, into the L1
            asm volatile("prefetch.global.L1 [%0];" ::"l"(p.cos + (long long)pos[i] * (HD / 2) + 32 * threadIdx.x));
            asm volatile("prefetch.global.L1 [%0];" ::"l"(p.sin + (long long)pos[i] * (HD / 2) + 32 * threadIdx.x));
        }
    }
#pragma unroll
    for (int i = 0; i < PROMPT_TOKENS; i++) {
        kept[i] = -1;
        if (caching && seq[i] >= 0 &&
            !(p.cache.ring_pages > 0 && pos[i] + p.cache.ring_pages * p.cache.tokens_per_page <= len_after[i] - 1))
            kept[i] = cache_offset(p.cache, cache_page(p.cache, slot[i], pos[i]), 0, p.n_kv_heads, pos[i], HD);
    }
    auto load_rows = [&](bool on, int i, int round, uint4 *raw) {
        const __nv_bfloat16 *row0 = (const __nv_bfloat16 *)p.qkv + (long long)(t0 + i) * total_heads * HD + l * 8;
#pragma unroll
        for (int u = 0; u < FAST_SLOTS; u++) {
            const int head = round * ROUND + warp * HPW + sub + u * FAST_WARPS * HPW;
            raw[u] = on && head < limit ? *(const uint4 *)(row0 + (long long)head * HD) : make_uint4(0, 0, 0, 0);
        }
    };
    pdl_wait();
    uint4 cur[FAST_SLOTS], next[FAST_SLOTS];
    load_rows(seq[0] >= 0, 0, 0, cur);
#pragma unroll
    for (int i = 0; i < PROMPT_TOKENS; i++) {
        float cs[8], sn[8];
        if (p.cos && seq[i] >= 0) {
            const float4 *c4 = (const float4 *)(p.cos + (long long)pos[i] * (HD / 2) + at), *s4 = (const float4 *)(p.sin + (long long)pos[i] * (HD / 2) + at);
            const float4 c0 = c4[0], c1 = c4[1], s0 = s4[0], s1 = s4[1];
            cs[0] = c0.x, cs[1] = c0.y, cs[2] = c0.z, cs[3] = c0.w, cs[4] = c1.x, cs[5] = c1.y, cs[6] = c1.z, cs[7] = c1.w;
            sn[0] = s0.x, sn[1] = s0.y, sn[2] = s0.z, sn[3] = s0.w, sn[4] = s1.x, sn[5] = s1.y, sn[6] = s1.z, sn[7] = s1.w;
        }
        __nv_bfloat16 *row0 = (__nv_bfloat16 *)p.qkv + (long long)(t0 + i) * total_heads * HD + l * 8;
        for (int round = 0; round < rounds; round++) {
            if (round + 1 < rounds) load_rows(seq[i] >= 0, i, round + 1, next);
            else if (i + 1 < PROMPT_TOKENS) load_rows(seq[i + 1 < PROMPT_TOKENS ? i + 1 : i] >= 0, i + 1, 0, next);
            if (seq[i] >= 0) {  // (the same for the whole CTA)
#pragma unroll
                for (int u = 0; u < FAST_SLOTS; u++) {
                    const int head = round * ROUND + warp * HPW + sub + u * FAST_WARPS * HPW;
                    if (head - sub >= limit) break;  // the whole warp is past the end (the shuffles are for whole warps)
                    prep_head<HD>(p, cur[u], head, head < limit, l, upper, cs, sn, row0, kept[i]);
                }
            }
#pragma unroll
            for (int u = 0; u < FAST_SLOTS; u++) cur[u] = next[u];
        }
    }
}

extern "C" int abk_qkv_prep(void *qkv, int dtype, int n_tokens, int n_heads, int n_kv_heads, int head_dim, int q_only,
                            const int *token_seq, const int *token_pos, const int *seq_slot, const int *seq_len_after,
                            const float *q_norm, const float *k_norm, float eps, const float *cos, const float *sin,
                            int rotary_dim, int interleaved, void *k_pool, void *v_pool, const int *page_table,
                            int table_width, int ring_pages, int tokens_per_page, void *stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim > MAX_HEAD_DIM || head_dim < 2 || head_dim % 2)
        ABK_REFUSE("qkv_prep: head_dim %d is not an even number up to %d", head_dim, MAX_HEAD_DIM);
    if (cos && (rotary_dim < 2 || rotary_dim % 2 || rotary_dim > head_dim))
        ABK_REFUSE("qkv_prep: rotary_dim %d does not fit head_dim %d", rotary_dim, head_dim);
    QkvPrep p;
    p.qkv = qkv, p.n_heads = n_heads, p.n_kv_heads = n_kv_heads, p.head_dim = head_dim, p.q_only = q_only;
    p.token_seq = token_seq, p.token_pos = token_pos, p.seq_slot = seq_slot, p.seq_len_after = seq_len_after;
    p.q_norm = q_norm, p.k_norm = k_norm, p.eps = eps, p.cos = cos, p.sin = sin;
    p.rotary_dim = rotary_dim, p.interleaved = interleaved, p.k_pool = k_pool, p.v_pool = v_pool;
    p.cache.page_table = page_table, p.cache.table_width = table_width, p.cache.ring_pages = ring_pages;
    p.cache.tokens_per_page = tokens_per_page;
    int total_heads = n_heads + 2 * n_kv_heads;
    dim3 grid(n_tokens, (total_heads + PREP_WARPS - 1) / PREP_WARPS);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ABK_BF16 && (head_dim == 64 || head_dim == 128 || head_dim == 256) &&
        (!cos || (rotary_dim == head_dim && !interleaved)) &&
        ((uintptr_t)qkv | (uintptr_t)cos | (uintptr_t)sin | (uintptr_t)q_norm | (uintptr_t)k_norm | (uintptr_t)k_pool |
         (uintptr_t)v_pool) % 16 == 0) {
        // prompts: a token's heads in one CTA; a decode step of few tokens: one round of its warps' heads to a CTA
        const int work = q_only ? n_heads : total_heads;
        if (n_tokens > 6 * abk_sm_count()) {  // more one-token CTAs than are resident at a time
            dim3 many((unsigned)((n_tokens + PROMPT_TOKENS - 1) / PROMPT_TOKENS));
            if (head_dim == 64) abk_launch(qkv_prep_prompt_kernel<64>, many, dim3(FAST_WARPS * 32), 0, s, p, n_tokens);
            else if (head_dim == 128) abk_launch(qkv_prep_prompt_kernel<128>, many, dim3(FAST_WARPS * 32), 0, s, p, n_tokens);
            else abk_launch(qkv_prep_prompt_kernel<256>, many, dim3(FAST_WARPS * 32), 0, s, p, n_tokens);
            return ABK_LAUNCH_RESULT();
        }
        const int per_cta = n_tokens >= 64 ? work : FAST_WARPS * (256 / head_dim);
        dim3 fast((unsigned)n_tokens, (unsigned)((work + per_cta - 1) / per_cta));
        if (head_dim == 64) abk_launch(qkv_prep_fast_kernel<64>, fast, dim3(FAST_WARPS * 32), 0, s, p, per_cta);
        else if (head_dim == 128) abk_launch(qkv_prep_fast_kernel<128>, fast, dim3(FAST_WARPS * 32), 0, s, p, per_cta);
        else abk_launch(qkv_prep_fast_kernel<256>, fast, dim3(FAST_WARPS * 32), 0, s, p, per_cta);
        return ABK_LAUNCH_RESULT();
    }
    if (dtype == ABK_BF16)
        abk_launch(qkv_prep_kernel<__nv_bfloat16>, grid, dim3(PREP_WARPS * 32), 0, s, p);
    else
        abk_launch(qkv_prep_kernel<float>, grid, dim3(PREP_WARPS * 32), 0, s, p);
    return ABK_LAUNCH_RESULT();
}

// ------------------------------------------------------------------ next decode step
// Moves a decode step one position on without the host: every real row's position, and every
// sequence's start and length, go up by one.
__global__ void advance_decode_kernel(const int *token_seq, int *token_pos, int n_rows, int *seq_pos0,
                                      int *seq_len_after, int n_seqs) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_rows && token_seq[i] >= 0) token_pos[i] += 1;
    if (i < n_seqs) seq_pos0[i] += 1, seq_len_after[i] += 1;
}

extern "C" int abk_advance_decode(const int *token_seq, int *token_pos, int n_rows, int *seq_pos0, int *seq_len_after,
                                  int n_seqs, void *stream) {
    int n = n_rows > n_seqs ? n_rows : n_seqs;
    if (n <= 0) return 0;
    advance_decode_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>(token_seq, token_pos, n_rows, seq_pos0,
                                                                            seq_len_after, n_seqs);
    return ABK_LAUNCH_RESULT();
}


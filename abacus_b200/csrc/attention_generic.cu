// Causal grouped-query attention over the paged cache, for any head size up to 256 that is a
// multiple of 8, any number of heads and groups, with or without a window. One block per
// (token, query head); float32 arithmetic with an online softmax over tiles of 128 keys (in the
// bfloat16 instantiation the probabilities are rounded to bfloat16 for the second product, as in
// the tensor-core kernels, and summed unrounded).
// It serves prefill and decode alike and is the kernel every size falls back to; the float32
// path of the model uses nothing else for attention.
//
// Formula (src/model.c:197-211): s_j = (q . k_j) * scale for the keys the token may see,
// p = softmax(s), out = sum_j p_j v_j; query head h reads kv head h / (Hq / Hkv).
// The result for a token depends only on its own position and keys: tiles start at the first
// visible key, never at a batch-dependent place.
#define ABK_DEFINE_ERROR
#include "common.cuh"

#define ATT_THREADS 128
#define ATT_MAX_HEAD_DIM 256

struct AttnGeneric {
    const void *q;      // row t, head h at q + (t * q_row + h * head_dim)
    long long q_row;    // elements between rows of q
    void *out;          // [tokens, n_heads * head_dim]
    int n_heads, n_kv_heads, head_dim;
    float scale;
    int window;         // 0: all earlier keys
    const int *token_seq, *token_pos, *seq_slot, *seq_start, *seq_pos0;
    // keys and values either in the paged cache ...
    const void *k_pool, *v_pool;
    PagedCache cache;
    // ... or in the rows of this step (k_step null: use the cache): position j of sequence s is
    // row seq_start[s] + j - seq_pos0[s]
    const void *k_step, *v_step;
    long long kv_row;   // elements between rows of k_step / v_step
};

template <typename T> __device__ __forceinline__ float dot_row(const float *q, const T *k, int hd);
template <> __device__ __forceinline__ float dot_row<float>(const float *q, const float *k, int hd) {
    float acc = 0.0f;
    for (int i = 0; i < hd; i += 4) {
        float4 v = *(const float4 *)(k + i);
        acc = fmaf(q[i], v.x, acc), acc = fmaf(q[i + 1], v.y, acc);
        acc = fmaf(q[i + 2], v.z, acc), acc = fmaf(q[i + 3], v.w, acc);
    }
    return acc;
}
template <> __device__ __forceinline__ float dot_row<__nv_bfloat16>(const float *q, const __nv_bfloat16 *k, int hd) {
    float acc = 0.0f;
    for (int i = 0; i < hd; i += 8) {
        uint4 raw = *(const uint4 *)(k + i);
        const __nv_bfloat162 *h = (const __nv_bfloat162 *)&raw;
#pragma unroll
        for (int u = 0; u < 4; u++) {
            float2 f = __bfloat1622float2(h[u]);
            acc = fmaf(q[i + 2 * u], f.x, acc), acc = fmaf(q[i + 2 * u + 1], f.y, acc);
        }
    }
    return acc;
}

template <typename T> __global__ void __launch_bounds__(ATT_THREADS) attention_generic_kernel(AttnGeneric p) {
    __shared__ float q_s[ATT_MAX_HEAD_DIM];
    __shared__ float p_s[ATT_THREADS];
    __shared__ long long v_off[ATT_THREADS];
    __shared__ float scratch[33];
    constexpr bool ROUNDED_P = sizeof(T) == 2;  // bfloat16: the probabilities are a stored tensor too
    int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, hd = p.head_dim;
    int seq = p.token_seq[t];
    T *out = (T *)p.out + ((long long)t * p.n_heads + h) * hd;
    if (seq < 0) {  // padding
        for (int d = tid; d < hd; d += ATT_THREADS) out[d] = from_float<T>(0.0f);
        return;
    }
    int pos = p.token_pos[t], slot = p.seq_slot[seq];
    int kvh = h / (p.n_heads / p.n_kv_heads);
    int lo = p.window > 0 && pos - p.window + 1 > 0 ? pos - p.window + 1 : 0;
    const T *q = (const T *)p.q + (long long)t * p.q_row + (long long)h * hd;
    for (int d = tid; d < hd; d += ATT_THREADS) q_s[d] = to_float(q[d]);
    __syncthreads();

    float m = -INFINITY, l = 0.0f, acc0 = 0.0f, acc1 = 0.0f;
    for (int base = lo; base <= pos; base += ATT_THREADS) {
        int j = base + tid;
        bool valid = j <= pos;
        float s = -INFINITY;
        if (valid) {
            const T *k;
            long long vo;
            if (p.k_step) {
                long long row = (long long)p.seq_start[seq] + j - p.seq_pos0[seq];
                vo = row * p.kv_row + (long long)kvh * hd;
                k = (const T *)p.k_step + vo;
            } else {
                int page = cache_page(p.cache, slot, j);
                vo = cache_offset(p.cache, page, kvh, p.n_kv_heads, j, hd);
                k = (const T *)p.k_pool + vo;
            }
            v_off[tid] = vo;
            s = dot_row<T>(q_s, k, hd) * (ROUNDED_P ? p.scale * 1.4426950408889634f : p.scale);
        }
        float m_new, pj, corr;
        if (ROUNDED_P) {
            // in units of log2, against the maximum rounded up to a whole number: a probability is then the same
            // bits times a power of two whatever tile it is in, and rounds to the same bfloat16 in every kernel
            m_new = fmaxf(m, ceilf(block_max(s, scratch)));
            pj = valid ? exp2f(s - m_new) : 0.0f;
            corr = exp2f(m - m_new);  // 0 on the first tile (m = -inf)
        } else {
            m_new = fmaxf(m, block_max(s, scratch));
            pj = valid ? expf(s - m_new) : 0.0f;
            corr = expf(m - m_new);
        }
        // the probabilities of the second product are a stored tensor: bfloat16 where the model's are (the
        // tensor-core kernels must round them, so every kernel does); the row's sum is of the unrounded ones
        p_s[tid] = to_float(from_float<T>(pj));
        l = l * corr + block_sum(pj, scratch);  // the barrier inside also publishes p_s and v_off
        m = m_new;
        int n_valid = pos - base + 1 < ATT_THREADS ? pos - base + 1 : ATT_THREADS;
        const T *v_base = (const T *)(p.k_step ? p.v_step : p.v_pool);
        acc0 *= corr, acc1 *= corr;
        if (tid < hd) {
            for (int jj = 0; jj < n_valid; jj++) {
                const T *v = v_base + v_off[jj];
                acc0 = fmaf(p_s[jj], to_float(v[tid]), acc0);
                if (tid + ATT_THREADS < hd) acc1 = fmaf(p_s[jj], to_float(v[tid + ATT_THREADS]), acc1);
            }
        }
        __syncthreads();  // p_s and v_off are rewritten by the next tile
    }
    if (tid < hd) out[tid] = from_float<T>(acc0 / l);
    if (tid + ATT_THREADS < hd) out[tid + ATT_THREADS] = from_float<T>(acc1 / l);
}

extern "C" int abk_attention_generic(const void *q, long long q_row, void *out, int dtype, int n_tokens, int n_heads,
                                     int n_kv_heads, int head_dim, float scale, int window, const int *token_seq,
                                     const int *token_pos, const int *seq_slot, const int *seq_start,
                                     const int *seq_pos0, const void *k_pool, const void *v_pool,
                                     const int *page_table, int table_width, int ring_pages, int tokens_per_page,
                                     const void *k_step, const void *v_step, long long kv_row, void *stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim > ATT_MAX_HEAD_DIM || head_dim % 8 || head_dim < 8)
        ABK_REFUSE("attention: head_dim %d is not a multiple of 8 up to %d", head_dim, ATT_MAX_HEAD_DIM);
    if (n_kv_heads < 1 || n_heads % n_kv_heads)
        ABK_REFUSE("attention: %d query heads do not divide into %d kv heads", n_heads, n_kv_heads);
    if (n_heads > 65535) ABK_REFUSE("attention: %d heads are more than a grid takes", n_heads);
    AttnGeneric p;
    p.q = q, p.q_row = q_row, p.out = out, p.n_heads = n_heads, p.n_kv_heads = n_kv_heads, p.head_dim = head_dim;
    p.scale = scale, p.window = window, p.token_seq = token_seq, p.token_pos = token_pos, p.seq_slot = seq_slot;
    p.seq_start = seq_start, p.seq_pos0 = seq_pos0, p.k_pool = k_pool, p.v_pool = v_pool;
    p.cache.page_table = page_table, p.cache.table_width = table_width, p.cache.ring_pages = ring_pages;
    p.cache.tokens_per_page = tokens_per_page;
    p.k_step = k_step, p.v_step = v_step, p.kv_row = kv_row;
    dim3 grid(n_tokens, n_heads);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ABK_BF16)
        attention_generic_kernel<__nv_bfloat16><<<grid, ATT_THREADS, 0, s>>>(p);
    else
        attention_generic_kernel<float><<<grid, ATT_THREADS, 0, s>>>(p);
    return ABK_LAUNCH_RESULT();
}

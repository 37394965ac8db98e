// Choosing the next token from float32 logits: the first maximum, or a draw from the
// highest-k logits at a temperature (src/main.c:31-56). A row is cut into slices, one block each.
#define ABK_DEFINE_ERROR
#include "common.cuh"

#define SAMPLE_MAX_K 64

struct Best {
    float v;
    int i;
};
// Order of src/main.c:31-36 and :43-48: larger logit first, earlier index first among equals.
__device__ __forceinline__ bool before(Best a, Best b) { return a.v > b.v || (a.v == b.v && a.i < b.i); }

__device__ __forceinline__ Best block_best(Best b, Best *scratch) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other;
        other.v = __shfl_xor_sync(0xffffffffu, b.v, o);
        other.i = __shfl_xor_sync(0xffffffffu, b.i, o);
        if (before(other, b)) b = other;
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = b;
    __syncthreads();
    if (warp == 0) {
        Best t;
        t.v = -INFINITY, t.i = 0x7fffffff;
        if (lane < n_warps) t = scratch[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best other;
            other.v = __shfl_xor_sync(0xffffffffu, t.v, o);
            other.i = __shfl_xor_sync(0xffffffffu, t.i, o);
            if (before(other, t)) t = other;
        }
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// The row is cut into gridDim.x slices, one block each; the last block of a row to finish (a ticket
// in `tickets`, left at zero) picks the best of the slices. `before` is a total order, so the result
// does not depend on which block came last.
#define ARGMAX_SLICES 32
#define ARGMAX_THREADS 256
__global__ void __launch_bounds__(ARGMAX_THREADS) argmax_kernel(const float *__restrict__ logits, long long row_stride,
                                                                int vocab, int *__restrict__ out, Best *part,
                                                                int *tickets) {
    __shared__ Best scratch[33];
    __shared__ int ticket;
    pdl_wait();
    const int row = blockIdx.y, slices = gridDim.x;
    const int per = (vocab + slices - 1) / slices, lo = blockIdx.x * per, hi = min(vocab, lo + per);
    const float *x = logits + (long long)row * row_stride;
    Best b;
    b.v = -INFINITY, b.i = 0x7fffffff;
    for (int j = lo + threadIdx.x; j < hi; j += blockDim.x) {
        Best c;
        c.v = x[j], c.i = j;
        if (before(c, b)) b = c;
    }
    b = block_best(b, scratch);
    if (threadIdx.x == 0) {
        part[(long long)row * slices + blockIdx.x] = b;
        __threadfence();
        ticket = atomicAdd(&tickets[row], 1);
    }
    __syncthreads();
    if (ticket != slices - 1) return;
    __threadfence();
    Best t;
    t.v = -INFINITY, t.i = 0x7fffffff;
    if (threadIdx.x < slices) {
        const volatile Best *q = part + (long long)row * slices + threadIdx.x;
        t.v = q->v, t.i = q->i;
    }
    t = block_best(t, scratch);
    if (threadIdx.x == 0) out[row] = t.i, tickets[row] = 0;
}

// Draw from the top_k logits at temperature temp: p_j = exp((l_j - l_top) / temp), the random
// number is one xorshift64 step of the row's state (src/main.c:49-55). The state is advanced.
//
// The row is cut into TOPK_SLICES slices, one block each. A block finds the top_k of its slice in two
// passes: the warps' ceil(top_k / warps)-th largest thread maxima give a value that at least top_k
// elements of the slice reach, so everything from that value up (some tens of elements) goes into
// shared memory, and one warp picks the top_k of those in the order of src/main.c:43-48. The last
// block of a row to finish (a ticket, left at zero) picks the top_k of the slices' and draws. `before`
// is a total order, so nothing depends on the order in which candidates or blocks come.
#define TOPK_SLICES 32
#define TOPK_THREADS 256
#define TOPK_CANDIDATES 1024

// The k best of cand[0..n) in order, by one warp; what is picked is taken out (its value set to -inf, index to max).
__device__ __forceinline__ void warp_pick(Best *cand, int n, int k, Best *picked, int lane) {
    for (int r = 0; r < k; r++) {
        Best b;
        b.v = -INFINITY, b.i = 0x7fffffff;
        int at = -1;
        for (int j = lane; j < n; j += 32)
            if (before(cand[j], b)) b = cand[j], at = j;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best other;
            other.v = __shfl_xor_sync(0xffffffffu, b.v, o), other.i = __shfl_xor_sync(0xffffffffu, b.i, o);
            int other_at = __shfl_xor_sync(0xffffffffu, at, o);
            if (before(other, b)) b = other, at = other_at;
        }
        if (lane == 0) {
            picked[r] = b;
            if (at >= 0) cand[at].v = -INFINITY, cand[at].i = 0x7fffffff;
        }
        __syncwarp();
    }
}

__global__ void __launch_bounds__(TOPK_THREADS) sample_topk_kernel(const float *__restrict__ logits, long long row_stride,
                                                                   int vocab, float temp, int top_k,
                                                                   unsigned long long *rng, const int *__restrict__ rng_index,
                                                                   int *__restrict__ out, Best *part, int *tickets) {
    __shared__ Best cand[TOPK_CANDIDATES + SAMPLE_MAX_K];  // (the last block's second half carries the first half's best along)
    __shared__ Best picked[SAMPLE_MAX_K];
    __shared__ Best scratch[33];
    __shared__ float warp_bound[TOPK_THREADS / 32];
    __shared__ int count, ticket;
    pdl_wait();
    const int row = blockIdx.y, slices = gridDim.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int per = (vocab + slices - 1) / slices, lo = min(vocab, blockIdx.x * per), hi = min(vocab, lo + per);
    const float *x = logits + (long long)row * row_stride;
    const int k = min(top_k, vocab);
    if (threadIdx.x == 0) count = 0;
    float bound = -INFINITY;
    if (hi - lo > TOPK_CANDIDATES) {
        float tmax = -INFINITY;
        for (int j = lo + threadIdx.x; j < hi; j += TOPK_THREADS) tmax = fmaxf(tmax, x[j]);
        // this warp's ceil(k / warps)-th largest thread maximum
        const int rounds = (k + TOPK_THREADS / 32 - 1) / (TOPK_THREADS / 32);
        float v = tmax, m = -INFINITY;
        for (int r = 0; r < rounds; r++) {
            m = warp_max(v);
            unsigned holders = __ballot_sync(0xffffffffu, v == m);
            if (lane == __ffs(holders) - 1) v = -INFINITY;  // one of them is taken out
        }
        if (lane == 0) warp_bound[warp] = m;
        __syncthreads();
        bound = warp_bound[0];
        for (int w = 1; w < TOPK_THREADS / 32; w++) bound = fminf(bound, warp_bound[w]);
    } else {
        __syncthreads();
    }
    for (int j = lo + threadIdx.x; j < hi; j += TOPK_THREADS) {
        const float v = x[j];
        if (v >= bound) {
            const int at = atomicAdd(&count, 1);
            if (at < TOPK_CANDIDATES) cand[at].v = v, cand[at].i = j;
        }
    }
    __syncthreads();
    Best *mine = part + ((long long)row * slices + blockIdx.x) * SAMPLE_MAX_K;
    if (count <= TOPK_CANDIDATES) {
        if (warp == 0) {
            warp_pick(cand, count, k, picked, lane);
            for (int r = lane; r < k; r += 32) mine[r] = picked[r];
        }
    } else {  // (many equal logits at the top: more candidates than there is room for) one at a time, from the slice itself
        Best prev;
        prev.v = 0.0f, prev.i = -1;
        for (int r = 0; r < k; r++) {
            Best b;
            b.v = -INFINITY, b.i = 0x7fffffff;
            for (int j = lo + threadIdx.x; j < hi; j += TOPK_THREADS) {
                Best c;
                c.v = x[j], c.i = j;
                if (prev.i >= 0 && !before(prev, c)) continue;
                if (before(c, b)) b = c;
            }
            prev = block_best(b, scratch);
            if (threadIdx.x == 0) mine[r] = prev;
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) ticket = atomicAdd(&tickets[row], 1);
    __syncthreads();
    if (ticket != slices - 1) return;
    __threadfence();
    // the last block of the row: the best k of the slices' best k
    const int n = slices * k;  // at most 32 * 64
    Best *all = cand;          // TOPK_CANDIDATES holds 32 x 32; more go through in two halves below
    if (n <= TOPK_CANDIDATES) {
        for (int j = threadIdx.x; j < n; j += TOPK_THREADS) {
            const volatile Best *q = part + ((long long)row * slices + j / k) * SAMPLE_MAX_K + j % k;
            all[j].v = q->v, all[j].i = q->i;
        }
        __syncthreads();
        if (warp == 0) warp_pick(all, n, k, picked, lane);
    } else {
        // first the lower half of the slices, then its k best together with the upper half
        const int half = slices / 2 * k;
        for (int j = threadIdx.x; j < half; j += TOPK_THREADS) {
            const volatile Best *q = part + ((long long)row * slices + j / k) * SAMPLE_MAX_K + j % k;
            all[j].v = q->v, all[j].i = q->i;
        }
        __syncthreads();
        if (warp == 0) warp_pick(all, half, k, picked, lane);
        __syncthreads();
        for (int j = threadIdx.x; j < n - half; j += TOPK_THREADS) {
            const volatile Best *q = part + ((long long)row * slices + (half + j) / k) * SAMPLE_MAX_K + (half + j) % k;
            all[j].v = q->v, all[j].i = q->i;
        }
        for (int j = threadIdx.x; j < k; j += TOPK_THREADS) all[n - half + j] = picked[j];
        __syncthreads();
        if (warp == 0) warp_pick(all, n - half + k, k, picked, lane);
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    tickets[row] = 0;
    float p[SAMPLE_MAX_K], sum = 0.0f;
    for (int j = 0; j < k; j++) sum += p[j] = expf((picked[j].v - picked[0].v) / temp);
    int which = rng_index ? rng_index[row] : row;  // e.g. the row's cache slot
    unsigned long long s = rng[which];
    s ^= s << 13, s ^= s >> 7, s ^= s << 17;
    rng[which] = s;
    float r = (float)(s >> 40) / (float)(1 << 24) * sum;
    int chosen = picked[k - 1].i;
    for (int j = 0; j < k; j++)
        if ((r -= p[j]) <= 0.0f) {
            chosen = picked[j].i;
            break;
        }
    out[row] = chosen;
}

extern "C" int abk_argmax_slices() { return ARGMAX_SLICES; }
extern "C" int abk_argmax(const float *logits, long long row_stride, int n_rows, int vocab, int *out, void *scratch,
                          int *tickets, void *stream) {
    if (n_rows <= 0) return 0;
    if (vocab < 1) ABK_REFUSE("argmax: vocabulary of %d", vocab);
    if (n_rows > 65535) ABK_REFUSE("argmax: %d rows are more than one launch takes", n_rows);
    int slices = vocab >= 8192 ? ARGMAX_SLICES : 1;
    abk_launch(argmax_kernel, dim3(slices, n_rows), dim3(ARGMAX_THREADS), 0, (cudaStream_t)stream, logits, row_stride,
               vocab, out, (Best *)scratch, tickets);
    return ABK_LAUNCH_RESULT();
}

// scratch: room for abk_sample_topk_scratch_bytes(n_rows) bytes; tickets: int32 [n_rows], zero before and after.
extern "C" long long abk_sample_topk_scratch_bytes(int n_rows) { return (long long)n_rows * TOPK_SLICES * SAMPLE_MAX_K * sizeof(Best); }
extern "C" int abk_sample_topk(const float *logits, long long row_stride, int n_rows, int vocab, float temp, int top_k,
                               unsigned long long *rng, const int *rng_index, int *out, void *scratch, int *tickets,
                               void *stream) {
    if (n_rows <= 0) return 0;
    if (vocab < 1) ABK_REFUSE("sample: vocabulary of %d", vocab);
    if (top_k < 1 || top_k > SAMPLE_MAX_K) ABK_REFUSE("sample: top_k %d is not in 1..%d", top_k, SAMPLE_MAX_K);
    if (!(temp > 0.0f)) ABK_REFUSE("sample: temperature %g is not positive (use argmax)", temp);
    if (n_rows > 65535) ABK_REFUSE("sample: %d rows exceed a grid", n_rows);
    int slices = TOPK_SLICES;
    while (slices > 1 && (vocab + slices - 1) / slices < TOPK_THREADS) slices >>= 1;  // a small vocabulary: fewer slices
    abk_launch(sample_topk_kernel, dim3(slices, n_rows), dim3(TOPK_THREADS), 0, (cudaStream_t)stream, logits, row_stride, vocab,
               temp, top_k, rng, rng_index, out, (Best *)scratch, tickets);
    return ABK_LAUNCH_RESULT();
}

// ---------------------------------------------------------------------------------------------------------------
// A draw from the whole vocabulary at a temperature (top_k = 0). abacus always cuts to the 20 most likely tokens
// (src/main.c:41); without the cut there is no short list to sort, so the tokens are walked in index order instead of
// by falling logit. The distribution is the same, p_j = exp((l_j - l_max) / temperature) over all j, and so is the
// generator (xorshift64, src/main.c:52): r = u24 / 2^24 * sum, the token is the first j whose running sum reaches r.
// Sums are float64 over float32 terms, so the grouping of the additions cannot move a boundary.
//   sample_all_sums_kernel: a block adds up p_j over its ALL_BLOCK logits.
//   sample_all_draw_kernel: one block a row: running sums of the blocks in order, the block r falls into, the walk in it.
#define ALL_BLOCK 1024
#define ALL_THREADS 256
#define ALL_MAX_BLOCKS 1024

__global__ void __launch_bounds__(ALL_THREADS) sample_all_sums_kernel(const float *__restrict__ logits, long long row_stride,
                                                                      int vocab, float inv_temp, const int *__restrict__ top,
                                                                      double *__restrict__ sums) {
    __shared__ double warp_sum_s[ALL_THREADS / 32];
    pdl_wait();
    const int row = blockIdx.y, lo = blockIdx.x * ALL_BLOCK, hi = min(vocab, lo + ALL_BLOCK);
    const float *x = logits + (long long)row * row_stride;
    const float m = x[top[row]];
    double acc = 0.0;
    for (int j = lo + threadIdx.x; j < hi; j += ALL_THREADS) acc += (double)expf((x[j] - m) * inv_temp);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) warp_sum_s[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < ALL_THREADS / 32; w++) t += warp_sum_s[w];
        sums[(long long)row * gridDim.x + blockIdx.x] = t;
    }
}

__global__ void __launch_bounds__(ALL_THREADS) sample_all_draw_kernel(const float *__restrict__ logits, long long row_stride,
                                                                      int vocab, float inv_temp, const int *__restrict__ top,
                                                                      const double *__restrict__ sums, int n_blocks,
                                                                      unsigned long long *rng, const int *rng_index,
                                                                      int *__restrict__ out) {
    __shared__ double before_block[ALL_MAX_BLOCKS + 1];  // running sum of the blocks before block b
    __shared__ float p_s[ALL_BLOCK];
    __shared__ int block_of_r;
    __shared__ double r_s;
    pdl_wait();
    const int row = blockIdx.x;
    const float *x = logits + (long long)row * row_stride;
    const float m = x[top[row]];
    if (threadIdx.x == 0) {
        double run = 0.0;
        for (int b = 0; b < n_blocks; b++) {
            before_block[b] = run;
            run += sums[(long long)row * n_blocks + b];
        }
        before_block[n_blocks] = run;
        const int which = rng_index ? rng_index[row] : row;
        unsigned long long s = rng[which];
        s ^= s << 13, s ^= s >> 7, s ^= s << 17;
        rng[which] = s;
        const double r = (double)(s >> 40) / (double)(1 << 24) * run;
        int b = 0;
        while (b + 1 < n_blocks && before_block[b + 1] < r) b++;  // the first block whose running sum reaches r
        block_of_r = b, r_s = r;
    }
    __syncthreads();
    const int lo = block_of_r * ALL_BLOCK, hi = min(vocab, lo + ALL_BLOCK);
    for (int j = lo + threadIdx.x; j < hi; j += ALL_THREADS) p_s[j - lo] = expf((x[j] - m) * inv_temp);
    __syncthreads();
    if (threadIdx.x == 0) {
        double run = before_block[block_of_r];
        int chosen = hi - 1;  // (rounding left r a hair above the block's last running sum)
        for (int j = lo; j < hi; j++) {
            run += (double)p_s[j - lo];
            if (run >= r_s) {
                chosen = j;
                break;
            }
        }
        out[row] = chosen;
    }
}

// Bytes of scratch abk_sample_all needs for n_rows rows of a vocabulary.
extern "C" long long abk_sample_all_scratch_bytes(int n_rows, int vocab) {
    return (long long)n_rows * ((vocab + ALL_BLOCK - 1) / ALL_BLOCK) * (long long)sizeof(double);
}
// top: int32 [n_rows], the index of each row's maximum (abk_argmax gives it); scratch as above.
extern "C" int abk_sample_all(const float *logits, long long row_stride, int n_rows, int vocab, float temp, const int *top,
                              unsigned long long *rng, const int *rng_index, int *out, void *scratch, void *stream) {
    if (n_rows <= 0) return 0;
    if (vocab < 1) ABK_REFUSE("sample: vocabulary of %d", vocab);
    if (!(temp > 0.0f)) ABK_REFUSE("sample: temperature %g is not positive (use argmax)", temp);
    const int n_blocks = (vocab + ALL_BLOCK - 1) / ALL_BLOCK;
    if (n_blocks > ALL_MAX_BLOCKS) ABK_REFUSE("sample: a vocabulary of %d is more than %d blocks of %d", vocab, ALL_MAX_BLOCKS, ALL_BLOCK);
    if (n_rows > 65535) ABK_REFUSE("sample: %d rows exceed a grid", n_rows);
    abk_launch(sample_all_sums_kernel, dim3(n_blocks, n_rows), dim3(ALL_THREADS), 0, (cudaStream_t)stream, logits, row_stride,
               vocab, 1.0f / temp, top, (double *)scratch);
    int rc = ABK_LAUNCH_RESULT();
    if (rc) return rc;
    abk_launch(sample_all_draw_kernel, dim3(n_rows), dim3(ALL_THREADS), 0, (cudaStream_t)stream, logits, row_stride, vocab,
               1.0f / temp, top, (const double *)scratch, n_blocks, rng, rng_index, out);
    return ABK_LAUNCH_RESULT();
}


// Choosing the next token from float32 logits: the first maximum, or a draw from the
// highest-k logits at a temperature (src/main.c:31-56). One block per row.
#define ABK_DEFINE_ERROR
#include "common.cuh"

#define SAMPLE_THREADS 1024
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

// The best element that comes strictly after `prev` in the order above (prev.i < 0: the very best).
__device__ __forceinline__ Best next_best(const float *row, int vocab, Best prev, Best *scratch) {
    Best b;
    b.v = -INFINITY, b.i = 0x7fffffff;
    for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
        Best c;
        c.v = row[j], c.i = j;
        if (prev.i >= 0 && !before(prev, c)) continue;
        if (before(c, b)) b = c;
    }
    return block_best(b, scratch);
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
__global__ void __launch_bounds__(SAMPLE_THREADS) sample_topk_kernel(const float *__restrict__ logits,
                                                                     long long row_stride, int vocab, float temp,
                                                                     int top_k, unsigned long long *rng,
                                                                     const int *__restrict__ rng_index,
                                                                     int *__restrict__ out) {
    __shared__ Best scratch[33];
    __shared__ Best top[SAMPLE_MAX_K];
    const float *row = logits + (long long)blockIdx.x * row_stride;
    Best prev;
    prev.v = 0.0f, prev.i = -1;
    int k = top_k < vocab ? top_k : vocab;
    for (int r = 0; r < k; r++) {
        prev = next_best(row, vocab, prev, scratch);
        if (threadIdx.x == 0) top[r] = prev;
    }
    if (threadIdx.x != 0) return;
    float p[SAMPLE_MAX_K], sum = 0.0f;
    for (int j = 0; j < k; j++) sum += p[j] = expf((top[j].v - top[0].v) / temp);
    int which = rng_index ? rng_index[blockIdx.x] : blockIdx.x;  // e.g. the row's cache slot
    unsigned long long s = rng[which];
    s ^= s << 13, s ^= s >> 7, s ^= s << 17;
    rng[which] = s;
    float r = (float)(s >> 40) / (float)(1 << 24) * sum;
    int chosen = top[k - 1].i;
    for (int j = 0; j < k; j++)
        if ((r -= p[j]) <= 0.0f) {
            chosen = top[j].i;
            break;
        }
    out[blockIdx.x] = chosen;
}

// scratch: 8 * ARGMAX_SLICES * n_rows bytes; tickets: int32 [n_rows], zero before and after.
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

extern "C" int abk_sample_topk(const float *logits, long long row_stride, int n_rows, int vocab, float temp, int top_k,
                               unsigned long long *rng, const int *rng_index, int *out, void *stream) {
    if (n_rows <= 0) return 0;
    if (vocab < 1) ABK_REFUSE("sample: vocabulary of %d", vocab);
    if (top_k < 1 || top_k > SAMPLE_MAX_K) ABK_REFUSE("sample: top_k %d is not in 1..%d", top_k, SAMPLE_MAX_K);
    if (!(temp > 0.0f)) ABK_REFUSE("sample: temperature %g is not positive (use argmax)", temp);
    sample_topk_kernel<<<n_rows, SAMPLE_THREADS, 0, (cudaStream_t)stream>>>(logits, row_stride, vocab, temp, top_k, rng,
                                                                           rng_index, out);
    return ABK_LAUNCH_RESULT();
}

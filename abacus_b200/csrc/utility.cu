// Utilities around the model: random weights made on the device, and guard words around buffers.
//
// Random weights. abacus gets its random test model from a library initialiser on the CPU
// (tools/tiny.py:15-20). Here a value depends only on (key, element index), so a tensor can be filled on
// the device in one pass, any slice of it can be made again on the host, and both agree bit for bit:
//   h_j  = mix(key + GAMMA * (3 i + j + 1)),  j = 0, 1, 2      (mix: the finaliser of splitmix64)
//   S    = the sum of the twelve 16-bit fields of h_0, h_1, h_2
//   z    = float(S - 393210) / 65536        (mean 0, variance 1 - 2^-32, within +-6; sum of 12 uniforms)
//   v    = mean + amplitude * z             (each operation rounded to float32, no fused multiply-add)
// Only integer arithmetic and two correctly rounded float32 operations: nothing a compiler or a maths
// library could round differently. weights/random_init.py holds the numpy twin.
//
// Guard words. A buffer handed out with guards has ABK_GUARD_WORDS words of a fixed pattern before and
// after it; abk_guard_check counts the words that no longer hold the pattern. With no memory checker on
// the device, this is what shows a store past the end of a workspace, a scratch area or a cache pool.
//
// A wait that runs out. Every wait of the kernels on a barrier is bounded (tc_common.cuh) and ends in a status word
// instead of a hang. abk_wait_that_runs_out is the smallest kernel with such a wait: a barrier that expects bytes
// nobody sends. It exists so that the way from a wait that ran out to the host's exception can be walked without
// breaking anything: the kernel returns, the context stays usable.
#define ABK_DEFINE_ERROR
#include "common.cuh"
#include "tc_common.cuh"

__host__ __device__ __forceinline__ unsigned long long abk_mix64(unsigned long long x) {
    x ^= x >> 30;
    x *= 0xbf58476d1ce4e5b9ull;
    x ^= x >> 27;
    x *= 0x94d049bb133111ebull;
    x ^= x >> 31;
    return x;
}

__device__ __forceinline__ float unit_normal(unsigned long long key, unsigned long long i) {
    unsigned int sum = 0;
#pragma unroll
    for (unsigned long long j = 1; j <= 3; j++) {
        unsigned long long h = abk_mix64(key + 0x9e3779b97f4a7c15ull * (3ull * i + j));
        sum += (unsigned int)(h & 0xffff) + (unsigned int)((h >> 16) & 0xffff) + (unsigned int)((h >> 32) & 0xffff) +
               (unsigned int)(h >> 48);
    }
    return __fmul_rn((float)((int)sum - 393210), 1.0f / 65536.0f);
}

template <typename T>
__global__ void fill_normal_kernel(T *out, long long n, long long first, unsigned long long key, float mean,
                                   float amplitude) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = from_float<T>(__fadd_rn(mean, __fmul_rn(amplitude, unit_normal(key, (unsigned long long)(first + i)))));
}

// out[i] = mean + amplitude * z(key, first + i) for i in [0, n): element `first + i` of the tensor that `key` names.
extern "C" int abk_fill_normal(void *out, int dtype, long long n, long long first, unsigned long long key, float mean,
                               float amplitude, void *stream) {
    if (n <= 0) return 0;
    if (dtype != ABK_F32 && dtype != ABK_BF16) ABK_REFUSE("fill_normal: dtype %d is neither float32 nor bfloat16", dtype);
    const int threads = 256;
    const long long blocks = (n + threads - 1) / threads;
    const int grid = (int)(blocks < abk_sm_count() * 16 ? blocks : abk_sm_count() * 16);
    if (dtype == ABK_F32)
        fill_normal_kernel<float><<<grid, threads, 0, (cudaStream_t)stream>>>((float *)out, n, first, key, mean, amplitude);
    else
        fill_normal_kernel<__nv_bfloat16><<<grid, threads, 0, (cudaStream_t)stream>>>((__nv_bfloat16 *)out, n, first, key,
                                                                                      mean, amplitude);
    return ABK_LAUNCH_RESULT();
}

#define ABK_GUARD_PATTERN 0xabac05c5u

__global__ void guard_fill_kernel(unsigned int *words, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) words[i] = ABK_GUARD_PATTERN;
}

__global__ void guard_check_kernel(const unsigned int *words, int n, int *damaged) {
    int bad = 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        bad += words[i] != ABK_GUARD_PATTERN;
    if (bad) atomicAdd(damaged, bad);
}

// Writes the pattern into `n` 32-bit words at `words`.
extern "C" int abk_guard_fill(void *words, int n, void *stream) {
    if (n <= 0) return 0;
    guard_fill_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>((unsigned int *)words, n);
    return ABK_LAUNCH_RESULT();
}

// Adds to *damaged how many of the `n` words at `words` no longer hold the pattern.
extern "C" int abk_guard_check(const void *words, int n, int *damaged, void *stream) {
    if (n <= 0) return 0;
    guard_check_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>((const unsigned int *)words, n, damaged);
    return ABK_LAUNCH_RESULT();
}

__global__ void wait_that_runs_out_kernel(int *status, int bit) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        tc::mbar_init(&bar, 1);
        tc::mbar_init_fence();
        tc::mbar_expect_tx(&bar, 16);             // 16 bytes that no copy will ever bring
        if (!tc::mbar_wait(&bar, 0)) atomicOr(status, bit);
    }
}

// Runs a kernel whose only wait cannot be satisfied and therefore runs out after this library's limit
// (abk_set_wait_limit_ns); it then sets `bit` in *status and returns.
extern "C" int abk_wait_that_runs_out(int *status, int bit, void *stream) {
    wait_that_runs_out_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, bit);
    return ABK_LAUNCH_RESULT();
}


// out[M, N] = x[M, K] . w[N, K]^T with float32 multiply-adds on the CUDA cores, for any M, N, K.
//
// This is the matrix product of the true 32-bit path (no tensor cores, no TF32), and the
// fallback of the bfloat16 path for shapes the tensor-core kernel refuses. Every output element
// is one thread's running sum over k = 0, 1, ..., K-1 in that order, so a row's result does not
// depend on how many other rows are in the batch or where its tile lies.
// Formula: src/model.c:299, 302, 307, 309, 324 (weights are [out, in] row-major, no bias).
#define ABK_DEFINE_ERROR
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const TX *__restrict__ x, const TW *__restrict__ w,
                                                        TO *__restrict__ out, int M, int N, int K, long long ldx,
                                                        long long ldw, long long ldo) {
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int idx = tid + i * 256, r = idx >> 4, k = idx & 15;
            int gm = m0 + r, gn = n0 + r, gk = k0 + k;
            xs[k][r] = (gm < M && gk < K) ? to_float(x[(long long)gm * ldx + gk]) : 0.0f;
            ws[k][r] = (gn < N && gk < K) ? to_float(w[(long long)gn * ldw + gk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = xs[k][ty * 4 + i], b[i] = ws[k][tx * 4 + i];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int gn = n0 + tx * 4 + j;
            if (gn < N) out[(long long)gm * ldo + gn] = from_float<TO>(acc[i][j]);
        }
    }
}

// x_dtype/w_dtype/out_dtype: ABK_F32 or ABK_BF16. Supported: all-float32; bf16 x and w with bf16 or f32 out.
extern "C" int abk_gemm_simt(const void *x, int x_dtype, const void *w, int w_dtype, void *out, int out_dtype, int M,
                             int N, int K, long long ldx, long long ldw, long long ldo, void *stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) ABK_REFUSE("gemm: K = %d", K);
    dim3 grid((M + BM - 1) / BM, (N + BN - 1) / BN);
    if (grid.y > 65535) ABK_REFUSE("gemm: %d output columns are more than one launch takes", N);
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
    if (x_dtype == ABK_F32 && w_dtype == ABK_F32 && out_dtype == ABK_F32)
        gemm_simt_kernel<<<grid, 256, 0, s>>>((const float *)x, (const float *)w, (float *)out, M, N, K, ldx, ldw, ldo);
    else if (x_dtype == ABK_BF16 && w_dtype == ABK_BF16 && out_dtype == ABK_BF16)
        gemm_simt_kernel<<<grid, 256, 0, s>>>((const bf *)x, (const bf *)w, (bf *)out, M, N, K, ldx, ldw, ldo);
    else if (x_dtype == ABK_BF16 && w_dtype == ABK_BF16 && out_dtype == ABK_F32)
        gemm_simt_kernel<<<grid, 256, 0, s>>>((const bf *)x, (const bf *)w, (float *)out, M, N, K, ldx, ldw, ldo);
    else
        ABK_REFUSE("gemm: dtype combination x=%d w=%d out=%d is not built", x_dtype, w_dtype, out_dtype);
    return ABK_LAUNCH_RESULT();
}

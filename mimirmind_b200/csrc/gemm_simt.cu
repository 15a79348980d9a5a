// C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]) on the fp32 FMA units: the matrix product of the
// true 32-bit path, and the any-shape fallback of the bfloat16 path.
//
// The reference computes Y[m,n] = sum_k X[m,k] * W[n,k] with W stored [N_out, K_in]
// (src/compute/Matmul.cpp:54-65) and adds a bias per output column
// (src/compute/Matmul.cpp:67-78).  Every output element is accumulated over k in
// ascending order by one thread, so its value does not depend on M, on the row's place
// in the batch, or on the tile it falls into.
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W,
                                                        const void* __restrict__ bias, int bias_dtype,
                                                        TC* __restrict__ C, int M, int N, int K, int lda, int ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, 4 x 4 outputs each
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k = 1024 elements per operand, 4 per thread
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int k = k0 + kk;
            float a = 0.0f, w = 0.0f;
            if (k < K) {
                if (m0 + r < M) a = to_f32<TA>(A[(size_t)(m0 + r) * lda + k]);
                if (n0 + r < N) w = to_f32<TW>(W[(size_t)(n0 + r) * K + k]);
            }
            As[kk][r] = a;
            Ws[kk][r] = w;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) {
                v += (bias_dtype == MM_F32) ? ((const float*)bias)[n] : __bfloat162float(((const __nv_bfloat16*)bias)[n]);
            }
            C[(size_t)m * ldc + n] = from_f32<TC>(v);
        }
    }
}

MM_EXPORT int mm_gemm_simt(const void* A, int a_dtype, const void* W, int w_dtype, const void* bias, int bias_dtype,
                           void* C, int c_dtype, int M, int N, int K, int lda, int ldc, void* stream) {
    MM_REQUIRE(M >= 0 && N > 0 && K > 0 && lda >= K && ldc >= N, "gemm: bad sizes");
    if (M == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(ceil_div(N, BN), ceil_div(M, BM));
#define MM_GEMM(TA, TW, TC) \
    gemm_simt_kernel<TA, TW, TC><<<grid, 256, 0, s>>>((const TA*)A, (const TW*)W, bias, bias_dtype, (TC*)C, M, N, K, lda, ldc)
    typedef __nv_bfloat16 bf;
    const int key = a_dtype * 4 + w_dtype * 2 + c_dtype;
    switch (key) {
        case 0: MM_GEMM(float, float, float); break;
        case 1: MM_GEMM(float, float, bf); break;
        case 2: MM_GEMM(float, bf, float); break;
        case 3: MM_GEMM(float, bf, bf); break;
        case 4: MM_GEMM(bf, float, float); break;
        case 5: MM_GEMM(bf, float, bf); break;
        case 6: MM_GEMM(bf, bf, float); break;
        case 7: MM_GEMM(bf, bf, bf); break;
        default: MM_REQUIRE(false, "gemm: dtypes must be float32 or bfloat16");
    }
#undef MM_GEMM
    MM_CHECK_LAUNCH();
    return MM_OK;
}

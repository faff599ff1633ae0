// True 32-bit matrix product on the CUDA cores: C[M,N] = A[M,K] * B[N,K]^T, the
// y = x W^T of every projection (xiyiji/paged-llm llama.py:141-144, :166-168,
// :208).  No tensor cores and no reduced-precision mode: every output element is
// one chain of float32 fused multiply-adds over k = 0..K-1 in order, so a row's
// result does not depend on which other rows are in the batch or on the tile
// shape that was chosen.
#include "common.cuh"

template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
sgemm_nt_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M, int N, int K,
                int lda, int ldb, int ldc) {
    constexpr int THREADS = (BM / TM) * (BN / TN);
    constexpr int PAD = 4;
    __shared__ float As[BK][BM + PAD];
    __shared__ float Bs[BK][BN + PAD];
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int e = tid; e < BM * BK; e += THREADS) {
            const int k = e % BK, m = e / BK;
            const int gm = m0 + m, gk = k0 + k;
            As[k][m] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.f;
        }
        for (int e = tid; e < BN * BK; e += THREADS) {
            const int k = e % BK, n = e / BK;
            const int gn = n0 + n, gk = k0 + k;
            Bs[k][n] = (gn < N && gk < K) ? B[(size_t)gn * ldb + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn < N) C[(size_t)gm * ldc + gn] = acc[i][j];
        }
    }
}

PL_EXPORT int pl_gemm_f32(const float* A, const float* B, float* C, int M, int N, int K, int lda, int ldb, int ldc,
                          cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    PL_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_f32: bad sizes M=%d N=%d K=%d", M, N, K);
    PL_REQUIRE(lda >= K && ldb >= K && ldc >= N, "gemm_f32: leading dimensions too small");
    if (M >= 512 && N >= 512) {
        dim3 grid((N + 127) / 128, (M + 127) / 128);
        sgemm_nt_kernel<128, 128, 8, 8, 8><<<grid, 256, 0, stream>>>(A, B, C, M, N, K, lda, ldb, ldc);
    } else {
        dim3 grid((N + 63) / 64, (M + 63) / 64);
        sgemm_nt_kernel<64, 64, 16, 4, 4><<<grid, 256, 0, stream>>>(A, B, C, M, N, K, lda, ldb, ldc);
    }
    PL_LAUNCHED("gemm_f32");
    return 0;
}

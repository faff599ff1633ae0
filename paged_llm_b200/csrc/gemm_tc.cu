// The many-token tcgen05 product (gemm_tc_duo.cuh: pairs of blocks on tiles of 256 tokens x 256 features).
#include "gemm_tc_duo.cuh"

// Waits inside the kernel that gave up since the library was loaded (0 unless something is broken).
PL_EXPORT int pl_gemm_tc_timeouts() {
    int n = 0;
    if (cudaMemcpyFromSymbol(&n, tc::g_timeouts, sizeof(int)) != cudaSuccess) return -1;
    return n;
}

// epi: 0 bfloat16 out, 1 float32 out, 2 SiLU (W = [Wg; Wu] of shape [2I, K], N = I outputs), 3 add (resid[M, N] +=,
// N a multiple of 4).  K a multiple of 64; rows of X and Y 16-byte aligned.
PL_EXPORT int pl_gemm_tc(const void* X, int ldx, const void* W, void* Y, int ldy, float* resid, int M, int N, int K, int epi,
                         cudaStream_t stream) {
    return gemm_tc_duo_launch(X, ldx, W, Y, ldy, resid, M, N, K, epi, stream);
}

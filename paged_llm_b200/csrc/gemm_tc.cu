// The many-token tcgen05 products: gemm_tc.cuh with every block fetching its own tiles, and gemm_tc_duo.cuh
// (pairs of blocks on one tile).
#include "gemm_tc_duo.cuh"

namespace {

struct SingleIO {
    static constexpr int CLUSTER = 1;
    static __device__ __forceinline__ void load_w(unsigned char* dst, const CUtensorMap* map, int k, int row_a, int row_b,
                                                  uint64_t* bar, uint32_t) {
        tc_tma(dst, map, k, row_a, bar);
        tc_tma(dst + 128 * 128, map, k, row_b, bar);
    }
    static __device__ __forceinline__ void release(uint64_t* bar) { tc::mma_commit(bar); }
};

}  // namespace

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
    return gemm_tc_launch<SingleIO>(X, ldx, W, Y, ldy, resid, M, N, K, epi, stream);
}

// The same interface, run by pairs of blocks (tcgen05.mma.cta_group::2) on tiles of 256 tokens.
PL_EXPORT int pl_gemm_tc_duo(const void* X, int ldx, const void* W, void* Y, int ldy, float* resid, int M, int N, int K,
                             int epi, cudaStream_t stream) {
    return gemm_tc_duo_launch(X, ldx, W, Y, ldy, resid, M, N, K, epi, stream);
}

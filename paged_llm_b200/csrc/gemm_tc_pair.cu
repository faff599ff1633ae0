// The many-token tcgen05 product (gemm_tc.cuh) with the blocks in pairs: the two blocks of a
// cluster work on two tiles of the same 256 features (consecutive 128-token tiles) in step, each
// fetches one half of the W tile of a stage, and the TMA unit delivers that half to the shared
// memory of both (one read of L2 for two blocks).  A block then has 32 KB instead of 48 KB on their
// way per stage, so the four stages of the ring cover half as much latency again.  A stage is
// given back when the products of both blocks have read it: the commit arrives on the `empty`
// barrier of both.
//
// This file is the only one of the package that names a TMA load that delivers to several blocks;
// the package runs without it (kernels/ops.py then uses gemm_tc.cu or the library product).
#include "gemm_tc.cuh"

namespace {

struct PairIO {
    static constexpr int CLUSTER = 2;
    // This block's half of the 256 rows (rank 0: the first box, rank 1: the second), to both blocks.
    static __device__ __forceinline__ void load_w(unsigned char* dst, const CUtensorMap* map, int k, int row_a, int row_b,
                                                  uint64_t* bar, uint32_t rank) {
        const uint16_t both = 3;
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.multicast::cluster "
            "[%0], [%1, {%2, %3}], [%4], %5;\n" ::"r"(tc::saddr(dst + rank * (128 * 128))),
            "l"(map), "r"(k), "r"(rank == 0 ? row_a : row_b), "r"(tc::saddr(bar)), "h"(both)
            : "memory");
    }
    static __device__ __forceinline__ void release(uint64_t* bar) {
        const uint16_t both = 3;
        asm volatile(
            "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n" ::"r"(
                tc::saddr(bar)),
            "h"(both)
            : "memory");
    }
};

}  // namespace

PL_EXPORT int pl_gemm_tc_pair_timeouts() {
    int n = 0;
    if (cudaMemcpyFromSymbol(&n, tc::g_timeouts, sizeof(int)) != cudaSuccess) return -1;
    return n;
}

// The same interface as pl_gemm_tc.
PL_EXPORT int pl_gemm_tc_pair(const void* X, int ldx, const void* W, void* Y, int ldy, float* resid, int M, int N, int K,
                              int epi, cudaStream_t stream) {
    return gemm_tc_launch<PairIO>(X, ldx, W, Y, ldy, resid, M, N, K, epi, stream);
}

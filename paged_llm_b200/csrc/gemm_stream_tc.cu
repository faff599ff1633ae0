// Matrix product for 17 to 128 tokens on the 5th-generation tensor cores:
// Y[M,N] = X[M,K] * W[N,K]^T, bfloat16 in, float32 accumulation in tensor memory.
//
// With so few tokens the product is still a read of W, so the roles are swapped: a tile of 128
// rows of W is the 128-row A operand of tcgen05.mma and the tokens (padded to 32, 64 or 128) are
// the N dimension, so one instruction multiplies the whole batch by 128 output features.  W and X
// tiles (64 k each) come through TMA (cp.async.bulk.tensor.2d, 128-byte swizzle) into a ring of
// four stages: one warp issues the copies, one thread the products, completion runs over
// mbarriers (TMA complete_tx, tcgen05.commit), every wait is bounded.  N / 128 tiles would leave
// most SMs idle for the narrow products of a decoder layer, so K is split over the blocks of a
// thread-block cluster (up to 8): each block multiplies its share of K, leaves its 128 x M partial
// result in its own shared memory, and after a cluster barrier every block adds up, over all
// blocks' shared memory (distributed shared memory), the rows it finishes.  No partial result
// touches global memory and the order of the sum is fixed.
//
// The 128 rows of a tile are chosen so that the epilogue needs no second kernel:
//   plain  rows n0..n0+127;                         y = acc (bfloat16 or float32)
//   SiLU   64 gate rows and the 64 matching up rows; y = silu(gate) * up   (xiyiji/paged-llm llama.py:171)
//   add    the product is a branch of the residual stream: x += bf16(acc) in float32 (llama.py:183-184)
// For a given token the order of summation does not depend on M or on the other tokens.
#include <cooperative_groups.h>

#include "tcgen05.cuh"
#include "tensor_map.cuh"

namespace cg = cooperative_groups;

enum { ST_BF16 = 0, ST_F32 = 1, ST_SILU = 2, ST_ADD = 3 };

struct StreamParams {
    void* Y;            // [M, ldy] (plain, SiLU)
    float* resid;       // [M, N] (add)
    int ldy, M, N, K, I;
    int epi;
    int tiles;          // row tiles of W (128 rows; SiLU: 64 gate + 64 up rows)
    int splitk;         // blocks per cluster
    int k_per_split;    // k of one block, a multiple of 64
};

namespace {

using namespace tc;

constexpr int ST_BK = 64, ST_STAGES = 4, ST_THREADS = 192;
constexpr int ST_W_BYTES = 128 * 128;          // 128 rows x 64 k

__device__ __forceinline__ void st_arrive_expect(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(saddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void st_tma(void* dst, const CUtensorMap* map, int col, int row, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::
            "r"(saddr(dst)), "l"(map), "r"(col), "r"(row), "r"(saddr(bar))
        : "memory");
}

template <int MPAD>
constexpr size_t st_smem_bytes() {
    // ring of stages (W tile + X tile); the partial result [128][MPAD + 1] float32 reuses it
    size_t ring = (size_t)ST_STAGES * (ST_W_BYTES + MPAD * 128);
    size_t part = (size_t)128 * (MPAD + 1) * 4;
    return (ring > part ? ring : part) + 1024;
}

template <int MPAD>
__global__ void __launch_bounds__(ST_THREADS, 1) gemm_stream_tc_kernel(StreamParams p, const __grid_constant__ CUtensorMap w_map,
                                                                      const __grid_constant__ CUtensorMap x_map) {
    constexpr int X_BYTES = MPAD * 128, STAGE_BYTES = ST_W_BYTES + X_BYTES;
    constexpr int TMEM_COLS = MPAD < 32 ? 32 : MPAD;
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full[ST_STAGES], empty[ST_STAGES], acc_done;
    __shared__ uint32_t tmem_base_slot;

    cg::cluster_group cluster = cg::this_cluster();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int C = p.splitk, rank = (int)cluster.block_rank();
    const int tile = blockIdx.x / C;
    const int k_lo = rank * p.k_per_split;
    const int k_hi = min(p.K, k_lo + p.k_per_split);
    const int k_steps = k_hi > k_lo ? (k_hi - k_lo) / ST_BK : 0;
    // rows of W behind the two 64-row boxes of a stage
    const int row_a = p.epi == ST_SILU ? tile * 64 : tile * 128;
    const int row_b = p.epi == ST_SILU ? p.I + tile * 64 : tile * 128 + 64;

    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(saddr(&tmem_base_slot)),
                     "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    if (tid == 0) {
        for (int s = 0; s < ST_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(&acc_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- copies
        if (lane == 0) {
            for (int ks = 0; ks < k_steps; ++ks) {
                const int s = ks % ST_STAGES;
                if (ks >= ST_STAGES) mbar_wait(&empty[s], ((ks / ST_STAGES) - 1) & 1);
                unsigned char* st = smem + (size_t)s * STAGE_BYTES;
                const int k = k_lo + ks * ST_BK;
                st_arrive_expect(&full[s], STAGE_BYTES);
                st_tma(st, &w_map, k, row_a, &full[s]);
                st_tma(st + 64 * 128, &w_map, k, row_b, &full[s]);
                st_tma(st + ST_W_BYTES, &x_map, k, 0, &full[s]);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- products
        if (lane == 0) {
            constexpr uint32_t IDESC = instr_desc(128, MPAD, false);
            for (int ks = 0; ks < k_steps; ++ks) {
                const int s = ks % ST_STAGES;
                mbar_wait(&full[s], (ks / ST_STAGES) & 1);
                fence_after_sync();
                const uint32_t wa = saddr(smem + (size_t)s * STAGE_BYTES), xa = wa + ST_W_BYTES;
#pragma unroll
                for (int kk = 0; kk < ST_BK / 16; ++kk)
                    mma_f16(tmem_base, smem_desc(wa + kk * 32, 16, 1024), smem_desc(xa + kk * 32, 16, 1024), IDESC,
                            ks > 0 || kk > 0);
                mma_commit(&empty[s]);
            }
            mma_commit(&acc_done);
        }
        __syncwarp();
    }
    // ---------------------------------------------------------------- partial result to shared memory
    float* part = reinterpret_cast<float*>(smem);            // [128][MPAD + 1]: the ring is free once acc_done fires
    if (warp >= 2) {
        const int f = (warp & 3) * 32 + lane;                 // row of the tile = lane of tensor memory
        if (k_steps > 0) {
            mbar_wait(&acc_done, 0);
            fence_after_sync();
            const uint32_t trow = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
#pragma unroll 1
            for (int cb = 0; cb < MPAD / 32; ++cb) {
                float v[32];
                tmem_ld32(trow + cb * 32, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) part[(size_t)f * (MPAD + 1) + cb * 32 + i] = v[i];
            }
        } else {
            for (int i = 0; i < MPAD; ++i) part[(size_t)f * (MPAD + 1) + i] = 0.f;
        }
    }
    fence_before_sync();
    cluster.sync();
    // ---------------------------------------------------------------- sum over the cluster and epilogue
    if (warp >= 2) {
        const int et = tid - 64;                              // 0..127
        const int rows_per = (64 + C - 1) / C;               // row pairs (f, f + 64) this block finishes
        const int f_lo = rank * rows_per;
        const int mine = max(0, min(rows_per, 64 - f_lo));
        for (int e = et; e < p.M * mine; e += 128) {
            const int tok = e / mine, f0 = f_lo + (e - tok * mine), f1 = f0 + 64;
            float v0 = 0.f, v1 = 0.f;
            for (int j = 0; j < C; ++j) {
                const float* pj = cluster.map_shared_rank(part, j);
                v0 += pj[(size_t)f0 * (MPAD + 1) + tok];
                v1 += pj[(size_t)f1 * (MPAD + 1) + tok];
            }
            if (p.epi == ST_SILU) {
                const int j = tile * 64 + f0;
                if (j < p.I) {
                    const float gate = __bfloat162float(__float2bfloat16_rn(v0));
                    const float up = __bfloat162float(__float2bfloat16_rn(v1));
                    ((__nv_bfloat16*)p.Y)[(size_t)tok * p.ldy + j] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
                }
            } else {
                const int n0 = tile * 128 + f0, n1 = n0 + 64;
                if (p.epi == ST_BF16) {
                    __nv_bfloat16* y = (__nv_bfloat16*)p.Y + (size_t)tok * p.ldy;
                    if (n0 < p.N) y[n0] = __float2bfloat16_rn(v0);
                    if (n1 < p.N) y[n1] = __float2bfloat16_rn(v1);
                } else if (p.epi == ST_F32) {
                    float* y = (float*)p.Y + (size_t)tok * p.ldy;
                    if (n0 < p.N) y[n0] = v0;
                    if (n1 < p.N) y[n1] = v1;
                } else {
                    // the branch is rounded to bfloat16 first, as a separate product would store it
                    float* x = p.resid + (size_t)tok * p.N;
                    if (n0 < p.N) x[n0] += __bfloat162float(__float2bfloat16_rn(v0));
                    if (n1 < p.N) x[n1] += __bfloat162float(__float2bfloat16_rn(v1));
                }
            }
        }
    }
    cluster.sync();                  // nobody leaves while its shared memory is still read
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS));
}

template <int MPAD>
int launch_stream(const StreamParams& p, const CUtensorMap* w_map, const CUtensorMap* x_map, cudaStream_t stream) {
    constexpr size_t smem = st_smem_bytes<MPAD>();
    auto kernel = gemm_stream_tc_kernel<MPAD>;
    static bool attr_set = false;
    if (!attr_set) {
        PL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.tiles * p.splitk);
    cfg.blockDim = dim3(ST_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = p.splitk;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static const bool no_pdl = getenv("PAGED_LLM_B200_NO_PDL") != nullptr;
    cfg.numAttrs = no_pdl ? 1 : 2;
    PL_CUDA(cudaLaunchKernelEx(&cfg, kernel, p, *w_map, *x_map));
    return 0;
}

int g_st_sms = 0;

}  // namespace

// Waits inside the kernel that gave up since the library was loaded (0 unless something is broken).
PL_EXPORT int pl_gemm_stream_tc_timeouts() {
    int n = 0;
    if (cudaMemcpyFromSymbol(&n, tc::g_timeouts, sizeof(int)) != cudaSuccess) return -1;
    return n;
}

// Whether the sizes fit this kernel (the caller uses the library product otherwise).
PL_EXPORT int pl_gemm_stream_tc_supported(int M, int N, int K, int ldx) {
    return M > 16 && M <= 128 && N >= 1 && K >= 64 && K % 64 == 0 && ldx % 8 == 0;
}

// epi: 0 bfloat16 out, 1 float32 out, 2 SiLU (W = [Wg; Wu] of shape [2I, K], N = I outputs), 3 add (resid[M, N] +=).
PL_EXPORT int pl_gemm_stream_tc(const void* X, int ldx, const void* W, void* Y, int ldy, float* resid, int M, int N, int K,
                                int epi, cudaStream_t stream) {
    PL_REQUIRE(pl_gemm_stream_tc_supported(M, N, K, ldx), "gemm_stream_tc: M=%d (17..128) N=%d K=%d (multiple of 64) ldx=%d",
               M, N, K, ldx);
    PL_REQUIRE(epi >= ST_BF16 && epi <= ST_ADD, "gemm_stream_tc: epilogue %d", epi);
    PL_REQUIRE(epi == ST_ADD ? resid != nullptr : (Y != nullptr && ldy >= N), "gemm_stream_tc: output missing or ldy < N");
    if (g_st_sms == 0) {
        int dev = 0;
        PL_CUDA(cudaGetDevice(&dev));
        PL_CUDA(cudaDeviceGetAttribute(&g_st_sms, cudaDevAttrMultiProcessorCount, dev));
    }
    StreamParams p = {};
    p.Y = Y;
    p.resid = resid;
    p.ldy = ldy;
    p.M = M;
    p.N = N;
    p.K = K;
    p.epi = epi;
    p.I = N;
    const int w_rows = epi == ST_SILU ? 2 * N : N;
    p.tiles = epi == ST_SILU ? (N + 63) / 64 : (N + 127) / 128;
    // blocks for about two per SM; K is cut in multiples of 64, every block of a cluster gets some
    // (clusters of 1, 2, 4 or 8: other sizes place badly on the GPCs and fewer of them run at a time)
    int split = 1;
    while (split < 8 && p.tiles * split * 2 <= 2 * g_st_sms) split *= 2;
    const int k_blocks = K / ST_BK;
    if (split > k_blocks) split = k_blocks;
    const int per = (k_blocks + split - 1) / split;
    p.k_per_split = per * ST_BK;
    p.splitk = (k_blocks + per - 1) / per;
    const int mpad = M <= 32 ? 32 : M <= 64 ? 64 : 128;
    alignas(64) CUtensorMap w_map, x_map;
    if (!tensor_map_bf16(&w_map, W, (unsigned long long)w_rows, (unsigned long long)K, (unsigned long long)K, 64) ||
        !tensor_map_bf16(&x_map, X, (unsigned long long)M, (unsigned long long)K, (unsigned long long)ldx, mpad))
        return 1;
    if (mpad == 32) return launch_stream<32>(p, &w_map, &x_map, stream);
    if (mpad == 64) return launch_stream<64>(p, &w_map, &x_map, stream);
    return launch_stream<128>(p, &w_map, &x_map, stream);
}

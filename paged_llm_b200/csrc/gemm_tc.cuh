// Matrix product for many tokens (prompt portions) on the 5th-generation tensor cores:
// Y[M,N] = X[M,K] * W[N,K]^T, bfloat16 in, float32 accumulation in tensor memory, with the
// elementwise work that follows a projection done in the epilogue.
//
// A block is persistent and walks output tiles of 128 tokens x 256 features.  One warp brings
// X and W tiles (64 k each) in with TMA (cp.async.bulk.tensor.2d, 128-byte swizzle) through a ring
// of four stages, one thread issues tcgen05.mma 128x256x16 into one of two accumulators in tensor
// memory (2 x 256 columns: all of it), and four warps drain the other accumulator meanwhile:
// tcgen05.ld, the epilogue's arithmetic, 16-byte stores.  Completion runs over mbarriers
// (TMA complete_tx, tcgen05.commit, arrivals of the epilogue threads); every wait is bounded.
// Tiles are taken feature-tile by feature-tile so that the blocks running at a time share W
// tiles in L2.
//
// Epilogues (the rows of W behind a tile are chosen so that no second kernel is needed):
//   plain  256 consecutive rows;                      y = acc (bfloat16 or float32)
//   SiLU   128 gate rows and the 128 matching up rows; y = silu(gate) * up  (xiyiji/paged-llm llama.py:171)
//   add    the product is a branch of the residual stream: x += bf16(acc) in float32 (llama.py:183-184)
#pragma once

#include "tcgen05.cuh"
#include "tensor_map.cuh"

enum { TC_BF16 = 0, TC_F32 = 1, TC_SILU = 2, TC_ADD = 3 };

struct TcParams {
    void* Y;            // [M, ldy] (plain, SiLU)
    float* resid;       // [M, N] (add)
    int ldy, M, N, K, I;
    int epi;
    int m_tiles, n_tiles;
};

namespace {

using namespace tc;

constexpr int TC_BM = 128, TC_BN = 256, TC_BK = 64, TC_STAGES = 4, TC_THREADS = 192;
constexpr int TC_A_BYTES = TC_BM * 128, TC_B_BYTES = TC_BN * 128, TC_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES;
constexpr size_t TC_SMEM = (size_t)TC_STAGES * TC_STAGE_BYTES + 1024;

__device__ __forceinline__ void tc_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(saddr(bar)) : "memory");
}
__device__ __forceinline__ void tc_arrive_expect(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(saddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tc_tma(void* dst, const CUtensorMap* map, int col, int row, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::
            "r"(saddr(dst)), "l"(map), "r"(col), "r"(row), "r"(saddr(bar))
        : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// The epilogue of one thread: row `tok` of the tile of feature tile `nt`, whose accumulator starts at `acc`
// (this thread's lane of tensor memory).
__device__ __forceinline__ void tc_drain_row(const TcParams& p, uint32_t acc, int tok, int nt) {
    if (p.epi == TC_SILU) {
        const int j0 = nt * 128;
#pragma unroll 1
        for (int cb = 0; cb < 4; ++cb) {
            float g[32], u[32];
            tmem_ld32(acc + cb * 32, g);
            tmem_ld32(acc + 128 + cb * 32, u);
            if (tok < p.M) {
                __nv_bfloat16* y = (__nv_bfloat16*)p.Y + (size_t)tok * p.ldy + j0 + cb * 32;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t w[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float o[2];
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const float gate = __bfloat162float(__float2bfloat16_rn(g[q * 8 + 2 * i + e]));
                            const float up = __bfloat162float(__float2bfloat16_rn(u[q * 8 + 2 * i + e]));
                            o[e] = gate / (1.0f + __expf(-gate)) * up;
                        }
                        w[i] = pack_bf16x2(o[0], o[1]);
                    }
                    if (j0 + cb * 32 + q * 8 + 8 <= p.I)
                        *reinterpret_cast<uint4*>(y + q * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                    else
                        for (int i = 0; i < 8; ++i)
                            if (j0 + cb * 32 + q * 8 + i < p.I)
                                y[q * 8 + i] = __ushort_as_bfloat16((unsigned short)((w[i >> 1] >> ((i & 1) * 16)) & 0xffff));
                }
            }
        }
    } else {
        const int n0 = nt * TC_BN;
#pragma unroll 1
        for (int cb = 0; cb < 8; ++cb) {
            float v[32];
            tmem_ld32(acc + cb * 32, v);
            if (tok >= p.M) continue;
            const int n = n0 + cb * 32;
            if (p.epi == TC_BF16) {
                __nv_bfloat16* y = (__nv_bfloat16*)p.Y + (size_t)tok * p.ldy + n;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    if (n + q * 8 + 8 <= p.N)
                        *reinterpret_cast<uint4*>(y + q * 8) =
                            make_uint4(pack_bf16x2(v[q * 8], v[q * 8 + 1]), pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]),
                                       pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]), pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]));
                    else
                        for (int i = 0; i < 8; ++i)
                            if (n + q * 8 + i < p.N) y[q * 8 + i] = __float2bfloat16_rn(v[q * 8 + i]);
                }
            } else if (p.epi == TC_F32) {
                float* y = (float*)p.Y + (size_t)tok * p.ldy + n;
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    if (n + q * 4 + 4 <= p.N)
                        *reinterpret_cast<float4*>(y + q * 4) = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
                    else
                        for (int i = 0; i < 4; ++i)
                            if (n + q * 4 + i < p.N) y[q * 4 + i] = v[q * 4 + i];
                }
            } else {
                // the branch is rounded to bfloat16 first, as a separate product would store it
                float* x = p.resid + (size_t)tok * p.N + n;
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    if (n + q * 4 + 4 <= p.N) {
                        float4 r = *reinterpret_cast<float4*>(x + q * 4);
                        r.x += __bfloat162float(__float2bfloat16_rn(v[q * 4]));
                        r.y += __bfloat162float(__float2bfloat16_rn(v[q * 4 + 1]));
                        r.z += __bfloat162float(__float2bfloat16_rn(v[q * 4 + 2]));
                        r.w += __bfloat162float(__float2bfloat16_rn(v[q * 4 + 3]));
                        *reinterpret_cast<float4*>(x + q * 4) = r;
                    } else {
                        for (int i = 0; i < 4; ++i)
                            if (n + q * 4 + i < p.N) x[q * 4 + i] += __bfloat162float(__float2bfloat16_rn(v[q * 4 + i]));
                    }
                }
            }
        }
    }
}

// IO says how the W tile of a stage comes in and how a stage is given back:
//   IO::CLUSTER            blocks per cluster (1, or 2 blocks that share every W tile)
//   IO::load_w(dst, map, k, row_a, row_b, bar, rank)   the 256 rows of W behind the tile, as two boxes of 128
//   IO::release(bar)       after the products of a stage: tcgen05.commit on its `empty` barrier
// The blocks of a cluster take tiles of the same 256 features and of consecutive 128 tokens, in step.
template <class IO>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(TcParams p, const __grid_constant__ CUtensorMap x_map,
                                                                const __grid_constant__ CUtensorMap w_map) {
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full[TC_STAGES], empty[TC_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_slot;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t rank = 0;
    if (IO::CLUSTER > 1) asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(rank));
    // a "tile" of the loops below is one tile per block of the cluster: m_tiles is a multiple of IO::CLUSTER
    const int m_groups = p.m_tiles / IO::CLUSTER;
    const int tiles = m_groups * p.n_tiles;
    const int first = blockIdx.x / IO::CLUSTER, stride = gridDim.x / IO::CLUSTER;
    const int k_steps = p.K / TC_BK;

    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(saddr(&tmem_base_slot)),
                     "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], IO::CLUSTER);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 128);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    if (IO::CLUSTER > 1) {        // the other block's barriers must exist before anything of ours reaches them
        asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    }
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- copies
        if (lane == 0) {
            int it = 0;
            for (int tile = first; tile < tiles; tile += stride) {
                const int nt = tile / m_groups, mt = (tile - nt * m_groups) * IO::CLUSTER + (int)rank;
                const int row_a = p.epi == TC_SILU ? nt * 128 : nt * 256;            // rows of W behind the two boxes
                const int row_b = p.epi == TC_SILU ? p.I + nt * 128 : nt * 256 + 128;
                for (int ks = 0; ks < k_steps; ++ks, ++it) {
                    const int s = it % TC_STAGES;
                    if (it >= TC_STAGES) mbar_wait(&empty[s], ((it / TC_STAGES) - 1) & 1);
                    unsigned char* st = smem + (size_t)s * TC_STAGE_BYTES;
                    tc_arrive_expect(&full[s], TC_STAGE_BYTES);
                    tc_tma(st, &x_map, ks * TC_BK, mt * TC_BM, &full[s]);
                    IO::load_w(st + TC_A_BYTES, &w_map, ks * TC_BK, row_a, row_b, &full[s], rank);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- products
        if (lane == 0) {
            constexpr uint32_t IDESC = instr_desc(TC_BM, TC_BN, false);
            int it = 0, n_tile = 0;
            for (int tile = first; tile < tiles; tile += stride, ++n_tile) {
                const int b = n_tile & 1;
                if (n_tile >= 2) mbar_wait(&acc_empty[b], ((n_tile >> 1) - 1) & 1);     // the epilogue has drained it
                fence_after_sync();
                for (int ks = 0; ks < k_steps; ++ks, ++it) {
                    const int s = it % TC_STAGES;
                    mbar_wait(&full[s], (it / TC_STAGES) & 1);
                    fence_after_sync();
                    const uint32_t xa = saddr(smem + (size_t)s * TC_STAGE_BYTES), wa = xa + TC_A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < TC_BK / 16; ++kk)
                        mma_f16(tmem_base + b * TC_BN, smem_desc(xa + kk * 32, 16, 1024), smem_desc(wa + kk * 32, 16, 1024),
                                IDESC, ks > 0 || kk > 0);
                    IO::release(&empty[s]);
                }
                mma_commit(&acc_full[b]);
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- epilogue: one thread per token row
        const int row = (warp & 3) * 32 + lane;
        const uint32_t trow = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        int n_tile = 0;
        for (int tile = first; tile < tiles; tile += stride, ++n_tile) {
            const int b = n_tile & 1;
            const int nt = tile / m_groups, mt = (tile - nt * m_groups) * IO::CLUSTER + (int)rank;
            const int tok = mt * TC_BM + row;
            mbar_wait(&acc_full[b], (n_tile >> 1) & 1);
            __syncwarp();
            fence_after_sync();
            tc_drain_row(p, trow + b * TC_BN, tok, nt);
            // this accumulator is in registers or stored: the product warp may write it again
            fence_before_sync();
            tc_arrive(&acc_empty[b]);
        }
    }
    fence_before_sync();
    __syncthreads();
    if (IO::CLUSTER > 1) {        // nobody leaves while the other block may still write to it or signal it
        asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    }
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512));
}


// Checks, tensor maps and launch, shared by the entry points.
template <class IO>
int gemm_tc_launch(const void* X, int ldx, const void* W, void* Y, int ldy, float* resid, int M, int N, int K, int epi,
                   cudaStream_t stream) {
    PL_REQUIRE(epi >= TC_BF16 && epi <= TC_ADD, "gemm_tc: epilogue %d", epi);
    PL_REQUIRE(M >= 1 && N >= 1 && K >= 64 && K % 64 == 0 && ldx % 8 == 0 && (epi == TC_ADD || ldy % 8 == 0),
               "gemm_tc: M=%d N=%d K=%d (multiple of 64) ldx=%d ldy=%d", M, N, K, ldx, ldy);
    PL_REQUIRE(epi == TC_ADD ? (resid != nullptr && N % 4 == 0 && ((uintptr_t)resid & 15) == 0)
                             : (Y != nullptr && ldy >= N && ((uintptr_t)Y & 15) == 0),
               "gemm_tc: output missing, misaligned or ldy < N");
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        PL_CUDA(cudaGetDevice(&dev));
        PL_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        PL_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<IO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM));
    }
    TcParams p = {};
    p.Y = Y;
    p.resid = resid;
    p.ldy = ldy;
    p.M = M;
    p.N = N;
    p.K = K;
    p.I = N;
    p.epi = epi;
    p.m_tiles = ((M + TC_BM - 1) / TC_BM + IO::CLUSTER - 1) / IO::CLUSTER * IO::CLUSTER;
    p.n_tiles = epi == TC_SILU ? (N + 127) / 128 : (N + TC_BN - 1) / TC_BN;
    const int w_rows = epi == TC_SILU ? 2 * N : N;
    alignas(64) CUtensorMap x_map, w_map;
    if (!tensor_map_bf16(&x_map, X, (unsigned long long)M, (unsigned long long)K, (unsigned long long)ldx, 128) ||
        !tensor_map_bf16(&w_map, W, (unsigned long long)w_rows, (unsigned long long)K, (unsigned long long)K, 128))
        return 1;
    const int groups = p.m_tiles / IO::CLUSTER * p.n_tiles;
    const int max_groups = sms / IO::CLUSTER;
    const int grid = (groups < max_groups ? groups : max_groups) * IO::CLUSTER;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = TC_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    static const bool no_pdl = getenv("PAGED_LLM_B200_NO_PDL") != nullptr;
    if (!no_pdl) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    if (IO::CLUSTER > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = IO::CLUSTER;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    PL_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc_kernel<IO>, p, x_map, w_map));
    return 0;
}

}  // namespace

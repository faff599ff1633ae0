// The many-token product (see gemm_tc.cuh) with the two blocks of a cluster on one tile of 256 tokens
// x 256 features (tcgen05.mma.cta_group::2): each block keeps its own 128 tokens of X and one half
// of the 256 rows of W behind the tile, the tensor cores of both SMs read both halves of W, and each
// block's tensor memory holds the accumulators of its own 128 tokens (all 256 features, twice: one
// is drained while the other is filled).  A stage of the TMA ring is 32 KB per block for 512 cycles
// of products, six stages deep.  Blocks are persistent; tiles are taken in bands (duo_tile).
//
// Roles per block: one thread brings this block's X and W boxes in (cp.async.bulk.tensor.2d with
// 128-byte swizzle and .cta_group::2, which lets the copy signal the barrier of the other block);
// one thread of the first block of the pair issues the products for both and commits on the
// barriers of both (tcgen05.commit with a block mask); four warps per block drain the accumulator
// of their own tokens (tcgen05.ld, the epilogue's arithmetic, 16-byte stores) and tell the first
// block when it may be written again.  No TMA load here delivers to more than one block.  Every
// wait is bounded; a thread that gave up once stops waiting at all.
//
// Measured against a block per 128 x 256 tile with four stages of 48 KB (the form this replaced):
// gate/up + SiLU-mul at 2,048 tokens 76.7 against 84.0 us, tensor pipe 65 against 61 % of active cycles.
#pragma once

#include "gemm_tc.cuh"

namespace {

// measured on the gate/up product at 2,048 tokens: 4 stages 2 % slower per prefill, 5 to 7 the same
constexpr int DUO_STAGES = 6;
constexpr int DUO_A_BYTES = 128 * 128, DUO_B_BYTES = 128 * 128, DUO_STAGE_BYTES = DUO_A_BYTES + DUO_B_BYTES;
constexpr size_t DUO_SMEM = (size_t)DUO_STAGES * DUO_STAGE_BYTES + 1024;

// The address, in the cluster's window, of `local` (an address in this block's shared memory) in block `rank`.
__device__ __forceinline__ uint32_t duo_map(uint32_t local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
__device__ __forceinline__ void duo_tma(void* dst, const CUtensorMap* map, int col, int row, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];\n" ::"r"(saddr(dst)),
        "l"(map), "r"(col), "r"(row), "r"(bar_cluster)
        : "memory");
}
__device__ __forceinline__ void duo_arrive(uint32_t bar_cluster) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(bar_cluster) : "memory");
}
__device__ __forceinline__ void duo_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.u32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// Arrives, once the products issued so far are done, on the barrier at this offset in both blocks.
__device__ __forceinline__ void duo_commit(uint64_t* bar) {
    const uint16_t both = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n" ::"r"(
            saddr(bar)),
        "h"(both)
        : "memory");
}

// The order of tiles: bands of DUO_BAND token tiles (pairs of 128), feature tile by feature tile within a
// band, so that the pairs running at a time share few rows of X and few rows of W (both stay in L2).
constexpr int DUO_BAND = 8;
__device__ __forceinline__ void duo_tile(int tile, int m_pairs, int n_tiles, int& nt, int& mp) {
    const int per_band = DUO_BAND * n_tiles;
    const int band = tile / per_band, in_band = tile - band * per_band;
    const int rows = min(DUO_BAND, m_pairs - band * DUO_BAND);
    nt = in_band / rows;
    mp = band * DUO_BAND + (in_band - nt * rows);
}

__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_duo_kernel(TcParams p, const __grid_constant__ CUtensorMap x_map,
                                                                    const __grid_constant__ CUtensorMap w_map) {
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full[DUO_STAGES], empty[DUO_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_slot;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(rank));
    const bool leader = rank == 0;
    const int m_pairs = p.m_tiles / 2;
    const int tiles = m_pairs * p.n_tiles;
    const int first = blockIdx.x / 2, stride = gridDim.x / 2;
    const int k_steps = p.K / TC_BK;

    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(saddr(&tmem_base_slot)),
                     "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::);
    }
    if (tid == 0) {
        for (int s = 0; s < DUO_STAGES; ++s) {
            mbar_init(&full[s], 1);         // the first block's arrival with the bytes of both blocks' boxes
            mbar_init(&empty[s], 1);        // the commit after the products of the stage
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);     // the commit after the last product of a tile
            mbar_init(&acc_empty[b], 256);  // the epilogue threads of both blocks (counted in the first block)
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    // the other block's barriers and tensor memory must exist before anything of ours reaches them
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- copies (both blocks)
        if (lane == 0) {
            bool alive = true;
            int it = 0;
            for (int tile = first; tile < tiles && alive; tile += stride) {
                int nt, mp;
                duo_tile(tile, m_pairs, p.n_tiles, nt, mp);
                const int mt = mp * 2 + (int)rank;
                // this block's half of the 256 rows of W: the first 128 (gate rows) or the second (up rows)
                const int w_row = p.epi == TC_SILU ? (leader ? nt * 128 : p.I + nt * 128) : nt * 256 + (int)rank * 128;
                for (int ks = 0; ks < k_steps; ++ks, ++it) {
                    const int s = it % DUO_STAGES;
                    if (it >= DUO_STAGES && !mbar_wait(&empty[s], ((it / DUO_STAGES) - 1) & 1)) {
                        alive = false;
                        break;
                    }
                    unsigned char* st = smem + (size_t)s * DUO_STAGE_BYTES;
                    if (leader) tc_arrive_expect(&full[s], 2 * DUO_STAGE_BYTES);
                    const uint32_t bar = duo_map(saddr(&full[s]), 0);
                    duo_tma(st, &x_map, ks * TC_BK, mt * TC_BM, bar);
                    duo_tma(st + DUO_A_BYTES, &w_map, ks * TC_BK, w_row, bar);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- products (the first block, for both)
        if (lane == 0 && leader) {
            constexpr uint32_t IDESC = instr_desc(256, TC_BN, false);
            bool alive = true;
            int it = 0, n_tile = 0;
            for (int tile = first; tile < tiles && alive; tile += stride, ++n_tile) {
                const int b = n_tile & 1;
                if (n_tile >= 2 && !mbar_wait(&acc_empty[b], ((n_tile >> 1) - 1) & 1)) break;
                fence_after_sync();
                for (int ks = 0; ks < k_steps; ++ks, ++it) {
                    const int s = it % DUO_STAGES;
                    if (!mbar_wait(&full[s], (it / DUO_STAGES) & 1)) {
                        alive = false;
                        break;
                    }
                    fence_after_sync();
                    const uint32_t xa = saddr(smem + (size_t)s * DUO_STAGE_BYTES), wa = xa + DUO_A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < TC_BK / 16; ++kk)
                        duo_mma(tmem_base + b * TC_BN, smem_desc(xa + kk * 32, 16, 1024), smem_desc(wa + kk * 32, 16, 1024),
                                IDESC, ks > 0 || kk > 0);
                    duo_commit(&empty[s]);
                }
                if (alive) duo_commit(&acc_full[b]);
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
            int nt, mp;
            duo_tile(tile, m_pairs, p.n_tiles, nt, mp);
            const int mt = mp * 2 + (int)rank;
            // all lanes leave together: the loads of tensor memory below are warp-wide
            const bool ready = mbar_wait(&acc_full[b], (n_tile >> 1) & 1);
            if (!__all_sync(0xffffffffu, ready)) break;
            fence_after_sync();
            tc_drain_row(p, trow + b * TC_BN, mt * TC_BM + row, nt);
            fence_before_sync();
            duo_arrive(duo_map(saddr(&acc_empty[b]), 0));
        }
    }
    fence_before_sync();
    __syncthreads();
    // nobody leaves while the other block may still read its shared memory or signal its barriers
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512));
}

// The same checks and interface as gemm_tc_launch.
int gemm_tc_duo_launch(const void* X, int ldx, const void* W, void* Y, int ldy, float* resid, int M, int N, int K, int epi,
                       cudaStream_t stream) {
    PL_REQUIRE(epi >= TC_BF16 && epi <= TC_ADD, "gemm_tc_duo: epilogue %d", epi);
    PL_REQUIRE(M >= 1 && N >= 1 && K >= 64 && K % 64 == 0 && ldx % 8 == 0 && (epi == TC_ADD || ldy % 8 == 0),
               "gemm_tc_duo: M=%d N=%d K=%d (multiple of 64) ldx=%d ldy=%d", M, N, K, ldx, ldy);
    PL_REQUIRE(epi == TC_ADD ? (resid != nullptr && N % 4 == 0 && ((uintptr_t)resid & 15) == 0)
                             : (Y != nullptr && ldy >= N && ((uintptr_t)Y & 15) == 0),
               "gemm_tc_duo: output missing, misaligned or ldy < N");
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        PL_CUDA(cudaGetDevice(&dev));
        PL_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        PL_CUDA(cudaFuncSetAttribute(gemm_tc_duo_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DUO_SMEM));
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
    p.m_tiles = ((M + TC_BM - 1) / TC_BM + 1) / 2 * 2;
    p.n_tiles = epi == TC_SILU ? (N + 127) / 128 : (N + TC_BN - 1) / TC_BN;
    const int w_rows = epi == TC_SILU ? 2 * N : N;
    alignas(64) CUtensorMap x_map, w_map;
    if (!tensor_map_bf16(&x_map, X, (unsigned long long)M, (unsigned long long)K, (unsigned long long)ldx, 128) ||
        !tensor_map_bf16(&w_map, W, (unsigned long long)w_rows, (unsigned long long)K, (unsigned long long)K, 128))
        return 1;
    const int pairs = p.m_tiles / 2 * p.n_tiles;
    const int max_pairs = sms / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((pairs < max_pairs ? pairs : max_pairs) * 2);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = DUO_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    static const bool no_pdl = getenv("PAGED_LLM_B200_NO_PDL") != nullptr;
    if (!no_pdl) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 2;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    PL_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc_duo_kernel, p, x_map, w_map));
    return 0;
}

}  // namespace

// Paged prefill attention on the 5th-generation tensor cores (tcgen05) with the
// accumulators in tensor memory, in bfloat16: a block-synchronous kernel for head size 64
// (namespace tc) and a warp-specialised one for head sizes 64 and 128 (namespace tc2).
//
// One thread block takes a tile of 128 query rows of one kv head (row = token * G
// + head within the group, as in attention_bf16.cuh) and walks its keys 128 at a
// time:
//   S = Q K^T     tcgen05.mma 128x128x64, Q and the key tile in shared memory
//                 (K-major, 128-byte swizzle), S in tensor memory (128 columns);
//   softmax       two threads per row, each with half of the columns: they read S
//                 from tensor memory (tcgen05.ld), mask by absolute position,
//                 exchange their maxima through shared memory, keep the running
//                 maximum and sum in float32, rescale O in tensor memory where a
//                 maximum moved, and write P in bfloat16 to shared memory;
//   O += P V      tcgen05.mma 128x64x128, P from shared memory, the value tile as
//                 the MN-major operand, O in tensor memory (64 columns).
// Keys and values come through the block table with cp.async into two swizzled
// stages, zero-filled outside the key range.  A block allocates 256 columns of
// tensor memory and 97 KiB of shared memory, so two blocks share an SM and one
// block's softmax overlaps the other's products.  Completion of the products is
// signalled by tcgen05.commit on mbarriers; every wait is bounded and counts a
// timeout instead of hanging (pl_attention_tc_timeouts).
//
// Semantics are those of attention_bf16.cuh (xiyiji/paged-llm
// pagedllm/attention/triton_kernel.py:22-93): float32 scores, maximum, sum and
// accumulator; P rounded to bfloat16 for the second product.
#pragma once

#include "attention_common.cuh"
#include "tcgen05.cuh"
#include "tensor_map.cuh"

namespace tc {

constexpr int BM = 128, BN = 128, D = 64;
constexpr int THREADS = 256;          // two threads per query row: each takes half of the columns
constexpr int TMEM_COLS = 256;           // S: columns 0..127, O: 128..191
constexpr int Q_BYTES = BM * 128, KV_STAGE_BYTES = BN * 128, P_BYTES = BM * BN * 2;
constexpr int SMEM_BYTES = Q_BYTES + 3 * KV_STAGE_BYTES + P_BYTES + 1024;     // + alignment slack
__global__ void __launch_bounds__(THREADS, 2) attn_tc_kernel(AttnParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const AttnItem it = attn_decode_item(p, blockIdx.x / p.nkv, BM, BN);
    if (!it.valid) return;

    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
    unsigned char* Qs = smem;                                  // [128][128 B]
    unsigned char* Ks = Qs + Q_BYTES;                          // [128][128 B]: free again once S is done
    unsigned char* Vs = Ks + KV_STAGE_BYTES;                   // [2][128][128 B]
    unsigned char* Ps = Vs + 2 * KV_STAGE_BYTES;               // [2 column blocks][128][128 B]
    __shared__ uint64_t bar_s, bar_o;
    __shared__ uint32_t tmem_base_slot;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kvh = blockIdx.x % p.nkv, G = p.nh / p.nkv;
    const __nv_bfloat16* q = (const __nv_bfloat16*)p.q;
    const __nv_bfloat16* kv = (const __nv_bfloat16*)p.kv;
    const int* bt = p.block_table + (size_t)it.seq * p.bt_stride;
    const size_t v_off = (size_t)p.nkv * p.ps * D;

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(saddr(&tmem_base_slot)),
                     "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    if (tid == 0) {
        mbar_init(&bar_s, 1);
        mbar_init(&bar_o, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }

    // Q tile: row R = token * G + head; eight 16-byte chunks per row
    for (int e = tid; e < BM * 8; e += THREADS) {
        const int r = e >> 3, c = e & 7;
        const int R = it.row_base + r;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (R < it.rows_total)
            v = *reinterpret_cast<const uint4*>(q + (size_t)(it.q0 + R / G) * p.q_stride + (kvh * G + R % G) * D + c * 8);
        *reinterpret_cast<uint4*>(Qs + swz(r, c)) = v;
    }

    // One tile of keys (sel 0) or values (sel 1): every thread looks up the pages of its rows
    // first, then issues the copies.
    auto load_tile = [&](unsigned char* dst, int kt, int sel) {
        constexpr int ITERS = BN * 8 / THREADS;
        int pg[ITERS];
#pragma unroll
        for (int i = 0; i < ITERS; ++i) {
            const int n = kt + ((tid + i * THREADS) >> 3);
            const int pi = p.ps_shift >= 0 ? n >> p.ps_shift : n / p.ps;
            pg[i] = n < it.key_hi ? bt[pi] : -1;
        }
#pragma unroll
        for (int i = 0; i < ITERS; ++i) {
            const int e = tid + i * THREADS;
            const int j = e >> 3, c = e & 7;
            const int n = kt + j;
            const int po = p.ps_shift >= 0 ? n & (p.ps - 1) : n % p.ps;
            const bool ok = pg[i] >= 0;
            const __nv_bfloat16* src =
                ok ? kv + ((((size_t)pg[i] * 2 + sel) * p.nkv + kvh) * p.ps + po) * D + c * 8 : kv;
            cp16(dst + swz(j, c), src, ok ? 16 : 0);
        }
        cp_commit();
    };

    const int n_tiles = (it.key_hi - it.key_lo + BN - 1) / BN;
    if (n_tiles > 0) {
        load_tile(Ks, it.key_lo, 0);
        load_tile(Vs, it.key_lo, 1);
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    const int half = warp >> 2;                                 // which half of the columns this thread takes
    const uint32_t tmem_row = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);   // this warp's 32 lanes
    const uint32_t tmem_s = tmem_row + half * 64, tmem_o = tmem_row + 128 + half * 32;
    __shared__ float xmax[2][BM];                               // the halves' maxima of the current tile

    const int r = (warp & 3) * 32 + lane;                       // this thread's row of the tile
    const int R = it.row_base + r;
    const int pos = R < it.rows_total ? it.lk - it.nq + R / G : -1;
    float m_run = -INFINITY, l_run = 0.f;
    const float scale_log2 = p.scale * 1.4426950408889634f;
    constexpr uint32_t IDESC_S = instr_desc(BM, BN, false), IDESC_O = instr_desc(BM, D, true);
    uint32_t phase_s = 0, phase_o = 0;

    // cp.async groups: at the top of iteration t the copies of K(t) and V(t) are in flight or done;
    // V(t+1) is requested there, K(t+1) as soon as S(t) is done with the key stage.
    for (int t = 0; t < n_tiles; ++t) {
        const int stage = t & 1;
        const bool more = t + 1 < n_tiles;
        if (t > 0) {
            // P V of the tile before must be done before its P, its value stage and O are touched
            mbar_wait(&bar_o, phase_o);
            phase_o ^= 1;
            __syncwarp();
            fence_after_sync();
        }
        if (more) load_tile(Vs + (stage ^ 1) * KV_STAGE_BYTES, it.key_lo + (t + 1) * BN, 1);
        if (more) cp_wait<1>(); else cp_wait<0>();             // all but V(t+1): K(t) and V(t) have landed
        fence_async_smem();                                     // cp.async and Q stores -> tensor-core reads
        __syncthreads();
        if (tid == 0) {
            fence_after_sync();
            const uint32_t qa = saddr(Qs), ka = saddr(Ks);
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk)
                mma_f16(tmem_base, smem_desc(qa + kk * 32, 16, 1024), smem_desc(ka + kk * 32, 16, 1024), IDESC_S, kk > 0);
            mma_commit(&bar_s);
        }
        mbar_wait(&bar_s, phase_s);
        phase_s ^= 1;
        __syncwarp();
        fence_after_sync();
        if (more) load_tile(Ks, it.key_lo + (t + 1) * BN, 0);   // the key stage is free again

        // softmax of this thread's half row, in two passes over S in tensor memory
        const int kbase = it.key_lo + t * BN;
        const int kcol = kbase + half * 64;
        const bool row_full = p.window <= 0 && kbase + BN <= it.key_hi && kbase + BN - 1 <= pos;
        const bool warp_full = __all_sync(0xffffffffu, row_full);
        float m_tile = -INFINITY;
        float sv[32];
        if (warp_full) {
#pragma unroll 1
            for (int cb = 0; cb < 2; ++cb) {
                tmem_ld32(tmem_s + cb * 32, sv);
#pragma unroll
                for (int i = 0; i < 32; ++i) m_tile = fmaxf(m_tile, sv[i]);
            }
            m_tile *= scale_log2;
        } else {
#pragma unroll 1
            for (int cb = 0; cb < 2; ++cb) {
                tmem_ld32(tmem_s + cb * 32, sv);
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int n = kcol + cb * 32 + i;
                    const bool vis = n < it.key_hi && n <= pos && (p.window <= 0 || n > pos - p.window);
                    m_tile = fmaxf(m_tile, vis ? sv[i] * scale_log2 : -INFINITY);
                }
            }
        }
        xmax[half][r] = m_tile;
        __syncthreads();
        m_tile = fmaxf(m_tile, xmax[half ^ 1][r]);
        const float m_new = fmaxf(m_run, m_tile);
        const float alpha = m_run == -INFINITY ? 0.f : ex2(m_run - m_new);
        const bool changed = m_new != m_run;
        m_run = m_new;
        l_run *= alpha;
        const float neg_m = m_run == -INFINITY ? 0.f : -m_run;
        float l_add = 0.f;
#pragma unroll 1
        for (int cb = 0; cb < 2; ++cb) {
            tmem_ld32(tmem_s + cb * 32, sv);
            uint32_t packed[16];
            if (warp_full) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float p0 = ex2(fmaf(sv[2 * i], scale_log2, neg_m));
                    const float p1 = ex2(fmaf(sv[2 * i + 1], scale_log2, neg_m));
                    l_add += p0 + p1;
                    __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
                    packed[i] = *reinterpret_cast<uint32_t*>(&b);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float pv[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int n = kcol + cb * 32 + 2 * i + e;
                        const bool vis = n < it.key_hi && n <= pos && (p.window <= 0 || n > pos - p.window);
                        pv[e] = vis ? ex2(fmaf(sv[2 * i + e], scale_log2, neg_m)) : 0.f;
                    }
                    l_add += pv[0] + pv[1];
                    __nv_bfloat162 b = __floats2bfloat162_rn(pv[0], pv[1]);
                    packed[i] = *reinterpret_cast<uint32_t*>(&b);
                }
            }
            unsigned char* blk = Ps + half * (BM * 128);            // this half's 64-key column block
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4)
                *reinterpret_cast<uint4*>(blk + swz(r, cb * 4 + c4)) =
                    make_uint4(packed[4 * c4], packed[4 * c4 + 1], packed[4 * c4 + 2], packed[4 * c4 + 3]);
        }
        l_run += l_add;
        // rescale O where a row's maximum moved (skipped when it moved in no row of the warp)
        if (t > 0 && __any_sync(0xffffffffu, changed)) {
            tmem_ld32(tmem_o, sv);
#pragma unroll
            for (int i = 0; i < 32; ++i) sv[i] *= alpha;
            tmem_st32(tmem_o, sv);
            tmem_st_wait();
        }
        fence_async_smem();                                     // P (generic stores) -> tensor-core reads
        fence_before_sync();
        __syncthreads();
        if (tid == 0) {
            fence_after_sync();
            const uint32_t pa = saddr(Ps), va = saddr(Vs + stage * KV_STAGE_BYTES);
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk)
                mma_f16(tmem_base + 128, smem_desc(pa + (kk >> 2) * (BM * 128) + (kk & 3) * 32, 16, 1024),
                        smem_desc(va + kk * 2048, 16, 1024), IDESC_O, t > 0 || kk > 0);
            mma_commit(&bar_o);
        }
    }
    if (n_tiles > 0) {
        mbar_wait(&bar_o, phase_o);
        __syncwarp();
        fence_after_sync();
        // the row sum is the sum of the halves' sums
        xmax[half][r] = l_run;
        __syncthreads();
        const float l_row = l_run + xmax[half ^ 1][r];
        // every lane takes part in the aligned load; only valid rows store their 32 columns
        const float inv = l_row > 0.f ? 1.0f / l_row : 0.f;
        const int Rc = pos >= 0 ? R : it.row_base;
        const int tok = Rc / G, head = kvh * G + Rc % G;
        __nv_bfloat16* o_row = (__nv_bfloat16*)p.out + (size_t)(it.q0 + tok) * p.out_stride + head * D + half * 32;
        float o[32];
        tmem_ld32(tmem_o, o);
        if (pos >= 0) {
#pragma unroll
            for (int c8 = 0; c8 < 4; ++c8) {
                __nv_bfloat162 b[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) b[i] = __floats2bfloat162_rn(o[c8 * 8 + 2 * i] * inv, o[c8 * 8 + 2 * i + 1] * inv);
                *reinterpret_cast<uint4*>(o_row + c8 * 8) = *reinterpret_cast<uint4*>(b);
            }
        }
        __syncwarp();
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS));
}

inline int launch(const AttnParams& p, cudaStream_t stream) {
    static bool attr_set = false;
    if (!attr_set) {
        PL_CUDA(cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        PL_CUDA(cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                     (int)cudaSharedmemCarveoutMaxShared));
        attr_set = true;
    }
    PL_CUDA(launch_pdl(attn_tc_kernel, dim3(p.n_work * p.nkv), dim3(THREADS), (size_t)SMEM_BYTES, stream, p));
    return 0;
}

}  // namespace tc

// ---------------------------------------------------------------------------------------------
// The same attention with the phases of a block running side by side instead of one after the
// other.  Warps have roles: four softmax warps (one thread per query row, the whole row of 64
// scores in registers), one warp that issues the tensor-core products, two warps that bring keys
// and values in with TMA: the pool of one layer is a 2-D tensor [pages * 2 * kv_heads *
// page_size, 64] whose rows are 128 bytes, a box is the rows of one page (at most 64) and lands in
// shared memory in the 128-byte swizzle the products read.  Scores are double-buffered in tensor
// memory (two tiles of 64 keys); P never leaves tensor memory: the softmax thread writes it, two
// bfloat16 per column, over the first half of the scores it has just read, and the second product
// takes it from there as its A operand.  Keys and values sit in rings of four stages each;
// everything is handed over through mbarriers:
//   k_full[s], v_full[s]    the boxes of a stage of keys / values have landed (TMA complete_tx)
//   k_empty[s], v_empty[s]  the product reading the stage is done              (tcgen05.commit)
//   s_full[b]    S[b] = Q K^T is in tensor memory        (tcgen05.commit)
//   p_full[b]    P[b] is in tensor memory, O is rescaled, stray value rows are zeroed (softmax threads)
//   pv_done[b]   O += P[b] V is done: S[b] may be written again (tcgen05.commit)
// The product warp issues P(t) V(t) and then S(t+2), while the softmax warps work on S(t+1).
// Key tiles start at multiples of 64 so that a box never straddles a page; keys outside the
// block's range are masked by position, and their value rows are zeroed in shared memory (a page
// may hold anything behind the last token).
// Head size 128 has the same shape with rows of two 64-element panels (the 128-byte swizzle spans
// one): a TMA box per page and panel, the first product over both panels, the second one 128
// columns wide (O takes 128 columns of tensor memory), rings of two stages.
// Needs a page size that is a power of two >= 8; other page sizes run the kernel above (head size
// 64) or the mma.sync kernel (head size 128).
namespace tc2 {

using tc::saddr;
using tc::mbar_init;
using tc::mbar_wait;
using tc::smem_desc;
using tc::instr_desc;
using tc::mma_f16;
using tc::mma_f16_ts;
using tc::mma_commit;
using tc::fence_before_sync;
using tc::fence_after_sync;
using tc::fence_async_smem;
using tc::tmem_st32;
using tc::tmem_st_wait;
using tc::ex2;
using tc::swz;


constexpr int BM = 128, BN = 64;
constexpr int SOFTMAX_WARPS = 4, MMA_WARP = 4, K_WARP = 5, V_WARP = 6;
constexpr int THREADS = (SOFTMAX_WARPS + 3) * 32;                   // 224
constexpr int TMEM_COLS = 256;               // S0 / P0: 0..63, S1 / P1: 64..127, O: 128..128+D-1
constexpr float LAZY_LOG2 = 8.f;
// A head of D elements is D / 64 panels of 64 elements (128 bytes, the span of the swizzle): Q,
// a stage of keys and a stage of values are each `PANELS` tiles of [rows][128 B], one behind the
// other.  Two blocks share an SM for either head size, so the deeper rows get the shallower ring.
template <int D>
struct Shape {
    static_assert(D == 64 || D == 128, "head sizes 64 and 128");
    static constexpr int PANELS = D / 64;
    static constexpr int STAGES = D == 64 ? 4 : 2;
    static constexpr int Q_PANEL = BM * 128, K_PANEL = BN * 128;
    static constexpr int Q_BYTES = PANELS * Q_PANEL, K_BYTES = PANELS * K_PANEL;
    static constexpr int SMEM_BYTES = Q_BYTES + 2 * STAGES * K_BYTES + 1024;
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(saddr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(saddr(bar)), "r"(bytes) : "memory");
}
// One box of the tensor map at rows [row, row + box rows), columns [col, col + 64) (col a
// multiple of 64), to shared memory; the bytes are counted on `bar`.
__device__ __forceinline__ void tma_box(void* dst, const CUtensorMap* map, int col, int row, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::
            "r"(saddr(dst)), "l"(map), "r"(col), "r"(row), "r"(saddr(bar))
        : "memory");
}
// Two float32 operations in one instruction (sm_100): the pair lives in a 64-bit register.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// 64 columns of this thread's lane of tensor memory, one wait for both halves.
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float (&v)[64]) {
    uint32_t r[64];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t* q = r + 32 * h;
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
            : "=r"(q[0]), "=r"(q[1]), "=r"(q[2]), "=r"(q[3]), "=r"(q[4]), "=r"(q[5]), "=r"(q[6]), "=r"(q[7]), "=r"(q[8]),
              "=r"(q[9]), "=r"(q[10]), "=r"(q[11]), "=r"(q[12]), "=r"(q[13]), "=r"(q[14]), "=r"(q[15]), "=r"(q[16]),
              "=r"(q[17]), "=r"(q[18]), "=r"(q[19]), "=r"(q[20]), "=r"(q[21]), "=r"(q[22]), "=r"(q[23]), "=r"(q[24]),
              "=r"(q[25]), "=r"(q[26]), "=r"(q[27]), "=r"(q[28]), "=r"(q[29]), "=r"(q[30]), "=r"(q[31])
            : "r"(taddr + 32 * h));
    }
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}

// WIDE (head size 128 only): O += P V as one product 128 x 128 x 16 per step, the value panels
// being the two 64-column groups of its MN-major operand, instead of one product per panel.
template <int D, bool WIDE>
__global__ void __launch_bounds__(THREADS, 2) attn_tc2_kernel(AttnParams p, const __grid_constant__ CUtensorMap kv_map) {
    using SH = Shape<D>;
    constexpr int PANELS = SH::PANELS, STAGES = SH::STAGES, Q_PANEL = SH::Q_PANEL, K_PANEL = SH::K_PANEL;
    constexpr int Q_BYTES = SH::Q_BYTES, K_BYTES = SH::K_BYTES;
    pdl_launch_dependents();
    pdl_wait();
    const AttnItem it = attn_decode_item(p, blockIdx.x / p.nkv, BM, BN);
    if (!it.valid) return;

    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
    unsigned char* Qs = smem;                                  // [PANELS][128][128 B]
    unsigned char* Ks = Qs + Q_BYTES;                          // [STAGES][PANELS][64 keys][128 B]
    unsigned char* Vs = Ks + STAGES * K_BYTES;                 // [STAGES][PANELS][64 keys][128 B]
    __shared__ uint64_t k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES];
    __shared__ uint64_t s_full[2], p_full[2], pv_done[2];
    __shared__ uint32_t tmem_base_slot;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kvh = blockIdx.x % p.nkv, G = p.nh / p.nkv;
    const __nv_bfloat16* q = (const __nv_bfloat16*)p.q;
    const int key0 = it.key_lo & ~(BN - 1);                    // tiles start at multiples of 64
    const int n_tiles = (it.key_hi - key0 + BN - 1) / BN;

    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(saddr(&tmem_base_slot)),
                     "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&s_full[b], 1);
            mbar_init(&p_full[b], SOFTMAX_WARPS * 32);
            mbar_init(&pv_done[b], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    // Q tile: row R = token * G + head; eight 16-byte chunks per row and panel
    for (int e = tid; e < BM * 8 * PANELS; e += THREADS) {
        const int r = e / (8 * PANELS), c16 = e % (8 * PANELS);
        const int R = it.row_base + r;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (R < it.rows_total)
            v = *reinterpret_cast<const uint4*>(q + (size_t)(it.q0 + R / G) * p.q_stride + (kvh * G + R % G) * D + c16 * 8);
        *reinterpret_cast<uint4*>(Qs + (c16 >> 3) * Q_PANEL + swz(r, c16 & 7)) = v;
    }
    fence_async_smem();
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp >= K_WARP) {
        // ---------------------------------------------------------------- copy warps (keys, values): lane i brings box i
        const bool values = warp == V_WARP;
        const int* bt = p.block_table + (size_t)it.seq * p.bt_stride;
        const int box_rows = min(p.ps, BN), boxes = BN / box_rows;
        const uint32_t box_bytes = box_rows * 128;
        const int row_add = values ? p.nkv * p.ps : 0;         // rows from a page's keys to its values
        unsigned char* ring = values ? Vs : Ks;
        uint64_t* full = values ? v_full : k_full;
        uint64_t* empty = values ? v_empty : k_empty;
        auto page_of = [&](int t) {                             // page of this lane's box of tile t, or -1
            const int n0 = key0 + t * BN + lane * box_rows;
            if (t >= n_tiles || lane >= boxes || n0 >= it.key_hi || n0 + box_rows <= it.key_lo) return -1;
            return bt[n0 >> p.ps_shift];
        };
        int pg_next = page_of(0);
        for (int t = 0; t < n_tiles; ++t) {
            const int s = t % STAGES;
            const int pg = pg_next;
            pg_next = page_of(t + 1);
            if (t >= STAGES) mbar_wait(&empty[s], ((t / STAGES) - 1) & 1);
            const bool ok = pg >= 0;
            const int n_ok = __popc(__ballot_sync(0xffffffffu, ok));
            if (lane == 0) mbar_arrive_expect(&full[s], n_ok * box_bytes * PANELS);
            __syncwarp();
            if (ok) {
                const int n0 = key0 + t * BN + lane * box_rows;
                const int row = (pg * 2 * p.nkv + kvh) * p.ps + (n0 & (p.ps - 1)) + row_add;
#pragma unroll
                for (int c = 0; c < PANELS; ++c)
                    tma_box(ring + s * K_BYTES + c * K_PANEL + lane * box_bytes, &kv_map, c * 64, row, &full[s]);
            }
        }
    } else if (warp == MMA_WARP) {
        // ---------------------------------------------------------------- product warp: one thread issues
        if (lane == 0) {
            constexpr uint32_t IDESC_S = instr_desc(BM, BN, false), IDESC_O = instr_desc(BM, WIDE ? D : 64, true);
            const uint32_t qa = saddr(Qs);
            auto issue_s = [&](int t) {                     // S[t & 1] = Q K(t)^T
                const int b = t & 1, s = t % STAGES;
                mbar_wait(&k_full[s], (t / STAGES) & 1);
                if (t >= 2) mbar_wait(&pv_done[b], ((t - 2) >> 1) & 1);    // P(t-2), which lies over S[b], is consumed
                fence_after_sync();
                const uint32_t ka = saddr(Ks + s * K_BYTES);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk)          // four steps of 16 elements per panel
                    mma_f16(tmem_base + b * 64, smem_desc(qa + (kk >> 2) * Q_PANEL + (kk & 3) * 32, 16, 1024),
                            smem_desc(ka + (kk >> 2) * K_PANEL + (kk & 3) * 32, 16, 1024), IDESC_S, kk > 0);
                mma_commit(&s_full[b]);
                mma_commit(&k_empty[s]);
            };
            // Scores run ahead of the second product: while the softmax works on S(u + 1), the
            // tensor cores do P(u) V(u) and then S(u + 2) into the columns P(u) leaves.
            if (n_tiles > 0) issue_s(0);
            if (n_tiles > 1) issue_s(1);
            for (int u = 0; u < n_tiles; ++u) {
                const int bu = u & 1, su = u % STAGES;
                mbar_wait(&v_full[su], (u / STAGES) & 1);
                mbar_wait(&p_full[bu], (u >> 1) & 1);
                fence_after_sync();
                const uint32_t va = saddr(Vs + su * K_BYTES);
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk) {        // P from tensor memory: 8 packed columns per step
                    if (WIDE) {
                        // groups of 64 columns of the MN-major operand lie a panel apart
                        mma_f16_ts(tmem_base + 128, tmem_base + bu * 64 + kk * 8, smem_desc(va + kk * 2048, K_PANEL, 1024),
                                   IDESC_O, u > 0 || kk > 0);
                    } else {
#pragma unroll
                        for (int c = 0; c < PANELS; ++c)
                            mma_f16_ts(tmem_base + 128 + c * 64, tmem_base + bu * 64 + kk * 8,
                                       smem_desc(va + c * K_PANEL + kk * 2048, 16, 1024), IDESC_O, u > 0 || kk > 0);
                    }
                }
                mma_commit(&pv_done[bu]);
                mma_commit(&v_empty[su]);
                if (u + 2 < n_tiles) issue_s(u + 2);
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- softmax warps: one thread per row
        const int r = tid;
        const int R = it.row_base + r;
        const int pos = R < it.rows_total ? it.lk - it.nq + R / G : -1;
        const uint32_t tmem_row = tmem_base + ((uint32_t)(warp * 32) << 16);
        const uint32_t tmem_o = tmem_row + 128;
        const float scale_log2 = p.scale * 1.4426950408889634f;
        float m_run = -INFINITY, l_run = 0.f;
        float sv[64];
        for (int t = 0; t < n_tiles; ++t) {
            const int b = t & 1;
            mbar_wait(&s_full[b], (t >> 1) & 1);
            __syncwarp();
            fence_after_sync();
            tmem_ld64(tmem_row + b * 64, sv);
            const int kbase = key0 + t * BN;
            const bool row_full = p.window <= 0 && kbase >= it.key_lo && kbase + BN <= it.key_hi && kbase + BN - 1 <= pos;
            const bool warp_full = __all_sync(0xffffffffu, row_full);
            if (!warp_full) {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const int n = kbase + i;
                    const bool vis = n >= it.key_lo && n < it.key_hi && n <= pos && (p.window <= 0 || n > pos - p.window);
                    sv[i] = vis ? sv[i] : -INFINITY;
                }
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < 32; ++i) mx[i & 3] = max3(mx[i & 3], sv[2 * i], sv[2 * i + 1]);
            const float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2;
            // The reference maximum moves only when the tile's maximum exceeds it by more than 2^8:
            // P stays below 256, exact enough in bfloat16 and float32, and O is seldom rescaled.
            const bool changed = m_tile > m_run + LAZY_LOG2;
            const float alpha = !changed ? 1.f : m_run == -INFINITY ? 0.f : ex2(m_run - m_tile);
            if (changed) m_run = m_tile;
            const float neg_m = m_run == -INFINITY ? 0.f : -m_run;
            // P goes back to tensor memory, two bfloat16 per column, over the first half of S[b]
            // (all of S[b] is in registers by now); the second product reads it from there.
            unsigned long long ls2[4] = {0ull, 0ull, 0ull, 0ull};           // four pairs of partial sums
            const unsigned long long scale2 = pack2(scale_log2, scale_log2), negm2 = pack2(neg_m, neg_m);
            float packed[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                // a masked score is -inf: fma gives -inf and the exponential 0
                float x0, x1;
                unpack2(fma2(pack2(sv[2 * i], sv[2 * i + 1]), scale2, negm2), x0, x1);
                const float p0 = ex2(x0), p1 = ex2(x1);
                ls2[i & 3] = add2(ls2[i & 3], pack2(p0, p1));
                __nv_bfloat162 bb = __floats2bfloat162_rn(p0, p1);
                packed[i] = __uint_as_float(*reinterpret_cast<uint32_t*>(&bb));
            }
            tmem_st32(tmem_row + b * 64, packed);
            float la, lb, lc, ld;
            unpack2(add2(ls2[0], ls2[1]), la, lb);
            unpack2(add2(ls2[2], ls2[3]), lc, ld);
            l_run = l_run * alpha + ((la + lb) + (lc + ld));
            // O is rescaled once the product of the tile before is done
            if (t >= 1 && __any_sync(0xffffffffu, changed)) {
                mbar_wait(&pv_done[b ^ 1], ((t - 1) >> 1) & 1);
                __syncwarp();
                fence_after_sync();
#pragma unroll
                for (int c = 0; c < PANELS; ++c) {
                    tmem_ld64(tmem_o + c * 64, sv);
#pragma unroll
                    for (int i = 0; i < 64; ++i) sv[i] *= alpha;
                    tmem_st32(tmem_o + c * 64, reinterpret_cast<const float(&)[32]>(sv[0]));
                    tmem_st32(tmem_o + c * 64 + 32, reinterpret_cast<const float(&)[32]>(sv[32]));
                    tmem_st_wait();
                }
            }
            if (kbase < it.key_lo || kbase + BN > it.key_hi) {
                // Value rows of keys outside the range are zeroed, so that 0 * anything stays 0 (a
                // page may hold anything behind the last token).
                mbar_wait(&v_full[t % STAGES], (t / STAGES) & 1);
                unsigned char* vd = Vs + (t % STAGES) * K_BYTES;
                for (int e = tid; e < BN * 8 * PANELS; e += SOFTMAX_WARPS * 32) {      // panels are [64 keys][8 chunks]
                    const int n = kbase + ((e >> 3) & (BN - 1));
                    if (n < it.key_lo || n >= it.key_hi) *reinterpret_cast<uint4*>(vd + e * 16) = make_uint4(0, 0, 0, 0);
                }
                fence_async_smem();                                  // generic stores -> tensor-core reads
            }
            tmem_st_wait();
            fence_before_sync();
            mbar_arrive(&p_full[b]);
        }
        if (n_tiles > 0) {
            const int last = n_tiles - 1;
            mbar_wait(&pv_done[last & 1], (last >> 1) & 1);
            __syncwarp();
            fence_after_sync();
            const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
            const int tok = R / G, head = kvh * G + R % G;
#pragma unroll
            for (int c = 0; c < PANELS; ++c) {
                tmem_ld64(tmem_o + c * 64, sv);                      // every thread of the warp takes part in the load
                if (pos >= 0) {
                    __nv_bfloat16* o_row = (__nv_bfloat16*)p.out + (size_t)(it.q0 + tok) * p.out_stride + head * D + c * 64;
#pragma unroll
                    for (int c8 = 0; c8 < 8; ++c8) {
                        __nv_bfloat162 bb[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            bb[i] = __floats2bfloat162_rn(sv[c8 * 8 + 2 * i] * inv, sv[c8 * 8 + 2 * i + 1] * inv);
                        *reinterpret_cast<uint4*>(o_row + c8 * 8) = *reinterpret_cast<uint4*>(bb);
                    }
                }
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == MMA_WARP)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS));
}

// The tensor map of one layer of a pool: rows of one head (p.d bfloat16), boxes of min(page
// size, 64) rows by 64 columns.
inline bool kv_tensor_map(CUtensorMap* out, const AttnParams& p) {
    return tensor_map_bf16(out, p.kv, (unsigned long long)p.num_pages * 2 * p.nkv * p.ps, p.d, p.d, p.ps < BN ? p.ps : BN);
}

// Whether this kernel takes the call: a page is a power of two of at least 8 tokens and the
// pool's row numbers fit the 32-bit coordinates of a box.
inline bool takes(const AttnParams& p) {
    return p.ps_shift >= 3 && p.num_pages > 0 && (long long)p.num_pages * 2 * p.nkv * p.ps < (1ll << 31) &&
           ((uintptr_t)p.kv & 15) == 0;
}

template <int D, bool WIDE>
inline int launch_as(const AttnParams& p, cudaStream_t stream) {
    static bool attr_set = false;
    auto kernel = attn_tc2_kernel<D, WIDE>;
    if (!attr_set) {
        PL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Shape<D>::SMEM_BYTES));
        PL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                     (int)cudaSharedmemCarveoutMaxShared));
        attr_set = true;
    }
    alignas(64) CUtensorMap map;
    if (!kv_tensor_map(&map, p)) return 1;
    PL_CUDA(launch_pdl(kernel, dim3(p.n_work * p.nkv), dim3(THREADS), (size_t)Shape<D>::SMEM_BYTES, stream, p, map));
    return 0;
}

// p.d must be D.
template <int D>
inline int launch(const AttnParams& p, cudaStream_t stream) {
    if constexpr (D == 128) {
        static const bool narrow = getenv("PAGED_LLM_B200_TC2_NARROW") != nullptr;   // one product per value panel
        return narrow ? launch_as<D, false>(p, stream) : launch_as<D, true>(p, stream);
    }
    return launch_as<D, false>(p, stream);
}

}  // namespace tc2

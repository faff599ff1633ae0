// Weight-streaming matrix product for few tokens (decode steps, small portions):
// Y[M,N] = X[M,K] * W[N,K]^T with M <= 16, bfloat16 in, float32 accumulation.
//
// At these sizes the product is a read of W at HBM speed and nothing else, so the
// kernel is built around that read.  It is persistent (one thread block per SM,
// each taking 16-row blocks of W round-robin) and warp-specialised: a producer
// warp pulls W into a ring of shared-memory stages with TMA bulk copies
// (cp.async.bulk, one row segment of 1,024 k each, completion counted on
// mbarriers) and runs ahead across block boundaries, so the stream never drains;
// eight consumer warps split every stage between them and feed the tensor cores
// (mma.sync m16n8k16 with W as the 16-row operand and the tokens as the 8-wide
// one); their partial sums meet in shared memory at the end of a block.  The
// producer starts before the kernel waits for the kernel in front of it
// (programmatic dependent launch): weights never depend on it, so the ring is
// full when the wait returns and consecutive products of a decode step stream
// weights back to back.  Every wait on a barrier is bounded: after a limit it
// counts a timeout (pl_gemm_skinny_timeouts) and goes on without hanging.
//
// The 16 rows of a block are chosen so that the epilogue needs no second kernel:
//   plain    rows n0..n0+15;                      y = acc (bfloat16 or float32)
//   SiLU     8 gate rows and the 8 matching up rows;   y = silu(gate) * up
//            (xiyiji/paged-llm llama.py:171)
//   rotary   8 elements of the first half of a head and their 8 partners of the
//            second half; q and k are rotated (llama.py:117-128), k and v are
//            written to their page slots (kv_cache.py:42-45), q goes to Y.
//   add      the product is a branch of the residual stream: x += y in float32
//            (llama.py:183-184); each block also leaves the sums of squares of
//            its 16 columns of the new x.
// And the prologue can normalise: with `norm` set, X is the float32 residual
// stream x, the sums of squares that an "add" product left are added up in a
// fixed order, and the operand is RMSNorm(x) * w (llama.py:80-83) formed while it
// is loaded.  So a layer of a decode step is five kernels: q/k/v + rotary + cache
// write, attention, o-proj + add, gate/up + SiLU, down + add.
// For a given token the order of summation never depends on M, so a token's
// result does not depend on what else is in the batch.
#include "common.cuh"

enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_SILU = 2, EPI_ROPE = 3, EPI_ADD = 4 };

struct SkinnyParams {
    const void* X;               // [M, ldx] bfloat16, or the float32 residual stream if norm is set
    const __nv_bfloat16* W;      // [N, K]
    void* Y;                     // [M, ldy]
    int ldx, ldy, M, N, K;
    int num_blocks;              // 16-row blocks of this product
    int I;                       // SiLU: N == 2 * I
    // rotary + cache write
    int nh, nkv, d, ps, bt_stride, num_pages, table_len, write;
    const float2* table;         // [positions, d/2] (cos, sin)
    const int* positions;        // [M]
    const int* token_seq;        // [M] row of the request of each token (-1: padding)
    const int* block_table;      // [requests, bt_stride]
    __nv_bfloat16* kv;           // [pages, 2, nkv, ps, d]
    // add: resid[M, N] += bf16(acc); part_out[block][16] = sums of squares of the block's columns
    float* resid;
    float* part_out;
    // normalising prologue: X = RMSNorm(x) * norm_w with sum(x^2) from part_in[K/16][16]
    const float* part_in;
    const void* norm_w;          // [K]
    int norm_w_bf16;
    float eps;
};

namespace {

constexpr int SK_CONSUMERS = 8;
constexpr int SK_THREADS = (SK_CONSUMERS + 1) * 32;
constexpr int SK_KC = 1024;              // k elements of one pipeline stage (2 KiB per row)
constexpr int SK_ROW_PAD = 64;           // bytes between rows of a stage beyond the data: no bank conflicts
constexpr int SK_STAGE_PITCH = SK_KC * 2 + SK_ROW_PAD;
constexpr int SK_STAGE_BYTES = 16 * SK_STAGE_PITCH;
constexpr int SK_STAGES = 6;
constexpr unsigned SK_SPIN_LIMIT = 1u << 21;

__device__ int g_skinny_timeouts = 0;    // waits that gave up (never expected; read by pl_gemm_skinny_timeouts)

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// X was written by the kernel in front, which may still have been running when this block
// started: read it through L2, not through a read-only path that assumes it never changes.
__device__ __forceinline__ uint4 ld_coherent(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(bar)) : "memory");
}
// Bounded wait: gives up after SK_SPIN_LIMIT polls, counts the timeout and returns false.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (unsigned i = 0; i < SK_SPIN_LIMIT; ++i) {
        uint32_t done;
        asm volatile(
            "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done)
            : "r"(smem_addr(bar)), "r"(parity)
            : "memory");
        if (done) return true;
    }
    atomicAdd(&g_skinny_timeouts, 1);
    return false;
}
// One row segment global -> shared through the TMA unit; completion is counted on `bar`.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                     smem_addr(dst)),
                 "l"(src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}
// Barrier among the consumer warps only (the producer warp runs on its own).
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(SK_CONSUMERS * 32) : "memory"); }

// Row of W that local row r (0..15) of block c stands for, or -1.
template <int EPI>
__device__ __forceinline__ int map_row(const SkinnyParams& p, int c, int r) {
    if (EPI == EPI_SILU) {
        const int j = c * 8 + (r & 7);
        return j < p.I ? (r < 8 ? j : p.I + j) : -1;
    }
    if (EPI == EPI_ROPE) {
        const int per_head = p.d / 16;
        const int head = c / per_head, blk = c - head * per_head;
        return head * p.d + (r < 8 ? 0 : p.d / 2) + blk * 8 + (r & 7);
    }
    const int n = c * 16 + r;
    return n < p.N ? n : -1;
}

// The 8 operand elements x[k..k+8) of one token as four bfloat16 pairs.
template <bool NORM>
__device__ __forceinline__ uint4 load_x(const SkinnyParams& p, const void* row, int k, float scale) {
    if (!NORM) return ld_coherent((const __nv_bfloat16*)row + k);
    const float4 a = __ldcg(reinterpret_cast<const float4*>((const float*)row + k));
    const float4 b = __ldcg(reinterpret_cast<const float4*>((const float*)row + k + 4));
    float w[8];
    if (p.norm_w_bf16) {
        const uint4 wv = *reinterpret_cast<const uint4*>((const __nv_bfloat16*)p.norm_w + k);
        const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            w[2 * i] = __low2float(w2[i]);
            w[2 * i + 1] = __high2float(w2[i]);
        }
    } else {
        const float4 w0 = *reinterpret_cast<const float4*>((const float*)p.norm_w + k);
        const float4 w1 = *reinterpret_cast<const float4*>((const float*)p.norm_w + k + 4);
        w[0] = w0.x; w[1] = w0.y; w[2] = w0.z; w[3] = w0.w;
        w[4] = w1.x; w[5] = w1.y; w[6] = w1.z; w[7] = w1.w;
    }
    __nv_bfloat162 o[4];
    o[0] = __floats2bfloat162_rn(a.x * scale * w[0], a.y * scale * w[1]);
    o[1] = __floats2bfloat162_rn(a.z * scale * w[2], a.w * scale * w[3]);
    o[2] = __floats2bfloat162_rn(b.x * scale * w[4], b.y * scale * w[5]);
    o[3] = __floats2bfloat162_rn(b.z * scale * w[6], b.w * scale * w[7]);
    return *reinterpret_cast<uint4*>(o);
}

// Shared memory: [stages][16 rows][SK_STAGE_PITCH] weights; red[2][8][NT][32][4]; inv[16] (+ scratch);
// full[stages], empty[stages] barriers.
// XC > 0: K has at most XC stages and the X fragments of all of them stay in registers for
// every row block of this thread block (they do not depend on the row block).  XC == 0: X is
// fetched stage by stage, one stage ahead.
template <int EPI, int NT, bool NORM, int XC>
__global__ void __launch_bounds__(SK_THREADS, 1) gemm_skinny_kernel(SkinnyParams p) {
    extern __shared__ __align__(128) unsigned char sk_smem[];
    unsigned char* wbuf = sk_smem;
    float* red = reinterpret_cast<float*>(sk_smem + (size_t)SK_STAGES * SK_STAGE_BYTES);   // [2][8][NT][32][4]
    float* inv = red + 2 * SK_CONSUMERS * NT * 128;                                        // [16] + [16][16] scratch
    uint64_t* full = reinterpret_cast<uint64_t*>(inv + 16 + 256);
    uint64_t* empty = full + SK_STAGES;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int chunks = (p.K + SK_KC - 1) / SK_KC;

    if (threadIdx.x == 0) {
        for (int s = 0; s < SK_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], SK_CONSUMERS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == SK_CONSUMERS) {
        // Producer.  Lanes 0..15 each fetch one row of a stage.  Rows outside the matrix read
        // row 0 (their results are dropped at the store).  It does not wait for the kernel in
        // front: the weights do not depend on it.
        int it = 0;
        for (int c = blockIdx.x; c < p.num_blocks; c += gridDim.x) {
            const int row = map_row<EPI>(p, c, lane & 15);
            const __nv_bfloat16* src = p.W + (size_t)max(row, 0) * p.K;
            for (int chunk = 0; chunk < chunks; ++chunk, ++it) {
                const int s = it % SK_STAGES, round = it / SK_STAGES;
                if (round > 0) mbar_wait(&empty[s], (round - 1) & 1);
                const int k0 = chunk * SK_KC;
                const uint32_t bytes = (uint32_t)min(SK_KC, p.K - k0) * 2u;
                if (lane == 0) mbar_expect_tx(&full[s], bytes * 16u);
                __syncwarp();
                if (lane < 16)
                    bulk_load(wbuf + (size_t)s * SK_STAGE_BYTES + (size_t)lane * SK_STAGE_PITCH, src + k0, bytes, &full[s]);
            }
        }
        return;
    }

    // Consumers.
    const int g = lane >> 2, t = lane & 3;
    // Rotary epilogue: position, request and page of the two tokens this thread finishes.  They
    // are step metadata, complete before any kernel of the step started, so they are fetched
    // before the wait for the kernel in front.
    int r_seq[2] = {-1, -1}, r_pos[2] = {-1, -1}, r_page[2] = {-1, -1};
    if (EPI == EPI_ROPE && warp < NT) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int tok = warp * 8 + 2 * t + e;
            if (tok < p.M) {
                r_seq[e] = p.token_seq[tok];
                r_pos[e] = p.positions[tok];
            }
        }
#pragma unroll
        for (int e = 0; e < 2; ++e)
            if (p.write && r_seq[e] >= 0 && r_pos[e] >= 0)
                r_page[e] = p.block_table[(size_t)r_seq[e] * p.bt_stride + r_pos[e] / p.ps];
    }
    pdl_wait();
    const unsigned char* x_row[NT];
    const size_t x_elem = NORM ? 4 : 2;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
        x_row[nt] = (const unsigned char*)p.X + (size_t)min(nt * 8 + g, p.M - 1) * p.ldx * x_elem;

    constexpr int SLABS_PER_WARP = SK_KC / 32 / SK_CONSUMERS;     // 4
    // With the normalising prologue the operand of a stage is fetched raw (float32 stream and
    // norm weights) and scaled and packed afterwards.  All loads go out before the first value
    // is used.
    struct RawX {
        float4 xa[NT][SLABS_PER_WARP], xb[NT][SLABS_PER_WARP];
        float w[SLABS_PER_WARP][8];
    };
    auto raw_load = [&](RawX& r, int chunk) {
        const int k_base = chunk * SK_KC + warp * SLABS_PER_WARP * 32 + 8 * t;
#pragma unroll
        for (int u = 0; u < SLABS_PER_WARP; ++u) {
            const int k = min(k_base + u * 32, p.K - 8);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                r.xa[nt][u] = __ldcg(reinterpret_cast<const float4*>((const float*)x_row[nt] + k));
                r.xb[nt][u] = __ldcg(reinterpret_cast<const float4*>((const float*)x_row[nt] + k + 4));
            }
            if (p.norm_w_bf16) {
                const uint4 wv = __ldg(reinterpret_cast<const uint4*>((const __nv_bfloat16*)p.norm_w + k));
                const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    r.w[u][2 * i] = __low2float(w2[i]);
                    r.w[u][2 * i + 1] = __high2float(w2[i]);
                }
            } else {
                const float4 w0 = __ldg(reinterpret_cast<const float4*>((const float*)p.norm_w + k));
                const float4 w1 = __ldg(reinterpret_cast<const float4*>((const float*)p.norm_w + k + 4));
                r.w[u][0] = w0.x; r.w[u][1] = w0.y; r.w[u][2] = w0.z; r.w[u][3] = w0.w;
                r.w[u][4] = w1.x; r.w[u][5] = w1.y; r.w[u][6] = w1.z; r.w[u][7] = w1.w;
            }
        }
    };
    // The first stage's raw values are asked for before the sums of squares: the two round trips
    // to L2 overlap.
    RawX raw0;
    if (NORM) raw_load(raw0, 0);
    float scale[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) scale[nt] = 1.f;
    if (NORM) {
        // sum(x^2) of every token from the partial sums the product in front left, in a fixed order
        float* slice_sum = inv + 16;
        const int tid = threadIdx.x, tok = tid & 15, slice = tid >> 4, nb = p.K / 16;
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
        int b = slice;
        for (; b + 112 < nb; b += 128) {                 // eight loads in flight per thread
            const float v0 = __ldcg(p.part_in + (size_t)b * 16 + tok), v1 = __ldcg(p.part_in + (size_t)(b + 16) * 16 + tok);
            const float v2 = __ldcg(p.part_in + (size_t)(b + 32) * 16 + tok), v3 = __ldcg(p.part_in + (size_t)(b + 48) * 16 + tok);
            const float v4 = __ldcg(p.part_in + (size_t)(b + 64) * 16 + tok), v5 = __ldcg(p.part_in + (size_t)(b + 80) * 16 + tok);
            const float v6 = __ldcg(p.part_in + (size_t)(b + 96) * 16 + tok), v7 = __ldcg(p.part_in + (size_t)(b + 112) * 16 + tok);
            s0 += v0; s1 += v1; s2 += v2; s3 += v3;
            s0 += v4; s1 += v5; s2 += v6; s3 += v7;
        }
        for (; b + 48 < nb; b += 64) {
            s0 += __ldcg(p.part_in + (size_t)b * 16 + tok);
            s1 += __ldcg(p.part_in + (size_t)(b + 16) * 16 + tok);
            s2 += __ldcg(p.part_in + (size_t)(b + 32) * 16 + tok);
            s3 += __ldcg(p.part_in + (size_t)(b + 48) * 16 + tok);
        }
        for (; b < nb; b += 16) s0 += __ldcg(p.part_in + (size_t)b * 16 + tok);
        slice_sum[slice * 16 + tok] = (s0 + s1) + (s2 + s3);
        consumer_sync();
        if (tid < 16) {
            float sum = 0.f;
#pragma unroll
            for (int sl = 0; sl < 16; ++sl) sum += slice_sum[sl * 16 + tid];
            inv[tid] = 1.0f / sqrtf(sum / (float)p.K + p.eps);
        }
        consumer_sync();
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) scale[nt] = inv[min(nt * 8 + g, 15)];
    }
    // X does not depend on the row block, only on the chunk: the fragments of the next chunk
    // are fetched while the current one is multiplied, so their latency hides behind the
    // wait for the weights.
    auto raw_finish = [&](uint4 (&dst)[NT][SLABS_PER_WARP], const RawX& r, int chunk) {
        const int k_base = chunk * SK_KC + warp * SLABS_PER_WARP * 32 + 8 * t;
#pragma unroll
        for (int u = 0; u < SLABS_PER_WARP; ++u)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const float sc = scale[nt];
                const float4 a = r.xa[nt][u], b = r.xb[nt][u];
                __nv_bfloat162 o[4];
                o[0] = __floats2bfloat162_rn(a.x * sc * r.w[u][0], a.y * sc * r.w[u][1]);
                o[1] = __floats2bfloat162_rn(a.z * sc * r.w[u][2], a.w * sc * r.w[u][3]);
                o[2] = __floats2bfloat162_rn(b.x * sc * r.w[u][4], b.y * sc * r.w[u][5]);
                o[3] = __floats2bfloat162_rn(b.z * sc * r.w[u][6], b.w * sc * r.w[u][7]);
                dst[nt][u] = (k_base + u * 32 < p.K) ? *reinterpret_cast<uint4*>(o) : make_uint4(0, 0, 0, 0);
            }
    };
    auto fetch_x = [&](uint4 (&dst)[NT][SLABS_PER_WARP], int chunk) {
        const int k_base = chunk * SK_KC + warp * SLABS_PER_WARP * 32 + 8 * t;
        if (!NORM) {
#pragma unroll
            for (int u = 0; u < SLABS_PER_WARP; ++u)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    dst[nt][u] = (k_base + u * 32 < p.K) ? load_x<false>(p, x_row[nt], k_base + u * 32, 1.f)
                                                         : make_uint4(0, 0, 0, 0);
            return;
        }
        RawX r;
        raw_load(r, chunk);
        raw_finish(dst, r, chunk);
    };
    auto multiply = [&](float (&acc)[NT][4], const uint4 (&x)[NT][SLABS_PER_WARP], int chunk, int it) {
        const int s = it % SK_STAGES;
        const int k_base = chunk * SK_KC + warp * SLABS_PER_WARP * 32 + 8 * t;
        mbar_wait(&full[s], (it / SK_STAGES) & 1);
        const unsigned char* st = wbuf + (size_t)s * SK_STAGE_BYTES + (size_t)(warp * SLABS_PER_WARP * 64 + 16 * t);
#pragma unroll
        for (int u = 0; u < SLABS_PER_WARP; ++u) {
            if (k_base + u * 32 < p.K) {
                const uint4 wl = *reinterpret_cast<const uint4*>(st + (size_t)g * SK_STAGE_PITCH + u * 64);
                const uint4 wh = *reinterpret_cast<const uint4*>(st + (size_t)(g + 8) * SK_STAGE_PITCH + u * 64);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    mma16816(acc[nt], wl.x, wh.x, wl.y, wh.y, x[nt][u].x, x[nt][u].y);
                    mma16816(acc[nt], wl.z, wh.z, wl.w, wh.w, x[nt][u].z, x[nt][u].w);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);            // the stage may be refilled
    };

    constexpr int XR = XC > 0 ? XC : 1;
    uint4 xres[XR][NT][SLABS_PER_WARP];
    uint4 xv[NT][SLABS_PER_WARP], xn[NT][SLABS_PER_WARP];
    if (XC > 0) {
        if (NORM) raw_finish(xres[0], raw0, 0);
        else fetch_x(xres[0], 0);
#pragma unroll
        for (int ch = 1; ch < XR; ++ch)
            if (ch < chunks) fetch_x(xres[ch], ch);
    } else {
        if (NORM) raw_finish(xv, raw0, 0);
        else fetch_x(xv, 0);
    }
    int it = 0, blk_i = 0;
    for (int c = blockIdx.x; c < p.num_blocks; c += gridDim.x, ++blk_i) {
        const int row_lo = map_row<EPI>(p, c, g), row_hi = map_row<EPI>(p, c, g + 8);
        // What the epilogue will read is requested now, so that its latency hides behind the
        // product: the residual values of the two tokens this thread finishes (warps < NT only).
        float x_lo[2] = {0.f, 0.f}, x_hi[2] = {0.f, 0.f};
        float2 r_cs[2] = {make_float2(1.f, 0.f), make_float2(1.f, 0.f)};      // (cos, sin) of the pair this thread rotates
        if (EPI == EPI_ROPE && warp < NT && row_lo >= 0) {
            const int head = row_lo / p.d, i_lo = row_lo - head * p.d;
#pragma unroll
            for (int e = 0; e < 2; ++e)
                if (head < p.nh + p.nkv && r_seq[e] >= 0 && r_pos[e] >= 0 && r_pos[e] < p.table_len)
                    r_cs[e] = __ldg(p.table + (size_t)r_pos[e] * (p.d / 2) + i_lo);
        }
        if (EPI == EPI_ADD && warp < NT) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int tok = warp * 8 + 2 * t + e;
                if (tok < p.M) {
                    if (row_lo >= 0) x_lo[e] = __ldcg(p.resid + (size_t)tok * p.N + row_lo);
                    if (row_hi >= 0) x_hi[e] = __ldcg(p.resid + (size_t)tok * p.N + row_hi);
                }
            }
        }
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;

        if (XC > 0) {
#pragma unroll
            for (int ch = 0; ch < XR; ++ch)
                if (ch < chunks) multiply(acc, xres[ch], ch, it++);
        } else {
            for (int chunk = 0; chunk < chunks; ++chunk, ++it) {
                fetch_x(xn, chunk + 1 < chunks ? chunk + 1 : 0);
                multiply(acc, xv, chunk, it);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int u = 0; u < SLABS_PER_WARP; ++u) xv[nt][u] = xn[nt][u];
            }
        }

        float* rbuf = red + (size_t)(blk_i & 1) * SK_CONSUMERS * NT * 128;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
            *reinterpret_cast<float4*>(rbuf + ((size_t)(warp * NT + nt) * 32 + lane) * 4) =
                make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
        consumer_sync();
        if (warp >= NT) continue;
        const int nt = warp;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int w = 0; w < SK_CONSUMERS; ++w) {
            const float4 f = *reinterpret_cast<const float4*>(rbuf + ((size_t)(w * NT + nt) * 32 + lane) * 4);
            v[0] += f.x;
            v[1] += f.y;
            v[2] += f.z;
            v[3] += f.w;
        }
        // v[0], v[1]: row_lo for tokens tok0, tok0 + 1; v[2], v[3]: row_hi for the same tokens
        const int tok0 = nt * 8 + 2 * t;
        float ss[2] = {0.f, 0.f};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int tok = tok0 + e;
            if (tok >= p.M) continue;
            const float lo = v[e], hi = v[2 + e];
            if (EPI == EPI_BF16) {
                __nv_bfloat16* y = (__nv_bfloat16*)p.Y + (size_t)tok * p.ldy;
                if (row_lo >= 0) y[row_lo] = __float2bfloat16_rn(lo);
                if (row_hi >= 0) y[row_hi] = __float2bfloat16_rn(hi);
            } else if (EPI == EPI_F32) {
                float* y = (float*)p.Y + (size_t)tok * p.ldy;
                if (row_lo >= 0) y[row_lo] = lo;
                if (row_hi >= 0) y[row_hi] = hi;
            } else if (EPI == EPI_ADD) {
                // the branch is rounded to bfloat16 first, as a separate product would store it
                float* x = p.resid + (size_t)tok * p.N;
                if (row_lo >= 0) {
                    const float nx = x_lo[e] + __bfloat162float(__float2bfloat16_rn(lo));
                    x[row_lo] = nx;
                    ss[e] += nx * nx;
                }
                if (row_hi >= 0) {
                    const float nx = x_hi[e] + __bfloat162float(__float2bfloat16_rn(hi));
                    x[row_hi] = nx;
                    ss[e] += nx * nx;
                }
            } else if (EPI == EPI_SILU) {
                if (row_lo >= 0) {
                    const float gate = __bfloat162float(__float2bfloat16_rn(lo));
                    const float up = __bfloat162float(__float2bfloat16_rn(hi));
                    ((__nv_bfloat16*)p.Y)[(size_t)tok * p.ldy + row_lo] =
                        __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
                }
            } else {
                const int head = row_lo / p.d, i_lo = row_lo - head * p.d, i_hi = i_lo + p.d / 2;
                float a = __bfloat162float(__float2bfloat16_rn(lo)), b = __bfloat162float(__float2bfloat16_rn(hi));
                const int s = r_seq[e];
                const int pos = r_pos[e];
                {
                    const float2 cs = r_cs[e];                  // (1, 0) where nothing is rotated
                    const float ra = a * cs.x - b * cs.y, rb = b * cs.x + a * cs.y;
                    a = ra;
                    b = rb;
                }
                const __nv_bfloat16 oa = __float2bfloat16_rn(a), ob = __float2bfloat16_rn(b);
                __nv_bfloat16* y = (__nv_bfloat16*)p.Y + (size_t)tok * p.ldy + head * p.d;
                y[i_lo] = oa;
                y[i_hi] = ob;
                if (head >= p.nh && p.write && s >= 0) {
                    const int page = r_page[e];
                    if (page >= 0 && page < p.num_pages) {
                        const int kvh = head - p.nh;
                        const int sel = kvh >= p.nkv ? 1 : 0;
                        const int hh = sel ? kvh - p.nkv : kvh;
                        __nv_bfloat16* dst = p.kv + ((((size_t)page * 2 + sel) * p.nkv + hh) * p.ps + pos % p.ps) * p.d;
                        dst[i_lo] = oa;
                        dst[i_hi] = ob;
                    }
                }
            }
        }
        if (EPI == EPI_ADD) {
            // sum over the 8 row pairs (lanes that share t); one lane per token pair stores
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                ss[e] += __shfl_xor_sync(0xffffffffu, ss[e], 4);
                ss[e] += __shfl_xor_sync(0xffffffffu, ss[e], 8);
                ss[e] += __shfl_xor_sync(0xffffffffu, ss[e], 16);
            }
            if (g == 0) {
                p.part_out[(size_t)c * 16 + tok0] = ss[0];
                p.part_out[(size_t)c * 16 + tok0 + 1] = ss[1];
            }
        }
    }
}

int g_num_sms = 0;

template <int EPI, int NT, bool NORM, int XC>
int launch_skinny(const SkinnyParams& p, cudaStream_t stream) {
    constexpr size_t smem = (size_t)SK_STAGES * SK_STAGE_BYTES + (size_t)2 * SK_CONSUMERS * NT * 128 * sizeof(float) +
                            (16 + 256) * sizeof(float) + 2 * SK_STAGES * sizeof(uint64_t);
    static bool attr_set = false;
    if (!attr_set) {
        PL_CUDA(cudaFuncSetAttribute(gemm_skinny_kernel<EPI, NT, NORM, XC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set = true;
    }
    if (g_num_sms == 0) {
        int dev = 0;
        PL_CUDA(cudaGetDevice(&dev));
        PL_CUDA(cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev));
    }
    const int grid = p.num_blocks < g_num_sms ? p.num_blocks : g_num_sms;
    PL_CUDA(launch_pdl(gemm_skinny_kernel<EPI, NT, NORM, XC>, dim3(grid), dim3(SK_THREADS), smem, stream, p));
    return 0;
}

template <int EPI, bool NORM>
int dispatch_skinny(const SkinnyParams& p, cudaStream_t stream) {
    const int chunks = (p.K + SK_KC - 1) / SK_KC;
    if (p.M <= 8) {
        if (chunks <= 2) return launch_skinny<EPI, 1, NORM, 2>(p, stream);
        if (chunks <= 6) return launch_skinny<EPI, 1, NORM, 6>(p, stream);
        return launch_skinny<EPI, 1, NORM, 0>(p, stream);
    }
    if (chunks <= 2) return launch_skinny<EPI, 2, NORM, 2>(p, stream);
    return launch_skinny<EPI, 2, NORM, 0>(p, stream);
}

int check_common(const SkinnyParams& p, const char* who) {
    PL_REQUIRE(p.M >= 1 && p.M <= 16, "%s: M=%d (1..16 tokens)", who, p.M);
    PL_REQUIRE(p.N >= 1 && p.K >= 32 && p.K % 32 == 0, "%s: N=%d K=%d (K must be a multiple of 32)", who, p.N, p.K);
    PL_REQUIRE(((uintptr_t)p.X & 15) == 0 && ((uintptr_t)p.W & 15) == 0, "%s: X and W must be 16-byte aligned", who);
    if (p.part_in != nullptr) {
        PL_REQUIRE(p.ldx % 4 == 0 && p.norm_w != nullptr && ((uintptr_t)p.norm_w & 15) == 0,
                   "%s: the float32 stream and the norm weight must be 16-byte aligned", who);
    } else {
        PL_REQUIRE(p.ldx % 8 == 0, "%s: rows of X must start on 16-byte boundaries", who);
    }
    return 0;
}

void set_norm(SkinnyParams& p, const float* part_in, const void* norm_w, int norm_w_dtype, float eps) {
    p.part_in = part_in;
    p.norm_w = norm_w;
    p.norm_w_bf16 = norm_w_dtype == PL_BF16;
    p.eps = eps;
}

}  // namespace

// Waits inside the kernel that gave up since the library was loaded (0 unless something is broken).
PL_EXPORT int pl_gemm_skinny_timeouts() {
    int n = 0;
    if (cudaMemcpyFromSymbol(&n, g_skinny_timeouts, sizeof(int)) != cudaSuccess) return -1;
    return n;
}

// Whether the sizes fit this kernel (the caller falls back to the library product otherwise).
PL_EXPORT int pl_gemm_skinny_supported(int M, int N, int K, int ldx) {
    return M >= 1 && M <= 16 && N >= 1 && K >= 32 && K % 32 == 0 && ldx % 8 == 0;
}

// In all entry points: with part_in non-null X is the float32 residual stream [M, ldx] and the
// operand is RMSNorm(X) * norm_w, sum(x^2) taken from part_in[K/16][16] (left by pl_gemm_skinny_add).

PL_EXPORT int pl_gemm_skinny(const void* X, int ldx, const void* W, void* Y, int ldy, int M, int N, int K,
                             int out_float32, const float* part_in, const void* norm_w, int norm_w_dtype, float eps,
                             cudaStream_t stream) {
    SkinnyParams p = {};
    p.X = X;
    p.W = (const __nv_bfloat16*)W;
    p.Y = Y;
    p.ldx = ldx;
    p.ldy = ldy;
    p.M = M;
    p.N = N;
    p.K = K;
    p.num_blocks = (N + 15) / 16;
    set_norm(p, part_in, norm_w, norm_w_dtype, eps);
    if (int rc = check_common(p, "gemm_skinny")) return rc;
    PL_REQUIRE(ldy >= N, "gemm_skinny: ldy=%d < N=%d", ldy, N);
    if (part_in) return out_float32 ? dispatch_skinny<EPI_F32, true>(p, stream) : dispatch_skinny<EPI_BF16, true>(p, stream);
    return out_float32 ? dispatch_skinny<EPI_F32, false>(p, stream) : dispatch_skinny<EPI_BF16, false>(p, stream);
}

// resid[M, N] += bf16(X W^T) in float32; part_out[ceil(N/16)][16] = sums of squares of each
// block's 16 columns of the new resid, per token.
PL_EXPORT int pl_gemm_skinny_add(const void* X, int ldx, const void* W, float* resid, int M, int N, int K,
                                 float* part_out, cudaStream_t stream) {
    SkinnyParams p = {};
    p.X = X;
    p.W = (const __nv_bfloat16*)W;
    p.ldx = ldx;
    p.ldy = N;
    p.M = M;
    p.N = N;
    p.K = K;
    p.num_blocks = (N + 15) / 16;
    p.resid = resid;
    p.part_out = part_out;
    if (int rc = check_common(p, "gemm_skinny_add")) return rc;
    return dispatch_skinny<EPI_ADD, false>(p, stream);
}

// Y[M, I] = silu(X Wg^T) * (X Wu^T), W = [Wg; Wu] of shape [2I, K].
PL_EXPORT int pl_gemm_skinny_silu(const void* X, int ldx, const void* W, void* Y, int ldy, int M, int I, int K,
                                  const float* part_in, const void* norm_w, int norm_w_dtype, float eps,
                                  cudaStream_t stream) {
    SkinnyParams p = {};
    p.X = X;
    p.W = (const __nv_bfloat16*)W;
    p.Y = Y;
    p.ldx = ldx;
    p.ldy = ldy;
    p.M = M;
    p.N = 2 * I;
    p.K = K;
    p.I = I;
    p.num_blocks = (I + 7) / 8;
    set_norm(p, part_in, norm_w, norm_w_dtype, eps);
    if (int rc = check_common(p, "gemm_skinny_silu")) return rc;
    PL_REQUIRE(ldy >= I, "gemm_skinny_silu: ldy=%d < I=%d", ldy, I);
    return part_in ? dispatch_skinny<EPI_SILU, true>(p, stream) : dispatch_skinny<EPI_SILU, false>(p, stream);
}

// Y[M, (nh + 2 nkv) d] = X W^T with q and k heads rotated (pairs i, i + d/2 over the whole
// head) and k, v written to their cache slots.
PL_EXPORT int pl_gemm_skinny_rope(const void* X, int ldx, const void* W, void* Y, int ldy, int M, int K, int nh,
                                  int nkv, int d, const float* table, int table_len, const int* positions,
                                  const int* token_seq, const int* block_table, int bt_stride, void* kv,
                                  int num_pages, int ps, int write, const float* part_in, const void* norm_w,
                                  int norm_w_dtype, float eps, cudaStream_t stream) {
    SkinnyParams p = {};
    p.X = X;
    p.W = (const __nv_bfloat16*)W;
    p.Y = Y;
    p.ldx = ldx;
    p.ldy = ldy;
    p.M = M;
    p.N = (nh + 2 * nkv) * d;
    p.K = K;
    p.nh = nh;
    p.nkv = nkv;
    p.d = d;
    p.ps = ps;
    p.bt_stride = bt_stride;
    p.num_pages = num_pages;
    p.table_len = table_len;
    p.write = write;
    p.table = (const float2*)table;
    p.positions = positions;
    p.token_seq = token_seq;
    p.block_table = block_table;
    p.kv = (__nv_bfloat16*)kv;
    p.num_blocks = (nh + 2 * nkv) * (d / 16);
    set_norm(p, part_in, norm_w, norm_w_dtype, eps);
    if (int rc = check_common(p, "gemm_skinny_rope")) return rc;
    PL_REQUIRE(d % 16 == 0 && d > 0 && nh > 0 && nkv > 0 && ps > 0, "gemm_skinny_rope: bad head sizes");
    PL_REQUIRE(ldy >= p.N, "gemm_skinny_rope: ldy=%d < %d", ldy, p.N);
    return part_in ? dispatch_skinny<EPI_ROPE, true>(p, stream) : dispatch_skinny<EPI_ROPE, false>(p, stream);
}

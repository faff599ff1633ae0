// Matrix product for many tokens (prompt portions) on the 5th-generation tensor cores:
// Y[M,N] = X[M,K] * W[N,K]^T, bfloat16 in, float32 accumulation in tensor memory, with the
// elementwise work that follows a projection done in the epilogue.  This header holds what the
// kernel (gemm_tc_duo.cuh) is made of: parameters, mbarrier and TMA helpers, and the epilogue of
// one accumulator row.
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

// a block's part of a tile: 128 tokens x 256 features, 64 k per stage
constexpr int TC_BM = 128, TC_BN = 256, TC_BK = 64, TC_THREADS = 192;

__device__ __forceinline__ void tc_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(saddr(bar)) : "memory");
}
__device__ __forceinline__ void tc_arrive_expect(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(saddr(bar)), "r"(bytes) : "memory");
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

}  // namespace

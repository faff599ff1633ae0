// Paged attention in bfloat16 on the tensor cores (mma.sync m16n8k16, float32
// accumulation), one instantiation per padded head size PL_DPAD.
//
// A thread block takes one item of the work list for one kv head: a tile of
// query rows (row = token * G + head within the group, so the G query heads that
// share a kv head sit in the same tile and read each key once) and a range of
// keys.  Keys and values are fetched page by page through the block table with
// cp.async into double-buffered shared memory, zero-filled outside the range, so
// stale or poisoned pages never reach a product.  Scores, running maximum, sum
// and the output accumulator are float32; probabilities are rounded to bfloat16
// for the second product, as the reference's kernel does
// (xiyiji/paged-llm pagedllm/attention/triton_kernel.py:76-89).
//
// Two shapes: "large" (4 warps x 16 rows, 64 keys per iteration) for prefill
// portions, and "small" (16 rows, 4 warps that each take other keys and are
// merged at the end) for decoding, where a split range per block keeps the
// machine busy on few requests.
#pragma once

#include <cooperative_groups.h>

#include "attention_common.cuh"

namespace {

namespace cg = cooperative_groups;

constexpr int kAttnMaxDevices = 64;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Rotates eight pairs (x[i], x[i + d/2]), i = i0..i0+7, of a head at position `pos`: lo and hi hold
// the two halves' elements as bfloat16; the angles come from the float32 table [positions][d/2]
// (cos, sin).  A position beyond the table is left unrotated (the engine refuses such a step earlier).
__device__ __forceinline__ void rotate_pair(uint4& lo, uint4& hi, const float2* table, int table_len, int pos, int d, int i0) {
    if (pos < 0 || pos >= table_len) return;
    __nv_bfloat162* a = reinterpret_cast<__nv_bfloat162*>(&lo);
    __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&hi);
    const float4* cs = reinterpret_cast<const float4*>(table + (size_t)pos * (d / 2) + i0);      // two (cos, sin) per float4
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float4 t = __ldg(cs + k);
        const float2 x = __bfloat1622float2(a[k]), y = __bfloat1622float2(b[k]);
        a[k] = __floats2bfloat162_rn(x.x * t.x - y.x * t.y, x.y * t.z - y.y * t.w);
        b[k] = __floats2bfloat162_rn(y.x * t.x + x.x * t.y, y.y * t.z + x.y * t.w);
    }
}

template <int DPAD, int MW, int NW, int KPW, int STAGES = 2>
struct AttnShape {
    static constexpr int BM = 16 * MW, BN = KPW * NW, PITCH = DPAD + 8, THREADS = 32 * MW * NW;
    static constexpr int Q_BYTES = BM * PITCH * 2;                                // Q tile
    static constexpr int SMEM_BYTES = Q_BYTES + 2 * STAGES * BN * PITCH * 2;      // then K and V stages
};

// CLUSTER: the blocks of a thread-block cluster take the splits of one (request, kv head) and
// merge their partial results through distributed shared memory: no partials in global memory,
// no counter, no work list.
// MOD: the score modifiers of AttnParams (cap, bias by distance) are applied; the kernel without
// them is the one the Llama decoder runs and carries none of their code.
// STAGES: key tiles in flight (a ring of that many K and V stages).
// ROPE (cluster form only): q, k, v arrive as the projection left them.  The queries are rotated as
// they are loaded (xiyiji/paged-llm llama.py:117-128: pairs i, i + d/2, float32 angles from the
// table), the step's own keys are rotated, written to their page slots together with the values
// (kv_cache.py:42-45) and taken from registers instead of from the cache: the separate kernel for
// rotary positions and the cache write is not needed.
// WP (small shape only): every warp runs a copy pipeline of its own for the keys it multiplies, so
// that the loop over key tiles has no block-wide barrier and the warps drift apart: one computes
// while another waits for its keys.
template <int DPAD, int MW, int NW, int KPW, bool CLUSTER = false, bool MOD = false, int STAGES = 2, bool ROPE = false,
          bool WP = false>
__global__ void __launch_bounds__(32 * MW * NW) attn_bf16_kernel(AttnParams p) {
    static_assert(!ROPE || CLUSTER, "rotary positions inside the kernel: cluster form only");
    static_assert(!WP || MW == 1, "warp-private pipelines: small shape only");
    using Shape = AttnShape<DPAD, MW, NW, KPW, STAGES>;
    constexpr int BM = Shape::BM, BN = Shape::BN, PITCH = Shape::PITCH, THREADS = Shape::THREADS;
    constexpr int CH = DPAD / 8;                          // 16-byte chunks per row
    constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;
    pdl_launch_dependents();
    // A cluster block (a decode step) waits for the kernel in front only after it has asked for its
    // first keys: lengths, block tables and all keys but the step's own are older than the step.
    if (!CLUSTER) {
        pdl_wait();
        attn_zero_padding<__nv_bfloat16>(p);
    }
    // kv heads of an item side by side: the list's longest-first order holds over heads
    const AttnItem it = CLUSTER ? attn_cluster_item(p, blockIdx.x / (p.cluster * p.nkv), blockIdx.x % p.cluster, p.cluster)
                                : attn_decode_item(p, blockIdx.x / p.nkv, BM, BN);
    if (!it.valid) {                 // the same for all blocks of a cluster
        if (CLUSTER) {
            pdl_wait();
            attn_zero_padding<__nv_bfloat16>(p);
        }
        return;
    }

    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem_raw + Shape::Q_BYTES);     // [STAGES][BN][PITCH]
    __nv_bfloat16* Vs = Ks + STAGES * BN * PITCH;                                          // [STAGES][BN][PITCH]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp % MW, wn = warp / MW;
    const int d = p.d, kvh = CLUSTER ? (blockIdx.x / p.cluster) % p.nkv : blockIdx.x % p.nkv, G = p.nh / p.nkv;
    const __nv_bfloat16* q = (const __nv_bfloat16*)p.q;
    const __nv_bfloat16* kv = (const __nv_bfloat16*)p.kv;
    const int* bt = p.block_table + (size_t)it.seq * p.bt_stride;
    const size_t v_off = (size_t)p.nkv * p.ps * d;
    // The step's own keys (the last nq of the request) are written by the kernel in front, or, with
    // ROPE, made here: then the tiles below stop in front of them and they come as a tile of their own.
    const int own_lo = CLUSTER ? it.lk - it.nq : 0x7fffffff;
    const int main_hi = ROPE ? min(it.key_hi, max(own_lo, it.key_lo)) : it.key_hi;
    int hi_cur = main_hi;                                  // keys at or behind it are not part of the tile at hand

    // One key tile: every thread first looks up the pages of all its rows (independent loads
    // that travel together), then issues the copies.
    constexpr int LOAD_ITERS = (BN * CH + THREADS - 1) / THREADS;
    // With warp-private pipelines a warp copies the KPW rows it multiplies (the same number of copies per
    // thread).  A thread's copies of a tile lie J_STEP rows apart in one 16-byte column, so that everything
    // but the page is known before the loop over the tiles.
    constexpr int E_STEP = WP ? 32 : THREADS, E_COUNT = WP ? KPW * CH : BN * CH, J_STEP = E_STEP / CH;
    static_assert(E_STEP % CH == 0, "a thread's copies stay in one column");
    const int e_first = WP ? lane : tid;
    const int c8 = e_first % CH, j0 = (WP ? wn * KPW : 0) + e_first / CH;
    const bool col_ok = c8 * 8 < d;
    const size_t page_stride = (size_t)2 * p.nkv * p.ps * d;
    const __nv_bfloat16* kv_head = kv + (size_t)kvh * p.ps * d + c8 * 8;
    const int smem_off0 = j0 * PITCH + c8 * 8;
    // Keys of the range at or behind `skip_from` are left alone (neither copied nor zero-filled).
    // With `only_from` set, only keys from there on are copied and nothing else is touched.
    auto load_tile = [&](int stage, int kt, int skip_from = 0x7fffffff, int only_from = -1) {
        __nv_bfloat16* kd = Ks + stage * BN * PITCH + smem_off0;
        __nv_bfloat16* vd = Vs + stage * BN * PITCH + smem_off0;
        int pg[LOAD_ITERS];
#pragma unroll
        for (int i = 0; i < LOAD_ITERS; ++i) {
            const int n = kt + j0 + i * J_STEP;
            const bool ok = e_first + i * E_STEP < E_COUNT && col_ok && n < main_hi && n < skip_from && n >= only_from;
            const int pi = p.ps_shift >= 0 ? n >> p.ps_shift : n / p.ps;
            pg[i] = ok ? bt[pi] : -1;
        }
#pragma unroll
        for (int i = 0; i < LOAD_ITERS; ++i) {
            if (e_first + i * E_STEP >= E_COUNT) break;
            const int n = kt + j0 + i * J_STEP;
            if (n >= skip_from && n < main_hi) continue;          // keys past the range are still zero-filled
            if (only_from >= 0 && (n < only_from || n >= main_hi)) continue;
            const int po = p.ps_shift >= 0 ? n & (p.ps - 1) : n % p.ps;
            const bool ok = pg[i] >= 0;
            const __nv_bfloat16* src = ok ? kv_head + (size_t)pg[i] * page_stride + po * d : kv;
            cp_async16(kd + i * J_STEP * PITCH, src, ok ? 16 : 0);
            cp_async16(vd + i * J_STEP * PITCH, ok ? src + v_off : kv, ok ? 16 : 0);
        }
        cp_async_commit();
    };

    const int g = lane >> 2, t4 = lane & 3;
    int pos[2];
    float slope[2];
    constexpr bool modified = MOD;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int R = it.row_base + wm * 16 + g + 8 * h;
        pos[h] = R < it.rows_total ? it.lk - it.nq + R / G : -1;
        slope[h] = MOD && p.slopes != nullptr && R < it.rows_total ? p.slopes[kvh * G + R % G] : 0.f;
    }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float oacc[DPAD / 8][4];
#pragma unroll
    for (int j = 0; j < DPAD / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[j][e] = 0.f;
    const float scale_log2 = p.scale * LOG2E;

    const int n_tiles = (main_hi - it.key_lo + BN - 1) / BN;
    // The first keys are on their way while Q is fetched.  A cluster block has not waited for the
    // kernel in front yet: the keys and values of this step's own tokens, which that kernel
    // writes, are left out of the first copy and fetched after the wait, in a group of their own
    // that the loop waits for together with the tile.
    if (n_tiles > 0) load_tile(0, it.key_lo, own_lo);
    else cp_async_commit();
    if (CLUSTER) {
        pdl_wait();
        attn_zero_padding<__nv_bfloat16>(p);
        // (with ROPE they are made further down instead)
        if (!ROPE && n_tiles > 0) load_tile(0, it.key_lo, 0x7fffffff, max(own_lo, it.key_lo));
        else cp_async_commit();
    }
    // the tiles behind the first, up to the depth of the ring; every position of the sequence of
    // copy groups is committed (empty if there is no such tile), so that the waits below can count
#pragma unroll
    for (int t = 1; t < STAGES - 1; ++t) {
        if (t < n_tiles) load_tile(t, it.key_lo + t * BN);
        else cp_async_commit();
    }
    if (ROPE) {
        // chunk c8 of the first half of a head with its partner in the second half; columns from d on are zero
        const int hc = d / 16;                               // chunks per half
        for (int e = tid; e < BM * hc; e += THREADS) {
            const int r = e / hc, c8 = e - r * hc;
            const int R = it.row_base + r;
            uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
            if (R < it.rows_total) {
                const __nv_bfloat16* src = q + (size_t)(it.q0 + R / G) * p.q_stride + (kvh * G + R % G) * d + c8 * 8;
                lo = *reinterpret_cast<const uint4*>(src);
                hi = *reinterpret_cast<const uint4*>(src + d / 2);
                rotate_pair(lo, hi, p.rope_table, p.rope_len, it.lk - it.nq + R / G, d, c8 * 8);
            }
            *reinterpret_cast<uint4*>(Qs + r * PITCH + c8 * 8) = lo;
            *reinterpret_cast<uint4*>(Qs + r * PITCH + d / 2 + c8 * 8) = hi;
        }
        const int padc = CH - 2 * hc;
        for (int e = tid; e < BM * padc; e += THREADS)
            *reinterpret_cast<uint4*>(Qs + (e / padc) * PITCH + d + (e % padc) * 8) = make_uint4(0, 0, 0, 0);
    } else {
        for (int e = tid; e < BM * CH; e += THREADS) {
            const int r = e / CH, c8 = e - r * CH;
            const int R = it.row_base + r;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (R < it.rows_total && c8 * 8 < d)
                v = *reinterpret_cast<const uint4*>(q + (size_t)(it.q0 + R / G) * p.q_stride + (kvh * G + R % G) * d + c8 * 8);
            *reinterpret_cast<uint4*>(Qs + r * PITCH + c8 * 8) = v;
        }
    }
    // scores, softmax and weighted values of the keys [tile_lo, tile_lo + BN) that lie in `stage`
    auto process_tile = [&](int stage, int tile_lo) {
        const __nv_bfloat16* kst = Ks + stage * BN * PITCH + wn * KPW * PITCH;
        const __nv_bfloat16* vst = Vs + stage * BN * PITCH + wn * KPW * PITCH;
        const int kbase = tile_lo + wn * KPW;
        if (kbase < hi_cur) {                                  // uniform per warp
            float sacc[KPW / 8][4];
#pragma unroll
            for (int j = 0; j < KPW / 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) sacc[j][e] = 0.f;
#pragma unroll
            for (int kk = 0; kk < DPAD / 16; ++kk) {
                uint32_t a[4];
                ldmatrix_x4(a, Qs + (wm * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + kk * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int n2 = 0; n2 < KPW / 16; ++n2) {
                    uint32_t b[4];
                    ldmatrix_x4(b, kst + (n2 * 16 + (lane & 7) + (lane >> 4) * 8) * PITCH + kk * 16 + ((lane >> 3) & 1) * 8);
                    mma_bf16(sacc[2 * n2], a, b[0], b[1]);
                    mma_bf16(sacc[2 * n2 + 1], a, b[2], b[3]);
                }
            }
            // scale, mask, running maximum.  A tile whose keys all lie at or before the first
            // row's position (and inside the window and the range) needs no mask.
            // (rows that pad the tile carry zero queries and are never stored: they need no mask)
            const int pos_min_warp = __reduce_min_sync(0xffffffffu, min(pos[0] < 0 ? 0x7fffffff : pos[0],
                                                                        pos[1] < 0 ? 0x7fffffff : pos[1]));
            const bool full_tile = !modified && p.window <= 0 && kbase + KPW <= hi_cur && kbase + KPW - 1 <= pos_min_warp;
            float mx[2] = {-INFINITY, -INFINITY};
            if (full_tile) {
#pragma unroll
                for (int j = 0; j < KPW / 8; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float s = sacc[j][e] * scale_log2;
                        sacc[j][e] = s;
                        mx[e >> 1] = fmaxf(mx[e >> 1], s);
                    }
            } else {
#pragma unroll
                for (int j = 0; j < KPW / 8; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int n = kbase + 8 * j + 2 * t4 + (e & 1);
                        const int pr = pos[e >> 1];
                        const bool vis = n < hi_cur && n <= pr && (p.window <= 0 || n > pr - p.window);
                        const float s = !vis ? -INFINITY
                                        : modified ? attn_score(p, sacc[j][e], slope[e >> 1], n, pr) * LOG2E
                                                   : sacc[j][e] * scale_log2;
                        sacc[j][e] = s;
                        mx[e >> 1] = fmaxf(mx[e >> 1], s);
                    }
            }
            float alpha[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                const float m_new = fmaxf(m_run[h], mx[h]);
                alpha[h] = m_run[h] == -INFINITY ? 0.f : fast_exp2(m_run[h] - m_new);
                m_run[h] = m_new;
                l_run[h] *= alpha[h];
            }
            uint32_t pa[KPW / 16][4];
#pragma unroll
            for (int j = 0; j < KPW / 8; ++j) {
                float pv[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float s = sacc[j][e];
                    pv[e] = s == -INFINITY ? 0.f : fast_exp2(s - m_run[e >> 1]);
                    l_run[e >> 1] += pv[e];
                }
                pa[j >> 1][(j & 1) * 2 + 0] = pack_bf16(pv[0], pv[1]);
                pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(pv[2], pv[3]);
            }
            // the accumulator is rescaled only if a row's maximum moved in this warp (a factor of exactly 1
            // changes nothing): after the first tiles of a long context it seldom does
            if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
                for (int j = 0; j < DPAD / 8; ++j) {
                    oacc[j][0] *= alpha[0];
                    oacc[j][1] *= alpha[0];
                    oacc[j][2] *= alpha[1];
                    oacc[j][3] *= alpha[1];
                }
            }
#pragma unroll
            for (int k2 = 0; k2 < KPW / 16; ++k2) {
#pragma unroll
                for (int d2 = 0; d2 < DPAD / 16; ++d2) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, vst + (k2 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + d2 * 16 + (lane >> 4) * 8);
                    mma_bf16(oacc[2 * d2], pa[k2], b[0], b[1]);
                    mma_bf16(oacc[2 * d2 + 1], pa[k2], b[2], b[3]);
                }
            }
        }
    };

    if (WP) __syncthreads();          // Q is in shared memory for all warps; from here on the warps run apart
    for (int t = 0; t < n_tiles; ++t) {
        // tile t + STAGES - 1 goes into the stage that tile t - 1 left (all warps are past it: the
        // barrier at the end of the iteration before); then all copies but those of the STAGES - 1
        // newest groups are awaited, which completes tile t (and the step's own keys)
        if (t + STAGES - 1 < n_tiles) load_tile((t + STAGES - 1) % STAGES, it.key_lo + (t + STAGES - 1) * BN);
        else cp_async_commit();
        cp_async_wait<STAGES - 1>();
        if (WP) __syncwarp(); else __syncthreads();
        process_tile(t % STAGES, it.key_lo + t * BN);
        if (WP) __syncwarp(); else __syncthreads();
    }
    if (ROPE && it.key_hi > main_hi) {
        // The step's own keys of this block's range, as a last tile in stage 0: rotated keys and values
        // straight from the projection, also written to their page slots; the rest of the first warp's
        // rows is zeroed (a masked score still multiplies its value row).
        if (WP) __syncthreads();                                          // all warps are out of stage 0
        const int own0 = main_hi, n_own = it.key_hi - main_hi;            // at most BM keys
        const int hc = d / 16, padc = CH - 2 * hc;
        for (int e = tid; e < KPW * hc; e += THREADS) {
            const int j = e / hc, c8 = e - j * hc;
            uint4 klo = make_uint4(0, 0, 0, 0), khi = klo, vlo = klo, vhi = klo;
            if (j < n_own) {
                const int n = own0 + j;                                    // position of the key
                const __nv_bfloat16* row = q + (size_t)(it.q0 + n - (it.lk - it.nq)) * p.q_stride;
                const __nv_bfloat16* ks = row + (size_t)(p.nh + kvh) * d + c8 * 8;
                const __nv_bfloat16* vs = row + (size_t)(p.nh + p.nkv + kvh) * d + c8 * 8;
                klo = *reinterpret_cast<const uint4*>(ks);
                khi = *reinterpret_cast<const uint4*>(ks + d / 2);
                vlo = *reinterpret_cast<const uint4*>(vs);
                vhi = *reinterpret_cast<const uint4*>(vs + d / 2);
                rotate_pair(klo, khi, p.rope_table, p.rope_len, n, d, c8 * 8);
                const int pi = p.ps_shift >= 0 ? n >> p.ps_shift : n / p.ps;
                const int po = p.ps_shift >= 0 ? n & (p.ps - 1) : n % p.ps;
                const int pg = bt[pi];
                if (pg >= 0 && (p.num_pages <= 0 || pg < p.num_pages)) {
                    __nv_bfloat16* dst = const_cast<__nv_bfloat16*>(kv) + ((((size_t)pg * 2) * p.nkv + kvh) * p.ps + po) * d + c8 * 8;
                    *reinterpret_cast<uint4*>(dst) = klo;
                    *reinterpret_cast<uint4*>(dst + d / 2) = khi;
                    *reinterpret_cast<uint4*>(dst + v_off) = vlo;
                    *reinterpret_cast<uint4*>(dst + v_off + d / 2) = vhi;
                }
            }
            *reinterpret_cast<uint4*>(Ks + j * PITCH + c8 * 8) = klo;
            *reinterpret_cast<uint4*>(Ks + j * PITCH + d / 2 + c8 * 8) = khi;
            *reinterpret_cast<uint4*>(Vs + j * PITCH + c8 * 8) = vlo;
            *reinterpret_cast<uint4*>(Vs + j * PITCH + d / 2 + c8 * 8) = vhi;
        }
        for (int e = tid; e < KPW * padc; e += THREADS) {
            *reinterpret_cast<uint4*>(Ks + (e / padc) * PITCH + d + (e % padc) * 8) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(Vs + (e / padc) * PITCH + d + (e % padc) * 8) = make_uint4(0, 0, 0, 0);
        }
        __syncthreads();
        hi_cur = it.key_hi;
        if (wn == 0) process_tile(0, own0);
        __syncthreads();
    }

    // merge the warps that took different keys, then write
    __syncthreads();          // the Q region is reused below, also when no key tile ran
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    float* red_ml = reinterpret_cast<float*>(smem_raw);                     // [NW][BM][2] in the Q region
    float* red_o = reinterpret_cast<float*>(smem_raw + Shape::Q_BYTES);     // [NW][BM][DPAD] in the K/V region
    float* cpart = red_o + (size_t)NW * BM * DPAD;                          // [BM][DPAD + 2]: this block's partial (CLUSTER)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = wm * 16 + g + 8 * h;
        if (t4 == 0) {
            red_ml[(wn * BM + r) * 2 + 0] = m_run[h];
            red_ml[(wn * BM + r) * 2 + 1] = l_run[h];
        }
#pragma unroll
        for (int j = 0; j < DPAD / 8; ++j) {
            float2 v = make_float2(oacc[j][2 * h], oacc[j][2 * h + 1]);
            *reinterpret_cast<float2*>(red_o + ((size_t)(wn * BM + r)) * DPAD + 8 * j + 2 * t4) = v;
        }
    }
    __syncthreads();
    for (int e = tid; e < BM * (DPAD / 2); e += THREADS) {
        const int r = e / (DPAD / 2), c = (e - r * (DPAD / 2)) * 2;
        const int R = it.row_base + r;
        if (R >= it.rows_total || c >= d) continue;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) M = fmaxf(M, red_ml[(w * BM + r) * 2]);
        float L = 0.f, o0 = 0.f, o1 = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float mw = red_ml[(w * BM + r) * 2];
            if (mw == -INFINITY) continue;
            const float f = NW == 1 ? 1.f : fast_exp2(mw - M);
            L += red_ml[(w * BM + r) * 2 + 1] * f;
            const float2 v = *reinterpret_cast<const float2*>(red_o + ((size_t)(w * BM + r)) * DPAD + c);
            o0 += v.x * f;
            o1 += v.y * f;
        }
        const int tok = R / G, head = kvh * G + R % G;
        if (CLUSTER) {
            float* part = cpart + (size_t)r * (DPAD + 2);
            if (c == 0) {
                part[0] = M;                          // base-2 units
                part[1] = L;
            }
            part[2 + c] = o0;
            part[3 + c] = o1;
        } else if (it.splits <= 1) {
            const float inv = L > 0.f ? 1.0f / L : 0.f;
            __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)(it.q0 + tok) * p.out_stride + head * d + c;
            *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(o0 * inv, o1 * inv);
        } else {
            if (!attn_partial_fits(p, it.scratch_base + tok)) continue;      // a row outside the declared scratch
            float* part = attn_partial(p, it.scratch_base + tok, head, it.split);
            if (c == 0) {
                part[0] = M == -INFINITY ? -INFINITY : M * LN2;
                part[1] = L;
            }
            part[2 + c] = o0;
            part[3 + c] = o1;
        }
    }
    if (CLUSTER) {
        // Every block of the cluster merges its share of the column pairs over all blocks'
        // partials, read from their shared memory.
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        const int C = it.splits, rank = it.split;
        const int pairs = d / 2;
        for (int e = tid; e < it.rows_total * pairs; e += THREADS) {
            const int R = e / pairs, cp = e - R * pairs;
            if (cp % C != rank) continue;
            const int c = cp * 2;
            float M = -INFINITY;
            for (int j = 0; j < C; ++j) M = fmaxf(M, cluster.map_shared_rank(cpart, j)[(size_t)R * (DPAD + 2)]);
            float L = 0.f, o0 = 0.f, o1 = 0.f;
            for (int j = 0; j < C; ++j) {
                const float* pj = cluster.map_shared_rank(cpart, j) + (size_t)R * (DPAD + 2);
                const float mj = pj[0];
                if (mj == -INFINITY) continue;
                const float f = fast_exp2(mj - M);
                L += pj[1] * f;
                const float2 v = *reinterpret_cast<const float2*>(pj + 2 + c);
                o0 += v.x * f;
                o1 += v.y * f;
            }
            const float inv = L > 0.f ? 1.0f / L : 0.f;
            const int tok = R / G, head = kvh * G + R % G;
            __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)(it.q0 + tok) * p.out_stride + head * d + c;
            *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(o0 * inv, o1 * inv);
        }
        cluster.sync();              // nobody leaves while its shared memory is still read
        return;
    }
    if (it.splits <= 1 || p.counters == nullptr) return;

    // The block of this request and kv head that finishes last merges the splits.
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (tid == 0) is_last = atomicAdd(&p.counters[(size_t)it.seq * p.nkv + kvh], 1u) == (unsigned)it.splits - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // (m, l) of every row and split go to shared memory in one parallel pass, the factors are
    // formed there, then every thread adds up one column pair over the splits.
    float* ml = reinterpret_cast<float*>(smem_raw);                          // [rows][splits][2] -> factors
    const int n_ml = it.rows_total * it.splits;
    for (int e = tid; e < n_ml; e += THREADS) {
        const int R = e / it.splits, j = e - R * it.splits;
        const float2 v = __ldcg(reinterpret_cast<const float2*>(attn_partial(p, it.scratch_base + R / G, kvh * G + R % G, j)));
        ml[2 * e] = v.x;
        ml[2 * e + 1] = v.y;
    }
    __syncthreads();
    for (int R = tid; R < it.rows_total; R += THREADS) {
        float M = -INFINITY;
        for (int j = 0; j < it.splits; ++j) M = fmaxf(M, ml[2 * (R * it.splits + j)]);
        float L = 0.f;
        for (int j = 0; j < it.splits; ++j) {
            const float mj = ml[2 * (R * it.splits + j)];
            const float f = mj == -INFINITY ? 0.f : __expf(mj - M);
            L += ml[2 * (R * it.splits + j) + 1] * f;
            ml[2 * (R * it.splits + j)] = f;
        }
        const float inv = L > 0.f ? 1.0f / L : 0.f;
        for (int j = 0; j < it.splits; ++j) ml[2 * (R * it.splits + j)] *= inv;
    }
    __syncthreads();
    for (int e = tid; e < it.rows_total * (d / 2); e += THREADS) {
        const int R = e / (d / 2), c = (e - R * (d / 2)) * 2;
        const int tok = R / G, head = kvh * G + R % G;
        const float* part0 = attn_partial(p, it.scratch_base + tok, head, 0) + 2 + c;
        const size_t stride = (size_t)(d + 2);
        float o0 = 0.f, o1 = 0.f;
        int j = 0;
        for (; j + 4 <= it.splits; j += 4) {
            const float2 v0 = __ldcg(reinterpret_cast<const float2*>(part0 + (j + 0) * stride));
            const float2 v1 = __ldcg(reinterpret_cast<const float2*>(part0 + (j + 1) * stride));
            const float2 v2 = __ldcg(reinterpret_cast<const float2*>(part0 + (j + 2) * stride));
            const float2 v3 = __ldcg(reinterpret_cast<const float2*>(part0 + (j + 3) * stride));
            const float f0 = ml[2 * (R * it.splits + j)], f1 = ml[2 * (R * it.splits + j + 1)];
            const float f2 = ml[2 * (R * it.splits + j + 2)], f3 = ml[2 * (R * it.splits + j + 3)];
            o0 += v0.x * f0 + v1.x * f1 + v2.x * f2 + v3.x * f3;
            o1 += v0.y * f0 + v1.y * f1 + v2.y * f2 + v3.y * f3;
        }
        for (; j < it.splits; ++j) {
            const float2 v = __ldcg(reinterpret_cast<const float2*>(part0 + j * stride));
            const float f = ml[2 * (R * it.splits + j)];
            o0 += v.x * f;
            o1 += v.y * f;
        }
        __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)(it.q0 + tok) * p.out_stride + head * d + c;
        *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(o0, o1);
    }
    if (tid == 0) p.counters[(size_t)it.seq * p.nkv + kvh] = 0u;      // ready for the next launch
}

template <int DPAD, int MW, int NW, int KPW, bool MOD = false, int STAGES = 2, bool WP = false>
int launch_attn_bf16(const AttnParams& p, cudaStream_t stream) {
    using Shape = AttnShape<DPAD, MW, NW, KPW, STAGES>;
    auto kernel = attn_bf16_kernel<DPAD, MW, NW, KPW, false, MOD, STAGES, false, WP>;
    static bool attr_set[kAttnMaxDevices] = {};         // function attributes are per device
    int dev = 0;
    PL_CUDA(cudaGetDevice(&dev));
    PL_REQUIRE(dev >= 0 && dev < kAttnMaxDevices, "attention_bf16: device index %d is out of range", dev);
    if (!attr_set[dev]) {
        PL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Shape::SMEM_BYTES));
        attr_set[dev] = true;
    }
    PL_CUDA(launch_pdl(kernel, dim3(p.n_work * p.nkv), dim3(Shape::THREADS), (size_t)Shape::SMEM_BYTES, stream, p));
    return 0;
}

// The cluster form of the small shape: p.n_work requests, p.cluster blocks per (request, kv head).
template <int DPAD, int KPW, bool MOD = false, int STAGES = 2, int NW = 4, bool ROPE = false, bool WP = false>
int launch_attn_cluster(const AttnParams& p, cudaStream_t stream) {
    using Shape = AttnShape<DPAD, 1, NW, KPW, STAGES>;
    // the merge of the warps reuses the K/V stages ([NW][BM][DPAD] float32); behind it, this block's partial.
    // (Letting the partial share the stages too would fit a third block of head size 128 on an SM; measured,
    // the decode step at Llama-3-8B sizes and batch 64 got 4 % slower by it: 512 blocks fall badly on 444 places.)
    constexpr size_t merge = (size_t)Shape::Q_BYTES + NW * Shape::BM * DPAD * 4;
    constexpr size_t smem = (Shape::SMEM_BYTES > merge ? Shape::SMEM_BYTES : merge) + Shape::BM * (DPAD + 2) * 4;
    auto kernel = attn_bf16_kernel<DPAD, 1, NW, KPW, true, MOD, STAGES, ROPE, WP>;
    static bool attr_set[kAttnMaxDevices] = {};
    int dev = 0;
    PL_CUDA(cudaGetDevice(&dev));
    PL_REQUIRE(dev >= 0 && dev < kAttnMaxDevices, "attention_bf16: device index %d is out of range", dev);
    if (!attr_set[dev]) {
        PL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        PL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));    // up to 16 blocks
        attr_set[dev] = true;
    }
    PL_REQUIRE(p.cluster >= 1 && p.cluster <= 16, "attention_bf16: clusters of 1 to 16 blocks, not %d", p.cluster);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.n_work * p.nkv * p.cluster);
    cfg.blockDim = dim3(Shape::THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = p.cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static const bool no_pdl = getenv("PAGED_LLM_B200_NO_PDL") != nullptr;
    cfg.numAttrs = no_pdl ? 1 : 2;
    PL_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
    return 0;
}

}  // namespace

#if PL_DPAD == 64 || PL_DPAD == 128
#include "attention_tc.cuh"
// Waits inside the tcgen05 kernel that gave up since the library was loaded (0 unless something is broken).
PL_EXPORT int pl_attention_tc_timeouts() {
    int n = 0;
    if (cudaMemcpyFromSymbol(&n, tc::g_timeouts, sizeof(int)) != cudaSuccess) return -1;
    return n;
}
#endif

#define PL_CAT_(a, b) a##b
#define PL_CAT(a, b) PL_CAT_(a, b)

// Tile rows of the two shapes, so that the host plans with the same numbers.
#define PL_LARGE_MW (PL_DPAD <= 128 ? 8 : 4)
PL_EXPORT int PL_CAT(pl_attention_bf16_rows_d, PL_DPAD)(int small) { return small ? 16 : 16 * PL_LARGE_MW; }

PL_EXPORT int PL_CAT(pl_attention_bf16_d, PL_DPAD)(const AttnParams* params, cudaStream_t stream) {
    AttnParams p = *params;
    if (p.n_work == 0) return 0;
    PL_REQUIRE(p.nh > 0 && p.nkv > 0 && p.nh % p.nkv == 0, "attention_bf16: %d query heads on %d kv heads", p.nh, p.nkv);
    PL_REQUIRE(p.d % 16 == 0 && p.d > 0 && p.d <= PL_DPAD, "attention_bf16: head_dim=%d does not fit this build (%d)",
               p.d, PL_DPAD);
    PL_REQUIRE(p.q_stride % 8 == 0 && p.out_stride % 2 == 0, "attention_bf16: row strides must keep 16-byte alignment");
    PL_REQUIRE(((uintptr_t)p.q & 15) == 0 && ((uintptr_t)p.kv & 15) == 0, "attention_bf16: q and kv must be 16-byte aligned");
    PL_REQUIRE(p.softcap >= 0.f, "attention_bf16: softcap=%f must not be negative", (double)p.softcap);
    // Shapes of the decode kernel, by measurement (B200; with so few warps per SM the dependent chain of a
    // warp and the shared memory a block takes decide): head sizes up to 64 walk 128 keys per tile, but 64
    // keys in a ring of three tiles where the work list says that the ranges are long (is_small == 2:
    // three blocks per SM, 18 against 26 us at 8 requests x 4,096 keys); head size 128 walks 64 keys per
    // tile in all forms (three blocks per SM instead of one: 1.7 times the speed); head size 256 keeps
    // 64 keys and two stages, which is what fits.
    constexpr int KPW_CLUSTER = PL_DPAD <= 64 ? 32 : 16;
    if (p.softcap > 0.f || p.slopes != nullptr) {
        PL_REQUIRE(p.rope_table == nullptr, "attention_bf16: score modifiers and rotary positions inside the kernel "
                                            "do not combine");
        // the score modifiers live in instantiations of their own of the mma.sync kernel (the tcgen05
        // kernels step aside for them)
        if (p.cluster > 0) return launch_attn_cluster<PL_DPAD, KPW_CLUSTER, true, 2, 4, false, true>(p, stream);
        if (p.is_small) return launch_attn_bf16<PL_DPAD, 1, 4, KPW_CLUSTER, true, 2, true>(p, stream);
        return launch_attn_bf16<PL_DPAD, PL_LARGE_MW, 1, 64, true>(p, stream);
    }
    // All forms of the small shape run warp-private copy pipelines (WP): 49 against 53 us at 64 requests x
    // 3,000 keys of head size 64, 110 against 115 at 8 x 16,384 of head size 128, no loss elsewhere.
    if (p.rope_table != nullptr) {
        // rotary positions and the cache write inside the kernel: the cluster form only (the caller knows)
        PL_REQUIRE(p.cluster > 0, "attention_bf16: rotary positions inside the kernel need the cluster form");
        PL_REQUIRE(p.d % 16 == 0 && p.rope_len > 0, "attention_bf16: bad rotary table");
#if PL_DPAD == 64
        return launch_attn_cluster<PL_DPAD, 16, false, 2, 8, true, true>(p, stream);
#else
        return launch_attn_cluster<PL_DPAD, KPW_CLUSTER, false, 2, 4, true, true>(p, stream);
#endif
    }
#if PL_DPAD == 64
    // eight warps of 16 keys each on a tile of 128 keys: shorter dependent chains per warp and twice the
    // warps per SM (13.5 against 14.2 us at 64 requests x 520 keys, 6.8 against 7.7 at 8, 5.1 against 5.8 at 1)
    if (p.cluster > 0) return launch_attn_cluster<PL_DPAD, 16, false, 2, 8, false, true>(p, stream);
    if (p.is_small == 2) return launch_attn_bf16<PL_DPAD, 1, 4, 16, false, 3, true>(p, stream);
    if (p.is_small) return launch_attn_bf16<PL_DPAD, 1, 8, 16, false, 2, true>(p, stream);
#elif PL_DPAD < 64
    if (p.cluster > 0) return launch_attn_cluster<PL_DPAD, KPW_CLUSTER, false, 2, 4, false, true>(p, stream);
    if (p.is_small == 2) return launch_attn_bf16<PL_DPAD, 1, 4, 16, false, 3, true>(p, stream);
    if (p.is_small) return launch_attn_bf16<PL_DPAD, 1, 4, KPW_CLUSTER, false, 2, true>(p, stream);
#else
    if (p.cluster > 0) return launch_attn_cluster<PL_DPAD, KPW_CLUSTER, false, 2, 4, false, true>(p, stream);
    if (p.is_small) return launch_attn_bf16<PL_DPAD, 1, 4, KPW_CLUSTER, false, 2, true>(p, stream);
#endif
#if PL_DPAD == 64 || PL_DPAD == 128
    // prefill tiles of head sizes 64 and 128 run on tcgen05 with tensor-memory accumulators
    static const bool no_tc = getenv("PAGED_LLM_B200_NO_TCGEN05") != nullptr;
#if PL_DPAD == 64
    static const bool serial_tc = getenv("PAGED_LLM_B200_TC_SERIAL") != nullptr;     // the block-synchronous variant
    if (p.d == 64 && !no_tc) return serial_tc || !tc2::takes(p) ? tc::launch(p, stream) : tc2::launch<64>(p, stream);
#else
    if (p.d == 128 && !no_tc && tc2::takes(p)) return tc2::launch<128>(p, stream);
#endif
#endif
    return launch_attn_bf16<PL_DPAD, PL_LARGE_MW, 1, 64>(p, stream);
}
